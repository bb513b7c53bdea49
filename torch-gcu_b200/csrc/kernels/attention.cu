// Scaled-dot-product attention forward (flash style) on tcgen05 tensor cores.
//
//   out = softmax(scale * Q K^T  [+ causal mask]) V,   lse = logsumexp rows
//   q (B,Hq,Sq,D), k/v (B,Hkv,Sk,D), D in {64,128}, Hq a multiple of Hkv (GQA),
//   bf16 or f16, last dim contiguous, other strides free.
//
// One CTA per (128 query rows, head, batch); 192 threads:
//   warp 0     TMA: Q tile once, then K / V tiles (128 keys) through a 2-stage ring
//   warp 1     tcgen05.mma: S_j = Q K_j^T into one of two S buffers in tensor
//              memory (so S_{j+1} is computed while the softmax of S_j runs), then
//              O += P_j V_j; V is consumed straight from its row-major tile as an
//              MN-major operand
//   warps 2-5  online softmax, one thread per query row: two passes over the S row
//              in tensor memory (max, then exp2 / sum), P_j written to shared
//              memory in the 128-byte-swizzled K-major layout the second MMA reads,
//              O rescaled in tensor memory only when a row maximum moved; at the
//              end O / l is rounded and stored, with lse.
// When the mask is not causal and groups*Sq <= 128 (decode), the query heads that
// share one KV head are packed into the 128 rows of one tile, so every K / V byte
// is read once per KV head instead of once per query head.
// Every barrier wait is bounded; loads never use cluster multicast.
#include "common.cuh"
#include "tc_common.cuh"

#include <cooperative_groups.h>
#include <math_constants.h>

namespace b200 {
unsigned int* device_error_word();

namespace {

using namespace tc;

constexpr int kAttThreads = 192;
constexpr int BQ = 128;   // query rows per tile (MMA M)
constexpr int BKV = 128;  // keys per tile
constexpr int kKVStages = 2;

struct AttnParams {
  int B, Hq, Hkv, Sq, Sk, D;
  int causal, packed, is_bf16;
  int pair_heads;    // prefill kernel: the CTA's two Q tiles are two heads of one KV group (else two row tiles)
  int items_x, items_y;   // prefill kernel: blocks of query rows, heads (or head pairs): the work items of its persistent CTAs
  float scale_log2;  // scale * log2(e)
  float scale;
  void* out;
  int64_t o_sb, o_sh, o_ss;  // element strides of out (B,Hq,Sq,D), D contiguous
  float* lse;                // (B,Hq,Sq) contiguous, may be null
  unsigned int* error_word;
};

template <int D> struct AttCfg {
  static constexpr int kHalves = D / 64;                 // 64-column (128-byte) slabs per row
  static constexpr int kQBytes = BQ * D * 2;
  static constexpr int kKVBytes = BKV * D * 2;
  static constexpr int kPBytes = BQ * BKV * 2;
  static constexpr int kSmem = kQBytes + kKVStages * 2 * kKVBytes + kPBytes + 1024 + 256;
  static constexpr int kOCol = 2 * BKV;                  // O accumulator after the two S buffers
  static constexpr int kTmemCols = 512;
};

template <int D>
__global__ void __launch_bounds__(kAttThreads, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const AttnParams p) {
  using Cfg = AttCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + Cfg::kQBytes;                      // [stage][K | V]
  uint8_t* sP = sKV + kKVStages * 2 * Cfg::kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + Cfg::kPBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;             // [2]
  uint64_t* v_full = bars + 3;             // [2]
  uint64_t* kv_empty = bars + 5;           // [2]
  uint64_t* s_full = bars + 7;             // [2]
  uint64_t* s_empty = bars + 9;            // [2]
  uint64_t* p_full = bars + 11;
  uint64_t* pv_done = bars + 12;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  int q0, hq, hkv, b = blockIdx.z;
  if (p.packed) {
    q0 = 0; hkv = blockIdx.y; hq = hkv * G;
  } else {
    const int qt = gridDim.x - 1 - blockIdx.x;  // longest (last) causal tiles first
    q0 = qt * BQ; hq = blockIdx.y; hkv = hq / G;
  }
  int n_kv = (p.Sk + BKV - 1) / BKV;
  if (p.causal) n_kv = min(n_kv, (q0 + BQ + BKV - 1) / BKV);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      prefetch_tmap(&tmap_q);
      prefetch_tmap(&tmap_k);
      prefetch_tmap(&tmap_v);
      if (p.packed) {
        // box (64, Sq, G, 1): rows ordered (group head, position); rest of the tile unused
        mbar_arrive_expect_tx(q_full, static_cast<uint32_t>(Cfg::kHalves * 128 * p.Sq * G));
#pragma unroll
        for (int h = 0; h < Cfg::kHalves; ++h) tma_load_4d(sQ + h * (BQ * 128), &tmap_q, q_full, h * 64, 0, hq, b);
      } else {
        mbar_arrive_expect_tx(q_full, Cfg::kQBytes);
#pragma unroll
        for (int h = 0; h < Cfg::kHalves; ++h) tma_load_4d(sQ + h * (BQ * 128), &tmap_q, q_full, h * 64, q0, hq, b);
      }
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1u) ^ 1u, abort_flag)) break;
        uint8_t* sK = sKV + st * 2 * Cfg::kKVBytes;
        uint8_t* sV = sK + Cfg::kKVBytes;
        mbar_arrive_expect_tx(&k_full[st], Cfg::kKVBytes);
#pragma unroll
        for (int h = 0; h < Cfg::kHalves; ++h) tma_load_4d(sK + h * (BKV * 128), &tmap_k, &k_full[st], h * 64, j * BKV, hkv, b);
        mbar_arrive_expect_tx(&v_full[st], Cfg::kKVBytes);
#pragma unroll
        for (int h = 0; h < Cfg::kHalves; ++h) tma_load_4d(sV + h * (BKV * 128), &tmap_v, &v_full[st], h * 64, j * BKV, hkv, b);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BQ, BKV, p.is_bf16 != 0, false, false);  // Q, K both K-major
      const uint32_t idesc_o = make_idesc(BQ, D, p.is_bf16 != 0, false, true);     // P K-major, V MN-major
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_s = [&](int j) {
        const uint32_t k_addr = smem_u32(sKV + (j & 1) * 2 * Cfg::kKVBytes);
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>((j & 1) * BKV);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (BQ * 128) + (kk % 4) * 32;
          umma_f16(d_tmem, smem_desc_sw128(q_addr + off, 16u, 1024u), smem_desc_sw128(k_addr + off, 16u, 1024u),
                   idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag) && n_kv > 0;
      if (ok) ok = mbar_wait(&k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < n_kv && ok; ++j) {
        if (j + 1 < n_kv) {
          const int jn = j + 1;
          if (!mbar_wait(&k_full[jn & 1], (jn >> 1) & 1u, abort_flag)) { ok = false; break; }
          if (!mbar_wait(&s_empty[jn & 1], ((jn >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_s(jn);
        }
        if (!mbar_wait(p_full, j & 1u, abort_flag)) { ok = false; break; }
        if (!mbar_wait(&v_full[j & 1], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sKV + (j & 1) * 2 * Cfg::kKVBytes + Cfg::kKVBytes);
        const uint32_t o_tmem = tmem_base + Cfg::kOCol;
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          // A = P: key slab kk/4, 32 bytes per step. B = V: 64-column slabs BKV*128 bytes
          // apart (LBO), 8-key groups 1024 bytes apart (SBO), 16 keys = 2048 bytes per step.
          const uint64_t da = smem_desc_sw128(p_addr + (kk / 4) * (BQ * 128) + (kk % 4) * 32, 16u, 1024u);
          const uint64_t db = smem_desc_sw128(v_addr + kk * 2048, BKV * 128, 1024u);
          umma_f16(o_tmem, da, db, idesc_o, (j | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&kv_empty[j & 1]);
        umma_commit(pv_done);
      }
    }
  } else {
    // ------------------------------------------------------ softmax / output --
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;             // row of the tile this thread owns
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    int qi, head;                                  // query position / head of this row
    bool row_valid;
    if (p.packed) {
      const int g = r / p.Sq;
      qi = r - g * p.Sq; head = hq + g; row_valid = r < G * p.Sq;
    } else {
      qi = q0 + r; head = hq; row_valid = qi < p.Sq;
    }
    float m = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int buf = j & 1;
      const int k0 = j * BKV;
      if (!mbar_wait(&s_full[buf], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_tmem = tmem_base + lane_sel + static_cast<uint32_t>(buf * BKV);
      const bool need_mask = (p.causal && k0 + BKV - 1 > q0) || (k0 + BKV > p.Sk);
      const int limit = p.causal ? min(p.Sk, qi + 1) : p.Sk;  // keys [0, limit) are visible
      // pass 1: row maximum
      float mx = -CUDART_INF_F;
#pragma unroll 1
      for (int c = 0; c < BKV; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(s_tmem + c, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(v[i]);
          if (need_mask && k0 + c + i >= limit) s = -CUDART_INF_F;
          mx = fmaxf(mx, s);
        }
      }
      const float m_new = fmaxf(m, mx);
      const float m_use = m_new == -CUDART_INF_F ? 0.f : m_new;
      const float alpha = exp2f((m - m_use) * p.scale_log2);  // m = -inf -> 0
      // P_{j-1} and the O accumulator are in use until the previous P.V finished
      if (j > 0) {
        if (!mbar_wait(pv_done, (j - 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, m_new > m)) {
#pragma unroll 1
          for (int c = 0; c < D; c += 16) {
            uint32_t o[16];
            tmem_ld_32x16(tmem_base + lane_sel + Cfg::kOCol + c, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x16(tmem_base + lane_sel + Cfg::kOCol + c, o);
          }
          tmem_wait_st();
        }
      }
      // pass 2: p = exp2((s - m) * scale*log2e), row sum, P tile to shared memory
      float sum = 0.f;
      const float mb = m_use * p.scale_log2;
#pragma unroll 1
      for (int c = 0; c < BKV; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(s_tmem + c, v);
        tmem_wait_ld();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float s0 = __uint_as_float(v[i]), s1 = __uint_as_float(v[i + 1]);
          float p0 = exp2f(fmaf(s0, p.scale_log2, -mb)), p1 = exp2f(fmaf(s1, p.scale_log2, -mb));
          if (need_mask) {
            if (k0 + c + i >= limit) p0 = 0.f;
            if (k0 + c + i + 1 >= limit) p1 = 0.f;
          }
          // the sum uses the rounded values, the ones the P.V product sees
          uint16_t b0, b1;
          if (p.is_bf16) { b0 = f32_to_bf16_bits(p0); b1 = f32_to_bf16_bits(p1); sum += bf16_bits_to_f32(b0) + bf16_bits_to_f32(b1); }
          else { b0 = f32_to_f16_bits(p0); b1 = f32_to_f16_bits(p1); sum += f16_bits_to_f32(b0) + f16_bits_to_f32(b1); }
          packed[i / 2] = static_cast<uint32_t>(b0) | (static_cast<uint32_t>(b1) << 16);
        }
        // row r, keys [c, c+32): slab c/64, four 16-byte chunks, XOR-swizzled by (r & 7)
        uint8_t* prow = sP + (c / 64) * (BQ * 128) + r * 128;
        const int chunk0 = (c % 64) / 8;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = (chunk0 + q) ^ (r & 7);
          *reinterpret_cast<uint4*>(prow + chunk * 16) =
              make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
        }
      }
      l = l * alpha + sum;
      m = m_new;
      // S_j consumed; P_j visible to the tensor core (async proxy); O rescaled
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[buf]);
        mbar_arrive(p_full);
      }
    }
    // epilogue: O / l
    if (ok && n_kv > 0) ok = mbar_wait(pv_done, (n_kv - 1) & 1u, abort_flag);
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      uint16_t* orow = static_cast<uint16_t*>(p.out) + b * p.o_sb + static_cast<int64_t>(head) * p.o_sh +
                       static_cast<int64_t>(qi) * p.o_ss;
      const bool vec_ok = (reinterpret_cast<uintptr_t>(orow) & 15) == 0;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t v[32];
        if (n_kv > 0) {
          tmem_ld_32x32(tmem_base + lane_sel + Cfg::kOCol + c, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (row_valid) {
          alignas(16) uint16_t o[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float x = __uint_as_float(v[i]) * inv;
            o[i] = p.is_bf16 ? f32_to_bf16_bits(x) : f32_to_f16_bits(x);
          }
          if (vec_ok) {
#pragma unroll
            for (int q = 0; q < 4; ++q) *reinterpret_cast<int4*>(orow + c + q * 8) = *reinterpret_cast<const int4*>(o + q * 8);
          } else {
            for (int i = 0; i < 32; ++i) orow[c + i] = o[i];
          }
        }
      }
      if (row_valid && p.lse) {
        const float lse = l > 0.f ? m * p.scale + logf(l) : -CUDART_INF_F;
        p.lse[(static_cast<int64_t>(b) * p.Hq + head) * p.Sq + qi] = lse;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_word, 2u);
}

// ---------------------------------------------------------------------------
// Prefill kernel: one CTA per (256 query rows, head, batch), 384 threads.
//   warp 0      TMA: two Q tiles once, K / V tiles through a 2-stage ring
//   warp 1      tcgen05.mma for both Q tiles in turn: S_t = Q_t K_j^T into that
//               tile's S buffer, then O_t += P_t V_j with P_t read from tensor memory
//   warps 4-7   softmax of tile 0, warps 8-11 softmax of tile 1 (2-3 idle), one thread per row:
//               the whole S row (128 fp32) is read once into registers, P_t is
//               written back over S_t as packed 16-bit pairs, so while one tile is
//               in its softmax the tensor core works on the other
// The running maximum is only advanced (and O rescaled) when it grew by more than
// 2^8 in the exponent, so most iterations touch O not at all; l and O stay
// consistent because both use the same stale maximum.
constexpr int kPrefillThreads = 384;  // registers are granted per 4 warps, so 10 warps cost as much as 12
constexpr float kRescaleThreshold = 8.0f;  // log2 units

template <int D> struct PrefillCfg {
  static constexpr int kHalves = D / 64;
  static constexpr int kQBytes = BQ * D * 2;     // one Q tile
  static constexpr int kKVBytes = BKV * D * 2;
  static constexpr int kOutBytes = 8 * 4096;   // per softmax warp: 32 rows x 64 columns staged for the output store
  static constexpr int kSmem = 2 * kQBytes + kKVStages * 2 * kKVBytes + kOutBytes + 1024 + 256;
  static constexpr int kSCol = 0;                // S_t at columns t*128 (P_t over its first 64)
  static constexpr int kOCol = 256;              // O_t at columns 256 + t*128
  static constexpr int kTmemCols = 512;
};

template <bool BF16> __device__ __forceinline__ uint32_t pack_pair(float lo, float hi) {
  if (BF16) return f32x2_to_bf16x2_bits(lo, hi);
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

template <int D, bool BF16>
__global__ void __launch_bounds__(kPrefillThreads, 1)
attention_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_o,
                         const AttnParams p) {
  using Cfg = PrefillCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                    // [tile]
  uint8_t* sKV = sQ + 2 * Cfg::kQBytes;                  // [stage][K | V]
  uint8_t* sO = sKV + kKVStages * 2 * Cfg::kKVBytes;     // [softmax warp] 32 rows x 128 bytes, 128-byte swizzle
  uint64_t* bars = reinterpret_cast<uint64_t*>(sO + Cfg::kOutBytes);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;             // [stage]
  uint64_t* v_full = bars + 3;             // [stage]
  uint64_t* kv_empty = bars + 5;           // [stage]
  uint64_t* s_full = bars + 7;             // [tile]
  uint64_t* p_full = bars + 9;             // [tile]
  uint64_t* o_done = bars + 11;            // [tile]
  uint64_t* q_empty = bars + 13;           // every S = Q K^T of the item has been computed: the Q buffers may be refilled
  uint64_t* o_free = bars + 14;            // [tile] the item's O has been read out of tensor memory
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int n_all = (p.Sk + BKV - 1) / BKV;
  const int tile_rows = p.pair_heads ? 0 : BQ, tile_heads = p.pair_heads ? 1 : 0;   // step from tile 0 to tile 1
  // Work items: (block of query rows, head or head pair, batch). The CTAs are persistent: CTA c takes items
  // c, c + gridDim.x, ... of a list ordered by length, longest causal blocks first, so every CTA gets a mix of
  // long and short items, and the barriers, the tensor memory and the pipeline are set up once per CTA, not once
  // per item; the loads of the next item start while the output of the current one is still being written.
  const int per_x = p.items_y * p.B;
  const int n_items = p.items_x * per_x;
  const int n_sweeps = (n_items + gridDim.x - 1) / gridDim.x;
  // Sweep k hands item k * gridDim.x + c to CTA c on even sweeps and to CTA gridDim.x - 1 - c on odd sweeps: the
  // lengths fall along the list, so the two directions cancel each other's slope. -1: no item in the last sweep.
  auto item_of_sweep = [&](int k) {
    const int pos = (k & 1) ? static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x) : static_cast<int>(blockIdx.x);
    const int idx = k * static_cast<int>(gridDim.x) + pos;
    return idx < n_items ? idx : -1;
  };

  // The two Q tiles of an item: with an even group size, the same 128 query rows of two query heads that share
  // the KV head (equal work and equal masks for both tiles, so the ping-pong never runs single-handed);
  // otherwise two consecutive row tiles of one head.
  struct Item {
    int b, q0, hq, hkv, n_t[2], n_max;
  };
  auto item_at = [&](int idx) {
    Item it;
    const int xr = idx / per_x, rest = idx - xr * per_x;
    const int first = p.items_x - 1 - xr;   // longest (last) causal blocks first
    const int y = rest % p.items_y;
    it.b = rest / p.items_y;
    it.q0 = p.pair_heads ? first * BQ : first * 2 * BQ;
    it.hq = p.pair_heads ? y * 2 : y;
    it.hkv = it.hq / G;
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int q0t = it.q0 + t * tile_rows;
      it.n_t[t] = q0t >= p.Sq ? 0 : (p.causal ? min(n_all, q0t / BKV + 1) : n_all);
    }
    it.n_max = max(it.n_t[0], it.n_t[1]);
    return it;
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&o_done[i], 1);
      mbar_init(&o_free[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      prefetch_tmap(&tmap_q);
      prefetch_tmap(&tmap_k);
      prefetch_tmap(&tmap_v);
      uint32_t kv_it = 0;   // K / V tiles loaded so far (ring position and phase)
      uint32_t q_it = 0;    // items started so far
      bool ok = true;
      for (int sweep = 0; sweep < n_sweeps && ok; ++sweep, ++q_it) {
        const int idx = item_of_sweep(sweep);
        if (idx < 0) break;
        const Item it = item_at(idx);
        for (int j = 0; j < it.n_max && ok; ++j, ++kv_it) {
          const int st = kv_it & 1;
          if (!mbar_wait(&kv_empty[st], ((kv_it >> 1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sK = sKV + st * 2 * Cfg::kKVBytes;
          uint8_t* sV = sK + Cfg::kKVBytes;
          mbar_arrive_expect_tx(&k_full[st], Cfg::kKVBytes);
#pragma unroll
          for (int h = 0; h < Cfg::kHalves; ++h) tma_load_4d(sK + h * (BKV * 128), &tmap_k, &k_full[st], h * 64, j * BKV, it.hkv, it.b);
          mbar_arrive_expect_tx(&v_full[st], Cfg::kKVBytes);
#pragma unroll
          for (int h = 0; h < Cfg::kHalves; ++h) tma_load_4d(sV + h * (BKV * 128), &tmap_v, &v_full[st], h * 64, j * BKV, it.hkv, it.b);
          if (j == 0) {
            // Q after the item's first K / V tile: that tile's buffer frees while the previous item is still
            // computing, the Q buffers only when its last S has been computed
            if (q_it > 0 && !mbar_wait(q_empty, (q_it - 1) & 1u, abort_flag)) { ok = false; break; }
            const int n_q = it.n_t[1] > 0 ? 2 : 1;
            mbar_arrive_expect_tx(q_full, static_cast<uint32_t>(n_q * Cfg::kQBytes));
            for (int t = 0; t < n_q; ++t)
#pragma unroll
              for (int h = 0; h < Cfg::kHalves; ++h)
                tma_load_4d(sQ + t * Cfg::kQBytes + h * (BQ * 128), &tmap_q, q_full, h * 64, it.q0 + t * tile_rows,
                            it.hq + t * tile_heads, it.b);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc(BQ, BKV, BF16, false, false);  // Q, K both K-major
      const uint32_t idesc_o = make_idesc(BQ, D, BF16, false, true);     // P from tensor memory, V MN-major
      uint32_t kv_base = 0;            // K / V tiles consumed before this item
      uint32_t q_it = 0;
      uint32_t p_cnt[2] = {0, 0};      // softmax results consumed so far, per tile
      uint32_t o_cnt[2] = {0, 0};      // items with work so far, per tile
      bool ok = true;
      for (int sweep = 0; sweep < n_sweeps && ok; ++sweep, ++q_it) {
        const int idx = item_of_sweep(sweep);
        if (idx < 0) break;
        const Item it = item_at(idx);
        auto issue_s = [&](int t, int j) {
          const uint32_t q_addr = smem_u32(sQ + t * Cfg::kQBytes);
          const uint32_t k_addr = smem_u32(sKV + ((kv_base + j) & 1u) * 2 * Cfg::kKVBytes);
          const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(Cfg::kSCol + t * BKV);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk / 4) * (BQ * 128) + (kk % 4) * 32;
            umma_f16(d_tmem, smem_desc_sw128(q_addr + off, 16u, 1024u), smem_desc_sw128(k_addr + off, 16u, 1024u),
                     idesc_s, kk != 0 ? 1u : 0u);
          }
          umma_commit(&s_full[t]);
        };
        auto k_phase = [&](int j) { return ((kv_base + j) >> 1) & 1u; };
        ok = mbar_wait(q_full, q_it & 1u, abort_flag) && mbar_wait(&k_full[kv_base & 1u], k_phase(0), abort_flag);
        if (ok) {
          tc_fence_after();
          issue_s(0, 0);
          if (it.n_t[1] > 0) issue_s(1, 0);
        }
        for (int j = 0; j < it.n_max && ok; ++j) {
          const int st = (kv_base + j) & 1;
          bool v_ready = false, k_ready = false;
          for (int t = 0; t < 2 && ok; ++t) {
            if (j >= it.n_t[t]) continue;
            if (!mbar_wait(&p_full[t], p_cnt[t] & 1u, abort_flag)) { ok = false; break; }
            ++p_cnt[t];
            if (!v_ready) {
              if (!mbar_wait(&v_full[st], k_phase(j), abort_flag)) { ok = false; break; }
              v_ready = true;
            }
            // the first P.V of an item overwrites O: the previous item's O must have been read out
            if (j == 0 && o_cnt[t] > 0 && !mbar_wait(&o_free[t], (o_cnt[t] - 1) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t v_addr = smem_u32(sKV + st * 2 * Cfg::kKVBytes + Cfg::kKVBytes);
            const uint32_t o_tmem = tmem_base + static_cast<uint32_t>(Cfg::kOCol + t * BKV);
            const uint32_t p_tmem = tmem_base + static_cast<uint32_t>(Cfg::kSCol + t * BKV);
#pragma unroll
            for (int kk = 0; kk < BKV / 16; ++kk) {
              // A = P_t: 16 keys = 8 packed columns per step. B = V: 64-column slabs BKV*128 bytes
              // apart (LBO), 8-key groups 1024 bytes apart (SBO), 16 keys = 2048 bytes per step.
              const uint64_t db = smem_desc_sw128(v_addr + kk * 2048, BKV * 128, 1024u);
              umma_f16_ts(o_tmem, p_tmem + kk * 8, db, idesc_o, (j | kk) != 0 ? 1u : 0u);
            }
            if (j + 1 < it.n_t[t]) {
              if (!k_ready) {
                if (!mbar_wait(&k_full[(kv_base + j + 1) & 1u], k_phase(j + 1), abort_flag)) { ok = false; break; }
                k_ready = true;
                tc_fence_after();
              }
              issue_s(t, j + 1);   // executes after the P.V above, which has then consumed P_t
            } else {
              umma_commit(&o_done[t]);
              ++o_cnt[t];
            }
          }
          if (ok) umma_commit(&kv_empty[st]);
        }
        if (ok) umma_commit(q_empty);   // arrives when every MMA of the item, its last S included, has completed
        kv_base += static_cast<uint32_t>(it.n_max);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------ softmax / output --
    const int t = (warp - 4) >> 2;                 // tile of this warp
    const int quarter = warp & 3;                  // tensor-memory lanes this warp may touch
    const int r = quarter * 32 + lane;             // row of the tile this thread owns
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_sel + static_cast<uint32_t>(Cfg::kSCol + t * BKV);
    const uint32_t o_tmem = tmem_base + lane_sel + static_cast<uint32_t>(Cfg::kOCol + t * BKV);
    const float sl2 = p.scale_log2;
    uint32_t s_cnt = 0;    // S tiles of this tile consumed so far
    uint32_t o_cnt = 0;    // items with work for this tile so far
    bool ok = true;
    for (int sweep = 0; sweep < n_sweeps && ok; ++sweep) {
      const int idx = item_of_sweep(sweep);
      if (idx < 0) break;
      const Item it = item_at(idx);
      const int b = it.b;
      const int q0t = it.q0 + t * tile_rows;
      const int head = it.hq + t * tile_heads;
      const int qi = q0t + r;
      const bool row_valid = qi < p.Sq;
      const int n_kv = it.n_t[t];
      float m = -CUDART_INF_F;   // maximum the exponentials are taken against (raw score units)
      float l = 0.f;
      for (int j = 0; j < n_kv && ok; ++j, ++s_cnt) {
        const int k0 = j * BKV;
        if (!mbar_wait(&s_full[t], s_cnt & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        uint32_t s[BKV];
#pragma unroll
        for (int c = 0; c < BKV; c += 32) tmem_ld_32x32_at(s_tmem + c, &s[c]);
        tmem_wait_ld();
        const bool need_mask = (p.causal && k0 + BKV - 1 > q0t) || (k0 + BKV > p.Sk);
        if (need_mask) {
          const int vis = (p.causal ? min(p.Sk, qi + 1) : p.Sk) - k0;  // columns [0, vis) are visible
#pragma unroll
          for (int i = 0; i < BKV; ++i)
            if (i >= vis) s[i] = 0xff800000u;  // -inf
        }
        float mx0 = -CUDART_INF_F, mx1 = -CUDART_INF_F, mx2 = -CUDART_INF_F, mx3 = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < BKV; i += 8) {
          mx0 = fmaxf(mx0, fmaxf(__uint_as_float(s[i]), __uint_as_float(s[i + 1])));
          mx1 = fmaxf(mx1, fmaxf(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3])));
          mx2 = fmaxf(mx2, fmaxf(__uint_as_float(s[i + 4]), __uint_as_float(s[i + 5])));
          mx3 = fmaxf(mx3, fmaxf(__uint_as_float(s[i + 6]), __uint_as_float(s[i + 7])));
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        // advance the maximum only when it grew by more than the threshold
        const bool grow = (mx - m) * sl2 > kRescaleThreshold;   // true on the first tile (m = -inf)
        float alpha = 1.f;
        if (grow) {
          alpha = ex2_approx((m - mx) * sl2);                    // m = -inf -> 0
          m = mx;
        }
        if (j > 0 && __any_sync(0xffffffffu, grow)) {
          // the P.V of the previous tile finished before this S was written, so O is stable
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t o[32];
            tmem_ld_32x32(o_tmem + c, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(o_tmem + c, o);
          }
        }
        const float mb = (m == -CUDART_INF_F ? 0.f : m) * sl2;
        float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
#pragma unroll
        for (int i = 0; i < BKV; i += 4) {
          const float p0 = ex2_approx(fmaf(__uint_as_float(s[i]), sl2, -mb));
          const float p1 = ex2_approx(fmaf(__uint_as_float(s[i + 1]), sl2, -mb));
          const float p2 = ex2_approx(fmaf(__uint_as_float(s[i + 2]), sl2, -mb));
          const float p3 = ex2_approx(fmaf(__uint_as_float(s[i + 3]), sl2, -mb));
          sum0 += p0; sum1 += p1; sum2 += p2; sum3 += p3;
          s[i / 2] = pack_pair<BF16>(p0, p1);
          s[i / 2 + 1] = pack_pair<BF16>(p2, p3);
        }
        l = l * alpha + ((sum0 + sum1) + (sum2 + sum3));
        tmem_st_32x32(s_tmem, &s[0]);
        tmem_st_32x32(s_tmem + 32, &s[32]);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[t]);
      }
      // epilogue: O / l
      if (ok && n_kv > 0) {
        ok = mbar_wait(&o_done[t], o_cnt & 1u, abort_flag);
        ++o_cnt;
      }
      if (ok && n_kv > 0) {
        tc_fence_after();
        const float inv = l > 0.f ? 1.0f / l : 0.f;
        // The warp's 32 rows go out through shared memory, 64 columns at a time, as one tensor store each (rows past
        // the end of the sequence are clipped by the store): a thread holds a whole row, so direct stores would
        // touch 32 different lines per instruction.
        const uint32_t stage = smem_u32(sO + (warp - 4) * 4096);
        const uint32_t stage_row = stage + static_cast<uint32_t>(lane) * 128u;
        const int row_first = q0t + quarter * 32;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32(o_tmem + c, v);
          tmem_wait_ld();
          if (c + 32 >= D) {
            // O is in registers: the next item's first P.V may overwrite the accumulator
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_free[t]);
          }
          uint32_t o[16];
#pragma unroll
          for (int i = 0; i < 16; ++i)
            o[i] = pack_pair<BF16>(__uint_as_float(v[2 * i]) * inv, __uint_as_float(v[2 * i + 1]) * inv);
          if ((c & 63) == 0) {
            if (lane == 0) bulk_wait_read_all();   // the store that last read this buffer has finished reading it
            __syncwarp();
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint32_t chunk = static_cast<uint32_t>((c & 63) / 8 + q);
            st_shared_v4(stage_row + ((chunk ^ static_cast<uint32_t>(lane & 7)) << 4), o[q * 4], o[q * 4 + 1], o[q * 4 + 2],
                         o[q * 4 + 3]);
          }
          if ((c & 63) == 32) {
            fence_proxy_async();
            __syncwarp();
            if (lane == 0 && row_first < p.Sq) {
              tma_store_4d(&tmap_o, stage, c & ~63, row_first, head, b);
              bulk_commit();
            }
          }
        }
        if (row_valid && p.lse) {
          const float lse = l > 0.f ? m * p.scale + logf(l) : -CUDART_INF_F;
          p.lse[(static_cast<int64_t>(b) * p.Hq + head) * p.Sq + qi] = lse;
        }
      }
    }
    if (lane == 0) bulk_wait_all();   // the output stores have left shared memory and are complete
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_word, 2u);
}

// ---------------------------------------------------------------------------
// Decode kernel (few query rows against a long KV cache, D = 128): the problem is
// transposed so that the KEYS fill the 128 rows of the MMA and the R = groups*Sq
// query rows (R <= 16, padded to N = 16) its narrow N side:
//   S^T (128 keys x N)  = K_j (A, K-major)      x  Q^T (B, K-major)
//   O^T (128 dims x N) += V_j^T (A, MN-major)   x  P^T (B, K-major, shared memory)
// so every K / V byte is read once per KV head, tensor-core and softmax work scale
// with N instead of 128, and one thread owns one key of the tile. The maximum over
// keys is a warp reduction plus one 128-thread named barrier per tile. A cluster
// of `splits` CTAs shares one (batch, KV head): each walks a contiguous slice of
// the keys and the partial (O, m, l) are merged by CTA 0 through distributed
// shared memory. 192 threads: warp 0 TMA, warp 1 MMA, warps 2-5 softmax and output.
// K and V tiles travel through one ring of three 32 KB slots (K0 V0 K1 | V1 K2 V2 | ...),
// each slot released as soon as the MMA that reads it has finished, so a CTA needs
// 110 KB and two of them share an SM: one streams while the other sets up or merges.
constexpr int kDecThreads = 192;
constexpr int kDecSlots = 3;
constexpr int kDecD = 128;

template <int N> struct DecCfg {
  static constexpr int kQBytes = N * 128 * 2;             // N rows, two 64-column slabs
  static constexpr int kKVBytes = BKV * kDecD * 2;
  static constexpr int kPBytes = N * 128 * 2;             // N rows x 128 keys, two 64-key slabs
  static constexpr int kSmem = kQBytes + kDecSlots * kKVBytes + 2 * kPBytes + 1024 + 1024;
  static constexpr int kSCol = 0;                         // S^T buffers at 0 and N
  static constexpr int kOCol = 2 * N;
  static constexpr int kTmemCols = N == 16 ? 64 : 128;
  static_assert(N == 16, "shared memory is budgeted for N = 16");
};

__device__ __forceinline__ float warp_max_f32(float v) {
  // order-preserving map to unsigned, hardware integer reduction, and back
  uint32_t u = __float_as_uint(v);
  u ^= (u >> 31) ? 0xffffffffu : 0x80000000u;
  u = __reduce_max_sync(0xffffffffu, u);
  u ^= (u >> 31) ? 0x80000000u : 0xffffffffu;
  return __uint_as_float(u);
}

template <int N, bool BF16>
__global__ void __launch_bounds__(kDecThreads, 2)
attention_decode_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const AttnParams p, const int splits) {
  using Cfg = DecCfg<N>;
  constexpr int D = kDecD;
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ uint8_t smem_raw[];
  // the same offset in every CTA of the cluster, so peers can be addressed by mapping
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + Cfg::kQBytes;                       // [slot]: tile t (K_i: t = 2i, V_i: t = 2i+1) in slot t % 3
  uint8_t* sP = sKV + kDecSlots * Cfg::kKVBytes;          // [2]
  uint8_t* tail = sP + 2 * Cfg::kPBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tail);
  uint64_t* q_full = bars;
  uint64_t* slot_full = bars + 1;          // [3]
  uint64_t* slot_empty = bars + 4;         // [3]
  uint64_t* s_full = bars + 7;             // [2]
  uint64_t* p_full = bars + 9;             // [2]
  uint64_t* pv_done = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(tail + 128);      // [2][4][N] warp maxima; later [4][N] warp sums
  float* comb_ml = red + 2 * 4 * N;                       // [2][N]: m, l of this CTA
  float* comb_o = reinterpret_cast<float*>(sKV);          // [N][128] partial O, over the drained K/V ring

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int R = G * p.Sq;
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int hq0 = hkv * G;
  const int n_tiles = (p.Sk + BKV - 1) / BKV;
  const int per = (n_tiles + splits - 1) / splits;
  const int t_begin = min(split * per, n_tiles), t_end = min(t_begin + per, n_tiles);
  const int n_my = t_end - t_begin;

  // zero the Q tile: the load fills only its first R rows
  for (int i = threadIdx.x; i < Cfg::kQBytes / 16; i += kDecThreads) reinterpret_cast<uint4*>(sQ)[i] = make_uint4(0, 0, 0, 0);
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < kDecSlots; ++i) {
      mbar_init(&slot_full[i], 1);
      mbar_init(&slot_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
    }
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tmem_relinquish();
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // set-up above runs under the predecessor's tail; Q, K and V are read from here on

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0 && n_my > 0) {
      prefetch_tmap(&tmap_q);
      prefetch_tmap(&tmap_k);
      prefetch_tmap(&tmap_v);
      // box (64, Sq, G, 1): rows ordered (group head, position)
      mbar_arrive_expect_tx(q_full, static_cast<uint32_t>(2 * 128 * R));
#pragma unroll
      for (int h = 0; h < 2; ++h) tma_load_4d(sQ + h * (N * 128), &tmap_q, q_full, h * 64, 0, hq0, b);
      for (int t = 0; t < 2 * n_my; ++t) {
        const int slot = t % kDecSlots, use = t / kDecSlots;
        if (!mbar_wait(&slot_empty[slot], (use & 1u) ^ 1u, abort_flag)) break;
        uint8_t* dst = sKV + slot * Cfg::kKVBytes;
        const int key0 = (t_begin + (t >> 1)) * BKV;
        const CUtensorMap* tm = (t & 1) ? &tmap_v : &tmap_k;
        mbar_arrive_expect_tx(&slot_full[slot], Cfg::kKVBytes);
#pragma unroll
        for (int h = 0; h < 2; ++h) tma_load_4d(dst + h * (BKV * 128), tm, &slot_full[slot], h * 64, key0, hkv, b);
      }
      pdl_launch_dependents();   // all loads issued
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0 && n_my > 0) {
      const uint32_t idesc_s = make_idesc(BKV, N, BF16, false, false);  // K tile, Q both K-major
      const uint32_t idesc_o = make_idesc(D, N, BF16, true, false);     // V^T MN-major, P^T K-major
      const uint32_t q_addr = smem_u32(sQ);
      bool ok = mbar_wait(q_full, 0, abort_flag);
      auto issue_pv = [&](int i) -> bool {
        const int t = 2 * i + 1, slot = t % kDecSlots, use = t / kDecSlots, buf = i & 1;
        if (!mbar_wait(&p_full[buf], (i >> 1) & 1u, abort_flag)) return false;
        if (!mbar_wait(&slot_full[slot], use & 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sKV + slot * Cfg::kKVBytes);
        const uint32_t p_addr = smem_u32(sP + buf * Cfg::kPBytes);
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          // A = V^T: 64-dim slabs BKV*128 bytes apart (LBO), 8-key groups 1024 bytes apart (SBO),
          // 16 keys = 2048 bytes per step. B = P^T: key slab kk/4, 32 bytes per step.
          const uint64_t da = smem_desc_sw128(v_addr + kk * 2048, BKV * 128, 1024u);
          const uint64_t db = smem_desc_sw128(p_addr + (kk / 4) * (N * 128) + (kk % 4) * 32, 16u, 1024u);
          umma_f16(tmem_base + Cfg::kOCol, da, db, idesc_o, (i | kk) != 0 ? 1u : 0u);
        }
        umma_commit(&slot_empty[slot]);
        umma_commit(pv_done);
        return true;
      };
      for (int i = 0; i < n_my && ok; ++i) {
        const int t = 2 * i, slot = t % kDecSlots, use = t / kDecSlots, buf = i & 1;
        if (!mbar_wait(&slot_full[slot], use & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        // S^T buffer `buf` was read by the softmax of tile i-2, whose P this thread has already waited for
        const uint32_t k_addr = smem_u32(sKV + slot * Cfg::kKVBytes);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t koff = (kk / 4) * (BKV * 128) + (kk % 4) * 32;
          const uint32_t qoff = (kk / 4) * (N * 128) + (kk % 4) * 32;
          umma_f16(tmem_base + Cfg::kSCol + buf * N, smem_desc_sw128(k_addr + koff, 16u, 1024u),
                   smem_desc_sw128(q_addr + qoff, 16u, 1024u), idesc_s, kk != 0 ? 1u : 0u);
        }
        umma_commit(&slot_empty[slot]);   // K_i is free once S^T_i has been computed
        umma_commit(&s_full[buf]);
        if (i > 0) ok = issue_pv(i - 1);
      }
      if (ok) issue_pv(n_my - 1);
    }
  } else {
    // ------------------------------------------------------ softmax / output --
    const int quarter = warp & 3;
    const int tid = quarter * 32 + lane;            // key of the tile, later output dim
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const float sl2 = p.scale_log2;
    float m[N], lsum[N];
#pragma unroll
    for (int n = 0; n < N; ++n) { m[n] = -CUDART_INF_F; lsum[n] = 0.f; }
    bool ok = true;
    for (int i = 0; i < n_my && ok; ++i) {
      const int buf = i & 1;
      if (!mbar_wait(&s_full[buf], (i >> 1) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[N];
      if (N == 16) tmem_ld_32x16(tmem_base + lane_sel + Cfg::kSCol + buf * N, *reinterpret_cast<uint32_t(*)[16]>(&sv[0]));
      else tmem_ld_32x32_at(tmem_base + lane_sel + Cfg::kSCol + buf * N, &sv[0]);
      tmem_wait_ld();
      const bool visible = (t_begin + i) * BKV + tid < p.Sk;
      float* redb = red + buf * 4 * N;
#pragma unroll
      for (int n = 0; n < N; ++n) {
        if (!visible) sv[n] = 0xff800000u;
        const float wm = warp_max_f32(__uint_as_float(sv[n]));
        if (lane == 0) redb[quarter * N + n] = wm;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float alpha[N];
      bool grow = false;
#pragma unroll
      for (int n = 0; n < N; ++n) {
        const float mx = fmaxf(fmaxf(redb[n], redb[N + n]), fmaxf(redb[2 * N + n], redb[3 * N + n]));
        alpha[n] = 1.f;
        if ((mx - m[n]) * sl2 > kRescaleThreshold) {   // also the first tile (m = -inf)
          alpha[n] = ex2_approx((m[n] - mx) * sl2);
          m[n] = mx;
          grow = true;
        }
      }
      if (grow) {   // same decision in every thread: m is replicated
#pragma unroll
        for (int n = 0; n < N; ++n) lsum[n] *= alpha[n];
        if (i > 0) {
          if (!mbar_wait(pv_done, (i - 1) & 1u, abort_flag)) { ok = false; break; }
          tc_fence_after();
          uint32_t o[N];
          if (N == 16) tmem_ld_32x16(tmem_base + lane_sel + Cfg::kOCol, *reinterpret_cast<uint32_t(*)[16]>(&o[0]));
          else tmem_ld_32x32_at(tmem_base + lane_sel + Cfg::kOCol, &o[0]);
          tmem_wait_ld();
#pragma unroll
          for (int n = 0; n < N; ++n) o[n] = __float_as_uint(__uint_as_float(o[n]) * alpha[n]);
          if (N == 16) tmem_st_32x16(tmem_base + lane_sel + Cfg::kOCol, *reinterpret_cast<const uint32_t(*)[16]>(&o[0]));
          else tmem_st_32x32(tmem_base + lane_sel + Cfg::kOCol, &o[0]);
          tmem_wait_st();
        }
      }
      // P^T row n, key tid: slab tid/64, 16-byte chunk (tid%64)/8 XOR-swizzled by (n & 7)
      uint8_t* pb = sP + buf * Cfg::kPBytes + (tid >> 6) * (N * 128) + (tid & 7) * 2;
      const int chunk = (tid & 63) >> 3;
#pragma unroll
      for (int n = 0; n < N; ++n) {
        const float mb = (m[n] == -CUDART_INF_F ? 0.f : m[n]) * sl2;
        const float pe = ex2_approx(fmaf(__uint_as_float(sv[n]), sl2, -mb));
        lsum[n] += pe;
        const uint16_t bits = BF16 ? f32_to_bf16_bits(pe) : f32_to_f16_bits(pe);
        *reinterpret_cast<uint16_t*>(pb + n * 128 + ((chunk ^ (n & 7)) << 4)) = bits;
      }
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[buf]);
    }
    // this CTA's partial result: O^T row `tid` (an output dim), m, l
    if (ok && n_my > 0) ok = mbar_wait(pv_done, (n_my - 1) & 1u, abort_flag);
    asm volatile("bar.sync 1, 128;" ::: "memory");   // every softmax thread is past its last read of `red`
#pragma unroll
    for (int n = 0; n < N; ++n) {
      float v = lsum[n];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) red[quarter * N + n] = v;
    }
    uint32_t o[N];
    if (ok && n_my > 0) {
      tc_fence_after();
      if (N == 16) tmem_ld_32x16(tmem_base + lane_sel + Cfg::kOCol, *reinterpret_cast<uint32_t(*)[16]>(&o[0]));
      else tmem_ld_32x32_at(tmem_base + lane_sel + Cfg::kOCol, &o[0]);
      tmem_wait_ld();
    } else {
#pragma unroll
      for (int n = 0; n < N; ++n) o[n] = 0u;
    }
#pragma unroll
    for (int n = 0; n < N; ++n) comb_o[n * 128 + tid] = __uint_as_float(o[n]);
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (tid < N) {
      float mm = m[0];   // m is a register array: select without dynamic indexing
#pragma unroll
      for (int n = 1; n < N; ++n) mm = tid == n ? m[n] : mm;
      comb_ml[tid] = mm;
      comb_ml[N + tid] = (red[tid] + red[N + tid]) + (red[2 * N + tid] + red[3 * N + tid]);
    }
  }

  // ---- merge the splits: CTA 0 of the cluster reads every partial through DSMEM --
  cluster.sync();
  if (split == 0 && warp >= 2 && !*abort_flag) {
    const int tid = (warp & 3) * 32 + lane;
    for (int n = 0; n < R; ++n) {
      float M = -CUDART_INF_F;
      for (int c = 0; c < splits; ++c) {
        const float* ml = cluster.map_shared_rank(comb_ml, c);
        if (ml[N + n] > 0.f) M = fmaxf(M, ml[n]);
      }
      float L = 0.f, acc = 0.f;
      for (int c = 0; c < splits; ++c) {
        const float* ml = cluster.map_shared_rank(comb_ml, c);
        const float lc = ml[N + n];
        if (lc > 0.f) {
          const float w = ex2_approx((ml[n] - M) * p.scale_log2);
          L += w * lc;
          acc += w * cluster.map_shared_rank(comb_o, c)[n * 128 + tid];
        }
      }
      const int g = n / p.Sq, s = n - g * p.Sq;
      const float val = L > 0.f ? acc / L : 0.f;
      uint16_t* orow = static_cast<uint16_t*>(p.out) + b * p.o_sb + static_cast<int64_t>(hq0 + g) * p.o_sh +
                       static_cast<int64_t>(s) * p.o_ss;
      orow[tid] = BF16 ? f32_to_bf16_bits(val) : f32_to_f16_bits(val);
      if (tid == 0 && p.lse)
        p.lse[(static_cast<int64_t>(b) * p.Hq + hq0 + g) * p.Sq + s] = L > 0.f ? M * p.scale + logf(L) : -CUDART_INF_F;
    }
  }
  cluster.sync();   // peers keep their shared memory alive until CTA 0 has read it

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_word, 2u);
}

bool make_qkv_map(CUtensorMap* m, const b200Tensor* t, uint32_t box_rows, uint32_t box_heads, const char** err) {
  // t: (B, H, S, D) view; tensor-map dims innermost first: D, S, H, B
  const uint64_t dims[4] = {(uint64_t)t->sizes[3], (uint64_t)t->sizes[2], (uint64_t)t->sizes[1], (uint64_t)t->sizes[0]};
  auto st = [&](int d) { return static_cast<uint64_t>(t->sizes[d] == 1 ? t->sizes[3] * 8 : t->strides[d]) * 2; };
  const uint64_t strides[3] = {st(2), st(1), st(0)};
  const uint32_t box[4] = {64, box_rows, box_heads, 1};
  return tc::encode_tmap_16bit(m, t->data, 4, dims, strides, box, err);
}

template <int D>
b200Status launch_attention(const b200Tensor* q, const b200Tensor* k, const b200Tensor* v, const b200Tensor* out, AttnParams p,
                           cudaStream_t s) {
  using Cfg = AttCfg<D>;
  CUtensorMap tq, tk, tv;
  const char* err = "";
  const int G = p.Hq / p.Hkv;
  const bool q_ok = p.packed ? make_qkv_map(&tq, q, (uint32_t)p.Sq, (uint32_t)G, &err) : make_qkv_map(&tq, q, BQ, 1, &err);
  B200_REQUIRE(q_ok && make_qkv_map(&tk, k, BKV, 1, &err) && make_qkv_map(&tv, v, BKV, 1, &err), B200_NOT_SUPPORTED,
               "b200_sdpa_flash_fwd: %s", err);
  static thread_local int last_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != last_dev) {
    cudaError_t e = cudaFuncSetAttribute(attention_fwd_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_prefill_kernel<D, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, PrefillCfg<D>::kSmem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_prefill_kernel<D, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, PrefillCfg<D>::kSmem);
    B200_REQUIRE(e == cudaSuccess, B200_LAUNCH_FAILED, "b200_sdpa_flash_fwd: %s", cudaGetErrorString(e));
    last_dev = dev;
  }
  if (p.packed) {
    attention_fwd_kernel<D><<<dim3(1, p.Hkv, p.B), kAttThreads, Cfg::kSmem, s>>>(tq, tk, tv, p);
  } else {
    p.pair_heads = (p.Hq / p.Hkv) % 2 == 0 ? 1 : 0;
    p.items_x = p.pair_heads ? (p.Sq + BQ - 1) / BQ : (p.Sq + 2 * BQ - 1) / (2 * BQ);
    p.items_y = p.pair_heads ? p.Hq / 2 : p.Hq;
    const int64_t items = static_cast<int64_t>(p.items_x) * p.items_y * p.B;
    B200_REQUIRE(items < (int64_t(1) << 31), B200_NOT_SUPPORTED, "b200_sdpa_flash_fwd: too many query tiles");
    const int sms = sm_count_current_device();
    const int grid = static_cast<int>(items < sms ? items : sms);   // persistent CTAs, one per SM
    CUtensorMap to;   // output: 64 columns x the 32 rows of one softmax warp per store
    B200_REQUIRE(make_qkv_map(&to, out, 32, 1, &err), B200_NOT_SUPPORTED, "b200_sdpa_flash_fwd: output: %s", err);
    if (p.is_bf16) attention_prefill_kernel<D, true><<<grid, kPrefillThreads, PrefillCfg<D>::kSmem, s>>>(tq, tk, tv, to, p);
    else attention_prefill_kernel<D, false><<<grid, kPrefillThreads, PrefillCfg<D>::kSmem, s>>>(tq, tk, tv, to, p);
  }
  return check_launch("b200_sdpa_flash_fwd");
}

template <bool BF16>
b200Status launch_decode(const b200Tensor* q, const b200Tensor* k, const b200Tensor* v, AttnParams p, cudaStream_t s) {
  using Cfg = DecCfg<16>;
  CUtensorMap tq, tk, tv;
  const char* err = "";
  const int G = p.Hq / p.Hkv;
  B200_REQUIRE(make_qkv_map(&tq, q, (uint32_t)p.Sq, (uint32_t)G, &err) && make_qkv_map(&tk, k, BKV, 1, &err) &&
               make_qkv_map(&tv, v, BKV, 1, &err), B200_NOT_SUPPORTED, "b200_sdpa_flash_fwd: %s", err);
  static thread_local int last_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != last_dev) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<16, BF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
    B200_REQUIRE(e == cudaSuccess, B200_LAUNCH_FAILED, "b200_sdpa_flash_fwd: %s", cudaGetErrorString(e));
    last_dev = dev;
  }
  // Split the keys of one (batch, KV head) over a cluster only while the split grid still fits the device at once
  // (two CTAs per SM): a split costs the cluster's co-scheduling and the merge, and more CTAs than places gain
  // nothing. Measured at batch 64 x 8 KV heads x 4096 keys: 168 us unsplit, 190 us in two, 215 us in four; at
  // 64 x 1 x 4096: 62 / 40 / 30 / 41 us for 1 / 2 / 4 / 8.
  const int n_tiles = (p.Sk + BKV - 1) / BKV;
  const int ctas = p.B * p.Hkv;
  const int places = 2 * sm_count_current_device();
  int splits = 1;
  while (splits < 8 && ctas * splits * 2 <= places && n_tiles >= splits * 2 * 8) splits *= 2;   // >= 8 tiles per CTA
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits, p.Hkv, p.B);
  cfg.blockDim = dim3(kDecThreads);
  cfg.dynamicSmemBytes = Cfg::kSmem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, attention_decode_kernel<16, BF16>, tq, tk, tv, p, splits);
  B200_REQUIRE(e == cudaSuccess, B200_LAUNCH_FAILED, "b200_sdpa_flash_fwd: %s", cudaGetErrorString(e));
  return check_launch("b200_sdpa_flash_fwd");
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" b200Status b200_sdpa_flash_fwd(const b200Tensor* out, const b200Tensor* lse, const b200Tensor* q,
                                          const b200Tensor* k, const b200Tensor* v, int32_t is_causal, double scale,
                                          b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(q) && valid(k) && valid(v), B200_BAD_PARAM, "b200_sdpa_flash_fwd: invalid tensor view");
  B200_REQUIRE(q->ndim == 4 && k->ndim == 4 && v->ndim == 4 && out->ndim == 4, B200_BAD_PARAM,
               "b200_sdpa_flash_fwd: q, k, v, out must be (B,H,S,D)");
  B200_REQUIRE((q->dtype == B200_BF16 || q->dtype == B200_F16) && k->dtype == q->dtype && v->dtype == q->dtype &&
               out->dtype == q->dtype, B200_NOT_SUPPORTED, "b200_sdpa_flash_fwd: bf16 or f16 operands of one dtype");
  AttnParams p{};
  p.B = (int)q->sizes[0]; p.Hq = (int)q->sizes[1]; p.Sq = (int)q->sizes[2]; p.D = (int)q->sizes[3];
  p.Hkv = (int)k->sizes[1]; p.Sk = (int)k->sizes[2];
  B200_REQUIRE(same_shape(out, q) && same_shape(k, v) && k->sizes[0] == p.B && k->sizes[3] == p.D, B200_BAD_PARAM,
               "b200_sdpa_flash_fwd: shape mismatch");
  B200_REQUIRE(p.Hkv > 0 && p.Hq % p.Hkv == 0, B200_BAD_PARAM, "b200_sdpa_flash_fwd: Hq must be a multiple of Hkv");
  B200_REQUIRE(p.D == 64 || p.D == 128, B200_NOT_SUPPORTED, "b200_sdpa_flash_fwd: head dim 64 or 128");
  B200_REQUIRE(scale > 0.0, B200_NOT_SUPPORTED, "b200_sdpa_flash_fwd: scale must be positive");
  B200_REQUIRE(!is_causal || p.Sq == p.Sk, B200_NOT_SUPPORTED,
               "b200_sdpa_flash_fwd: causal needs Sq == Sk (a single decode query attends everything: is_causal=0)");
  if (numel(q) == 0) return B200_OK;
  B200_REQUIRE(p.Sk > 0, B200_NOT_SUPPORTED, "b200_sdpa_flash_fwd: empty key sequence");
  for (const b200Tensor* t : {q, k, v, out}) {
    B200_REQUIRE(t->strides[3] == 1 && reinterpret_cast<uintptr_t>(t->data) % 16 == 0, B200_NOT_SUPPORTED,
                 "b200_sdpa_flash_fwd: last dim must be contiguous and the base 16-byte aligned");
    for (int d = 0; d < 3; ++d)
      B200_REQUIRE(t->sizes[d] == 1 || t->strides[d] % 8 == 0, B200_NOT_SUPPORTED,
                   "b200_sdpa_flash_fwd: strides must be multiples of 8 elements");
  }
  if (lse) {
    B200_REQUIRE(valid(lse) && lse->dtype == B200_F32 && is_contiguous(lse) && numel(lse) == (int64_t)p.B * p.Hq * p.Sq,
                 B200_BAD_PARAM, "b200_sdpa_flash_fwd: lse must be contiguous f32 (B,Hq,Sq)");
    p.lse = static_cast<float*>(lse->data);
  }
  p.causal = (is_causal && p.Sq > 1) ? 1 : 0;   // a single query row sees every key either way
  const int G = p.Hq / p.Hkv;
  p.packed = (!p.causal && G * p.Sq <= BQ && p.Sq <= 256 && G <= 256 && (G == 1 || q->strides[1] > 0)) ? 1 : 0;
  p.is_bf16 = q->dtype == B200_BF16;
  p.scale = static_cast<float>(scale);
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.out = out->data; p.o_sb = out->strides[0]; p.o_sh = out->strides[1]; p.o_ss = out->strides[2];
  p.error_word = device_error_word();
  B200_REQUIRE(p.error_word, B200_LAUNCH_FAILED, "b200_sdpa_flash_fwd: device error word unavailable");
  B200_REQUIRE(p.B <= 65535 && p.Hq <= 65535, B200_NOT_SUPPORTED, "b200_sdpa_flash_fwd: batch / heads too large");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p.packed && p.D == 128 && G * p.Sq <= 16)
    return p.is_bf16 ? launch_decode<true>(q, k, v, p, s) : launch_decode<false>(q, k, v, p, s);
  if (p.D == 128) return launch_attention<128>(q, k, v, out, p, s);
  return launch_attention<64>(q, k, v, out, p, s);
}
