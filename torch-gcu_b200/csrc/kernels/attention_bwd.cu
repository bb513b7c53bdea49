// Flash-attention backward on tcgen05 tensor cores, D = 128, bf16 / f16, GQA, causal
// or full. Three launches, no atomics, so gradients do not depend on timing:
//   1. delta[b,h,q] = sum_d dO * O                                  (row kernel)
//   2. dQ: one CTA per (128 query rows, query head, batch) walks the key tiles:
//        S = Q K^T, dP = dO V^T  -> P = exp(S*scale - lse), dS = P * (dP - delta) * scale
//        dQ += dS K          (dS handed to the tensor core in tensor memory)
//   3. dK, dV: one CTA per (128 keys, KV head, batch) walks the query tiles of every
//      query head of the group, on the transposed problem so that P^T and dS^T are
//      already laid out as the A operand of the accumulating products:
//        S^T = K Q^T, dP^T = V dO^T -> P^T, dS^T
//        dV += P^T dO,  dK += dS^T Q
// Roles per CTA: warp 0 TMA producer, warp 1 MMA issuer, then the pointwise warps (one thread
// per accumulator row): four in the dQ kernel; eight in the dK/dV kernel, which works on
// 64-query half tiles with two S^T / dP^T buffers in tensor memory so that the next half's
// products run under the pointwise stage. All barrier waits are bounded; loads never use
// cluster multicast.
// (reference: aot_ops/gcu_attention.cpp:135-203 _scaled_dot_product_flash_attention_backward.)
#include "common.cuh"
#include "tc_common.cuh"

#include <math_constants.h>

namespace b200 {
unsigned int* device_error_word();

namespace {

using namespace tc;

constexpr int kThreadsBwd = 192;
constexpr int BT = 128;     // rows of every tile (queries or keys)
constexpr int D = 128;
constexpr int kTileBytes = BT * D * 2;   // 32 KB
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
  int B, Hq, Hkv, Sq, Sk;
  int causal;
  float scale, scale_log2;
  const float* lse;     // (B,Hq,Sq)
  const float* delta;   // (B,Hq,Sq)
  void* dq; int64_t dq_sb, dq_sh, dq_ss;
  void* dk; int64_t dk_sb, dk_sh, dk_ss;
  void* dv; int64_t dv_sb, dv_sh, dv_ss;
  unsigned int* error_word;
};

template <bool BF16> __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if (BF16) return f32x2_to_bf16x2_bits(lo, hi);
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Stores one fp32 accumulator row (128 columns in tensor memory) as 16-bit values.
template <bool BF16>
__device__ __forceinline__ void store_acc_row(uint32_t tmem_row, uint16_t* dst, bool row_valid) {
  const bool vec_ok = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
#pragma unroll 1
  for (int c = 0; c < D; c += 32) {
    uint32_t v[32];
    tmem_ld_32x32(tmem_row + c, v);
    tmem_wait_ld();
    if (row_valid) {
      uint32_t o[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) o[i] = pack2<BF16>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
      if (vec_ok) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(dst + c + q * 8) = make_uint4(o[q * 4], o[q * 4 + 1], o[q * 4 + 2], o[q * 4 + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          dst[c + 2 * i] = static_cast<uint16_t>(o[i] & 0xffffu);
          dst[c + 2 * i + 1] = static_cast<uint16_t>(o[i] >> 16);
        }
      }
    }
  }
}

// ------------------------------------------------------------------ delta ----
template <typename T>
__global__ void __launch_bounds__(256)
delta_kernel(float* delta, const T* dout, const T* out, int64_t rows, int H, int S, int64_t g_sb, int64_t g_sh, int64_t g_ss,
             int64_t o_sb, int64_t o_sh, int64_t o_ss) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * 8;
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5); r < rows; r += warps) {
    const int64_t b = r / (static_cast<int64_t>(H) * S);
    const int64_t rem = r - b * H * S;
    const int64_t h = rem / S, s = rem - h * S;
    const T* g = dout + b * g_sb + h * g_sh + s * g_ss;
    const T* o = out + b * o_sb + h * o_sh + s * o_ss;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < D / 32; ++k)
      acc += static_cast<float>(load_as_math(g[lane + 32 * k])) * static_cast<float>(load_as_math(o[lane + 32 * k]));
    acc = warp_sum(acc);
    if (lane == 0) delta[r] = acc;
  }
}

// --------------------------------------------------------------------- dQ ----
constexpr int kSmemDq = 2 * kTileBytes + 2 * 2 * kTileBytes + 1024 + 256;   // Q, dO, 2 x (K, V)

template <bool BF16>
__global__ void __launch_bounds__(kThreadsBwd, 1)
attention_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                        const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                        const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + kTileBytes;
  uint8_t* sKV = sdO + kTileBytes;                 // [stage][K | V]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + 4 * kTileBytes);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;       // [2]
  uint64_t* kv_empty = bars + 3;      // [2]
  uint64_t* sdp_full = bars + 5;      // S and dP of the tile are in tensor memory
  uint64_t* ds_full = bars + 6;       // dS written back (4 warps)
  uint64_t* acc_done = bars + 7;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int qt = gridDim.x - 1 - blockIdx.x;       // longest causal tiles first
  const int q0 = qt * BT, hq = blockIdx.y, hkv = hq / G, b = blockIdx.z;
  int n_kv = (p.Sk + BT - 1) / BT;
  if (p.causal) n_kv = min(n_kv, qt + 1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    mbar_init(sdp_full, 1);
    mbar_init(ds_full, 4);
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kS = 0, kDP = 128, kAcc = 256;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_arrive_expect_tx(q_full, 2 * kTileBytes);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        tma_load_4d(sQ + h * (BT * 128), &tmap_q, q_full, h * 64, q0, hq, b);
        tma_load_4d(sdO + h * (BT * 128), &tmap_do, q_full, h * 64, q0, hq, b);
      }
      for (int j = 0; j < n_kv; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1u) ^ 1u, abort_flag)) break;
        uint8_t* sK = sKV + st * 2 * kTileBytes;
        uint8_t* sV = sK + kTileBytes;
        mbar_arrive_expect_tx(&kv_full[st], 2 * kTileBytes);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          tma_load_4d(sK + h * (BT * 128), &tmap_k, &kv_full[st], h * 64, j * BT, hkv, b);
          tma_load_4d(sV + h * (BT * 128), &tmap_v, &kv_full[st], h * 64, j * BT, hkv, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_kk = make_idesc(BT, BT, BF16, false, false);   // both operands K-major (over d)
      const uint32_t idesc_acc = make_idesc(BT, D, BF16, false, true);    // A from tensor memory, B = K tile MN-major
      const uint32_t q_addr = smem_u32(sQ), do_addr = smem_u32(sdO);
      bool ok = n_kv > 0 && mbar_wait(q_full, 0, abort_flag);
      for (int j = 0; j < n_kv && ok; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_full[st], (j >> 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t k_addr = smem_u32(sKV + st * 2 * kTileBytes), v_addr = k_addr + kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (BT * 128) + (kk % 4) * 32;
          umma_f16(tmem_base + kS, smem_desc_sw128(q_addr + off, 16u, 1024u), smem_desc_sw128(k_addr + off, 16u, 1024u),
                   idesc_kk, kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (BT * 128) + (kk % 4) * 32;
          umma_f16(tmem_base + kDP, smem_desc_sw128(do_addr + off, 16u, 1024u), smem_desc_sw128(v_addr + off, 16u, 1024u),
                   idesc_kk, kk != 0 ? 1u : 0u);
        }
        umma_commit(sdp_full);
        if (!mbar_wait(ds_full, j & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)   // dQ += dS (keys as K, 8 packed columns per step) x K tile (MN-major)
          umma_f16_ts(tmem_base + kAcc, tmem_base + kDP + kk * 8, smem_desc_sw128(k_addr + kk * 2048, BT * 128, 1024u), idesc_acc,
                      (j | kk) != 0 ? 1u : 0u);
        umma_commit(&kv_empty[st]);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const int qi = q0 + r;
    const bool row_valid = qi < p.Sq;
    const int64_t stat = (static_cast<int64_t>(b) * p.Hq + hq) * p.Sq + qi;
    const float lse2 = row_valid ? p.lse[stat] * kLog2e : CUDART_INF_F;   // invalid rows: p = 0
    const float dl = row_valid ? p.delta[stat] : 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv && ok; ++j) {
      const int k0 = j * BT;
      if (!mbar_wait(sdp_full, j & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int vis = (p.causal ? min(p.Sk, qi + 1) : p.Sk) - k0;   // columns [0, vis) are visible
#pragma unroll 1
      for (int c = 0; c < BT; c += 32) {
        uint32_t s[32], dp[32];
        tmem_ld_32x32(tmem_base + lane_sel + kS + c, s);
        tmem_ld_32x32(tmem_base + lane_sel + kDP + c, dp);
        tmem_wait_ld();
        uint32_t ds[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(s[i]), p.scale_log2, -lse2));
          float p1 = ex2_approx(fmaf(__uint_as_float(s[i + 1]), p.scale_log2, -lse2));
          if (c + i >= vis) p0 = 0.f;
          if (c + i + 1 >= vis) p1 = 0.f;
          ds[i / 2] = pack2<BF16>(p0 * (__uint_as_float(dp[i]) - dl) * p.scale, p1 * (__uint_as_float(dp[i + 1]) - dl) * p.scale);
        }
        // dS over the first half of the dP region: column c/2 .. c/2+15, always behind the reads
        tmem_st_32x16(tmem_base + lane_sel + kDP + c / 2, ds);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok && n_kv > 0) ok = mbar_wait(acc_done, 0, abort_flag);
    if (ok && n_kv > 0) {
      tc_fence_after();
      uint16_t* dst = static_cast<uint16_t*>(p.dq) + b * p.dq_sb + static_cast<int64_t>(hq) * p.dq_sh + static_cast<int64_t>(qi) * p.dq_ss;
      store_acc_row<BF16>(tmem_base + lane_sel + kAcc, dst, row_valid);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_word, 2u);
}

// ------------------------------------------------------------------ dK, dV ----
// 10 warps: TMA, MMA, and two groups of four pointwise warps that split the 64 query columns of a half tile
constexpr int kThreadsDkv = 320;
constexpr int kSmemDkv = 2 * kTileBytes + 2 * 2 * kTileBytes + 2 * 2 * BT * 4 + 1024 + 256;   // K, V, 2 x (Q, dO), 2 x (lse, delta)

template <bool BF16>
__global__ void __launch_bounds__(kThreadsDkv, 1)
attention_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_do,
                         const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                         const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + kTileBytes;
  uint8_t* sQdO = sV + kTileBytes;                 // [stage][Q | dO]
  float* sStat = reinterpret_cast<float*>(sQdO + 4 * kTileBytes);   // [stage][lse*log2e (128) | delta (128)]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sStat + 2 * 2 * BT);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;      // [2]
  uint64_t* qdo_empty = bars + 3;     // [2]
  uint64_t* sdp_full = bars + 5;      // [2]: S^T / dP^T of a half tile are in tensor-memory buffer i
  uint64_t* pds_full = bars + 7;      // [2]: P^T / dS^T written back into buffer i (4 warps)
  uint64_t* acc_done = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.Hq / p.Hkv;
  const int kt = blockIdx.x, k0 = kt * BT, hkv = blockIdx.y, b = blockIdx.z;
  const int n_q_all = (p.Sq + BT - 1) / BT;
  const int q_first = p.causal ? kt : 0;           // query tiles that see this key tile
  const int n_q = max(0, n_q_all - q_first);
  const int n_it = n_q * G;                        // (group head, query tile) pairs, head-major

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sdp_full[i], 1); mbar_init(&pds_full[i], 8); }
    mbar_init(acc_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // a query tile is worked in two halves of 64 queries; half-iteration h uses buffer h & 1:
  // S^T at kBuf*(h&1), dP^T 64 columns further; P^T / dS^T packed over their first 32 columns
  constexpr uint32_t kBuf = 128, kDPoff = 64, kDV = 256, kDK = 384;
  constexpr int HQ = BT / 2;                      // queries per half iteration

  if (warp == 0) {
    if (lane == 0 && n_it > 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_do); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_arrive_expect_tx(kv_full, 2 * kTileBytes);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        tma_load_4d(sK + h * (BT * 128), &tmap_k, kv_full, h * 64, k0, hkv, b);
        tma_load_4d(sV + h * (BT * 128), &tmap_v, kv_full, h * 64, k0, hkv, b);
      }
      for (int it = 0; it < n_it; ++it) {
        const int st = it & 1;
        const int g = it / n_q, qt = q_first + (it - g * n_q);
        if (!mbar_wait(&qdo_empty[st], ((it >> 1) & 1u) ^ 1u, abort_flag)) break;
        uint8_t* dQ_ = sQdO + st * 2 * kTileBytes;
        uint8_t* ddO = dQ_ + kTileBytes;
        mbar_arrive_expect_tx(&qdo_full[st], 2 * kTileBytes);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          tma_load_4d(dQ_ + h * (BT * 128), &tmap_q, &qdo_full[st], h * 64, qt * BT, hkv * G + g, b);
          tma_load_4d(ddO + h * (BT * 128), &tmap_do, &qdo_full[st], h * 64, qt * BT, hkv * G + g, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_it > 0) {
      const uint32_t idesc_kk = make_idesc(BT, HQ, BF16, false, false);   // 128 keys x 64 queries
      const uint32_t idesc_acc = make_idesc(BT, D, BF16, false, true);    // A from tensor memory, B MN-major
      const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      const int n_half = 2 * n_it;
      bool ok = mbar_wait(kv_full, 0, abort_flag);
      // S^T = K Q_half^T and dP^T = V dO_half^T of half-iteration h into buffer h & 1
      auto issue_sdp = [&](int h) -> bool {
        const int it = h >> 1, st = it & 1, half = h & 1;
        if (half == 0 && !mbar_wait(&qdo_full[st], (it >> 1) & 1u, abort_flag)) return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQdO + st * 2 * kTileBytes) + half * (HQ * 128), do_addr = q_addr + kTileBytes;
        const uint32_t buf = tmem_base + kBuf * (h & 1);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (BT * 128) + (kk % 4) * 32;
          umma_f16(buf, smem_desc_sw128(k_addr + off, 16u, 1024u), smem_desc_sw128(q_addr + off, 16u, 1024u), idesc_kk,
                   kk != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk / 4) * (BT * 128) + (kk % 4) * 32;
          umma_f16(buf + kDPoff, smem_desc_sw128(v_addr + off, 16u, 1024u), smem_desc_sw128(do_addr + off, 16u, 1024u), idesc_kk,
                   kk != 0 ? 1u : 0u);
        }
        umma_commit(&sdp_full[h & 1]);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int h = 0; h < n_half && ok; ++h) {
        // the next half's products run while the pointwise stage works on this one; its buffer was
        // read by the accumulating MMAs of half h-1, which were issued before (in-order execution)
        if (h + 1 < n_half && !issue_sdp(h + 1)) { ok = false; break; }
        if (!mbar_wait(&pds_full[h & 1], (h >> 1) & 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const int it = h >> 1, st = it & 1, half = h & 1;
        const uint32_t q_addr = smem_u32(sQdO + st * 2 * kTileBytes) + half * (HQ * 128), do_addr = q_addr + kTileBytes;
        const uint32_t buf = tmem_base + kBuf * (h & 1);
#pragma unroll
        for (int kk = 0; kk < HQ / 16; ++kk) {  // dV += P^T dO ; dK += dS^T Q   (the 64 queries are the K dimension)
          umma_f16_ts(tmem_base + kDV, buf + kk * 8, smem_desc_sw128(do_addr + kk * 2048, BT * 128, 1024u), idesc_acc,
                      (h | kk) != 0 ? 1u : 0u);
          umma_f16_ts(tmem_base + kDK, buf + kDPoff + kk * 8, smem_desc_sw128(q_addr + kk * 2048, BT * 128, 1024u), idesc_acc,
                      (h | kk) != 0 ? 1u : 0u);
        }
        if (half == 1) umma_commit(&qdo_empty[st]);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int quarter = warp & 3;
    const int colgroup = (warp - 2) >> 2;            // which 32 query columns of a half tile this warp takes
    const int tid = quarter * 32 + lane;             // key row of the tile
    const uint32_t lane_sel = static_cast<uint32_t>(quarter * 32) << 16;
    const int key = k0 + tid;
    const bool key_valid = key < p.Sk;
    bool ok = true;
    float next_lse = CUDART_INF_F, next_delta = 0.f;
    auto load_stats = [&](int it_) {
      const int g_ = it_ / n_q, qi = (q_first + (it_ - g_ * n_q)) * BT + tid;
      const bool qv = qi < p.Sq;
      const int64_t off = (static_cast<int64_t>(b) * p.Hq + hkv * G + g_) * p.Sq + qi;
      next_lse = qv ? p.lse[off] * kLog2e : CUDART_INF_F;
      next_delta = qv ? p.delta[off] : 0.f;
    };
    if (colgroup == 0 && n_it > 0) load_stats(0);
    for (int h = 0; h < 2 * n_it && ok; ++h) {
      const int it = h >> 1, st = it & 1, half = h & 1;
      const int g = it / n_q, qt = q_first + (it - g * n_q);
      const int q0 = qt * BT;
      float* stat = sStat + st * 2 * BT;
      if (half == 0) {
        // statistics of this query tile (fetched one tile ahead into registers), one per row thread of
        // group 0, shared through smem
        if (colgroup == 0) {
          stat[tid] = next_lse;
          stat[BT + tid] = next_delta;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
      } else if (colgroup == 0 && it + 1 < n_it) {
        load_stats(it + 1);   // in flight while this half and the next tile's first products run
      }
      if (!mbar_wait(&sdp_full[h & 1], (h >> 1) & 1u, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t buf = tmem_base + lane_sel + kBuf * (h & 1);
      const int qbase = half * HQ;                       // first query of this half inside the tile
      // query column q (of the tile) is visible to this key when q0 + q >= key (causal) and the key exists
      const int first_vis = !key_valid ? BT : (p.causal ? max(0, key - q0) : 0);
      {
        const int c = colgroup * 32;
        uint32_t s[32], dp[32];
        tmem_ld_32x32(buf + c, s);
        tmem_ld_32x32(buf + kDPoff + c, dp);
        tmem_wait_ld();
        // the packed results of one group land on columns the other group reads: everyone has loaded first
        asm volatile("bar.sync 2, 256;" ::: "memory");
        float ls[32], dl[32];
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 a4 = *reinterpret_cast<const float4*>(stat + qbase + c + i);
          const float4 d4 = *reinterpret_cast<const float4*>(stat + BT + qbase + c + i);
          ls[i] = a4.x; ls[i + 1] = a4.y; ls[i + 2] = a4.z; ls[i + 3] = a4.w;
          dl[i] = d4.x; dl[i + 1] = d4.y; dl[i + 2] = d4.z; dl[i + 3] = d4.w;
        }
        uint32_t pt[16], ds[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(s[i]), p.scale_log2, -ls[i]));
          float p1 = ex2_approx(fmaf(__uint_as_float(s[i + 1]), p.scale_log2, -ls[i + 1]));
          if (qbase + c + i < first_vis) p0 = 0.f;
          if (qbase + c + i + 1 < first_vis) p1 = 0.f;
          pt[i / 2] = pack2<BF16>(p0, p1);
          ds[i / 2] = pack2<BF16>(p0 * (__uint_as_float(dp[i]) - dl[i]) * p.scale, p1 * (__uint_as_float(dp[i + 1]) - dl[i + 1]) * p.scale);
        }
        // packed results over the first half of each region: columns c/2 .. c/2+15, always behind the reads
        tmem_st_32x16(buf + c / 2, pt);
        tmem_st_32x16(buf + kDPoff + c / 2, ds);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full[h & 1]);
    }
    if (ok && n_it > 0) ok = mbar_wait(acc_done, 0, abort_flag);
    if (n_it == 0 || ok) {
      tc_fence_after();
      uint16_t* dkr = static_cast<uint16_t*>(p.dk) + b * p.dk_sb + static_cast<int64_t>(hkv) * p.dk_sh + static_cast<int64_t>(key) * p.dk_ss;
      uint16_t* dvr = static_cast<uint16_t*>(p.dv) + b * p.dv_sb + static_cast<int64_t>(hkv) * p.dv_sh + static_cast<int64_t>(key) * p.dv_ss;
      if (n_it > 0) {   // one group stores dV, the other dK
        if (colgroup == 0) store_acc_row<BF16>(tmem_base + lane_sel + kDV, dvr, key_valid);
        else store_acc_row<BF16>(tmem_base + lane_sel + kDK, dkr, key_valid);
      } else if (key_valid && colgroup == 0) {   // no query sees these keys: zero gradient
        for (int c = 0; c < D; ++c) { dkr[c] = 0; dvr[c] = 0; }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_word, 2u);
}

bool make_map4(CUtensorMap* m, const b200Tensor* t, const char** err) {
  const uint64_t dims[4] = {(uint64_t)t->sizes[3], (uint64_t)t->sizes[2], (uint64_t)t->sizes[1], (uint64_t)t->sizes[0]};
  auto st = [&](int d) { return static_cast<uint64_t>(t->sizes[d] == 1 ? t->sizes[3] * 8 : t->strides[d]) * 2; };
  const uint64_t strides[3] = {st(2), st(1), st(0)};
  const uint32_t box[4] = {64, BT, 1, 1};
  return tc::encode_tmap_16bit(m, t->data, 4, dims, strides, box, err);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_sdpa_flash_bwd_workspace_size(const b200Tensor* q) {
  if (!q || q->ndim != 4) return 0;
  return static_cast<size_t>(q->sizes[0] * q->sizes[1] * q->sizes[2]) * sizeof(float) + 256;
}

b200Status b200_sdpa_flash_bwd(const b200Tensor* dq, const b200Tensor* dk, const b200Tensor* dv, const b200Tensor* dout,
                               const b200Tensor* q, const b200Tensor* k, const b200Tensor* v, const b200Tensor* out,
                               const b200Tensor* lse, int32_t is_causal, double scale, void* workspace, size_t workspace_bytes,
                               b200Stream stream) {
  const char* name = "b200_sdpa_flash_bwd";
  for (const b200Tensor* t : {dq, dk, dv, dout, q, k, v, out})
    B200_REQUIRE(valid(t) && t->ndim == 4, B200_BAD_PARAM, "%s: dq, dk, dv, dout, q, k, v, out must be (B,H,S,D) views", name);
  B200_REQUIRE((q->dtype == B200_BF16 || q->dtype == B200_F16), B200_NOT_SUPPORTED, "%s: bf16 or f16", name);
  for (const b200Tensor* t : {dq, dk, dv, dout, k, v, out})
    B200_REQUIRE(t->dtype == q->dtype, B200_BAD_PARAM, "%s: all operands must share one dtype", name);
  BwdParams p{};
  p.B = (int)q->sizes[0]; p.Hq = (int)q->sizes[1]; p.Sq = (int)q->sizes[2];
  p.Hkv = (int)k->sizes[1]; p.Sk = (int)k->sizes[2];
  B200_REQUIRE(q->sizes[3] == D && k->sizes[3] == D, B200_NOT_SUPPORTED, "%s: head dim 128", name);
  B200_REQUIRE(same_shape(dq, q) && same_shape(dout, q) && same_shape(out, q) && same_shape(k, v) && same_shape(dk, k) &&
               same_shape(dv, v) && k->sizes[0] == p.B, B200_BAD_PARAM, "%s: shape mismatch", name);
  B200_REQUIRE(p.Hkv > 0 && p.Hq % p.Hkv == 0, B200_BAD_PARAM, "%s: Hq must be a multiple of Hkv", name);
  B200_REQUIRE(!is_causal || p.Sq == p.Sk, B200_NOT_SUPPORTED, "%s: causal needs Sq == Sk", name);
  B200_REQUIRE(scale > 0.0, B200_NOT_SUPPORTED, "%s: scale must be positive", name);
  B200_REQUIRE(valid(lse) && lse->dtype == B200_F32 && is_contiguous(lse) && numel(lse) == (int64_t)p.B * p.Hq * p.Sq,
               B200_BAD_PARAM, "%s: lse must be contiguous f32 (B,Hq,Sq)", name);
  if (numel(q) == 0 || numel(k) == 0) return B200_OK;
  for (const b200Tensor* t : {dq, dk, dv, dout, q, k, v, out}) {
    B200_REQUIRE(t->strides[3] == 1 && reinterpret_cast<uintptr_t>(t->data) % 16 == 0, B200_NOT_SUPPORTED,
                 "%s: last dim must be contiguous and the base 16-byte aligned", name);
    for (int d = 0; d < 3; ++d)
      B200_REQUIRE(t->sizes[d] == 1 || t->strides[d] % 8 == 0, B200_NOT_SUPPORTED, "%s: strides must be multiples of 8 elements", name);
  }
  B200_REQUIRE(workspace && workspace_bytes >= b200_sdpa_flash_bwd_workspace_size(q) &&
               reinterpret_cast<uintptr_t>(workspace) % 256 == 0, B200_WORKSPACE_TOO_SMALL,
               "%s: workspace of %zu bytes (256-byte aligned) required", name, b200_sdpa_flash_bwd_workspace_size(q));
  B200_REQUIRE(p.B <= 65535 && p.Hq <= 65535, B200_NOT_SUPPORTED, "%s: batch / heads too large", name);
  p.causal = is_causal ? 1 : 0;
  p.scale = static_cast<float>(scale);
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.lse = static_cast<const float*>(lse->data);
  float* delta = static_cast<float*>(workspace);
  p.delta = delta;
  p.dq = dq->data; p.dq_sb = dq->strides[0]; p.dq_sh = dq->strides[1]; p.dq_ss = dq->strides[2];
  p.dk = dk->data; p.dk_sb = dk->strides[0]; p.dk_sh = dk->strides[1]; p.dk_ss = dk->strides[2];
  p.dv = dv->data; p.dv_sb = dv->strides[0]; p.dv_sh = dv->strides[1]; p.dv_ss = dv->strides[2];
  p.error_word = device_error_word();
  B200_REQUIRE(p.error_word, B200_LAUNCH_FAILED, "%s: device error word unavailable", name);
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  CUtensorMap tq, tdo, tk, tv;
  const char* err = "";
  B200_REQUIRE(make_map4(&tq, q, &err) && make_map4(&tdo, dout, &err) && make_map4(&tk, k, &err) && make_map4(&tv, v, &err),
               B200_NOT_SUPPORTED, "%s: %s", name, err);
  const bool bf = q->dtype == B200_BF16;
  static thread_local int last_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != last_dev) {
    cudaError_t e = cudaFuncSetAttribute(attention_bwd_dq_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDq);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_bwd_dq_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDq);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_bwd_dkv_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDkv);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(attention_bwd_dkv_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemDkv);
    B200_REQUIRE(e == cudaSuccess, B200_LAUNCH_FAILED, "%s: %s", name, cudaGetErrorString(e));
    last_dev = dev;
  }
  const int64_t rows = static_cast<int64_t>(p.B) * p.Hq * p.Sq;
  const int dgrid = grid_for(rows * 32, 256, 8);
  if (bf)
    delta_kernel<bf16_t><<<dgrid, 256, 0, s>>>(delta, static_cast<const bf16_t*>(dout->data), static_cast<const bf16_t*>(out->data), rows,
                                               p.Hq, p.Sq, dout->strides[0], dout->strides[1], dout->strides[2], out->strides[0],
                                               out->strides[1], out->strides[2]);
  else
    delta_kernel<f16_t><<<dgrid, 256, 0, s>>>(delta, static_cast<const f16_t*>(dout->data), static_cast<const f16_t*>(out->data), rows,
                                              p.Hq, p.Sq, dout->strides[0], dout->strides[1], dout->strides[2], out->strides[0],
                                              out->strides[1], out->strides[2]);
  const dim3 gq((p.Sq + BT - 1) / BT, p.Hq, p.B), gk((p.Sk + BT - 1) / BT, p.Hkv, p.B);
  if (bf) {
    attention_bwd_dq_kernel<true><<<gq, kThreadsBwd, kSmemDq, s>>>(tq, tdo, tk, tv, p);
    attention_bwd_dkv_kernel<true><<<gk, kThreadsDkv, kSmemDkv, s>>>(tq, tdo, tk, tv, p);
  } else {
    attention_bwd_dq_kernel<false><<<gq, kThreadsBwd, kSmemDq, s>>>(tq, tdo, tk, tv, p);
    attention_bwd_dkv_kernel<false><<<gk, kThreadsDkv, kSmemDkv, s>>>(tq, tdo, tk, tv, p);
  }
  note_launches(2);
  return check_launch(name);
}

}  // extern "C"
