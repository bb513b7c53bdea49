// bf16 / f16 matrix multiply on the 5th-generation tensor cores.
//
//   out[b] = alpha * A[b] @ B[b] + beta * Cin[b],  fp32 accumulation.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0     TMA producer: 128 x 64 tiles of A and BN x 64 tiles of B into a
//              ring of shared-memory stages (128-byte swizzle), mbarrier-tracked
//   warp 1     allocates tensor memory and issues tcgen05.mma (128 x BN x 16),
//              one elected thread; commits free the stage / publish the tile
//   warps 2-5  epilogue: tcgen05.ld the fp32 accumulator (each warp its 32-lane
//              quarter), scale, add beta*Cin, round, store 64-byte row segments
// Two accumulators live in tensor memory (2 x BN columns), so the epilogue of
// tile i overlaps the main loop of tile i+1. Tiles are walked in groups of 8
// row-tiles so that concurrently running CTAs share A and B tiles through L2.
// Either operand may be K-major (K contiguous) or MN-major (M / N contiguous);
// the layout goes into the tensor maps and the MMA descriptors, no copy is made.
// Loads never use cluster multicast. Every barrier wait is bounded.
#include "common.cuh"
#include "gemm_simt.cuh"
#include "tc_common.cuh"

#include <cooperative_groups.h>
#include <mutex>

namespace b200 {
unsigned int* device_error_word();  // index.cu: address of the device error word

namespace tc {

bool encode_tmap_16bit(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box, const char** err) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
    else
      cudaGetLastError();
  });
  if (!fn) {
    *err = "cuTensorMapEncodeTiled is not available from this driver";
    return false;
  }
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base),
                  reinterpret_cast<const cuuint64_t*>(dims), reinterpret_cast<const cuuint64_t*>(strides_bytes),
                  reinterpret_cast<const cuuint32_t*>(box), estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    *err = "cuTensorMapEncodeTiled rejected the operand layout";
    return false;
  }
  return true;
}

}  // namespace tc

namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BK = 64;           // 64 x 16-bit = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kGemmThreads = 192;
constexpr int kBandBytes = 32 << 20;   // rows of A kept hot in L2 while one band of row-tiles sweeps all of B

struct GemmParams {
  int M, N, K, batch;
  int a_mn_major, b_mn_major;    // 0: K contiguous, 1: M (resp. N) contiguous
  int is_bf16;
  float alpha, beta;
  void* out;
  int64_t o_sb, o_sm;            // out: column stride 1
  const void* cin;
  int64_t c_sb, c_sm, c_sn;
  unsigned int* error_word;
  int up_offset;                 // fused SwiGLU: row of B where the "up" half starts (= output columns F)
  int group_m;                   // row-tiles per band of the tile walk
  // fused RoPE epilogue: rotate-half over 128-wide heads of the first rope_cols output columns;
  // f32 (positions, 64) tables, position of row m = m % rope_seq
  const float* rope_cos;
  const float* rope_sin;
  int rope_seq, rope_cols;
};

template <int BN> struct GemmCfg {
  static constexpr int kStageA = BM * BK * 2;
  static constexpr int kStageB = BN * BK * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kStages = (196608 / kStage) > 8 ? 8 : (196608 / kStage);
  static constexpr int kSmem = kStages * kStage + 1024 /* alignment slack */ + 256 /* barriers */;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;  // power of two for BN in {64,128,256}
};

// Row-tiles per band: as many as keep the band's rows of A (tile_rows x K each) within kBandBytes,
// so that B is streamed from DRAM once per band and A once in total.
inline int band_rows(int tile_rows, int64_t K) {
  static const int forced = [] { const char* e = getenv("B200_GEMM_BAND"); return e ? atoi(e) : 0; }();   // tuning aid
  if (forced > 0) return forced;
  const int64_t per_tile = static_cast<int64_t>(tile_rows) * K * 2;
  int64_t g = per_tile > 0 ? kBandBytes / per_tile : 8;
  return static_cast<int>(g < 8 ? 8 : (g > 64 ? 64 : g));   // never narrower than 8: a long K needs B reuse more
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int GROUP_M, int& b, int& tm, int& tn) {
  const int per_batch = tiles_m * tiles_n;
  b = tile / per_batch;
  int t = tile - b * per_batch;
  const int group = t / (GROUP_M * tiles_n);
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, tiles_m - first_m);
  t -= group * GROUP_M * tiles_n;
  tm = first_m + t % rows;
  tn = t / rows;
}

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kStages * Cfg::kStage);
  uint64_t* full = bars;                       // [kStages]
  uint64_t* empty = bars + Cfg::kStages;       // [kStages]
  uint64_t* acc_full = empty + Cfg::kStages;   // [2]
  uint64_t* acc_empty = acc_full + 2;          // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int n_tiles = tiles_m * tiles_n * p.batch;
  const int n_k = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < Cfg::kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
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
  pdl_wait();   // barriers and tensor memory were set up under the predecessor's tail; operands are read from here on

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      prefetch_tmap(&tmap_a);
      prefetch_tmap(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        int b, tm, tn;
        tile_coords(tile, tiles_m, tiles_n, p.group_m, b, tm, tn);
        for (int k = 0; k < n_k; ++k) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::kStage;
          uint8_t* sb = sa + Cfg::kStageA;
          mbar_arrive_expect_tx(&full[stage], Cfg::kStage);
          if (!p.a_mn_major) {
            tma_load_3d(sa, &tmap_a, &full[stage], k * BK, tm * BM, b);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_3d(sa + j * 8192, &tmap_a, &full[stage], tm * BM + j * 64, k * BK, b);
          }
          if (!p.b_mn_major) {
            tma_load_3d(sb, &tmap_b, &full[stage], k * BK, tn * BN, b);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sb + j * 8192, &tmap_b, &full[stage], tn * BN + j * 64, k * BK, b);
          }
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
        }
      }
      // every load of this CTA is issued: the successor may take SM resources as they come free
      // (it is triggered late, so a waiting successor never sits on SMs for longer than one tile)
      pdl_launch_dependents();
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BM, BN, p.is_bf16 != 0, p.a_mn_major != 0, p.b_mn_major != 0);
      // K-major: rows of 128 B, 8-row groups 1024 B apart, 32 B per UMMA_K step.
      // MN-major: 64-element groups 8192 B apart (one TMA box each), 8-k groups
      // 1024 B apart, 2048 B per UMMA_K step.
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u, a_step = p.a_mn_major ? 2048u : 32u;
      const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u, b_step = p.b_mn_major ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
        const int ab = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(&acc_empty[ab], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(ab * BN);
        for (int k = 0; k < n_k; ++k) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::kStage);
          const uint32_t sb = sa + Cfg::kStageA;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = smem_desc_sw128(sa + kk * a_step, a_lbo, 1024u);
            const uint64_t db = smem_desc_sw128(sb + kk * b_step, b_lbo, 1024u);
            umma_f16(d_tmem, da, db, idesc, (k | kk) != 0 ? 1u : 0u);
          }
          umma_commit(&empty[stage]);  // stage reusable once these MMAs have read it
          if (++stage == Cfg::kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&acc_full[ab]);  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue --
    const int quarter = warp & 3;  // the TMEM lanes this warp may read
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
      const int ab = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      int b, tm, tn;
      tile_coords(tile, tiles_m, tiles_n, p.group_m, b, tm, tn);
      if (!mbar_wait(&acc_full[ab], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      uint16_t* orow = static_cast<uint16_t*>(p.out) + b * p.o_sb + static_cast<int64_t>(row) * p.o_sm;
      const uint16_t* crow = p.cin ? static_cast<const uint16_t*>(p.cin) + b * p.c_sb + static_cast<int64_t>(row) * p.c_sm
                                   : nullptr;
      const bool vec_ok = (p.o_sm % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) + 2 * b * p.o_sb) % 16 == 0);
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(ab * BN + c), r);
        tmem_wait_ld();
        const int col0 = tn * BN + c;
        if (row_ok && col0 < p.N) {
          alignas(16) uint16_t o[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float v = p.alpha * __uint_as_float(r[j]);
            if (crow && col0 + j < p.N) {
              const uint16_t cb = crow[static_cast<int64_t>(col0 + j) * p.c_sn];
              v += p.beta * (p.is_bf16 ? bf16_bits_to_f32(cb) : f16_bits_to_f32(cb));
            }
            o[j] = p.is_bf16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v);
          }
          if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              *reinterpret_cast<int4*>(orow + col0 + q * 8) = *reinterpret_cast<const int4*>(o + q * 8);
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) orow[col0 + j] = o[j];
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[ab]);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_word, 2u);  // bit 1: a barrier wait timed out
}

struct Operand {
  const void* base;
  bool mn_major;
  uint64_t dims[3];
  uint64_t strides[2];
  uint32_t box[3];
};

// Describes a (rows x K) operand (A: rows = M; B: rows = N) for TMA, or fails.
bool describe_operand(const void* data, int64_t rows, int64_t K, int64_t batch, int64_t s_row, int64_t s_k,
                      int64_t s_b, int tile_rows, Operand* o) {
  if (reinterpret_cast<uintptr_t>(data) % 16) return false;
  if (batch > 1 && (s_b % 8 != 0 || s_b <= 0)) return false;
  auto align16 = [](uint64_t x) { return (x + 15) & ~uint64_t(15); };
  o->base = data;
  if ((s_k == 1 || K == 1) && s_row % 8 == 0 && s_row >= K) {
    o->mn_major = false;
    o->dims[0] = K; o->dims[1] = rows; o->dims[2] = batch;
    o->strides[0] = static_cast<uint64_t>(s_row) * 2;
    o->strides[1] = batch > 1 ? static_cast<uint64_t>(s_b) * 2 : align16(static_cast<uint64_t>(s_row) * rows * 2);
    o->box[0] = BK; o->box[1] = tile_rows; o->box[2] = 1;
    return true;
  }
  if ((s_row == 1 || rows == 1) && s_k % 8 == 0 && s_k >= rows) {
    o->mn_major = true;
    o->dims[0] = rows; o->dims[1] = K; o->dims[2] = batch;
    o->strides[0] = static_cast<uint64_t>(s_k) * 2;
    o->strides[1] = batch > 1 ? static_cast<uint64_t>(s_b) * 2 : align16(static_cast<uint64_t>(s_k) * K * 2);
    o->box[0] = 64; o->box[1] = BK; o->box[2] = 1;
    return true;
  }
  return false;
}

template <int BN>
b200Status launch_tc(const Operand& oa, const Operand& ob, GemmParams p, cudaStream_t s) {
  using Cfg = GemmCfg<BN>;
  CUtensorMap ta, tb;
  const char* err = "";
  B200_REQUIRE(encode_tmap_16bit(&ta, oa.base, 3, oa.dims, oa.strides, oa.box, &err), B200_NOT_SUPPORTED, "matmul: %s", err);
  B200_REQUIRE(encode_tmap_16bit(&tb, ob.base, 3, ob.dims, ob.strides, ob.box, &err), B200_NOT_SUPPORTED, "matmul: %s", err);
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
  });
  // the attribute is per device: set it again when this device has not seen it
  static thread_local int last_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != last_dev) {
    attr_err = cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmem);
    last_dev = dev;
  }
  B200_REQUIRE(attr_err == cudaSuccess, B200_LAUNCH_FAILED, "matmul: %s", cudaGetErrorString(attr_err));
  p.group_m = band_rows(BM, p.K);
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * p.batch;
  const int sms = gemm_sm_budget();
  const int grid = tiles < sms ? tiles : sms;
  cudaError_t le = launch_pdl(gemm_tc_kernel<BN>, grid, kGemmThreads, Cfg::kSmem, s, ta, tb, p);
  B200_REQUIRE(le == cudaSuccess, B200_LAUNCH_FAILED, "matmul: %s", cudaGetErrorString(le));
  return check_launch("matmul (tcgen05)");
}

// ---------------------------------------------------------------------------
// Two-CTA variant (cta_group::2): a cluster of two CTAs on neighbouring SMs owns a
// 256 x 256 output tile. Each CTA loads its 128 rows of A and its 128 columns of B
// (32 KB per stage instead of 48, six stages instead of four), one thread of the
// even CTA issues 256 x 256 x 16 MMAs that read both CTAs' shared memory, and each
// CTA's tensor memory receives its own 128 accumulator rows. Operand traffic per SM
// drops by a third, which is what bounds the one-CTA kernel.
//   full[s]      lives in the even CTA; both CTAs' TMA loads complete on it
//   empty[s]     in each CTA, released by a commit that arrives in both CTAs
//   acc_full[a]  in each CTA (same commit form); acc_empty[a] in the even CTA,
//                eight arrivals: the four epilogue warps of both CTAs
constexpr int BN2 = 256;            // columns of the pair's tile
constexpr int BM2 = 2 * BM;         // rows of the pair's tile
constexpr int kStageHalfB = (BN2 / 2) * BK * 2;
constexpr int kStage2 = BM * BK * 2 + kStageHalfB;   // 32 KB per CTA
constexpr int kStages2 = 6;
constexpr int kSmem2 = kStages2 * kStage2 + 1024 + 256;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}
// Tile load into this CTA's shared memory whose completion is counted on a barrier of the even CTA.
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* m, uint32_t bar_cluster_addr, int x,
                                                 int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once
// every MMA issued so far has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask)
               : "memory");
}

// SWIGLU: B is a (2F x K) gate/up weight (gate rows first). The even CTA loads 128
// gate rows, the odd CTA the matching 128 up rows, so accumulator columns [0,128)
// hold gate and [128,256) up for the same 128 output columns, and the epilogue
// stores silu(gate) * up (computed on the fp32 accumulators): the 2F-wide
// intermediate never exists in memory. p.N is F here.
// EPI 2 (RoPE): output columns below p.rope_cols are heads of 128 (a 256-wide tile holds two) and get the
// rotate-half rotary embedding applied to the fp32 accumulators before the one rounding; the rest are stored
// as they are (the v part of a fused qkv projection).
template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const GemmParams p) {
  constexpr bool SWIGLU = EPI == 1, ROPE = EPI == 2;
  constexpr int BNO = SWIGLU ? BN2 / 2 : BN2;   // output columns per tile
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages2 * kStage2);
  uint64_t* full = bars;                       // [kStages2], used in the even CTA
  uint64_t* empty = bars + kStages2;           // [kStages2]
  uint64_t* acc_full = empty + kStages2;       // [2]
  uint64_t* acc_empty = acc_full + 2;          // [2], used in the even CTA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();     // 0: issues the MMAs
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_m = (p.M + BM2 - 1) / BM2, tiles_n = (p.N + BNO - 1) / BNO;
  const int n_tiles = tiles_m * tiles_n * p.batch;
  const int n_k = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages2; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // both CTAs' barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();   // set-up above runs under the predecessor's tail; operands are read from here on

  if (warp == 0) {
    // ------------------------------------------------------------ producer --
    if (lane == 0) {
      prefetch_tmap(&tmap_a);
      prefetch_tmap(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
        int b, tm, tn;
        tile_coords(tile, tiles_m, tiles_n, p.group_m, b, tm, tn);
        const int row0 = tm * BM2 + static_cast<int>(rank) * BM;          // this CTA's rows of A
        const int col0 = SWIGLU ? tn * BNO + static_cast<int>(rank) * p.up_offset   // gate rows / up rows of B
                                : tn * BN2 + static_cast<int>(rank) * (BN2 / 2);    // this CTA's columns of B
        for (int k = 0; k < n_k; ++k) {
          if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = smem + stage * kStage2;
          uint8_t* sb = sa + BM * BK * 2;
          const uint32_t bar = map_to_cta(smem_u32(&full[stage]), 0);
          if (rank == 0) mbar_arrive_expect_tx(&full[stage], 2 * kStage2);   // the bytes of both CTAs
          if (!p.a_mn_major) {
            tma_load_3d_pair(sa, &tmap_a, bar, k * BK, row0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_3d_pair(sa + j * 8192, &tmap_a, bar, row0 + j * 64, k * BK, b);
          }
          if (!p.b_mn_major) {
            tma_load_3d_pair(sb, &tmap_b, bar, k * BK, col0, b);
          } else {
#pragma unroll
            for (int j = 0; j < BN2 / 2 / 64; ++j) tma_load_3d_pair(sb + j * 8192, &tmap_b, bar, col0 + j * 64, k * BK, b);
          }
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
      }
      pdl_launch_dependents();   // all loads issued: at most one tile of work is left
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer --
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc(BM2, BN2, p.is_bf16 != 0, p.a_mn_major != 0, p.b_mn_major != 0);
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u, a_step = p.a_mn_major ? 2048u : 32u;
      const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u, b_step = p.b_mn_major ? 2048u : 32u;
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++it) {
        const int ab = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (!mbar_wait(&acc_empty[ab], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(ab * BN2);
        for (int k = 0; k < n_k; ++k) {
          if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kStage2);
          const uint32_t sb = sa + BM * BK * 2;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint64_t da = smem_desc_sw128(sa + kk * a_step, a_lbo, 1024u);
            const uint64_t db = smem_desc_sw128(sb + kk * b_step, b_lbo, 1024u);
            umma_f16_pair(d_tmem, da, db, idesc, (k | kk) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty[stage]);
          if (++stage == kStages2) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit_pair(&acc_full[ab]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue --
    const int quarter = warp & 3;
    int it = 0;
    bool ok = true;
    for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++it) {
      const int ab = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      int b, tm, tn;
      tile_coords(tile, tiles_m, tiles_n, p.group_m, b, tm, tn);
      if (!mbar_wait(&acc_full[ab], acc_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM2 + static_cast<int>(rank) * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      uint16_t* orow = static_cast<uint16_t*>(p.out) + b * p.o_sb + static_cast<int64_t>(row) * p.o_sm;
      const uint16_t* crow = p.cin ? static_cast<const uint16_t*>(p.cin) + b * p.c_sb + static_cast<int64_t>(row) * p.c_sm
                                   : nullptr;
      const bool vec_ok = (p.o_sm % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.out) + 2 * b * p.o_sb) % 16 == 0);
      if (SWIGLU) {
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(ab * BN2);
#pragma unroll 1
        for (int c = 0; c < BNO; c += 32) {
          uint32_t rg[32], ru[32];
          tmem_ld_32x32(t_row + c, rg);
          tmem_ld_32x32(t_row + BNO + c, ru);
          tmem_wait_ld();
          const int col0 = tn * BNO + c;
          if (row_ok && col0 < p.N) {
            uint32_t o[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float g0 = __uint_as_float(rg[2 * j]), g1 = __uint_as_float(rg[2 * j + 1]);
              const float v0 = __fdividef(g0, 1.0f + __expf(-g0)) * __uint_as_float(ru[2 * j]);
              const float v1 = __fdividef(g1, 1.0f + __expf(-g1)) * __uint_as_float(ru[2 * j + 1]);
              if (p.is_bf16) {
                o[j] = f32x2_to_bf16x2_bits(v0, v1);
              } else {
                __half2 h = __floats2half2_rn(v0, v1);
                o[j] = *reinterpret_cast<uint32_t*>(&h);
              }
            }
            if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
              for (int q = 0; q < 4; ++q)
                *reinterpret_cast<uint4*>(orow + col0 + q * 8) = make_uint4(o[q * 4], o[q * 4 + 1], o[q * 4 + 2], o[q * 4 + 3]);
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j)
                orow[col0 + j] = static_cast<uint16_t>(j & 1 ? o[j >> 1] >> 16 : o[j >> 1] & 0xffffu);
            }
          }
        }
      } else if (ROPE && tn * BN2 < p.rope_cols) {
        const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(ab * BN2);
        const int pos = row_ok ? row % p.rope_seq : 0;
        const float* cs = p.rope_cos + static_cast<int64_t>(pos) * 64;
        const float* sn = p.rope_sin + static_cast<int64_t>(pos) * 64;
#pragma unroll 1
        for (int hc = 0; hc < 128; hc += 32) {       // (head of the tile, 32-column chunk of its first half)
          const int hd = hc >> 6, c = hc & 32;        // hc = 0, 32 -> head 0; 64, 96 -> head 1
          uint32_t x1[32], x2[32];
          tmem_ld_32x32(t_row + hd * 128 + c, x1);
          tmem_ld_32x32(t_row + hd * 128 + c + 64, x2);
          tmem_wait_ld();
          const int col0 = tn * BN2 + hd * 128 + c;
          if (row_ok && col0 < p.N) {
            const bool rot = col0 < p.rope_cols;
            uint32_t o1[16], o2[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              float a0 = p.alpha * __uint_as_float(x1[j]), a1 = p.alpha * __uint_as_float(x1[j + 1]);
              float b0 = p.alpha * __uint_as_float(x2[j]), b1 = p.alpha * __uint_as_float(x2[j + 1]);
              if (rot) {
                const float c0 = cs[c + j], c1 = cs[c + j + 1], s0 = sn[c + j], s1 = sn[c + j + 1];
                const float r0 = a0 * c0 - b0 * s0, r1 = a1 * c1 - b1 * s1;
                b0 = b0 * c0 + a0 * s0;
                b1 = b1 * c1 + a1 * s1;
                a0 = r0;
                a1 = r1;
              }
              if (p.is_bf16) {
                o1[j / 2] = f32x2_to_bf16x2_bits(a0, a1);
                o2[j / 2] = f32x2_to_bf16x2_bits(b0, b1);
              } else {
                __half2 h1 = __floats2half2_rn(a0, a1), h2 = __floats2half2_rn(b0, b1);
                o1[j / 2] = *reinterpret_cast<uint32_t*>(&h1);
                o2[j / 2] = *reinterpret_cast<uint32_t*>(&h2);
              }
            }
            if (vec_ok && col0 + 96 <= p.N) {
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                *reinterpret_cast<uint4*>(orow + col0 + q * 8) = make_uint4(o1[q * 4], o1[q * 4 + 1], o1[q * 4 + 2], o1[q * 4 + 3]);
                *reinterpret_cast<uint4*>(orow + col0 + 64 + q * 8) = make_uint4(o2[q * 4], o2[q * 4 + 1], o2[q * 4 + 2], o2[q * 4 + 3]);
              }
            } else {
              for (int j = 0; j < 32; ++j) {
                if (col0 + j < p.N) orow[col0 + j] = static_cast<uint16_t>(j & 1 ? o1[j >> 1] >> 16 : o1[j >> 1] & 0xffffu);
                if (col0 + 64 + j < p.N) orow[col0 + 64 + j] = static_cast<uint16_t>(j & 1 ? o2[j >> 1] >> 16 : o2[j >> 1] & 0xffffu);
              }
            }
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN2; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(ab * BN2 + c), r);
        tmem_wait_ld();
        const int col0 = tn * BN2 + c;
        if (row_ok && col0 < p.N) {
          alignas(16) uint16_t o[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float v = p.alpha * __uint_as_float(r[j]);
            if (crow && col0 + j < p.N) {
              const uint16_t cb = crow[static_cast<int64_t>(col0 + j) * p.c_sn];
              v += p.beta * (p.is_bf16 ? bf16_bits_to_f32(cb) : f16_bits_to_f32(cb));
            }
            o[j] = p.is_bf16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v);
          }
          if (vec_ok && col0 + 32 <= p.N) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              *reinterpret_cast<int4*>(orow + col0 + q * 8) = *reinterpret_cast<const int4*>(o + q * 8);
          } else {
            for (int j = 0; j < 32 && col0 + j < p.N; ++j) orow[col0 + j] = o[j];
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[ab]), 0));
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // nothing of the peer is touched after this point
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_word, 2u);
}

template <int EPI>
b200Status launch_tc2(const Operand& oa, const Operand& ob, GemmParams p, cudaStream_t s) {
  CUtensorMap ta, tb;
  const char* err = "";
  B200_REQUIRE(encode_tmap_16bit(&ta, oa.base, 3, oa.dims, oa.strides, oa.box, &err), B200_NOT_SUPPORTED, "matmul: %s", err);
  B200_REQUIRE(encode_tmap_16bit(&tb, ob.base, 3, ob.dims, ob.strides, ob.box, &err), B200_NOT_SUPPORTED, "matmul: %s", err);
  static thread_local int last_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != last_dev) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc2_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem2);
    B200_REQUIRE(e == cudaSuccess, B200_LAUNCH_FAILED, "matmul: %s", cudaGetErrorString(e));
    last_dev = dev;
  }
  constexpr int bno = EPI == 1 ? BN2 / 2 : BN2;
  p.group_m = band_rows(BM2, p.K);
  const int tiles = ((p.M + BM2 - 1) / BM2) * ((p.N + bno - 1) / bno) * p.batch;
  const int pairs = gemm_sm_budget() / 2;
  const int grid = 2 * (tiles < pairs ? tiles : pairs);
  cudaError_t le = launch_pdl(gemm_tc2_kernel<EPI>, grid, kGemmThreads, kSmem2, s, ta, tb, p);
  B200_REQUIRE(le == cudaSuccess, B200_LAUNCH_FAILED, "matmul: %s", cudaGetErrorString(le));
  return check_launch("matmul (tcgen05, two-CTA)");
}

// ---------------------------------------------------------------------------
// Split-K variant for skinny products (M <= 128, e.g. one decode token per
// sequence): streaming the weight matrix is all that matters, so the grid is one
// wave of CTAs, two per SM, each with a 96 KB ring in flight. A cluster of `splits`
// CTAs (2, 4 or 8) shares one 128 x 128 output tile; each CTA runs the TMA / MMA pipeline over its slice of K, parks its fp32
// partial tile in shared memory, and after a cluster barrier every CTA sums one
// band of rows over all partials through distributed shared memory, always in rank
// order, so the result does not depend on timing.
constexpr int BNS = 128;
constexpr int kStageS = BM * BK * 2 + BNS * BK * 2;   // 32 KB
constexpr int kStagesS = 3;                           // 96 KB: two CTAs per SM
constexpr int kPartialStride = BNS + 4;               // padded: 16-byte accesses along rows and along columns without bank conflicts
constexpr int kSmemS = kStagesS * kStageS + 1024 + 256;
static_assert(BM * kPartialStride * 4 <= kStagesS * kStageS, "the partial tile reuses the drained stage ring");

// SWIGLU: B is a fused gate/up weight (2F, K), p.N = F output columns. A tile holds 64 gate rows and the 64 up rows
// that go with them (two boxes of 64 rows), so the summed tile has a gate half and an up half, and the band owner
// stores silu(gate) * up: 64 output columns per tile.
template <bool SWIGLU>
__global__ void __launch_bounds__(kGemmThreads, 2)
gemm_splitk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const GemmParams p, const int splits) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStagesS * kStageS);
  uint64_t* full = bars;
  uint64_t* empty = bars + kStagesS;
  uint64_t* acc_full = empty + kStagesS;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* partial = reinterpret_cast<float*>(smem);   // [BM][kPartialStride], valid after the ring drained

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster.block_rank());
  constexpr int kCols = SWIGLU ? BNS / 2 : BNS;   // output columns per tile
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + kCols - 1) / kCols;
  int b, tm, tn;
  tile_coords(static_cast<int>(blockIdx.x) / splits, tiles_m, tiles_n, p.group_m, b, tm, tn);
  const int n_k = (p.K + BK - 1) / BK;
  const int per = (n_k + splits - 1) / splits;
  const int k_begin = min(rank * per, n_k), k_end = min(k_begin + per, n_k);
  const int n_my = k_end - k_begin;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStagesS; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, BNS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) {
    // under the predecessor's tail: the descriptors, and the first ring's worth of B (a weight, as a rule) asked into
    // L2, where the loads below find it whatever the predecessor was still doing
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    if (!p.b_mn_major)
      for (int i = 0; i < min(n_my, kStagesS); ++i) {
        tma_prefetch_l2_3d(&tmap_b, (k_begin + i) * BK, tn * kCols, b);
        if (SWIGLU) tma_prefetch_l2_3d(&tmap_b, (k_begin + i) * BK, p.up_offset + tn * kCols, b);
      }
  }
  pdl_wait();   // set-up above runs under the predecessor's tail; operands are read from here on

  if (warp == 0) {
    if (lane == 0) {
      for (int i = 0; i < n_my; ++i) {
        const int stage = i % kStagesS;
        const uint32_t phase = (i / kStagesS) & 1u;
        if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) break;
        uint8_t* sa = smem + stage * kStageS;
        uint8_t* sb = sa + BM * BK * 2;
        const int k = k_begin + i;
        mbar_arrive_expect_tx(&full[stage], kStageS);
        if (!p.a_mn_major) {
          tma_load_3d(sa, &tmap_a, &full[stage], k * BK, tm * BM, b);
        } else {
#pragma unroll
          for (int j = 0; j < BM / 64; ++j) tma_load_3d(sa + j * 8192, &tmap_a, &full[stage], tm * BM + j * 64, k * BK, b);
        }
        if (SWIGLU) {
          tma_load_3d(sb, &tmap_b, &full[stage], k * BK, tn * kCols, b);                              // gate rows
          tma_load_3d(sb + kCols * BK * 2, &tmap_b, &full[stage], k * BK, p.up_offset + tn * kCols, b);   // up rows
        } else if (!p.b_mn_major) {
          tma_load_3d(sb, &tmap_b, &full[stage], k * BK, tn * BNS, b);
        } else {
#pragma unroll
          for (int j = 0; j < BNS / 64; ++j) tma_load_3d(sb + j * 8192, &tmap_b, &full[stage], tn * BNS + j * 64, k * BK, b);
        }
      }
      pdl_launch_dependents();   // all loads issued
    }
  } else if (warp == 1) {
    if (lane == 0 && n_my > 0) {
      const uint32_t idesc = make_idesc(BM, BNS, p.is_bf16 != 0, p.a_mn_major != 0, p.b_mn_major != 0);
      const uint32_t a_lbo = p.a_mn_major ? 8192u : 16u, a_step = p.a_mn_major ? 2048u : 32u;
      const uint32_t b_lbo = p.b_mn_major ? 8192u : 16u, b_step = p.b_mn_major ? 2048u : 32u;
      bool ok = true;
      for (int i = 0; i < n_my; ++i) {
        const int stage = i % kStagesS;
        const uint32_t phase = (i / kStagesS) & 1u;
        if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * kStageS);
        const uint32_t sb = sa + BM * BK * 2;
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk)
          umma_f16(tmem_base, smem_desc_sw128(sa + kk * a_step, a_lbo, 1024u), smem_desc_sw128(sb + kk * b_step, b_lbo, 1024u),
                   idesc, (i | kk) != 0 ? 1u : 0u);
        umma_commit(&empty[stage]);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    // this CTA's partial tile: tensor memory -> shared memory (zeros when the slice of K is empty); rows past the
    // end of the product are never read
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int valid = min(BM, p.M - tm * BM);
    bool ok = true;
    if (n_my > 0) ok = mbar_wait(acc_full, 0, abort_flag);
    tc_fence_after();
    if (quarter * 32 < valid) {
#pragma unroll 1
      for (int c = 0; c < BNS; c += 32) {
        uint32_t r[32];
        if (n_my > 0 && ok) {
          tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(c), r);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) r[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<uint4*>(&partial[row * kPartialStride + c + j]) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
      }
    }
  }

  tc_fence_before();
  cluster.sync();
  if (warp >= 2) {
    // The rows of the tile that exist are dealt out in bands, one per CTA of the cluster; a CTA sums its band over
    // the partials in rank order, four columns per thread and step, every partial's load issued before the first add.
    const int tid = (warp - 2) * 32 + lane;
    const int valid = min(BM, p.M - tm * BM);
    const int band = (valid + splits - 1) / splits;
    const int r0 = min(valid, rank * band), r1 = min(valid, r0 + band);
    const float* src[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) src[c] = cluster.map_shared_rank(partial, c < splits ? c : 0);
    const bool is_bf16 = p.is_bf16 != 0;
    if constexpr (SWIGLU) {
      for (int u = tid; u < (r1 - r0) * (kCols / 4); u += 128) {
        const int lr = r0 + u / (kCols / 4), col = (u % (kCols / 4)) * 4;
        const int grow = tm * BM + lr, gcol = tn * kCols + col;
        float4 vg[8], vu[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if (c < splits) {
            vg[c] = *reinterpret_cast<const float4*>(src[c] + lr * kPartialStride + col);
            vu[c] = *reinterpret_cast<const float4*>(src[c] + lr * kPartialStride + kCols + col);
          }
        float g[4] = {0.f, 0.f, 0.f, 0.f}, up[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if (c < splits) {
            g[0] += vg[c].x; g[1] += vg[c].y; g[2] += vg[c].z; g[3] += vg[c].w;
            up[0] += vu[c].x; up[1] += vu[c].y; up[2] += vu[c].z; up[3] += vu[c].w;
          }
        if (gcol >= p.N) continue;
        uint16_t bits[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float o = __fdividef(g[j], 1.0f + __expf(-g[j])) * up[j];   // the epilogue of the other SwiGLU kernels
          bits[j] = is_bf16 ? f32_to_bf16_bits(o) : f32_to_f16_bits(o);
        }
        uint16_t* dst = static_cast<uint16_t*>(p.out) + static_cast<int64_t>(grow) * p.o_sm + gcol;
        if (gcol + 3 < p.N && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
          *reinterpret_cast<uint2*>(dst) = make_uint2(bits[0] | (static_cast<uint32_t>(bits[1]) << 16),
                                                      bits[2] | (static_cast<uint32_t>(bits[3]) << 16));
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (gcol + j < p.N) dst[j] = bits[j];
        }
      }
    } else {
      for (int u = tid; u < (r1 - r0) * (BNS / 4); u += 128) {
        const int lr = r0 + u / (BNS / 4), col = (u % (BNS / 4)) * 4;
        const int grow = tm * BM + lr, gcol = tn * BNS + col;
        float4 v[8];
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if (c < splits) v[c] = *reinterpret_cast<const float4*>(src[c] + lr * kPartialStride + col);
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 8; ++c)
          if (c < splits) {
            acc[0] += v[c].x; acc[1] += v[c].y; acc[2] += v[c].z; acc[3] += v[c].w;
          }
        if (gcol >= p.N) continue;
        uint16_t bits[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float o = p.alpha * acc[j];
          if (p.cin && gcol + j < p.N) {
            const uint16_t cb = static_cast<const uint16_t*>(p.cin)[b * p.c_sb + static_cast<int64_t>(grow) * p.c_sm +
                                                                  static_cast<int64_t>(gcol + j) * p.c_sn];
            o += p.beta * (is_bf16 ? bf16_bits_to_f32(cb) : f16_bits_to_f32(cb));
          }
          bits[j] = is_bf16 ? f32_to_bf16_bits(o) : f32_to_f16_bits(o);
        }
        uint16_t* dst = static_cast<uint16_t*>(p.out) + b * p.o_sb + static_cast<int64_t>(grow) * p.o_sm + gcol;
        if (gcol + 3 < p.N && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
          *reinterpret_cast<uint2*>(dst) = make_uint2(bits[0] | (static_cast<uint32_t>(bits[1]) << 16),
                                                      bits[2] | (static_cast<uint32_t>(bits[3]) << 16));
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (gcol + j < p.N) dst[j] = bits[j];
        }
      }
    }
  }
  cluster.sync();   // peers keep their partials alive until everyone has read them

  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, BNS);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_word, 2u);
}

template <bool SWIGLU>
b200Status launch_splitk(const Operand& oa, Operand ob, GemmParams p, int splits, cudaStream_t s) {
  if (SWIGLU) ob.box[1] = BNS / 2;   // gate and up rows of a tile are loaded as two boxes
  CUtensorMap ta, tb;
  const char* err = "";
  B200_REQUIRE(encode_tmap_16bit(&ta, oa.base, 3, oa.dims, oa.strides, oa.box, &err), B200_NOT_SUPPORTED, "matmul: %s", err);
  B200_REQUIRE(encode_tmap_16bit(&tb, ob.base, 3, ob.dims, ob.strides, ob.box, &err), B200_NOT_SUPPORTED, "matmul: %s", err);
  static thread_local int last_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != last_dev) {
    cudaError_t e = cudaFuncSetAttribute(gemm_splitk_kernel<SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemS);
    B200_REQUIRE(e == cudaSuccess, B200_LAUNCH_FAILED, "matmul: %s", cudaGetErrorString(e));
    last_dev = dev;
  }
  p.group_m = 8;
  constexpr int kCols = SWIGLU ? BNS / 2 : BNS;
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + kCols - 1) / kCols) * p.batch;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(tiles * splits);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = kSmemS;
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
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_splitk_kernel<SWIGLU>, ta, tb, p, splits);
  B200_REQUIRE(e == cudaSuccess, B200_LAUNCH_FAILED, "matmul: %s", cudaGetErrorString(e));
  return check_launch("matmul (tcgen05, split-K)");
}

// ---------------------------------------------------------------------------
// One-wave kernel for a single row-tile (M <= 128) against a WIDE weight: the product is bound by
// streaming the weight once, so what matters is that every SM streams an equal share. A tile
// count fixed by a 128- or 256-column tile leaves the last wave part empty (28672 weight rows in
// 256-row tiles: 112 tiles on 148 SMs); here the tile width is a run-time value, a multiple of 16
// chosen so that the tiles fill one wave (28672 rows: 138 tiles of 208), one tile per CTA, the
// whole K range per CTA, no split and no merge. With SWIGLU the tile's weight rows are bn/2 "gate"
// rows and the matching bn/2 "up" rows (two TMA boxes per stage) and the epilogue stores
// silu(gate) * up: bn/2 output columns per tile.
constexpr int kWideRing = 196608;        // stages of 16 KB of A + bn x 128 B of weight rows: as many as fit (at most 12)
constexpr int kWideMaxStages = 12;       // narrow tiles need depth: the stream per SM is stages x weight bytes per round trip
constexpr int kSmemWide = kWideRing + 1024 + 256;

template <bool SWIGLU>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_wide_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmParams p, const int bn) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kWideRing);
  uint64_t* full = bars;
  uint64_t* empty = bars + kWideMaxStages;
  uint64_t* acc_full = empty + kWideMaxStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tn = blockIdx.x;
  const int n_k = (p.K + BK - 1) / BK;
  const int half = bn / 2;
  const int stage_stride = BM * BK * 2 + bn * BK * 2;   // a multiple of 2 KB (bn is a multiple of 16)
  const int n_stages = min(kWideMaxStages, kWideRing / stage_stride);

  if (threadIdx.x == 0) {
    for (int i = 0; i < n_stages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) {
    // under the predecessor's tail: the descriptors, and the first ring's worth of the weight asked into L2
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    for (int k = 0; k < min(n_k, n_stages); ++k) {
      if (SWIGLU) {
        tma_prefetch_l2_3d(&tmap_b, k * BK, tn * half, 0);
        tma_prefetch_l2_3d(&tmap_b, k * BK, p.up_offset + tn * half, 0);
      } else {
        tma_prefetch_l2_3d(&tmap_b, k * BK, tn * bn, 0);
      }
    }
  }
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t stage_bytes = static_cast<uint32_t>(stage_stride);
      for (int k = 0; k < n_k; ++k) {
        const int stage = k % n_stages;
        const uint32_t phase = (k / n_stages) & 1u;
        if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag)) break;
        uint8_t* sa = smem + stage * stage_stride;
        uint8_t* sb = sa + BM * BK * 2;
        mbar_arrive_expect_tx(&full[stage], stage_bytes);
        tma_load_3d(sa, &tmap_a, &full[stage], k * BK, 0, 0);
        if (SWIGLU) {
          tma_load_3d(sb, &tmap_b, &full[stage], k * BK, tn * half, 0);                              // gate rows
          tma_load_3d(sb + half * (BK * 2), &tmap_b, &full[stage], k * BK, p.up_offset + tn * half, 0);   // up rows
        } else {
          tma_load_3d(sb, &tmap_b, &full[stage], k * BK, tn * bn, 0);
        }
      }
      pdl_launch_dependents();
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = make_idesc(BM, bn, p.is_bf16 != 0, false, false);
      bool ok = true;
      for (int k = 0; k < n_k; ++k) {
        const int stage = k % n_stages;
        const uint32_t phase = (k / n_stages) & 1u;
        if (!mbar_wait(&full[stage], phase, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sa = smem_u32(smem + stage * stage_stride);
        const uint32_t sb = sa + BM * BK * 2;
#pragma unroll
        for (int kk = 0; kk < BK / UMMA_K; ++kk)
          umma_f16(tmem_base, smem_desc_sw128(sa + kk * 32, 16u, 1024u), smem_desc_sw128(sb + kk * 32, 16u, 1024u), idesc,
                   (k | kk) != 0 ? 1u : 0u);
        umma_commit(&empty[stage]);
      }
      if (ok) umma_commit(acc_full);
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const bool row_ok = row < p.M;
    if (mbar_wait(acc_full, 0, abort_flag)) {
      tc_fence_after();
      uint16_t* orow = static_cast<uint16_t*>(p.out) + static_cast<int64_t>(row) * p.o_sm;
      const uint16_t* crow = p.cin ? static_cast<const uint16_t*>(p.cin) + static_cast<int64_t>(row) * p.c_sm : nullptr;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const int cols = SWIGLU ? half : bn;     // output columns of this tile
#pragma unroll 1
      for (int c = 0; c < cols; c += 32) {
        uint32_t r[32], ru[32];
        tmem_ld_32x32(t_row + static_cast<uint32_t>(c), r);
        if (SWIGLU) tmem_ld_32x32(t_row + static_cast<uint32_t>(half + c), ru);
        tmem_wait_ld();
        const int col0 = tn * cols + c;
        if (!row_ok) continue;
        for (int j = 0; j < 32; ++j) {
          const int col = col0 + j;
          if (c + j >= cols || col >= p.N) break;
          float v;
          if (SWIGLU) {
            const float g0 = __uint_as_float(r[j]);
            v = __fdividef(g0, 1.0f + __expf(-g0)) * __uint_as_float(ru[j]);
          } else {
            v = p.alpha * __uint_as_float(r[j]);
            if (crow) {
              const uint16_t cb = crow[static_cast<int64_t>(col) * p.c_sn];
              v += p.beta * (p.is_bf16 ? bf16_bits_to_f32(cb) : f16_bits_to_f32(cb));
            }
          }
          orow[col] = p.is_bf16 ? f32_to_bf16_bits(v) : f32_to_f16_bits(v);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  if (threadIdx.x == 0 && *abort_flag) atomicOr(p.error_word, 2u);
}

// Columns per tile for the one-wave kernel: the smallest multiple of `unit` that covers `width` columns in at
// most `sms` tiles; 0 when the product does not suit the kernel (fewer than `at_least` columns per SM: too narrow
// to give every SM a worthwhile stream; or more than `at_most`: too wide for one wave).
// Slices of K for the few-row SwiGLU product on 64-column tiles: the rule of the plain skinny product (one wave of two
// CTAs per SM, at least 4 k-steps per slice); 1 = no split.
int swiglu_splits(int64_t F, int64_t K) {
  const int64_t tiles = (F + BNS / 2 - 1) / (BNS / 2), n_k = (K + BK - 1) / BK;
  const int sms = gemm_sm_budget();
  int splits = 1;
  while (splits < 8 && tiles * splits * 2 <= 2 * sms && n_k >= splits * 2 * 4) splits *= 2;
  return splits;
}

constexpr int kWideMinHalf = 64;   // gate (and up) rows per tile below which mm_swiglu leaves the one-wave kernel

int wide_tile_width(int64_t width, int unit, int at_least, int at_most, int sms) {
  int64_t bn = (width + sms - 1) / sms;
  bn = (bn + unit - 1) / unit * unit;
  if (bn < at_least || bn > at_most) return 0;
  return static_cast<int>(bn);
}

template <bool SWIGLU>
b200Status launch_wide(const Operand& oa, Operand ob, GemmParams p, int bn, cudaStream_t s) {
  ob.box[1] = static_cast<uint32_t>(SWIGLU ? bn / 2 : bn);
  CUtensorMap ta, tb;
  const char* err = "";
  B200_REQUIRE(encode_tmap_16bit(&ta, oa.base, 3, oa.dims, oa.strides, oa.box, &err), B200_NOT_SUPPORTED, "matmul: %s", err);
  B200_REQUIRE(encode_tmap_16bit(&tb, ob.base, 3, ob.dims, ob.strides, ob.box, &err), B200_NOT_SUPPORTED, "matmul: %s", err);
  static thread_local int last_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != last_dev) {
    cudaError_t e = cudaFuncSetAttribute(gemm_wide_kernel<SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemWide);
    B200_REQUIRE(e == cudaSuccess, B200_LAUNCH_FAILED, "matmul: %s", cudaGetErrorString(e));
    last_dev = dev;
  }
  const int cols = SWIGLU ? bn / 2 : bn;
  const int tiles = (p.N + cols - 1) / cols;
  cudaError_t le = launch_pdl(gemm_wide_kernel<SWIGLU>, tiles, kGemmThreads, kSmemWide, s, ta, tb, p, bn);
  B200_REQUIRE(le == cudaSuccess, B200_LAUNCH_FAILED, "matmul: %s", cudaGetErrorString(le));
  return check_launch("matmul (tcgen05, one wave)");
}

// B200_GEMM_PAIR=0 keeps every product on the one-CTA kernel (for A/B timing).
bool pair_kernel_enabled() {
  static const bool on = [] {
    const char* e = getenv("B200_GEMM_PAIR");
    return !(e && e[0] == '0');
  }();
  return on;
}

}  // namespace

// Shared implementation of mm / addmm / bmm / baddbmm.
b200Status matmul_impl(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, const b200Tensor* cin,
                       double alpha, double beta, bool batched, cudaStream_t s, const char* name) {
  B200_REQUIRE(valid(out) && valid(a) && valid(b), B200_BAD_PARAM, "%s: invalid tensor view", name);
  const int nd = batched ? 3 : 2;
  B200_REQUIRE(out->ndim == nd && a->ndim == nd && b->ndim == nd, B200_BAD_PARAM, "%s: operands must be %d-D", name, nd);
  B200_REQUIRE(a->dtype == b->dtype && a->dtype == out->dtype, B200_BAD_PARAM, "%s: dtype mismatch", name);
  const int o = batched ? 1 : 0;
  const int64_t batch = batched ? out->sizes[0] : 1;
  const int64_t M = out->sizes[o], N = out->sizes[o + 1], K = a->sizes[o + 1];
  B200_REQUIRE(a->sizes[o] == M && b->sizes[o] == K && b->sizes[o + 1] == N &&
               (!batched || (a->sizes[0] == batch && b->sizes[0] == batch)), B200_BAD_PARAM,
               "%s: shapes do not multiply", name);
  if (cin && beta != 0.0) {
    B200_REQUIRE(valid(cin) && same_shape(cin, out) && cin->dtype == out->dtype, B200_BAD_PARAM,
                 "%s: the addend must be expanded to the output's shape and share its dtype", name);
  } else {
    cin = nullptr;
  }
  if (M == 0 || N == 0 || batch == 0) return B200_OK;
  if (K == 0) {  // out = beta * cin
    if (!cin) return b200_fill(out, 0.0, s);
    return b200_mul_scalar(out, cin, beta, s);
  }

  const bool tc_type = a->dtype == B200_BF16 || a->dtype == B200_F16;
  const bool out_ok = (out->strides[o + 1] == 1 || N == 1) && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31) &&
                      batch < 65536;
  if (tc_type && out_ok) {
    // BN: the widest tile that still gives every SM work
    const int sms = sm_count_current_device();
    auto tiles = [&](int bn) { return ((M + BM - 1) / BM) * ((N + bn - 1) / bn) * batch; };
    int bn = 256;
    if (tiles(256) < sms && N > 128) bn = 128;
    if (tiles(bn) < sms && N > 64) bn = 64;
    if (N <= 64) bn = 64; else if (N <= 128 && bn > 128) bn = 128;
    // enough 256 x 256 tiles for two rounds of CTA pairs: the two-CTA kernel
    const bool pair_kernel = ((M + BM2 - 1) / BM2) * ((N + BN2 - 1) / BN2) * batch >= sms && pair_kernel_enabled();
    if (pair_kernel) bn = BN2 / 2;   // B is loaded in per-CTA halves
    // skinny product that cannot fill the SMs with tiles alone: split K over a cluster
    int splits = 1;
    bool skinny = false;
    if (!pair_kernel && M <= BM && pair_kernel_enabled()) {
      // one wave of two CTAs per SM: double the splits while tiles x splits fits and a slice keeps >= 4 k-steps
      const int64_t t128 = ((N + BNS - 1) / BNS) * batch, n_k = (K + BK - 1) / BK;
      while (splits < 8 && t128 * splits * 2 <= 2 * sms && n_k >= splits * 2 * 4) splits *= 2;
      // (without a split the persistent one-CTA kernel is faster: 56 us against 65 us on 64 x 28672 x 4096)
      skinny = splits > 1;
      if (skinny) bn = BNS;
    }
    Operand oa, ob;
    const bool a_ok = describe_operand(a->data, M, K, batch, a->strides[o], a->strides[o + 1], batched ? a->strides[0] : 0, BM, &oa);
    const bool b_ok = describe_operand(b->data, N, K, batch, b->strides[o + 1], b->strides[o], batched ? b->strides[0] : 0, bn, &ob);
    if (a_ok && b_ok) {
      GemmParams p{};
      p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = (int)batch;
      p.a_mn_major = oa.mn_major; p.b_mn_major = ob.mn_major;
      p.is_bf16 = a->dtype == B200_BF16;
      p.alpha = (float)alpha; p.beta = (float)beta;
      p.out = out->data; p.o_sb = batched ? out->strides[0] : 0; p.o_sm = out->strides[o];
      if (cin) {
        p.cin = cin->data; p.c_sb = batched ? cin->strides[0] : 0; p.c_sm = cin->strides[o]; p.c_sn = cin->strides[o + 1];
      }
      p.error_word = device_error_word();
      B200_REQUIRE(p.error_word, B200_LAUNCH_FAILED, "%s: device error word unavailable", name);
      if (pair_kernel) return launch_tc2<0>(oa, ob, p, s);
      if (skinny) return launch_splitk<false>(oa, ob, p, splits, s);
      if (bn == 256) return launch_tc<256>(oa, ob, p, s);
      if (bn == 128) return launch_tc<128>(oa, ob, p, s);
      return launch_tc<64>(oa, ob, p, s);
    }
  }
  simt::MatmulArgs q{};
  q.a = a->data; q.b = b->data; q.cin = cin ? cin->data : nullptr; q.out = out->data;
  q.M = M; q.N = N; q.K = K; q.batch = batch;
  q.a_sb = batched ? a->strides[0] : 0; q.a_sm = a->strides[o]; q.a_sk = a->strides[o + 1];
  q.b_sb = batched ? b->strides[0] : 0; q.b_sk = b->strides[o]; q.b_sn = b->strides[o + 1];
  if (cin) { q.c_sb = batched ? cin->strides[0] : 0; q.c_sm = cin->strides[o]; q.c_sn = cin->strides[o + 1]; }
  q.o_sb = batched ? out->strides[0] : 0; q.o_sm = out->strides[o]; q.o_sn = out->strides[o + 1];
  q.alpha = alpha; q.beta = beta;
  return simt::launch(q, a->dtype, s);
}

// out (M, F) = silu(a @ w[:F].T) * (a @ w[F:].T); a (M, K) and w (2F, K) with K contiguous.
b200Status mm_swiglu_impl(const b200Tensor* out, const b200Tensor* a, const b200Tensor* w, cudaStream_t s) {
  const char* name = "b200_mm_swiglu";
  B200_REQUIRE(valid(out) && valid(a) && valid(w), B200_BAD_PARAM, "%s: invalid tensor view", name);
  B200_REQUIRE(out->ndim == 2 && a->ndim == 2 && w->ndim == 2, B200_BAD_PARAM, "%s: operands must be 2-D", name);
  B200_REQUIRE((a->dtype == B200_BF16 || a->dtype == B200_F16) && w->dtype == a->dtype && out->dtype == a->dtype,
               B200_NOT_SUPPORTED, "%s: bf16 or f16 operands of one dtype", name);
  const int64_t M = a->sizes[0], K = a->sizes[1], F = out->sizes[1];
  B200_REQUIRE(out->sizes[0] == M && w->sizes[0] == 2 * F && w->sizes[1] == K, B200_BAD_PARAM,
               "%s: expected a (M,K), w (2F,K), out (M,F)", name);
  if (M == 0 || F == 0) return B200_OK;
  B200_REQUIRE(K > 0, B200_BAD_PARAM, "%s: K must be positive", name);
  B200_REQUIRE(M < (1ll << 31) && F < (1ll << 30) && K < (1ll << 31) && (out->strides[1] == 1 || F == 1),
               B200_NOT_SUPPORTED, "%s: sizes or output layout not supported", name);
  Operand oa, ob;
  const bool a_ok = describe_operand(a->data, M, K, 1, a->strides[0], a->strides[1], 0, BM, &oa) && !oa.mn_major;
  const bool b_ok = describe_operand(w->data, 2 * F, K, 1, w->strides[0], w->strides[1], 0, BN2 / 2, &ob) && !ob.mn_major;
  B200_REQUIRE(a_ok && b_ok, B200_NOT_SUPPORTED, "%s: operands must be K-contiguous, 16-byte aligned, leading dimension a multiple of 8", name);
  GemmParams p{};
  p.M = (int)M; p.N = (int)F; p.K = (int)K; p.batch = 1;
  p.is_bf16 = a->dtype == B200_BF16;
  p.alpha = 1.f; p.beta = 0.f;
  p.out = out->data; p.o_sm = out->strides[0];
  p.up_offset = (int)F;
  p.error_word = device_error_word();
  B200_REQUIRE(p.error_word, B200_LAUNCH_FAILED, "%s: device error word unavailable", name);
  if (M <= BM) {
    // one row-tile against a wide weight (a decode step): one wave of equal tiles instead of 256-row pair tiles.
    // Gate and up halves of a tile are multiples of 8 rows (one 128-byte-swizzle atom), 64 to 128 each
    // (measured: with narrower tiles the pair kernel is faster: 25.0 against 29.7 us at F = 3584, 24.0 against
    // 27.1 us at F = 1792, and at F = 7168, halves of 56 rows, the split-K product followed by the activation
    // kernel beats both: 27 + 4 us against 34; with wide tiles this kernel wins: 51 against 56 us at F = 14336).
    const int half = wide_tile_width(F, 8, kWideMinHalf, 128, gemm_sm_budget());
    if (half > 0) return launch_wide<true>(oa, ob, p, 2 * half, s);
    // a narrower weight: K split over a cluster, 64 gate + 64 up rows per tile, the activation applied by the band owner
    const int splits = swiglu_splits(F, K);
    if (splits > 1) return launch_splitk<true>(oa, ob, p, splits, s);
  }
  return launch_tc2<1>(oa, ob, p, s);
}

// out (M, N) = a @ w^T with the rotate-half rotary embedding applied to the first rope_cols columns
// (heads of 128), in the GEMM's epilogue. a (M,K), w (N,K) K-contiguous; cos / sin f32 (P, 64).
b200Status mm_rope_impl(const b200Tensor* out, const b200Tensor* a, const b200Tensor* w, const b200Tensor* cos_t,
                        const b200Tensor* sin_t, int64_t seq_len, int64_t rope_cols, cudaStream_t s) {
  const char* name = "b200_mm_rope";
  B200_REQUIRE(valid(out) && valid(a) && valid(w) && valid(cos_t) && valid(sin_t), B200_BAD_PARAM, "%s: invalid tensor view", name);
  B200_REQUIRE(out->ndim == 2 && a->ndim == 2 && w->ndim == 2, B200_BAD_PARAM, "%s: operands must be 2-D", name);
  B200_REQUIRE((a->dtype == B200_BF16 || a->dtype == B200_F16) && w->dtype == a->dtype && out->dtype == a->dtype,
               B200_NOT_SUPPORTED, "%s: bf16 or f16 operands of one dtype", name);
  const int64_t M = a->sizes[0], K = a->sizes[1], N = w->sizes[0];
  B200_REQUIRE(out->sizes[0] == M && out->sizes[1] == N && w->sizes[1] == K, B200_BAD_PARAM, "%s: expected a (M,K), w (N,K), out (M,N)", name);
  B200_REQUIRE(rope_cols >= 0 && rope_cols <= N && rope_cols % 128 == 0 && seq_len > 0, B200_BAD_PARAM,
               "%s: rope_cols must be a multiple of the head size 128 within N, seq_len positive", name);
  B200_REQUIRE(cos_t->dtype == B200_F32 && sin_t->dtype == B200_F32 && cos_t->ndim == 2 && same_shape(cos_t, sin_t) &&
               cos_t->sizes[1] == 64 && cos_t->sizes[0] >= seq_len && is_contiguous(cos_t) && is_contiguous(sin_t), B200_BAD_PARAM,
               "%s: cos / sin must be contiguous f32 (positions >= seq_len, 64)", name);
  if (M == 0 || N == 0) return B200_OK;
  B200_REQUIRE(K > 0 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31) && (out->strides[1] == 1 || N == 1), B200_NOT_SUPPORTED,
               "%s: sizes or output layout not supported", name);
  Operand oa, ob;
  const bool a_ok = describe_operand(a->data, M, K, 1, a->strides[0], a->strides[1], 0, BM, &oa) && !oa.mn_major;
  const bool b_ok = describe_operand(w->data, N, K, 1, w->strides[0], w->strides[1], 0, BN2 / 2, &ob) && !ob.mn_major;
  B200_REQUIRE(a_ok && b_ok, B200_NOT_SUPPORTED, "%s: operands must be K-contiguous, 16-byte aligned, leading dimension a multiple of 8", name);
  GemmParams p{};
  p.M = (int)M; p.N = (int)N; p.K = (int)K; p.batch = 1;
  p.is_bf16 = a->dtype == B200_BF16;
  p.alpha = 1.f; p.beta = 0.f;
  p.out = out->data; p.o_sm = out->strides[0];
  p.rope_cos = static_cast<const float*>(cos_t->data);
  p.rope_sin = static_cast<const float*>(sin_t->data);
  p.rope_seq = (int)seq_len; p.rope_cols = (int)rope_cols;
  p.error_word = device_error_word();
  B200_REQUIRE(p.error_word, B200_LAUNCH_FAILED, "%s: device error word unavailable", name);
  return launch_tc2<2>(oa, ob, p, s);
}

}  // namespace b200

using namespace b200;

extern "C" {

b200Status b200_mm_rope(const b200Tensor* out, const b200Tensor* a, const b200Tensor* w, const b200Tensor* cos_table,
                        const b200Tensor* sin_table, int64_t seq_len, int64_t rope_cols, b200Stream stream) {
  return mm_rope_impl(out, a, w, cos_table, sin_table, seq_len, rope_cols, static_cast<cudaStream_t>(stream));
}

b200Status b200_mm_swiglu(const b200Tensor* out, const b200Tensor* a, const b200Tensor* w_gate_up, b200Stream stream) {
  return mm_swiglu_impl(out, a, w_gate_up, static_cast<cudaStream_t>(stream));
}

int b200_mm_swiglu_few_rows(int64_t M, int64_t F, int64_t K) {
  if (M <= 0 || M > BM || F <= 0 || K <= 0 || !pair_kernel_enabled()) return 0;
  return wide_tile_width(F, 8, kWideMinHalf, 128, gemm_sm_budget()) > 0 || swiglu_splits(F, K) > 1 ? 1 : 0;
}

b200Status b200_mm(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, b200Stream stream) {
  return matmul_impl(out, a, b, nullptr, 1.0, 0.0, false, static_cast<cudaStream_t>(stream), "b200_mm");
}
b200Status b200_addmm(const b200Tensor* out, const b200Tensor* self, const b200Tensor* a, const b200Tensor* b,
                      double beta, double alpha, b200Stream stream) {
  return matmul_impl(out, a, b, self, alpha, beta, false, static_cast<cudaStream_t>(stream), "b200_addmm");
}
b200Status b200_bmm(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, b200Stream stream) {
  return matmul_impl(out, a, b, nullptr, 1.0, 0.0, true, static_cast<cudaStream_t>(stream), "b200_bmm");
}
b200Status b200_baddbmm(const b200Tensor* out, const b200Tensor* self, const b200Tensor* a, const b200Tensor* b,
                        double beta, double alpha, b200Stream stream) {
  return matmul_impl(out, a, b, self, alpha, beta, true, static_cast<cudaStream_t>(stream), "b200_baddbmm");
}

}  // extern "C"
