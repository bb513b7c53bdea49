// Index kernels: index_select (and embedding), gather, advanced index with
// int32/int64 indices, and the deterministic scatter_add / index_put.
//
// Pure moves (index_select, gather, index) copy the widest unit the layout
// allows -- 128-bit for the row-shaped cases -- with the index read once.
//
// scatter_add / index_put(accumulate) must equal CPU ATen bit for bit, and the
// CPU adds the sources of one destination in ascending source order starting
// from self's value. The kernels therefore invert the index first: a stable
// least-significant-digit radix sort of (destination, source) pairs (8-bit
// digits, hand-written: per pass a per-tile digit histogram, one scan and a
// stable per-tile ranking with warp match), then one warp per destination row walks its
// segment in order, several source rows in flight, adding sequentially. No
// floating-point atomics anywhere, so results are run-to-run identical.
#include "common.cuh"

#include <cooperative_groups.h>

#include <mutex>

namespace b200 {

// Device-side error word: kernels OR a bit in instead of trapping.
__device__ unsigned int g_device_error_word = 0;
enum : unsigned int { kErrIndexOutOfRange = 1u };

// Device address of the error word (for kernels in other translation units).
unsigned int* device_error_word() {
  void* p = nullptr;
  if (cudaGetSymbolAddress(&p, g_device_error_word) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  return static_cast<unsigned int*>(p);
}

namespace {

constexpr int kThreads = 256;

template <typename I> __device__ __forceinline__ int64_t load_index(const void* p, int64_t i);
template <> __device__ __forceinline__ int64_t load_index<int64_t>(const void* p, int64_t i) {
  return static_cast<const int64_t*>(p)[i];
}
template <> __device__ __forceinline__ int64_t load_index<int32_t>(const void* p, int64_t i) {
  return static_cast<const int32_t*>(p)[i];
}

// ------------------------------------------------------------ row gather ----
// dst row r = (o, k) takes src row (o, index[k]). Rows are `upr` copy units
// long. A group of 2^g_log lanes moves one chunk of a row (4 units per lane).
struct RowGatherArgs {
  const void* src;
  void* dst;
  const void* index;
  int64_t index_stride;   // elements between consecutive indices
  int64_t n_rows;         // outer * K destination rows
  int64_t K;              // indices per outer slice
  int64_t S;              // size of the indexed source dim (bounds check / wrap)
  int64_t upr;            // units per row
  int64_t src_outer_stride, src_row_stride;  // in units
  int64_t chunks_per_row;
  int g_log;
  int wrap_negative;
};

template <typename U, typename I, typename W /* item arithmetic */>
__global__ void __launch_bounds__(kThreads)
row_gather_kernel(RowGatherArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int G = 1 << a.g_log;
  const W lane = threadIdx.x & (G - 1);
  const W groups_per_block = kThreads >> a.g_log;
  const W n_items = static_cast<W>(a.n_rows) * static_cast<W>(a.chunks_per_row);
  const W step = static_cast<W>(gridDim.x) * groups_per_block;
  const U* src = static_cast<const U*>(a.src);
  U* dst = static_cast<U*>(a.dst);
  for (W item = static_cast<W>(blockIdx.x) * groups_per_block + (threadIdx.x >> a.g_log); item < n_items;
       item += step) {
    const W row = item / static_cast<W>(a.chunks_per_row);
    const W chunk = item - row * static_cast<W>(a.chunks_per_row);
    W o = 0, k = row;
    if (a.n_rows != a.K) {
      o = row / static_cast<W>(a.K);
      k = row - o * static_cast<W>(a.K);
    }
    int64_t idx = load_index<I>(a.index, static_cast<int64_t>(k) * a.index_stride);
    if (a.wrap_negative && idx < 0) idx += a.S;
    const bool ok = idx >= 0 && idx < a.S;
    if (!ok) {
      if (lane == 0) atomicOr(&g_device_error_word, kErrIndexOutOfRange);
      idx = 0;
    }
    const U* s = src + static_cast<int64_t>(o) * a.src_outer_stride + idx * a.src_row_stride;
    U* d = dst + static_cast<int64_t>(row) * a.upr;
    const int64_t c0 = static_cast<int64_t>(chunk) * (G * 4) + lane;
    U v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t c = c0 + u * G;
      if (c < a.upr) v[u] = s[c];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t c = c0 + u * G;
      if (c < a.upr) d[c] = v[u];
    }
  }
}

// Widest copy unit (bytes) for rows of `row_bytes` at the given addresses/strides.
inline int pick_unit(int64_t row_bytes, const void* p0, const void* p1, int64_t stride_bytes0,
                     int64_t stride_bytes1, int64_t min_unit) {
  for (int64_t w = 16; w > min_unit; w >>= 1) {
    if (row_bytes % w == 0 && reinterpret_cast<uintptr_t>(p0) % w == 0 &&
        reinterpret_cast<uintptr_t>(p1) % w == 0 && stride_bytes0 % w == 0 && stride_bytes1 % w == 0)
      return static_cast<int>(w);
  }
  return static_cast<int>(min_unit);
}

template <typename I>
b200Status launch_row_gather_i(RowGatherArgs a, int unit, cudaStream_t s) {
  int g_log = 0;
  while ((1 << g_log) < 32 && (int64_t(1) << g_log) * 4 < a.upr) ++g_log;
  a.g_log = g_log;
  a.chunks_per_row = (a.upr + (int64_t(4) << g_log) - 1) / (int64_t(4) << g_log);
  const int64_t items = a.n_rows * a.chunks_per_row;
  if (items == 0) return B200_OK;
  const int64_t groups_per_block = kThreads >> g_log;
  int64_t need = (items + groups_per_block - 1) / groups_per_block;
  const bool small = items < (int64_t(1) << 31) && a.n_rows < (int64_t(1) << 31);
#define B200_RG(U)                                                                                                  \
  do {                                                                                                              \
    if (small)                                                                                                      \
      launch_pdl(row_gather_kernel<U, I, uint32_t>, wave_grid<row_gather_kernel<U, I, uint32_t>>(need, kThreads, kStreamWaves), kThreads, 0, s, a); \
    else                                                                                                            \
      launch_pdl(row_gather_kernel<U, I, int64_t>, wave_grid<row_gather_kernel<U, I, int64_t>>(need, kThreads, kStreamWaves), kThreads, 0, s, a); \
  } while (0)
  switch (unit) {
    case 16: B200_RG(int4); break;
    case 8: B200_RG(uint64_t); break;
    case 4: B200_RG(uint32_t); break;
    case 2: B200_RG(uint16_t); break;
    default: B200_RG(uint8_t); break;
  }
#undef B200_RG
  return check_launch("row gather");
}

b200Status launch_row_gather(const RowGatherArgs& a, int unit, int32_t index_dtype, cudaStream_t s) {
  if (index_dtype == B200_I64) return launch_row_gather_i<int64_t>(a, unit, s);
  if (index_dtype == B200_I32) return launch_row_gather_i<int32_t>(a, unit, s);
  return fail(B200_BAD_PARAM, "index dtype must be int32 or int64");
}

// ---------------------------------------------------------------- gather ----
// Fast form: index/out (rows, cols) contiguous, dim = last, self rows aligned
// with index rows. Four outputs per thread.
template <typename U, typename I>
__global__ void __launch_bounds__(kThreads)
gather_lastdim_kernel(U* __restrict__ out, const U* __restrict__ self, const I* __restrict__ index,
                      int64_t n4, int64_t cols, int64_t self_cols) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t v = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; v < n4; v += stride) {
    const int64_t e = v * 4;
    const int64_t row = e / cols;
    alignas(16) I idx[4];
    if constexpr (sizeof(I) == 8) {
      int4 a = __ldcs(reinterpret_cast<const int4*>(index + e));
      int4 b = __ldcs(reinterpret_cast<const int4*>(index + e) + 1);
      *reinterpret_cast<int4*>(&idx[0]) = a;
      *reinterpret_cast<int4*>(&idx[2]) = b;
    } else {
      int4 a = __ldcs(reinterpret_cast<const int4*>(index + e));
      *reinterpret_cast<int4*>(&idx[0]) = a;
    }
    const U* srow = self + row * self_cols;
    struct alignas(sizeof(U) * 4 > 16 ? 16 : sizeof(U) * 4) Pack { U v[4]; } r;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      int64_t j = idx[k];
      if (j < 0 || j >= self_cols) {
        atomicOr(&g_device_error_word, kErrIndexOutOfRange);
        j = 0;
      }
      r.v[k] = srow[j];
    }
    *reinterpret_cast<Pack*>(out + e) = r;
  }
}

template <typename U, typename I>
__global__ void __launch_bounds__(kThreads)
gather_generic_kernel(U* out, const U* self, const I* index, int64_t n, StridedIndexer<3> ix,
                      int64_t self_dim_stride, int64_t self_dim_size) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t off[3];
    ix.offsets(i, off);
    int64_t j = index[off[1]];
    if (j < 0 || j >= self_dim_size) {
      atomicOr(&g_device_error_word, kErrIndexOutOfRange);
      j = 0;
    }
    out[off[0]] = self[off[2] + j * self_dim_stride];
  }
}

// ------------------------------------------------------- advanced index ----
constexpr int kMaxIndexTensors = 4;
struct IndexArgs {
  const void* idx[kMaxIndexTensors];
  int64_t sizes[kMaxIndexTensors];
  int64_t strides[kMaxIndexTensors];
  int n;
};

template <typename U, typename I>
__global__ void __launch_bounds__(kThreads)
index_generic_kernel(U* out, const U* src, int64_t n, StridedIndexer<2 + kMaxIndexTensors> ix, IndexArgs a) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t off[2 + kMaxIndexTensors];
    ix.offsets(i, off);
    int64_t so = off[1];
#pragma unroll
    for (int k = 0; k < kMaxIndexTensors; ++k) {
      if (k < a.n) {
        int64_t j = static_cast<const I*>(a.idx[k])[off[2 + k]];
        if (j < 0) j += a.sizes[k];
        if (j < 0 || j >= a.sizes[k]) {
          atomicOr(&g_device_error_word, kErrIndexOutOfRange);
          j = 0;
        }
        so += j * a.strides[k];
      }
    }
    out[off[0]] = src[so];
  }
}

// ------------------------------------------------ stable LSD radix sort ----
// Sorts n (key, value) uint32 pairs by key, 8 bits per pass, stable.
// Tile = 256 threads x 4 items; warp w owns items [w*128, (w+1)*128) of the
// tile, read 32 consecutive items per round.
constexpr int kSortThreads = 256;
constexpr int kItemsPerThread = 4;
constexpr int kTile = kSortThreads * kItemsPerThread;  // 1024
constexpr int kWarps = kSortThreads / 32;

// hist[digit * nblocks + block]: digit counts of every tile, for one pass. The
// histogram is taken again before each pass because the previous pass has
// permuted which keys sit in which tile.
__device__ __forceinline__ void hist_tile(const uint32_t* __restrict__ keys, int64_t n, int pass, int nblocks, int tile,
                                          uint32_t* __restrict__ hist, uint32_t* sh /* [256] */) {
  sh[threadIdx.x] = 0;
  __syncthreads();
  const int64_t base = static_cast<int64_t>(tile) * kTile;
  const int shift = 8 * pass;
#pragma unroll 4
  for (int r = 0; r < kItemsPerThread; ++r) {
    const int64_t i = base + r * kSortThreads + threadIdx.x;
    if (i < n) atomicAdd(&sh[((keys[i] & 0x7fffffffu) >> shift) & 255u], 1u);   // bit 31 is a flag, never a digit
  }
  __syncthreads();
  hist[static_cast<int64_t>(threadIdx.x) * nblocks + tile] = sh[threadIdx.x];
  __syncthreads();
}

__global__ void __launch_bounds__(kSortThreads)
radix_hist_kernel(const uint32_t* __restrict__ keys, int64_t n, int pass, int nblocks,
                  uint32_t* __restrict__ hist) {
  __shared__ uint32_t sh[256];
  hist_tile(keys, n, pass, nblocks, blockIdx.x, hist, sh);
}

// Exclusive scan over the 256 threads of a block; *total gets the sum. `sh` holds
// one word per warp and may be reused after the call returns.
__device__ __forceinline__ uint32_t block_scan_256(uint32_t v, uint32_t* sh, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  __syncthreads();   // earlier readers of sh are done
  if (lane == 31) sh[warp] = inc;
  __syncthreads();
  uint32_t before = 0, all = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const uint32_t c = sh[w];
    if (w < warp) before += c;
    all += c;
  }
  *total = all;
  return before + inc - v;
}

// Block d scans, in place, the row of tile counts of digit d (exclusive) and
// leaves the digit's total in totals[d]; the scatter kernel adds the scan over
// the 256 totals itself.
__device__ __forceinline__ void scan_row(uint32_t* __restrict__ hist, int nblocks, int digit, uint32_t* __restrict__ totals,
                                         uint32_t* sh /* [kWarps] */) {
  uint32_t* row = hist + static_cast<int64_t>(digit) * nblocks;
  uint32_t carry = 0;
  for (int base = 0; base < nblocks; base += kSortThreads) {
    const int i = base + threadIdx.x;
    const uint32_t v = i < nblocks ? row[i] : 0u;
    uint32_t total;
    const uint32_t ex = block_scan_256(v, sh, &total);
    if (i < nblocks) row[i] = carry + ex;
    carry += total;
  }
  if (threadIdx.x == 0) totals[digit] = carry;
  __syncthreads();
}

__global__ void __launch_bounds__(kSortThreads)
radix_scan_rows_kernel(uint32_t* __restrict__ hist, int nblocks, uint32_t* __restrict__ totals) {
  __shared__ uint32_t sh[kWarps];
  scan_row(hist, nblocks, blockIdx.x, totals, sh);
}

// vals_in == nullptr: the value of item i is i (first pass).
struct ScatterSmem {
  uint32_t warp_count[kWarps][256];  // sweep 1: counts; then exclusive base per warp
  uint32_t digit_base[256];
  uint32_t scan_sh[kWarps];
};

__device__ __forceinline__ void scatter_tile(const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                                             uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out, int64_t n,
                                             int pass, int nblocks, int tile, const uint32_t* __restrict__ hist_scanned,
                                             const uint32_t* __restrict__ totals, ScatterSmem& sm) {
  auto& warp_count = sm.warp_count;
  auto& digit_base = sm.digit_base;
  uint32_t* scan_sh = sm.scan_sh;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < kWarps * 256; i += kSortThreads) (&warp_count[0][0])[i] = 0;
  {
    uint32_t all;
    const uint32_t first = block_scan_256(totals[threadIdx.x], scan_sh, &all);   // where digit threadIdx.x starts
    digit_base[threadIdx.x] = first + hist_scanned[static_cast<int64_t>(threadIdx.x) * nblocks + tile];
  }
  __syncthreads();

  const int64_t wbase = static_cast<int64_t>(tile) * kTile + warp * (kItemsPerThread * 32);
  uint32_t key[kItemsPerThread];
  const int shift = 8 * pass;
#pragma unroll
  for (int r = 0; r < kItemsPerThread; ++r) {
    const int64_t i = wbase + r * 32 + lane;
    key[r] = i < n ? keys_in[i] : 0xffffffffu;
  }
  // sweep 1: per-warp digit counts
#pragma unroll
  for (int r = 0; r < kItemsPerThread; ++r) {
    const int64_t i = wbase + r * 32 + lane;
    const bool live = i < n;
    const uint32_t d = live ? (((key[r] & 0x7fffffffu) >> shift) & 255u) : (256u + lane);
    const uint32_t peers = __match_any_sync(0xffffffffu, d);
    if (live && lane == (__ffs(peers) - 1)) warp_count[warp][d] += __popc(peers);
    __syncwarp();
  }
  __syncthreads();
  // exclusive prefix over warps, per digit (thread = digit)
  {
    uint32_t run = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      uint32_t c = warp_count[w][threadIdx.x];
      warp_count[w][threadIdx.x] = run;
      run += c;
    }
  }
  __syncthreads();
  // sweep 2: stable ranks and scatter
#pragma unroll
  for (int r = 0; r < kItemsPerThread; ++r) {
    const int64_t i = wbase + r * 32 + lane;
    const bool live = i < n;
    const uint32_t d = live ? (((key[r] & 0x7fffffffu) >> shift) & 255u) : (256u + lane);
    const uint32_t peers = __match_any_sync(0xffffffffu, d);
    uint32_t pos = 0;
    if (live) {
      const uint32_t before = __popc(peers & ((1u << lane) - 1u));
      pos = digit_base[d] + warp_count[warp][d] + before;
    }
    __syncwarp();
    if (live && lane == (__ffs(peers) - 1)) warp_count[warp][d] += __popc(peers);
    __syncwarp();
    if (live) {
      keys_out[pos] = key[r];
      // bit 31 of a key marks an out-of-range index: it rides along unsorted
      // (masked out of every digit, the top one of a four-pass sort included) and turns the
      // value into an invalid id
      vals_out[pos] = (key[r] >> 31) ? 0xffffffffu : (vals_in ? vals_in[i] : static_cast<uint32_t>(i));
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kSortThreads)
radix_scatter_kernel(const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                     uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out, int64_t n,
                     int pass, int nblocks, const uint32_t* __restrict__ hist_scanned,
                     const uint32_t* __restrict__ totals) {
  __shared__ ScatterSmem sm;
  scatter_tile(keys_in, vals_in, keys_out, vals_out, n, pass, nblocks, blockIdx.x, hist_scanned, totals, sm);
}

// seg_start[d] = first sorted position whose key is >= d, for d in [0, n_dst]; positions first, first + stride, ...
__device__ __forceinline__ void segment_bounds(const uint32_t* sorted_keys, int64_t n, int64_t n_dst, uint32_t* seg_start,
                                               int64_t first, int64_t stride) {
  for (int64_t p = first; p <= n; p += stride) {
    const int64_t lo = p == 0 ? 0 : static_cast<int64_t>(sorted_keys[p - 1] & 0x7fffffffu) + 1;
    int64_t hi = p == n ? n_dst : static_cast<int64_t>(sorted_keys[p] & 0x7fffffffu);
    if (hi > n_dst) hi = n_dst;
    for (int64_t d = lo; d <= hi; ++d) seg_start[d] = static_cast<uint32_t>(p);
  }
}

// All passes in one cooperative launch: histogram, row scans and scatter of a pass are
// separated by grid-wide barriers instead of kernel boundaries (three launches per pass
// otherwise, each a few microseconds of ramp for a few hundred kilobytes of keys).
__global__ void __launch_bounds__(kSortThreads)
radix_sort_fused_kernel(uint32_t* keys_a, uint32_t* keys_b, uint32_t* vals_a, uint32_t* vals_b, int64_t n, int passes,
                        int nblocks, uint32_t* hist, uint32_t* totals, uint32_t* seg_start, int64_t n_dst) {
  namespace cg = cooperative_groups;
  cg::grid_group grid = cg::this_grid();
  __shared__ ScatterSmem sm;
  uint32_t *kin = keys_a, *kout = keys_b, *vin = nullptr, *vout = vals_a, *vother = vals_b;
  for (int pass = 0; pass < passes; ++pass) {
    for (int tile = blockIdx.x; tile < nblocks; tile += gridDim.x) hist_tile(kin, n, pass, nblocks, tile, hist, sm.digit_base);
    grid.sync();
    for (int d = blockIdx.x; d < 256; d += gridDim.x) scan_row(hist, nblocks, d, totals, sm.scan_sh);
    grid.sync();
    for (int tile = blockIdx.x; tile < nblocks; tile += gridDim.x)
      scatter_tile(kin, vin, kout, vout, n, pass, nblocks, tile, hist, totals, sm);
    grid.sync();
    uint32_t* t = kin; kin = kout; kout = t;
    vin = vout;
    vout = vother;
    vother = vin;
  }
  // the segment bounds of the sorted keys, when the caller wants them (the last pass ended with a grid barrier)
  if (seg_start)
    segment_bounds(kin, n, n_dst, seg_start, static_cast<int64_t>(blockIdx.x) * kSortThreads + threadIdx.x,
                   static_cast<int64_t>(gridDim.x) * kSortThreads);
}

// ---- grouping source rows by destination without a global sort (row form) ----------------
// The ordered walk needs, for every destination row, its source rows in ascending order. A stable
// sort of (destination, source) pairs gives that, but for a megabyte of keys its dependent passes
// are all latency. Instead: count the sources of every destination (one atomic each), scan the
// counts into segment starts, drop every source id into its segment at an atomically claimed
// position (the order inside a segment is then arbitrary), and sort each segment by source id:
// ids are unique, so the result is exactly the stable order. Segments are short for any spread-out
// index (four ids on average in the benchmark's case): up to 8 ids are sorted in registers, up to
// 32 by insertion in place, and longer ones are queued for a block-wide radix sort of their own.
constexpr int kScanThreads = 256;
constexpr int kScanItems = 16;
constexpr int kScanChunk = kScanThreads * kScanItems;   // counts per scan block
constexpr uint32_t kBigSegment = 32;                     // longer segments go to the block-wide sort

struct BucketHeader {      // zeroed before every call, together with the scan status words and the counts
  unsigned int ticket;     // dynamic block order of the scan
  unsigned int big_n;      // number of queued long segments
  unsigned int pad[62];
};

template <typename I>
__global__ void __launch_bounds__(kThreads)
bucket_count_kernel(const I* __restrict__ index, int64_t index_stride, int64_t n, int64_t n_dst, int wrap_negative,
                    uint32_t* __restrict__ keys, uint32_t* __restrict__ slot, uint32_t* __restrict__ count) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t d = index[i * index_stride];
    if (wrap_negative && d < 0) d += n_dst;
    if (d < 0 || d >= n_dst) {
      atomicOr(&g_device_error_word, kErrIndexOutOfRange);
      keys[i] = 0xffffffffu;   // dropped: belongs to no segment
    } else {
      keys[i] = static_cast<uint32_t>(d);
      slot[i] = atomicAdd(&count[d], 1u);   // the position this source claims inside its segment (arbitrary order)
    }
  }
}

// Exclusive scan of count[0, n_dst) into seg_start[0, n_dst]. Blocks take chunks in ticket order and chain
// their totals through status words (bits 63-62: 1 = chunk total, 2 = inclusive prefix; low 32 bits: the
// value). The look-back reads 32 predecessors at a time, one per lane, so a chain of a few dozen chunks
// costs one round trip, not one per chunk. A block only ever waits for blocks that took an earlier ticket,
// which are running or done, and the wait is bounded.
__global__ void __launch_bounds__(kScanThreads)
bucket_scan_kernel(const uint32_t* __restrict__ count, uint32_t* __restrict__ seg_start, int64_t n_dst, BucketHeader* header,
                   unsigned long long* status) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ uint32_t sh[kWarps];
  __shared__ uint32_t s_chunk, s_before;
  if (threadIdx.x == 0) s_chunk = atomicAdd(&header->ticket, 1u);
  __syncthreads();
  const uint32_t chunk = s_chunk;
  const int lane = threadIdx.x & 31;
  // thread t takes items t, t + 256, ... of the chunk's 16 rows of 256: coalesced loads
  const int64_t cbase = static_cast<int64_t>(chunk) * kScanChunk;
  uint32_t v[kScanItems];
#pragma unroll
  for (int j = 0; j < kScanItems; ++j) {
    const int64_t i = cbase + j * kScanThreads + threadIdx.x;
    v[j] = i < n_dst ? count[i] : 0u;
  }
  // row j of the chunk is scanned across the block; rows are chained through `row_before`
  uint32_t ex[kScanItems];
  uint32_t row_before = 0;
#pragma unroll
  for (int j = 0; j < kScanItems; ++j) {
    uint32_t total;
    ex[j] = row_before + block_scan_256(v[j], sh, &total);
    row_before += total;
  }
  const uint32_t total = row_before;
  if (threadIdx.x < 32) {
    volatile unsigned long long* st = status;
    uint32_t before = 0;
    if (lane == 0) st[chunk] = ((chunk == 0 ? 2ull : 1ull) << 62) | total;
    __threadfence();
    int64_t b = static_cast<int64_t>(chunk) - 1;
    while (b >= 0) {
      const int64_t idx = b - lane;
      unsigned long long w = 2ull << 62;   // lanes past chunk 0 read "inclusive prefix 0"
      if (idx >= 0) {
        w = st[idx];
        for (int spin = 0; (w >> 62) == 0 && spin < (1 << 22); ++spin) w = st[idx];
        if ((w >> 62) == 0) {   // gave up: flag it and treat the chunk as empty
          atomicOr(&g_device_error_word, 2u);
          w = 2ull << 62;
        }
      }
      const unsigned done = __ballot_sync(0xffffffffu, (w >> 62) == 2);
      const int stop = done ? __ffs(done) - 1 : 32;   // nearest predecessor that already holds an inclusive prefix
      uint32_t part = lane <= stop ? static_cast<uint32_t>(w) : 0u;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      before += part;
      if (done) break;
      b -= 32;
    }
    if (lane == 0) {
      if (chunk != 0) {
        __threadfence();
        st[chunk] = (2ull << 62) | static_cast<unsigned long long>(before + total);
      }
      s_before = before;
    }
  }
  __syncthreads();
  const uint32_t before = s_before;
#pragma unroll
  for (int j = 0; j < kScanItems; ++j) {
    const int64_t i = cbase + j * kScanThreads + threadIdx.x;
    if (i < n_dst) seg_start[i] = before + ex[j];
    if (i + 1 == n_dst) seg_start[n_dst] = before + ex[j] + v[j];
  }
}

__global__ void __launch_bounds__(kThreads)
bucket_scatter_kernel(const uint32_t* __restrict__ keys, const uint32_t* __restrict__ slot, int64_t n,
                      const uint32_t* __restrict__ seg_start, uint32_t* __restrict__ ids) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    const uint32_t d = keys[i];
    if (d != 0xffffffffu) ids[seg_start[d] + slot[i]] = static_cast<uint32_t>(i);
  }
}

__device__ __forceinline__ void cswap(uint32_t& a, uint32_t& b) {
  const uint32_t lo = min(a, b), hi = max(a, b);
  a = lo;
  b = hi;
}

// One thread per destination row: its ids into ascending order.
__global__ void __launch_bounds__(kThreads)
bucket_sort_segments_kernel(uint32_t* __restrict__ ids, const uint32_t* __restrict__ seg_start, int64_t n_dst, int64_t n_src,
                            BucketHeader* header, uint32_t* __restrict__ big_list) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t d = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; d < n_dst; d += stride) {
    const uint32_t beg = seg_start[d], end = seg_start[d + 1];
    if (end <= beg + 1 || end > n_src) continue;
    const uint32_t k = end - beg;
    uint32_t* seg = ids + beg;
    if (k <= 8) {
      uint32_t a[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] = static_cast<uint32_t>(j) < k ? seg[j] : 0xffffffffu;
      // 19-comparator network for 8 keys (padding sorts to the end)
      cswap(a[0], a[1]); cswap(a[2], a[3]); cswap(a[4], a[5]); cswap(a[6], a[7]);
      cswap(a[0], a[2]); cswap(a[1], a[3]); cswap(a[4], a[6]); cswap(a[5], a[7]);
      cswap(a[1], a[2]); cswap(a[5], a[6]); cswap(a[0], a[4]); cswap(a[3], a[7]);
      cswap(a[1], a[5]); cswap(a[2], a[6]);
      cswap(a[1], a[4]); cswap(a[3], a[6]);
      cswap(a[2], a[4]); cswap(a[3], a[5]);
      cswap(a[3], a[4]);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (static_cast<uint32_t>(j) < k) seg[j] = a[j];
    } else if (k <= kBigSegment) {
      uint32_t a[kBigSegment];   // thread-local copy: the insertion sort's dependent accesses stay in L1
      for (uint32_t i = 0; i < k; ++i) a[i] = seg[i];
      for (uint32_t i = 1; i < k; ++i) {
        const uint32_t x = a[i];
        uint32_t j = i;
        while (j > 0 && a[j - 1] > x) {
          a[j] = a[j - 1];
          --j;
        }
        a[j] = x;
      }
      for (uint32_t i = 0; i < k; ++i) seg[i] = a[i];
    } else {
      big_list[atomicAdd(&header->big_n, 1u)] = static_cast<uint32_t>(d);
    }
  }
}

// The queued long segments: one block sorts one segment by source id, 8 bits per pass, between the
// segment's stretch of `ids` and the same stretch of `tmp`.
__global__ void __launch_bounds__(kSortThreads)
bucket_sort_big_kernel(uint32_t* ids, uint32_t* tmp, const uint32_t* __restrict__ seg_start, int64_t n_src, int passes,
                       const BucketHeader* header, const uint32_t* __restrict__ big_list) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ uint32_t warp_count[kWarps][256];
  __shared__ uint32_t digit_base[256];
  __shared__ uint32_t scan_sh[kWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t n_big = header->big_n;
  for (uint32_t b = blockIdx.x; b < n_big; b += gridDim.x) {
    const uint32_t d = big_list[b];
    const uint32_t beg = seg_start[d], end = seg_start[d + 1];
    if (end <= beg || end > n_src) continue;
    const uint32_t k = end - beg;
    uint32_t* in = ids + beg;
    uint32_t* out = tmp + beg;
    for (int pass = 0; pass < passes; ++pass) {
      const int shift = 8 * pass;
      digit_base[threadIdx.x] = 0;
      __syncthreads();
      for (uint32_t i = threadIdx.x; i < k; i += kSortThreads) atomicAdd(&digit_base[(in[i] >> shift) & 255u], 1u);
      __syncthreads();
      {
        uint32_t all;
        const uint32_t first = block_scan_256(digit_base[threadIdx.x], scan_sh, &all);
        __syncthreads();
        digit_base[threadIdx.x] = first;
      }
      __syncthreads();
      for (uint32_t c0 = 0; c0 < k; c0 += kSortThreads) {
        for (int i = threadIdx.x; i < kWarps * 256; i += kSortThreads) (&warp_count[0][0])[i] = 0;
        __syncthreads();
        const uint32_t i = c0 + threadIdx.x;
        const bool live = i < k;
        const uint32_t key = live ? in[i] : 0u;
        const uint32_t dg = live ? ((key >> shift) & 255u) : (256u + lane);
        const uint32_t peers = __match_any_sync(0xffffffffu, dg);
        const uint32_t before = __popc(peers & ((1u << lane) - 1u));
        if (live && lane == (__ffs(peers) - 1)) warp_count[warp][dg] = __popc(peers);
        __syncthreads();
        uint32_t tile_total = 0;
        {
          uint32_t run = 0;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) {
            const uint32_t cnt = warp_count[w][threadIdx.x];
            warp_count[w][threadIdx.x] = run;
            run += cnt;
          }
          tile_total = run;
        }
        __syncthreads();
        if (live) out[digit_base[dg] + warp_count[warp][dg] + before] = key;
        __syncthreads();
        digit_base[threadIdx.x] += tile_total;
        __syncthreads();
      }
      uint32_t* t = in; in = out; out = t;
    }
    if (in != ids + beg)   // an odd number of passes ended in tmp
      for (uint32_t i = threadIdx.x; i < k; i += kSortThreads) ids[beg + i] = in[i];
    __syncthreads();
  }
}

// keys for the element form: linear offset of the destination element.
template <typename I>
__global__ void __launch_bounds__(kThreads)
element_keys_kernel(const I* __restrict__ index, int64_t n, StridedIndexer<2> ix, int64_t dim_stride,
                    int64_t dim_size, int64_t out_numel, uint32_t* __restrict__ keys) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t off[2];  // [0]: index element, [1]: destination offset without the dim term
    ix.offsets(i, off);
    int64_t j = index[off[0]];
    int64_t dst = off[1] + j * dim_stride;
    if (j < 0 || j >= dim_size) {
      atomicOr(&g_device_error_word, kErrIndexOutOfRange);
      dst = 0x80000000ll;
    }
    keys[i] = static_cast<uint32_t>(dst);
  }
}

// Sequential add in the element type: 16-bit floats round after every add, as
// the CPU's `self[idx] += src` does.
template <typename T> __device__ __forceinline__ T seq_add(T a, T b) { return a + b; }
template <> __device__ __forceinline__ float seq_add<float>(float a, float b) { return __fadd_rn(a, b); }
template <> __device__ __forceinline__ bf16_t seq_add<bf16_t>(bf16_t a, bf16_t b) {
  return bf16_t{f32_to_bf16_bits(__fadd_rn(bf16_bits_to_f32(a.bits), bf16_bits_to_f32(b.bits)))};
}
template <> __device__ __forceinline__ f16_t seq_add<f16_t>(f16_t a, f16_t b) {
  return f16_t{f32_to_f16_bits(__fadd_rn(f16_bits_to_f32(a.bits), f16_bits_to_f32(b.bits)))};
}

// Accumulator type of the segment kernels. 16-bit floats either round after
// every add (ACC32 = false, what CPU index_put does) or accumulate in fp32 and
// round once (ACC32 = true, what CPU scatter_add does).
template <typename T, bool ACC32> struct AccT { using type = T; };
template <> struct AccT<bf16_t, true> { using type = float; };
template <> struct AccT<f16_t, true> { using type = float; };
template <typename A, typename T> __device__ __forceinline__ A to_accum(T v) { return v; }
template <> __device__ __forceinline__ float to_accum<float, bf16_t>(bf16_t v) { return bf16_bits_to_f32(v.bits); }
template <> __device__ __forceinline__ float to_accum<float, f16_t>(f16_t v) { return f16_bits_to_f32(v.bits); }
template <typename T, typename A> __device__ __forceinline__ T from_accum(A v) { return v; }
template <> __device__ __forceinline__ bf16_t from_accum<bf16_t, float>(float v) { return bf16_t{f32_to_bf16_bits(v)}; }
template <> __device__ __forceinline__ f16_t from_accum<f16_t, float>(float v) { return f16_t{f32_to_f16_bits(v)}; }

// One warp per (destination row, 64-vector column chunk).
// MODE 0: out = self + sum(sources in order); MODE 1: out = last source (or self).
template <typename T, int V, int MODE, bool ACC32>
__global__ void __launch_bounds__(kThreads)
segment_rows_kernel(T* __restrict__ out, const T* __restrict__ self, const T* __restrict__ src,
                    const uint32_t* __restrict__ sorted_src, const uint32_t* __restrict__ seg_start,
                    int64_t n_dst, int64_t n_src, int64_t inner /* elements per row */,
                    int64_t chunks_per_row) {
  pdl_wait();
  struct alignas(sizeof(T) * V) VecT { T v[V]; };
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
  const int64_t vpr = inner / V;
  const int64_t n_items = n_dst * chunks_per_row;
  for (int64_t item = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5);
       item < n_items; item += warps) {
    const int64_t r = item / chunks_per_row;
    const int64_t chunk = item - r * chunks_per_row;
    const int64_t c0 = chunk * 64 + lane, c1 = c0 + 32;
    const bool h0 = c0 < vpr, h1 = c1 < vpr;
    uint32_t beg = seg_start[r], end = seg_start[r + 1];
    if (end > n_src || beg > end) beg = end = 0;  // never walk outside the sorted list
    const VecT* self_row = reinterpret_cast<const VecT*>(self + r * inner);
    VecT* out_row = reinterpret_cast<VecT*>(out + r * inner);
    if (MODE == 1) {
      uint32_t last = beg < end ? sorted_src[end - 1] : 0u;
      if (last >= n_src) last = 0;
      const VecT* from = beg < end ? reinterpret_cast<const VecT*>(src + static_cast<int64_t>(last) * inner) : self_row;
      if (from != out_row) {
        if (h0) out_row[c0] = from[c0];
        if (h1) out_row[c1] = from[c1];
      }
      continue;
    }
    using A = typename AccT<T, ACC32>::type;
    A a0[V], a1[V];
    if (h0) {
      const VecT t = self_row[c0];
#pragma unroll
      for (int e = 0; e < V; ++e) a0[e] = to_accum<A>(t.v[e]);
    }
    if (h1) {
      const VecT t = self_row[c1];
#pragma unroll
      for (int e = 0; e < V; ++e) a1[e] = to_accum<A>(t.v[e]);
    }
    for (uint32_t p = beg; p < end; p += 32) {
      const uint32_t cnt = min(32u, end - p);
      const uint32_t mine = lane < cnt ? sorted_src[p + lane] : 0xffffffffu;
      for (uint32_t k = 0; k < cnt; k += 4) {  // four source rows in flight, added in order
        VecT b0[4], b1[4];
        bool okr[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const uint32_t sid = __shfl_sync(0xffffffffu, mine, (k + u) & 31u);
          // past the end of the segment, or an out-of-range source parked with an invalid id
          okr[u] = k + u < cnt && sid < n_src;
          const VecT* srow = reinterpret_cast<const VecT*>(src + static_cast<int64_t>(okr[u] ? sid : 0u) * inner);
          if (h0 && okr[u]) b0[u] = srow[c0];
          if (h1 && okr[u]) b1[u] = srow[c1];
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (!okr[u]) continue;
#pragma unroll
          for (int e = 0; e < V; ++e) {
            if (h0) a0[e] = seq_add(a0[e], to_accum<A>(b0[u].v[e]));
            if (h1) a1[e] = seq_add(a1[e], to_accum<A>(b1[u].v[e]));
          }
        }
      }
    }
    if (h0) {
      VecT t;
#pragma unroll
      for (int e = 0; e < V; ++e) t.v[e] = from_accum<T>(a0[e]);
      out_row[c0] = t;
    }
    if (h1) {
      VecT t;
#pragma unroll
      for (int e = 0; e < V; ++e) t.v[e] = from_accum<T>(a1[e]);
      out_row[c1] = t;
    }
  }
}

// MODE 0 with the row reads staged through shared memory. The register-resident walk above keeps at
// most 4 source rows (4 KB) per warp in flight and is bound by latency (49 % of DRAM throughput, 80 % of
// stall cycles on the row loads): registers limit both the rows per warp and the warps per SM. Here every
// warp owns a contiguous range of destination rows and a ring of kRingSlots (4) 1 KB slots that it fills with
// cp.async: the rows it needs, in the order it needs them (row of self, then its sources in sorted
// order, then the next destination row ...), always kRingSlots rows ahead of the one it is adding. A lane
// reads back exactly the 2 x 16 bytes it copied itself, so cp.async.wait_group is the only
// synchronisation. Segment bounds and source ids of a window of rows are staged per warp (no block-wide
// barrier anywhere). The order of additions is the one of the register walk.
constexpr int kWarpRows = 64;      // destination rows per staged window
constexpr int kWarpIds = 447;      // source ids staged per window (a longer stretch is read from global)
__host__ __device__ constexpr int warp_smem(int slots) { return slots * 1024 + (kWarpRows + 1 + kWarpIds) * 4; }
static_assert(warp_smem(4) % 16 == 0 && warp_smem(1) % 16 == 0, "every warp's ring starts 16-byte aligned");

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
               "l"(gmem_src)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T, int V, bool ACC32, int kRingSlots, int MINB>
__global__ void __launch_bounds__(kThreads, MINB)
segment_rows_ring_kernel(T* out, const T* self, const T* __restrict__ src,
                         const uint32_t* __restrict__ sorted_src, const uint32_t* __restrict__ seg_start,
                         int64_t n_dst, int64_t n_src, int64_t inner /* elements per row */,
                         int64_t chunks_per_row, int64_t rows_per_warp) {
  pdl_wait();
  static_assert(sizeof(T) * V == 16, "one 16-byte vector per copy");
  struct alignas(16) VecT { T v[V]; };
  using A = typename AccT<T, ACC32>::type;
  extern __shared__ __align__(16) uint8_t ring_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int kWarpSmem = warp_smem(kRingSlots);
  uint8_t* ring = ring_smem + warp * kWarpSmem;
  uint32_t* s_seg = reinterpret_cast<uint32_t*>(ring + kRingSlots * 1024);
  uint32_t* s_ids = s_seg + kWarpRows + 1;
  const int64_t vpr = inner / V;
  const int64_t gw = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + warp;
  const int64_t ra = gw * rows_per_warp, rb = min(n_dst, ra + rows_per_warp);

  for (int64_t w0 = ra; w0 < rb; w0 += kWarpRows) {
    const int rows = static_cast<int>(min(static_cast<int64_t>(kWarpRows), rb - w0));
    __syncwarp();   // the previous window's readers are done with the staged words
    for (int i = lane; i <= rows; i += 32) s_seg[i] = seg_start[w0 + i];
    __syncwarp();
    const uint32_t g_beg = s_seg[0], g_end = s_seg[rows];
    const uint32_t staged = (g_beg <= g_end && g_end <= n_src) ? min(g_end - g_beg, static_cast<uint32_t>(kWarpIds)) : 0u;
    for (uint32_t i = lane; i < staged; i += 32) s_ids[i] = sorted_src[g_beg + i];
    __syncwarp();
    auto id_at = [&](uint32_t p) -> uint32_t {
      const uint32_t o = p - g_beg;
      return o < staged ? s_ids[o] : sorted_src[p];
    };
    auto seg_of = [&](int lr, uint32_t& beg, uint32_t& end) {
      beg = s_seg[lr];
      end = s_seg[lr + 1];
      if (end > n_src || beg > end) beg = end = 0;   // never walk outside the sorted list
    };
    for (int64_t chunk = 0; chunk < chunks_per_row; ++chunk) {
      const int64_t c0 = chunk * 64 + lane, c1 = c0 + 32;
      const bool h0 = c0 < vpr, h1 = c1 < vpr;
      // the item sequence of a row: k = -1 is the row of self, k >= 0 the k-th source of its segment
      int ir = 0, ik = -1;          // next item to copy
      uint32_t ibeg, iend;
      seg_of(0, ibeg, iend);
      auto issue = [&](int slot) {
        if (ir < rows) {
          const T* rowp = nullptr;
          if (ik < 0) {
            rowp = self + (w0 + ir) * inner;
          } else {
            const uint32_t sid = id_at(ibeg + static_cast<uint32_t>(ik));
            if (sid < n_src) rowp = src + static_cast<int64_t>(sid) * inner;   // an invalid id copies nothing
          }
          if (rowp) {
            uint8_t* dst = ring + slot * 1024 + lane * 16;
            if (h0) cp_async16(dst, rowp + c0 * V);
            if (h1) cp_async16(dst + 512, rowp + c1 * V);
          }
          ++ik;
          if (ibeg + static_cast<uint32_t>(ik) >= iend) {
            ++ir;
            ik = -1;
            if (ir < rows) seg_of(ir, ibeg, iend);
          }
        }
        cp_async_commit();   // one group per slot, also when nothing was copied
      };
#pragma unroll 1
      for (int sl = 0; sl < kRingSlots; ++sl) issue(sl);

      int cr = 0, ck = -1, slot = 0;   // item being added
      uint32_t cbeg, cend;
      seg_of(0, cbeg, cend);
      A a0[V], a1[V];
#pragma unroll 1
      while (cr < rows) {
        cp_async_wait<kRingSlots - 1>();   // the oldest group, the one of `slot`, has landed
        const uint8_t* from = ring + slot * 1024 + lane * 16;
        bool use = true;
        if (ck >= 0) use = id_at(cbeg + static_cast<uint32_t>(ck)) < n_src;
        if (use) {
          VecT v0, v1;
          if (h0) v0 = *reinterpret_cast<const VecT*>(from);
          if (h1) v1 = *reinterpret_cast<const VecT*>(from + 512);
          if (ck < 0) {
#pragma unroll
            for (int e = 0; e < V; ++e) {
              if (h0) a0[e] = to_accum<A>(v0.v[e]);
              if (h1) a1[e] = to_accum<A>(v1.v[e]);
            }
          } else {
#pragma unroll
            for (int e = 0; e < V; ++e) {
              if (h0) a0[e] = seq_add(a0[e], to_accum<A>(v0.v[e]));
              if (h1) a1[e] = seq_add(a1[e], to_accum<A>(v1.v[e]));
            }
          }
        }
        ++ck;
        if (cbeg + static_cast<uint32_t>(ck) >= cend) {   // the row is complete
          VecT* out_row = reinterpret_cast<VecT*>(out + (w0 + cr) * inner);
          if (h0) {
            VecT t;
#pragma unroll
            for (int e = 0; e < V; ++e) t.v[e] = from_accum<T>(a0[e]);
            out_row[c0] = t;
          }
          if (h1) {
            VecT t;
#pragma unroll
            for (int e = 0; e < V; ++e) t.v[e] = from_accum<T>(a1[e]);
            out_row[c1] = t;
          }
          ++cr;
          ck = -1;
          if (cr < rows) seg_of(cr, cbeg, cend);
        }
        issue(slot);   // the slot just read takes the item kRingSlots ahead
        slot = slot + 1 == kRingSlots ? 0 : slot + 1;
      }
      cp_async_wait<0>();
    }
  }
}

// Element form: the thread that holds the head of a segment walks it.
template <typename T>
__global__ void __launch_bounds__(kThreads)
segment_elements_kernel(T* out, const T* self, const T* __restrict__ src,
                        const uint32_t* __restrict__ sorted_keys, const uint32_t* __restrict__ sorted_src,
                        int64_t n, int64_t out_numel) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t p = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; p < n; p += stride) {
    const uint32_t key = sorted_keys[p] & 0x7fffffffu;
    if (key >= out_numel) continue;
    if (p > 0 && (sorted_keys[p - 1] & 0x7fffffffu) == key) continue;
    using A = typename AccT<T, true>::type;
    A acc = to_accum<A>(self[key]);
    for (int64_t q = p; q < n && (sorted_keys[q] & 0x7fffffffu) == key; ++q) {
      const uint32_t sidx = sorted_src[q];
      if (sidx < n) acc = seq_add(acc, to_accum<A>(src[sidx]));
    }
    out[key] = from_accum<T>(acc);
  }
}

struct SortPlan {
  int64_t n;
  int passes;
  int nblocks;
  size_t keys_bytes, hist_bytes, seg_bytes, total;
  // row form only (n_dst_rows >= 0): header + scan status + counts (zeroed every call), then the queue of long segments
  int scan_blocks;
  size_t zero_bytes, bucket_bytes;
};

inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

SortPlan make_plan(int64_t n, int64_t key_range /* keys in [0, key_range) */, int64_t n_dst_rows) {
  SortPlan p{};
  p.n = n;
  int bits = 1;
  while ((int64_t(1) << bits) < key_range && bits < 31) ++bits;
  p.passes = (bits + 7) / 8;
  p.nblocks = static_cast<int>((n + kTile - 1) / kTile);
  if (p.nblocks < 1) p.nblocks = 1;
  p.keys_bytes = align256(static_cast<size_t>(n) * 4);
  p.hist_bytes = align256((static_cast<size_t>(256) * p.nblocks + 256) * 4);   // tile counts, then digit totals
  p.seg_bytes = n_dst_rows >= 0 ? align256(static_cast<size_t>(n_dst_rows + 2) * 4) : 0;
  if (n_dst_rows >= 0) {
    p.scan_blocks = static_cast<int>((n_dst_rows + kScanChunk - 1) / kScanChunk);
    if (p.scan_blocks < 1) p.scan_blocks = 1;
    p.zero_bytes = align256(sizeof(BucketHeader) + static_cast<size_t>(p.scan_blocks) * 8 + static_cast<size_t>(n_dst_rows + 1) * 4);
    p.bucket_bytes = p.zero_bytes + align256((static_cast<size_t>(n) / kBigSegment + 2) * 4);
  }
  p.total = 4 * p.keys_bytes + p.hist_bytes + p.seg_bytes + p.bucket_bytes;
  return p;
}

// Runs the sort. On return *sorted_keys / *sorted_vals point into the workspace.
b200Status run_sort(const SortPlan& p, uint32_t* keys_a, uint32_t* keys_b, uint32_t* vals_a,
                    uint32_t* vals_b, uint32_t* hist, cudaStream_t s, uint32_t** sorted_keys,
                    uint32_t** sorted_vals, uint32_t* seg_start = nullptr, int64_t n_dst = 0,
                    bool* bounds_done = nullptr) {
  if (bounds_done) *bounds_done = false;
  uint32_t *kin = keys_a, *kout = keys_b, *vin = nullptr, *vout = vals_a, *vother = vals_b;
  uint32_t* totals = hist + static_cast<size_t>(256) * p.nblocks;
  // one cooperative launch when the device can hold the grid, else three launches per pass
  static thread_local int coop_dev = -1, coop_blocks = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != coop_dev) {
    int supported = 0, per_sm = 0;
    cudaDeviceGetAttribute(&supported, cudaDevAttrCooperativeLaunch, dev);
    if (supported && cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, radix_sort_fused_kernel, kSortThreads, 0) == cudaSuccess)
      coop_blocks = per_sm * sm_count_current_device();
    else
      coop_blocks = 0;
    cudaGetLastError();
    coop_dev = dev;
  }
  bool fused = false;
  if (coop_blocks > 0) {
    int grid = p.nblocks > 256 ? p.nblocks : 256;
    if (grid > coop_blocks) grid = coop_blocks;
    int64_t n = p.n;
    int passes = p.passes, nblocks = p.nblocks;
    void* args[] = {&keys_a, &keys_b, &vals_a, &vals_b, &n, &passes, &nblocks, &hist, &totals, &seg_start, &n_dst};
    fused = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(radix_sort_fused_kernel), dim3(grid), dim3(kSortThreads), args, 0, s) ==
            cudaSuccess;
    if (!fused) cudaGetLastError();
    else if (bounds_done && seg_start) *bounds_done = true;
  }
  for (int pass = 0; pass < p.passes; ++pass) {
    if (!fused) {
      radix_hist_kernel<<<p.nblocks, kSortThreads, 0, s>>>(kin, p.n, pass, p.nblocks, hist);
      radix_scan_rows_kernel<<<256, kSortThreads, 0, s>>>(hist, p.nblocks, totals);
      radix_scatter_kernel<<<p.nblocks, kSortThreads, 0, s>>>(kin, vin, kout, vout, p.n, pass, p.nblocks, hist, totals);
    }
    uint32_t* t = kin; kin = kout; kout = t;
    vin = vout;
    vout = vother;
    vother = vin;
  }
  *sorted_keys = kin;
  *sorted_vals = vin;
  if (!fused) note_launches(3 * p.passes - 1);
  return check_launch("radix sort");
}

// Decides whether scatter_add(dim) can use the row form, and its geometry.
struct ScatterGeom {
  bool row_form;
  int64_t n_src, n_dst, inner;
  int64_t index_stride;
};

bool row_form_geometry(const b200Tensor* self, int64_t dim, const b200Tensor* index,
                       const b200Tensor* src, ScatterGeom* g) {
  if (dim != 0 || self->ndim < 1 || index->ndim != self->ndim || src->ndim != self->ndim) return false;
  if (!is_contiguous(self) || !is_contiguous(src)) return false;
  int64_t inner = 1;
  for (int d = 1; d < self->ndim; ++d) {
    if (index->sizes[d] != src->sizes[d] || index->sizes[d] != self->sizes[d]) return false;
    if (index->sizes[d] != 1 && index->strides[d] != 0) return false;  // must be broadcast along the row
    inner *= self->sizes[d];
  }
  if (index->sizes[0] != src->sizes[0]) return false;
  g->row_form = true;
  g->n_src = index->sizes[0];
  g->n_dst = self->sizes[0];
  g->inner = inner;
  g->index_stride = index->sizes[0] > 1 ? index->strides[0] : 1;
  return true;
}

template <typename T, int MODE, bool ACC32>
b200Status launch_segment_rows(void* out, const void* self, const void* src, const uint32_t* sorted_src,
                               const uint32_t* seg_start, int64_t n_dst, int64_t n_src, int64_t inner,
                               cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  const bool vec = inner % V == 0 && aligned16(out) && aligned16(self) && aligned16(src);
  const int64_t vpr = vec ? inner / V : inner;
  const int64_t cpr = (vpr + 63) / 64;
  const int64_t items = n_dst * cpr;
  if (items == 0) return B200_OK;
  if constexpr (MODE == 0) {
    // B200_WALK_RING=0 keeps the register-resident walk (for A/B timing)
    static const bool ring = [] { const char* e = getenv("B200_WALK_RING"); return !(e && e[0] == '0'); }();
    if (ring && vec) {
      // 4 slots and three blocks per SM: measured 114 us per scatter_add call against 117 (8 slots, two blocks),
      // 119 (10, two) and 162 (16, one): past a few KB per warp, more warps are worth more than a deeper ring
      constexpr int kSlots = 4, kBlocksPerSm = 3;
      auto kernel = segment_rows_ring_kernel<T, V, ACC32, kSlots, kBlocksPerSm>;
      constexpr size_t smem = static_cast<size_t>(kThreads / 32) * warp_smem(kSlots);
      static thread_local int last_dev = -1;
      int dev = 0;
      cudaGetDevice(&dev);
      if (dev != last_dev) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        B200_REQUIRE(e == cudaSuccess, B200_LAUNCH_FAILED, "segment rows: %s", cudaGetErrorString(e));
        last_dev = dev;
      }
      // one resident wave; every warp walks one contiguous range of destination rows
      const int grid = wave_grid<segment_rows_ring_kernel<T, V, ACC32, kSlots, kBlocksPerSm>>((n_dst + 7) / 8, kThreads, 1, smem);
      const int64_t total_warps = static_cast<int64_t>(grid) * (kThreads / 32);
      const int64_t rows_per_warp = (n_dst + total_warps - 1) / total_warps;
      cudaError_t le = launch_pdl(kernel, grid, kThreads, smem, s, (T*)out, (const T*)self, (const T*)src, sorted_src,
                                  seg_start, n_dst, n_src, inner, cpr, rows_per_warp);
      B200_REQUIRE(le == cudaSuccess, B200_LAUNCH_FAILED, "segment rows: %s", cudaGetErrorString(le));
      return check_launch("segment rows (ring)");
    }
  }
  int64_t need = (items + 7) / 8;
  const int64_t cap = static_cast<int64_t>(sm_count_current_device()) * 8;
  const int grid = static_cast<int>(need < cap ? need : cap);
  if (vec)
    launch_pdl(segment_rows_kernel<T, V, MODE, ACC32>, grid, kThreads, 0, s, (T*)out, (const T*)self, (const T*)src,
               sorted_src, seg_start, n_dst, n_src, inner, cpr);
  else
    launch_pdl(segment_rows_kernel<T, 1, MODE, ACC32>, grid, kThreads, 0, s, (T*)out, (const T*)self, (const T*)src,
               sorted_src, seg_start, n_dst, n_src, inner, cpr);
  return check_launch("segment rows");
}

// Row-form pipeline shared by scatter_add and index_put.
// mode 0: accumulate in the element type; 1: assign (last source wins);
// 2: accumulate, 16-bit floats in fp32 with one final rounding.
template <typename T>
b200Status scatter_rows(void* out, const void* self, const void* src, const b200Tensor* index,
                        int64_t index_stride, int64_t n_src, int64_t n_dst, int64_t inner, int mode,
                        int wrap_negative, void* workspace, size_t workspace_bytes, cudaStream_t s) {
  B200_REQUIRE(n_src < (int64_t(1) << 31) && n_dst < (int64_t(1) << 31) - 2, B200_NOT_SUPPORTED,
               "scatter: more than 2^31 rows");
  if (n_src == 0) {
    if (out != self) {
      cudaError_t e = cudaMemcpyAsync(out, self, static_cast<size_t>(n_dst) * inner * sizeof(T),
                                      cudaMemcpyDeviceToDevice, s);
      if (e != cudaSuccess) return fail(B200_LAUNCH_FAILED, "scatter: %s", cudaGetErrorString(e));
    }
    return B200_OK;
  }
  SortPlan p = make_plan(n_src, n_dst, n_dst);
  B200_REQUIRE(workspace && workspace_bytes >= p.total, B200_WORKSPACE_TOO_SMALL,
               "scatter: workspace of %zu bytes needed, %zu given", p.total, workspace_bytes);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, B200_BAD_PARAM,
               "scatter: workspace must be 256-byte aligned");
  char* w = static_cast<char*>(workspace);
  uint32_t* keys_a = reinterpret_cast<uint32_t*>(w);
  uint32_t* keys_b = reinterpret_cast<uint32_t*>(w + p.keys_bytes);
  uint32_t* vals_a = reinterpret_cast<uint32_t*>(w + 2 * p.keys_bytes);
  uint32_t* vals_b = reinterpret_cast<uint32_t*>(w + 3 * p.keys_bytes);
  uint32_t* hist = reinterpret_cast<uint32_t*>(w + 4 * p.keys_bytes);
  uint32_t* seg = reinterpret_cast<uint32_t*>(w + 4 * p.keys_bytes + p.hist_bytes);
  (void)hist;
  // grouping by destination: count, scan, claim, sort the (short) segments -- five small dependent launches
  char* bucket = w + 4 * p.keys_bytes + p.hist_bytes + p.seg_bytes;
  BucketHeader* header = reinterpret_cast<BucketHeader*>(bucket);
  unsigned long long* status = reinterpret_cast<unsigned long long*>(bucket + sizeof(BucketHeader));
  uint32_t* count = reinterpret_cast<uint32_t*>(bucket + sizeof(BucketHeader) + static_cast<size_t>(p.scan_blocks) * 8);
  uint32_t* big_list = reinterpret_cast<uint32_t*>(bucket + p.zero_bytes);
  uint32_t* sv = vals_a;   // the source ids, grouped by destination and ascending inside every group
  {
    cudaError_t e = cudaMemsetAsync(bucket, 0, p.zero_bytes, s);
    B200_REQUIRE(e == cudaSuccess, B200_LAUNCH_FAILED, "scatter: %s", cudaGetErrorString(e));
  }
  const int kgrid = grid_for(n_src, kThreads, 8);
  cudaError_t le;
  if (index->dtype == B200_I64)
    le = launch_pdl(bucket_count_kernel<int64_t>, kgrid, kThreads, 0, s, (const int64_t*)index->data, index_stride, n_src, n_dst,
                    wrap_negative, keys_a, vals_b, count);
  else
    le = launch_pdl(bucket_count_kernel<int32_t>, kgrid, kThreads, 0, s, (const int32_t*)index->data, index_stride, n_src, n_dst,
                    wrap_negative, keys_a, vals_b, count);
  if (le == cudaSuccess)
    le = launch_pdl(bucket_scan_kernel, p.scan_blocks, kScanThreads, 0, s, (const uint32_t*)count, seg, n_dst, header, status);
  if (le == cudaSuccess)
    le = launch_pdl(bucket_scatter_kernel, kgrid, kThreads, 0, s, (const uint32_t*)keys_a, (const uint32_t*)vals_b, n_src,
                    (const uint32_t*)seg, sv);
  if (le == cudaSuccess)
    le = launch_pdl(bucket_sort_segments_kernel, grid_for(n_dst, kThreads, 8), kThreads, 0, s, sv, (const uint32_t*)seg, n_dst, n_src,
                    header, big_list);
  int id_bits = 1;
  while ((int64_t(1) << id_bits) < n_src) ++id_bits;
  if (le == cudaSuccess)
    le = launch_pdl(bucket_sort_big_kernel, sm_count_current_device(), kSortThreads, 0, s, sv, keys_b, (const uint32_t*)seg, n_src,
                    (id_bits + 7) / 8, (const BucketHeader*)header, (const uint32_t*)big_list);
  B200_REQUIRE(le == cudaSuccess, B200_LAUNCH_FAILED, "scatter: %s", cudaGetErrorString(le));
  note_launches(6);   // the memset and the five grouping kernels; the segment walk counts itself
  if (mode == 1) return launch_segment_rows<T, 1, false>(out, self, src, sv, seg, n_dst, n_src, inner, s);
  if (mode == 2 && sizeof(T) == 2) return launch_segment_rows<T, 0, true>(out, self, src, sv, seg, n_dst, n_src, inner, s);
  return launch_segment_rows<T, 0, false>(out, self, src, sv, seg, n_dst, n_src, inner, s);
}

#define B200_DISPATCH_SCATTER(DT, T, ...)                                        \
  switch (DT) {                                                                  \
    case B200_F32: { using T = float; __VA_ARGS__; break; }                      \
    case B200_BF16: { using T = ::b200::bf16_t; __VA_ARGS__; break; }            \
    case B200_F16: { using T = ::b200::f16_t; __VA_ARGS__; break; }              \
    case B200_F64: { using T = double; __VA_ARGS__; break; }                     \
    case B200_I64: { using T = int64_t; __VA_ARGS__; break; }                    \
    case B200_I32: { using T = int32_t; __VA_ARGS__; break; }                    \
    default: return ::b200::fail(B200_NOT_SUPPORTED, "%s: dtype %d not supported", __func__, (int)(DT)); \
  }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

// Reads and clears the device error word (bit 0: an index was out of range and
// was replaced by 0 / skipped; bit 1: a bounded barrier wait in a tensor-core
// kernel gave up). Synchronises the device; meant for debug modes.
b200Status b200_device_error_fetch(uint32_t* flags) {
  B200_REQUIRE(flags, B200_BAD_PARAM, "b200_device_error_fetch: null");
  unsigned int v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_device_error_word, sizeof(v));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_device_error_word, &zero, sizeof(zero));
  if (e != cudaSuccess) return fail(B200_LAUNCH_FAILED, "b200_device_error_fetch: %s", cudaGetErrorString(e));
  *flags = v;
  return B200_OK;
}

b200Status b200_index_select(const b200Tensor* out, const b200Tensor* self, int64_t dim,
                             const b200Tensor* index, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(self) && valid(index), B200_BAD_PARAM, "b200_index_select: invalid tensor view");
  B200_REQUIRE(index->ndim <= 1, B200_BAD_PARAM, "b200_index_select: index must be 1-D");
  B200_REQUIRE(out->dtype == self->dtype, B200_BAD_PARAM, "b200_index_select: dtype mismatch");
  B200_REQUIRE(is_contiguous(self) && is_contiguous(out), B200_NOT_SUPPORTED,
               "b200_index_select: self/out must be contiguous");
  const int64_t K = numel(index);
  int64_t outer = 1, S = 1, inner = 1;
  if (self->ndim == 0) {
    B200_REQUIRE(dim == 0, B200_BAD_PARAM, "b200_index_select: dim");
  } else {
    B200_REQUIRE(dim >= 0 && dim < self->ndim, B200_BAD_PARAM, "b200_index_select: dim %lld", (long long)dim);
    for (int d = 0; d < dim; ++d) outer *= self->sizes[d];
    S = self->sizes[dim];
    for (int d = (int)dim + 1; d < self->ndim; ++d) inner *= self->sizes[d];
  }
  B200_REQUIRE(numel(out) == outer * K * inner, B200_BAD_PARAM, "b200_index_select: out shape");
  if (numel(out) == 0) return B200_OK;
  const int64_t es = static_cast<int64_t>(dtype_size(self->dtype));
  const int unit = pick_unit(inner * es, self->data, out->data, 0, 0, es);
  RowGatherArgs a{};
  a.src = self->data; a.dst = out->data; a.index = index->data;
  a.index_stride = index->ndim == 1 && K > 1 ? index->strides[0] : 1;
  a.n_rows = outer * K; a.K = K; a.S = S;
  a.upr = inner * es / unit;
  a.src_outer_stride = S * a.upr; a.src_row_stride = a.upr;
  a.wrap_negative = 0;
  return launch_row_gather(a, unit, index->dtype, static_cast<cudaStream_t>(stream));
}

b200Status b200_gather(const b200Tensor* out, const b200Tensor* self, int64_t dim,
                       const b200Tensor* index, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(self) && valid(index), B200_BAD_PARAM, "b200_gather: invalid tensor view");
  B200_REQUIRE(same_shape(out, index), B200_BAD_PARAM, "b200_gather: out and index shapes differ");
  B200_REQUIRE(out->dtype == self->dtype, B200_BAD_PARAM, "b200_gather: dtype mismatch");
  B200_REQUIRE(index->dtype == B200_I64 || index->dtype == B200_I32, B200_BAD_PARAM, "b200_gather: index dtype");
  const int64_t n = numel(out);
  if (n == 0) return B200_OK;
  B200_REQUIRE(self->ndim == index->ndim || (self->ndim == 0 && index->ndim <= 1) ||
               (index->ndim == 0 && self->ndim <= 1), B200_BAD_PARAM, "b200_gather: rank mismatch");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t es = static_cast<int64_t>(dtype_size(self->dtype));
  const int nd = index->ndim;
  int64_t dim_size = self->ndim ? self->sizes[dim] : 1, dim_stride = self->ndim ? self->strides[dim] : 0;
  if (nd > 0) B200_REQUIRE(dim >= 0 && dim < nd, B200_BAD_PARAM, "b200_gather: dim");

  bool fast = nd >= 1 && self->ndim == nd && dim == nd - 1 && is_contiguous(out) && is_contiguous(index) &&
              is_contiguous(self) && index->sizes[nd - 1] % 4 == 0 && (es == 4 || es == 2 || es == 8) &&
              aligned16(index->data) && aligned16(out->data);
  for (int d = 0; fast && d < nd - 1; ++d) fast = self->sizes[d] == index->sizes[d];
  if (fast) {
    const int64_t cols = index->sizes[nd - 1], n4 = n / 4;
    const int grid = grid_for(n4, kThreads, 8);
#define B200_GL(U)                                                                                     \
  do {                                                                                                 \
    if (index->dtype == B200_I64)                                                                      \
      launch_pdl(gather_lastdim_kernel<U, int64_t>, grid, kThreads, 0, s, (U*)out->data, (const U*)self->data, \
                 (const int64_t*)index->data, n4, cols, dim_size);                                     \
    else                                                                                               \
      launch_pdl(gather_lastdim_kernel<U, int32_t>, grid, kThreads, 0, s, (U*)out->data, (const U*)self->data, \
                 (const int32_t*)index->data, n4, cols, dim_size);                                     \
  } while (0)
    if (es == 4) B200_GL(uint32_t); else if (es == 2) B200_GL(uint16_t); else B200_GL(uint64_t);
#undef B200_GL
    return check_launch("b200_gather");
  }
  // generic: walk index's shape; self contributes every stride except dim's
  b200Tensor self_view = *index;
  self_view.data = self->data;
  self_view.dtype = self->dtype;
  for (int d = 0; d < nd; ++d) self_view.strides[d] = (d == dim || self->ndim == 0) ? 0 : self->strides[d];
  const b200Tensor* ts[3] = {out, index, &self_view};
  auto ix = make_indexer<3>(ts);
  const int grid = grid_for(n, kThreads, 8);
#define B200_GG(U)                                                                                      \
  do {                                                                                                  \
    if (index->dtype == B200_I64)                                                                       \
      gather_generic_kernel<U, int64_t><<<grid, kThreads, 0, s>>>((U*)out->data, (const U*)self->data,  \
                                                                  (const int64_t*)index->data, n, ix, dim_stride, dim_size); \
    else                                                                                                \
      gather_generic_kernel<U, int32_t><<<grid, kThreads, 0, s>>>((U*)out->data, (const U*)self->data,  \
                                                                  (const int32_t*)index->data, n, ix, dim_stride, dim_size); \
  } while (0)
  B200_DISPATCH_BYTES(es, U, B200_GG(U));
#undef B200_GG
  return check_launch("b200_gather");
}

b200Status b200_index(const b200Tensor* out, const b200Tensor* src, const b200Tensor* const* indices,
                      int32_t n_indices, const int64_t* indexed_sizes, const int64_t* indexed_strides,
                      b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(src), B200_BAD_PARAM, "b200_index: invalid tensor view");
  B200_REQUIRE(n_indices >= 1 && n_indices <= kMaxIndexTensors && indices && indexed_sizes && indexed_strides,
               B200_NOT_SUPPORTED, "b200_index: between 1 and %d index tensors supported", kMaxIndexTensors);
  B200_REQUIRE(same_shape(out, src) && out->dtype == src->dtype, B200_BAD_PARAM,
               "b200_index: src must be restrided to out's shape");
  for (int k = 0; k < n_indices; ++k) {
    B200_REQUIRE(indices[k] && valid(indices[k]) && same_shape(out, indices[k]), B200_BAD_PARAM,
                 "b200_index: index %d must be broadcast to out's shape", k);
    B200_REQUIRE(indices[k]->dtype == indices[0]->dtype &&
                 (indices[k]->dtype == B200_I32 || indices[k]->dtype == B200_I64), B200_BAD_PARAM,
                 "b200_index: indices must all be int32 or all int64");
  }
  const int64_t n = numel(out);
  if (n == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t es = static_cast<int64_t>(dtype_size(out->dtype));

  // Row form: one index tensor, constant along a contiguous trailing block that
  // src and out both walk contiguously.
  if (n_indices == 1 && is_contiguous(out)) {
    const b200Tensor* idx = indices[0];
    int split = out->ndim;  // trailing dims [split, ndim) form the row
    int64_t row = 1;
    while (split > 0) {
      const int d = split - 1;
      if (out->sizes[d] != 1 && (idx->strides[d] != 0 || src->strides[d] != row)) break;
      row *= out->sizes[d];
      --split;
    }
    bool lead_ok = row > 1;
    int64_t K = 1, expect = 1;
    for (int d = split - 1; d >= 0 && lead_ok; --d) {  // leading dims: index contiguous, src stride 0
      if (out->sizes[d] == 1) continue;
      if (src->strides[d] != 0 || idx->strides[d] != expect) lead_ok = false;
      expect *= out->sizes[d];
      K *= out->sizes[d];
    }
    if (lead_ok) {
      const int unit = pick_unit(row * es, src->data, out->data, indexed_strides[0] * es, 0, es);
      RowGatherArgs a{};
      a.src = src->data; a.dst = out->data; a.index = idx->data;
      a.index_stride = 1;
      a.n_rows = K; a.K = K; a.S = indexed_sizes[0];
      a.upr = row * es / unit;
      a.src_outer_stride = 0; a.src_row_stride = indexed_strides[0] * es / unit;
      a.wrap_negative = 1;
      return launch_row_gather(a, unit, idx->dtype, s);
    }
  }

  b200Tensor dummy = *out;
  dummy.data = nullptr;
  for (int d = 0; d < dummy.ndim; ++d) dummy.strides[d] = 0;
  const b200Tensor* ts[2 + kMaxIndexTensors];
  ts[0] = out; ts[1] = src;
  IndexArgs ia{};
  ia.n = n_indices;
  for (int k = 0; k < kMaxIndexTensors; ++k) {
    ts[2 + k] = k < n_indices ? indices[k] : &dummy;
    ia.idx[k] = k < n_indices ? indices[k]->data : nullptr;
    ia.sizes[k] = k < n_indices ? indexed_sizes[k] : 1;
    ia.strides[k] = k < n_indices ? indexed_strides[k] : 0;
  }
  auto ix = make_indexer<2 + kMaxIndexTensors>(ts);
  const int grid = grid_for(n, kThreads, 8);
#define B200_IG(U)                                                                                   \
  do {                                                                                               \
    if (indices[0]->dtype == B200_I64)                                                               \
      index_generic_kernel<U, int64_t><<<grid, kThreads, 0, s>>>((U*)out->data, (const U*)src->data, n, ix, ia); \
    else                                                                                             \
      index_generic_kernel<U, int32_t><<<grid, kThreads, 0, s>>>((U*)out->data, (const U*)src->data, n, ix, ia); \
  } while (0)
  B200_DISPATCH_BYTES(es, U, B200_IG(U));
#undef B200_IG
  return check_launch("b200_index");
}

size_t b200_scatter_add_workspace_size(const b200Tensor* self, int64_t dim, const b200Tensor* index,
                                       const b200Tensor* src) {
  if (!self || !index || !src || !valid(self) || !valid(index) || !valid(src)) return 0;
  ScatterGeom g{};
  if (row_form_geometry(self, dim, index, src, &g)) return make_plan(g.n_src, g.n_dst, g.n_dst).total;
  return make_plan(numel(index), numel(self), -1).total;
}

b200Status b200_scatter_add(const b200Tensor* out, const b200Tensor* self, int64_t dim,
                            const b200Tensor* index, const b200Tensor* src, void* workspace,
                            size_t workspace_bytes, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(self) && valid(index) && valid(src), B200_BAD_PARAM,
               "b200_scatter_add: invalid tensor view");
  B200_REQUIRE(same_shape(out, self) && out->dtype == self->dtype && src->dtype == self->dtype, B200_BAD_PARAM,
               "b200_scatter_add: out/self/src must agree in dtype, out and self in shape");
  B200_REQUIRE(index->dtype == B200_I64 || index->dtype == B200_I32, B200_BAD_PARAM, "b200_scatter_add: index dtype");
  B200_REQUIRE(is_contiguous(out) && is_contiguous(self), B200_NOT_SUPPORTED,
               "b200_scatter_add: out/self must be contiguous");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (numel(self) == 0) return B200_OK;
  B200_REQUIRE(self->ndim == 0 || (dim >= 0 && dim < self->ndim), B200_BAD_PARAM, "b200_scatter_add: dim");

  ScatterGeom g{};
  if (row_form_geometry(self, dim, index, src, &g)) {
    B200_DISPATCH_SCATTER(self->dtype, T, {
      // CPU ATen runs scatter_add on bf16/f16 through an fp32 buffer: the sums
      // are accumulated in fp32 and rounded once (mode 2). index_put(accumulate)
      // instead adds in the element type, rounding after every add (mode 0).
      return scatter_rows<T>(out->data, self->data, src->data, index, g.index_stride, g.n_src, g.n_dst,
                             g.inner, 2, 0, workspace, workspace_bytes, s);
    });
  }

  // element form
  if (out->data != self->data) {
    b200Status st = b200_copy(out, self, stream);
    if (st != B200_OK) return st;
  }
  const int64_t n = numel(index);
  if (n == 0) return B200_OK;
  B200_REQUIRE(index->ndim == self->ndim && src->ndim == self->ndim, B200_BAD_PARAM,
               "b200_scatter_add: index/src rank must equal self's");
  B200_REQUIRE(same_shape(index, src) && is_contiguous(src), B200_NOT_SUPPORTED,
               "b200_scatter_add: element form needs src contiguous and shaped like index");
  const int64_t out_numel = numel(self);
  B200_REQUIRE(n < (int64_t(1) << 31) && out_numel < (int64_t(1) << 31), B200_NOT_SUPPORTED,
               "b200_scatter_add: element form limited to 2^31 sources and destinations");
  SortPlan p = make_plan(n, out_numel, -1);
  B200_REQUIRE(workspace && workspace_bytes >= p.total, B200_WORKSPACE_TOO_SMALL,
               "b200_scatter_add: workspace of %zu bytes needed, %zu given", p.total, workspace_bytes);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, B200_BAD_PARAM,
               "b200_scatter_add: workspace must be 256-byte aligned");
  char* w = static_cast<char*>(workspace);
  uint32_t* keys_a = reinterpret_cast<uint32_t*>(w);
  uint32_t* keys_b = reinterpret_cast<uint32_t*>(w + p.keys_bytes);
  uint32_t* vals_a = reinterpret_cast<uint32_t*>(w + 2 * p.keys_bytes);
  uint32_t* vals_b = reinterpret_cast<uint32_t*>(w + 3 * p.keys_bytes);
  uint32_t* hist = reinterpret_cast<uint32_t*>(w + 4 * p.keys_bytes);

  b200Tensor dst_view = *index;  // destination offsets without the dim term
  dst_view.data = out->data;
  for (int d = 0; d < index->ndim; ++d) dst_view.strides[d] = d == dim ? 0 : self->strides[d];
  b200Tensor idx_c = *index;
  // The sort's tie order is the row-major order of index's shape, so walk it
  // uncollapsed-by-value: make_indexer only merges dims, it keeps the order.
  const b200Tensor* ts[2] = {&idx_c, &dst_view};
  auto ix = make_indexer<2>(ts);
  const int64_t dim_stride = self->ndim ? self->strides[dim] : 0;
  const int64_t dim_size = self->ndim ? self->sizes[dim] : 1;
  const int kgrid = grid_for(n, kThreads, 8);
  if (index->dtype == B200_I64)
    element_keys_kernel<int64_t><<<kgrid, kThreads, 0, s>>>((const int64_t*)index->data, n, ix, dim_stride, dim_size, out_numel, keys_a);
  else
    element_keys_kernel<int32_t><<<kgrid, kThreads, 0, s>>>((const int32_t*)index->data, n, ix, dim_stride, dim_size, out_numel, keys_a);
  note_launches(1);   // the key kernel above
  uint32_t *sk, *sv;
  b200Status st = run_sort(p, keys_a, keys_b, vals_a, vals_b, hist, s, &sk, &sv);
  if (st != B200_OK) return st;
  B200_DISPATCH_SCATTER(self->dtype, T, {
    segment_elements_kernel<T><<<kgrid, kThreads, 0, s>>>((T*)out->data, (const T*)self->data,
                                                         (const T*)src->data, sk, sv, n, out_numel);
  });
  return check_launch("b200_scatter_add");
}

// ---- scatter_add without any allocation -----------------------------------
// Scratch for b200_scatter_add_static: lives in the library image, so every GPU
// that loads the library holds these bytes until the process exits.
#define B200_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_static_scratch[B200_STATIC_SCRATCH_BYTES];

b200Status b200_scatter_add_static(const b200Tensor* out, const b200Tensor* self, int64_t dim,
                                   const b200Tensor* index, const b200Tensor* src, b200Stream stream) {
  // Argument and size checks come first: a call that is refused costs no device call at all.
  B200_REQUIRE(out && self && index && src, B200_BAD_PARAM, "b200_scatter_add_static: null tensor");
  B200_REQUIRE(valid(out) && valid(self) && valid(index) && valid(src), B200_BAD_PARAM,
               "b200_scatter_add_static: invalid tensor view");
  const size_t need = b200_scatter_add_workspace_size(self, dim, index, src);
  B200_REQUIRE(need <= B200_STATIC_SCRATCH_BYTES, B200_NOT_SUPPORTED,
               "b200_scatter_add_static: this problem needs %zu bytes of scratch, the built-in array holds %u; "
               "use b200_scatter_add with a caller workspace", need, (unsigned)B200_STATIC_SCRATCH_BYTES);
  // In host code `g_static_scratch` is only a handle for the symbol, not a device
  // address: the address is looked up once per device, with that device current.
  static void* scratch_of_device[64] = {nullptr};
  static std::mutex setup_mutex;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  B200_REQUIRE(e == cudaSuccess && dev >= 0 && dev < 64, B200_LAUNCH_FAILED, "b200_scatter_add_static: %s",
               e == cudaSuccess ? "device index out of range" : cudaGetErrorString(e));
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> g(setup_mutex);
    if (!scratch_of_device[dev]) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_static_scratch);
      if (e != cudaSuccess || !p) {
        (void)cudaGetLastError();
        return fail(B200_LAUNCH_FAILED, "b200_scatter_add_static: cannot resolve the scratch array on device %d: %s", dev,
                    cudaGetErrorString(e));
      }
      scratch_of_device[dev] = p;
    }
    scratch = scratch_of_device[dev];
  }
  // Nothing in the scratch has to start at zero: keys, histograms, sorted pairs and
  // segment starts are all fully rewritten by every call before they are read.
  return b200_scatter_add(out, self, dim, index, src, scratch, B200_STATIC_SCRATCH_BYTES, stream);
}

size_t b200_index_put_workspace_size(const b200Tensor* self, const b200Tensor* index,
                                     const b200Tensor* values) {
  if (!self || !index || !values || !valid(self) || !valid(index) || self->ndim < 1) return 0;
  return make_plan(numel(index), self->sizes[0], self->sizes[0]).total;
}

b200Status b200_index_put(const b200Tensor* self, const b200Tensor* index, const b200Tensor* values,
                          int32_t accumulate, void* workspace, size_t workspace_bytes, b200Stream stream) {
  B200_REQUIRE(valid(self) && valid(index) && valid(values), B200_BAD_PARAM, "b200_index_put: invalid tensor view");
  B200_REQUIRE(self->ndim >= 1 && index->ndim <= 1, B200_BAD_PARAM,
               "b200_index_put: self must have rank >= 1 and index rank 1");
  B200_REQUIRE(index->dtype == B200_I64 || index->dtype == B200_I32, B200_BAD_PARAM, "b200_index_put: index dtype");
  B200_REQUIRE(values->dtype == self->dtype, B200_BAD_PARAM, "b200_index_put: dtype mismatch");
  B200_REQUIRE(is_contiguous(self) && is_contiguous(values), B200_NOT_SUPPORTED,
               "b200_index_put: self/values must be contiguous");
  const int64_t n_src = numel(index), n_dst = self->sizes[0];
  int64_t inner = 1;
  for (int d = 1; d < self->ndim; ++d) inner *= self->sizes[d];
  B200_REQUIRE(numel(values) == n_src * inner, B200_BAD_PARAM,
               "b200_index_put: values must hold index.numel() rows of self's row shape");
  if (n_src == 0 || numel(self) == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t istride = index->ndim == 1 && n_src > 1 ? index->strides[0] : 1;
  // Negative indices wrap once, as ATen's index_put does.
  B200_DISPATCH_SCATTER(self->dtype, T, {
    return scatter_rows<T>(self->data, self->data, values->data, index, istride, n_src, n_dst, inner,
                           accumulate ? 0 : 1, 1, workspace, workspace_bytes, s);
  });
  return B200_OK;
}

}  // extern "C"
