// Row sort (sort / argsort / topk) and cumulative sum: what a sampling step needs around
// the logits (top-k, top-p). Stand-ins for the vendor calls behind the reference's generated
// aotops::sort_out (values_stable), argsort (stable), topk_out (values) and cumsum_out
// (codegen/gcu_native_functions.yaml rows sort.values_stable, argsort.stable, topk.values,
// cumsum.out).
//
// Sort: a stable least-significant-digit radix sort, one CTA per row, 8 bits per pass. Every
// element becomes an unsigned key whose integer order is the element order CPU ATen uses
// (NaN greater than every number, -0 equal to +0), inverted for a descending sort; the row
// position rides along as the value, so equal keys keep their original order (the stable
// contract) and the sorted values are gathered from the input by position at the end (the
// output holds the input's own bits, NaN payloads and zero signs included).
// A pass over a row: digit histogram in shared memory, exclusive scan, then the tiles of the
// row in order -- per tile the ranks come from warp-level match / popcount, a prefix over the
// warps, and a running per-digit base.
//
// Cumsum: along the last dimension a block scans a row in chunks (thread-local serial prefix,
// block scan of the thread totals, running carry); along any other dimension one thread walks
// one column serially (coalesced across the inner dimension), which is CPU ATen's own order.
// Accumulation follows CPU ATen: fp32 rows in fp64, bf16 / f16 in fp32, integers in int64.
#include "common.cuh"

#include <initializer_list>

namespace b200 {
namespace {

constexpr int kSortThreads = 512;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kSortItems = 4;
constexpr int kSortTile = kSortThreads * kSortItems;   // 2048 keys per step

// ---- element -> ordered unsigned key --------------------------------------------------
template <typename K> struct KeyOf;

__device__ __forceinline__ uint32_t key_f32(uint32_t u) {
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;        // NaN: above +inf
  if (u == 0x80000000u) u = 0;                                      // -0 orders as +0
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ uint32_t key_f16like(uint32_t u, uint32_t exp_mask) {
  if ((u & 0x7fffu) > exp_mask) return 0xffffu;
  if (u == 0x8000u) u = 0;
  return (u & 0x8000u) ? (~u & 0xffffu) : (u | 0x8000u);
}
__device__ __forceinline__ uint64_t key_f64(uint64_t u) {
  if ((u & 0x7fffffffffffffffull) > 0x7ff0000000000000ull) return ~0ull;
  if (u == 0x8000000000000000ull) u = 0;
  return (u & 0x8000000000000000ull) ? ~u : (u | 0x8000000000000000ull);
}

// dtype codes are b200DType; K is uint32_t for elements of up to 4 bytes, uint64_t for 8.
template <typename K>
__device__ __forceinline__ K load_key(const void* base, int64_t i, int dtype, bool descending);

template <>
__device__ __forceinline__ uint32_t load_key<uint32_t>(const void* base, int64_t i, int dtype, bool descending) {
  uint32_t k;
  switch (dtype) {
    case B200_F32: k = key_f32(static_cast<const uint32_t*>(base)[i]); break;
    case B200_BF16: k = key_f16like(static_cast<const uint16_t*>(base)[i], 0x7f80u); break;
    case B200_F16: k = key_f16like(static_cast<const uint16_t*>(base)[i], 0x7c00u); break;
    case B200_I32: k = static_cast<const uint32_t*>(base)[i] ^ 0x80000000u; break;
    case B200_I16: k = (static_cast<const uint16_t*>(base)[i] ^ 0x8000u) & 0xffffu; break;
    case B200_I8: k = (static_cast<const uint8_t*>(base)[i] ^ 0x80u) & 0xffu; break;
    default: k = static_cast<const uint8_t*>(base)[i]; break;   // u8, bool
  }
  return descending ? ~k : k;   // bits above the element's width are never taken as a digit
}
template <>
__device__ __forceinline__ uint64_t load_key<uint64_t>(const void* base, int64_t i, int dtype, bool descending) {
  const uint64_t u = static_cast<const uint64_t*>(base)[i];
  const uint64_t k = dtype == B200_F64 ? key_f64(u) : (u ^ 0x8000000000000000ull);
  return descending ? ~k : k;
}

struct SortSmem {
  uint32_t warp_count[kSortWarps][256];   // per tile: counts, then exclusive base per warp
  uint32_t digit_base[256];               // where the next key of each digit goes (running)
  uint32_t scan[kSortWarps];
};

// Exclusive scan of one value per thread over the first 256 threads (8 warps).
__device__ __forceinline__ uint32_t scan_256(uint32_t v, uint32_t* sh) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (warp < 8 && lane == 31) sh[warp] = inc;
  __syncthreads();
  uint32_t before = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w)
    if (w < warp) before += sh[w];
  __syncthreads();
  return before + inc - v;
}

// One CTA sorts one row per iteration of its row loop.
// in: (rows, n) contiguous elements. keys_* / idx_*: ping-pong scratch of rows * n entries each.
// values_out (element bytes `esize`, may be null) and indices_out (int64, may be null) take the first
// k sorted entries of every row.
template <typename K>
__global__ void __launch_bounds__(kSortThreads)
row_sort_kernel(const void* __restrict__ in, int dtype, int esize, int64_t rows, int64_t n, int64_t k, int descending,
                int passes, K* keys_a, K* keys_b, uint32_t* idx_a, uint32_t* idx_b, void* values_out,
                int64_t* indices_out) {
  __shared__ SortSmem sm;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const char* in_row = static_cast<const char*>(in) + row * n * esize;
    K* ka = keys_a + row * n;
    K* kb = keys_b + row * n;
    uint32_t* ia = idx_a + row * n;
    uint32_t* ib = idx_b + row * n;
    const K* kin = nullptr;          // pass 0 reads the elements themselves
    const uint32_t* iin = nullptr;   // ... and the value of item i is i
    K* kout = ka;
    uint32_t* iout = ia;
    for (int pass = 0; pass < passes; ++pass) {
      const int shift = 8 * pass;
      const bool last = pass == passes - 1;
      // 1. digit histogram of the row
      for (int i = threadIdx.x; i < 256; i += kSortThreads) sm.digit_base[i] = 0;
      __syncthreads();
      for (int64_t i = threadIdx.x; i < n; i += kSortThreads) {
        const K key = kin ? kin[i] : load_key<K>(in_row, i, dtype, descending != 0);
        atomicAdd(&sm.digit_base[static_cast<uint32_t>(key >> shift) & 255u], 1u);
      }
      __syncthreads();
      // 2. exclusive scan: first destination of every digit
      {
        const uint32_t c = threadIdx.x < 256 ? sm.digit_base[threadIdx.x] : 0u;
        const uint32_t ex = scan_256(c, sm.scan);
        if (threadIdx.x < 256) sm.digit_base[threadIdx.x] = ex;
      }
      __syncthreads();
      // 3. the tiles of the row in order
      for (int64_t base = 0; base < n; base += kSortTile) {
        for (int i = threadIdx.x; i < kSortWarps * 256; i += kSortThreads) (&sm.warp_count[0][0])[i] = 0;
        __syncthreads();
        const int64_t wbase = base + warp * (kSortItems * 32);
        K key[kSortItems];
        uint32_t val[kSortItems];
#pragma unroll
        for (int r = 0; r < kSortItems; ++r) {
          const int64_t i = wbase + r * 32 + lane;
          if (i < n) {
            key[r] = kin ? kin[i] : load_key<K>(in_row, i, dtype, descending != 0);
            val[r] = iin ? iin[i] : static_cast<uint32_t>(i);
          } else {
            key[r] = 0;
            val[r] = 0;
          }
        }
#pragma unroll
        for (int r = 0; r < kSortItems; ++r) {
          const bool live = wbase + r * 32 + lane < n;
          const uint32_t d = live ? (static_cast<uint32_t>(key[r] >> shift) & 255u) : (256u + lane);
          const uint32_t peers = __match_any_sync(0xffffffffu, d);
          if (live && lane == (__ffs(peers) - 1)) sm.warp_count[warp][d] += __popc(peers);
          __syncwarp();
        }
        __syncthreads();
        uint32_t tile_total = 0;
        if (threadIdx.x < 256) {   // exclusive prefix over the warps, per digit
          uint32_t run = 0;
#pragma unroll
          for (int w = 0; w < kSortWarps; ++w) {
            const uint32_t c = sm.warp_count[w][threadIdx.x];
            sm.warp_count[w][threadIdx.x] = run;
            run += c;
          }
          tile_total = run;
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kSortItems; ++r) {
          const bool live = wbase + r * 32 + lane < n;
          const uint32_t d = live ? (static_cast<uint32_t>(key[r] >> shift) & 255u) : (256u + lane);
          const uint32_t peers = __match_any_sync(0xffffffffu, d);
          uint32_t pos = 0;
          if (live) pos = sm.digit_base[d] + sm.warp_count[warp][d] + __popc(peers & ((1u << lane) - 1u));
          __syncwarp();
          if (live && lane == (__ffs(peers) - 1)) sm.warp_count[warp][d] += __popc(peers);
          __syncwarp();
          if (live) {
            if (!last) {
              kout[pos] = key[r];
              iout[pos] = val[r];
            } else if (pos < k) {
              if (indices_out) indices_out[row * k + pos] = static_cast<int64_t>(val[r]);
              if (values_out) {
                const char* src = in_row + static_cast<int64_t>(val[r]) * esize;
                char* dst = static_cast<char*>(values_out) + (row * k + pos) * esize;
                switch (esize) {
                  case 1: *dst = *src; break;
                  case 2: *reinterpret_cast<uint16_t*>(dst) = *reinterpret_cast<const uint16_t*>(src); break;
                  case 4: *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(src); break;
                  default: *reinterpret_cast<uint64_t*>(dst) = *reinterpret_cast<const uint64_t*>(src); break;
                }
              }
            }
          }
        }
        __syncthreads();
        if (threadIdx.x < 256) sm.digit_base[threadIdx.x] += tile_total;
        __syncthreads();
      }
      kin = kout;
      iin = iout;
      kout = (kout == ka) ? kb : ka;
      iout = (iout == ia) ? ib : ia;
    }
  }
}

// ---- cumulative sum -----------------------------------------------------------------------
template <typename T> struct ScanAcc { using type = int64_t; };
template <> struct ScanAcc<float> { using type = double; };
template <> struct ScanAcc<double> { using type = double; };
template <> struct ScanAcc<bf16_t> { using type = float; };
template <> struct ScanAcc<f16_t> { using type = float; };

template <typename T, typename A> __device__ __forceinline__ A scan_load(T v) { return static_cast<A>(v); }
template <> __device__ __forceinline__ float scan_load<bf16_t, float>(bf16_t v) { return bf16_bits_to_f32(v.bits); }
template <> __device__ __forceinline__ float scan_load<f16_t, float>(f16_t v) { return f16_bits_to_f32(v.bits); }
template <typename T, typename A> __device__ __forceinline__ T scan_store(A v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ bf16_t scan_store<bf16_t, float>(float v) { return bf16_t{f32_to_bf16_bits(v)}; }
template <> __device__ __forceinline__ f16_t scan_store<f16_t, float>(float v) { return f16_t{f32_to_f16_bits(v)}; }

constexpr int kScanThreads = 256;
constexpr int kScanItems = 8;

template <typename A>
__device__ __forceinline__ A shfl_up_any(A v, int o) {
  if constexpr (sizeof(A) == 8) {
    long long x = __shfl_up_sync(0xffffffffu, *reinterpret_cast<long long*>(&v), o);
    return *reinterpret_cast<A*>(&x);
  } else {
    return __shfl_up_sync(0xffffffffu, v, o);
  }
}

// One block per row of a (rows, n) contiguous view, scanning along n.
template <typename T>
__global__ void __launch_bounds__(kScanThreads)
cumsum_rows_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t rows, int64_t n) {
  using A = typename ScanAcc<T>::type;
  __shared__ A warp_tot[kScanThreads / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const T* src = in + row * n;
    T* dst = out + row * n;
    A carry = 0;
    for (int64_t base = 0; base < n; base += kScanThreads * kScanItems) {
      const int64_t first = base + static_cast<int64_t>(threadIdx.x) * kScanItems;
      A v[kScanItems];
      A run = 0;
#pragma unroll
      for (int j = 0; j < kScanItems; ++j) {
        const int64_t i = first + j;
        run += i < n ? scan_load<T, A>(src[i]) : A(0);
        v[j] = run;
      }
      A inc = run;   // inclusive scan of the thread totals over the block
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const A t = shfl_up_any<A>(inc, o);
        if (lane >= o) inc += t;
      }
      __syncthreads();   // readers of warp_tot from the previous chunk are done
      if (lane == 31) warp_tot[warp] = inc;
      __syncthreads();
      A before = carry, all = 0;
#pragma unroll
      for (int w = 0; w < kScanThreads / 32; ++w) {
        const A c = warp_tot[w];
        if (w < warp) before += c;
        all += c;
      }
      const A offset = before + inc - run;
#pragma unroll
      for (int j = 0; j < kScanItems; ++j) {
        const int64_t i = first + j;
        if (i < n) dst[i] = scan_store<T, A>(offset + v[j]);
      }
      carry += all;
    }
    __syncthreads();
  }
}

// (outer, n, inner) contiguous view, inner > 1: one thread per (outer, inner) column, serial along n.
template <typename T>
__global__ void __launch_bounds__(kScanThreads)
cumsum_columns_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t outer, int64_t n, int64_t inner) {
  using A = typename ScanAcc<T>::type;
  const int64_t total = outer * inner;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kScanThreads;
  for (int64_t c = static_cast<int64_t>(blockIdx.x) * kScanThreads + threadIdx.x; c < total; c += stride) {
    const int64_t o = c / inner, i = c - o * inner;
    const T* src = in + o * n * inner + i;
    T* dst = out + o * n * inner + i;
    A run = 0;
    for (int64_t j = 0; j < n; ++j) {
      run += scan_load<T, A>(src[j * inner]);
      dst[j * inner] = scan_store<T, A>(run);
    }
  }
}

int sort_passes(int32_t dtype) { return static_cast<int>(dtype_size(dtype)); }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_sort_rows_workspace_size(const b200Tensor* in) {
  if (!in || !valid(in)) return 0;
  const size_t count = static_cast<size_t>(numel(in));
  const size_t key = dtype_size(in->dtype) == 8 ? 8 : 4;
  return 2 * ((count * key + 255) / 256 * 256) + 2 * ((count * 4 + 255) / 256 * 256);
}

b200Status b200_sort_rows(const b200Tensor* values, const b200Tensor* indices, const b200Tensor* in, int32_t descending,
                          void* workspace, size_t workspace_bytes, b200Stream stream) {
  B200_REQUIRE(valid(in) && in->ndim == 2 && is_contiguous(in), B200_BAD_PARAM,
               "b200_sort_rows: in must be a contiguous (rows, n) view");
  B200_REQUIRE(values || indices, B200_BAD_PARAM, "b200_sort_rows: no output given");
  const int64_t rows = in->sizes[0], n = in->sizes[1];
  int64_t k = -1;
  for (const b200Tensor* o : {values, indices}) {
    if (!o) continue;
    B200_REQUIRE(valid(o) && o->ndim == 2 && is_contiguous(o) && o->sizes[0] == rows && o->sizes[1] <= n, B200_BAD_PARAM,
                 "b200_sort_rows: outputs must be contiguous (rows, k) with k <= n");
    B200_REQUIRE(k < 0 || k == o->sizes[1], B200_BAD_PARAM, "b200_sort_rows: values and indices disagree in k");
    k = o->sizes[1];
  }
  B200_REQUIRE(!values || values->dtype == in->dtype, B200_BAD_PARAM, "b200_sort_rows: values must have in's dtype");
  B200_REQUIRE(!indices || indices->dtype == B200_I64, B200_BAD_PARAM, "b200_sort_rows: indices must be int64");
  B200_REQUIRE(n < (int64_t(1) << 32), B200_NOT_SUPPORTED, "b200_sort_rows: rows of up to 2^32 - 1 elements");
  if (rows == 0 || n == 0 || k == 0) return B200_OK;
  const size_t need = b200_sort_rows_workspace_size(in);
  B200_REQUIRE(workspace && workspace_bytes >= need, B200_WORKSPACE_TOO_SMALL,
               "b200_sort_rows: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  B200_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, B200_BAD_PARAM,
               "b200_sort_rows: workspace must be 256-byte aligned");
  const size_t count = static_cast<size_t>(rows * n);
  const int esize = static_cast<int>(dtype_size(in->dtype));
  const size_t key_bytes = (count * (esize == 8 ? 8 : 4) + 255) / 256 * 256, idx_bytes = (count * 4 + 255) / 256 * 256;
  char* w = static_cast<char*>(workspace);
  uint32_t* idx_a = reinterpret_cast<uint32_t*>(w + 2 * key_bytes);
  uint32_t* idx_b = reinterpret_cast<uint32_t*>(w + 2 * key_bytes + idx_bytes);
  const int grid = static_cast<int>(rows < 4 * sm_count_current_device() ? rows : 4 * sm_count_current_device());
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  void* vout = values ? values->data : nullptr;
  int64_t* iout = indices ? static_cast<int64_t*>(indices->data) : nullptr;
  if (esize == 8)
    row_sort_kernel<uint64_t><<<grid, kSortThreads, 0, s>>>(in->data, in->dtype, esize, rows, n, k, descending, sort_passes(in->dtype),
                                                            reinterpret_cast<uint64_t*>(w), reinterpret_cast<uint64_t*>(w + key_bytes),
                                                            idx_a, idx_b, vout, iout);
  else
    row_sort_kernel<uint32_t><<<grid, kSortThreads, 0, s>>>(in->data, in->dtype, esize, rows, n, k, descending, sort_passes(in->dtype),
                                                            reinterpret_cast<uint32_t*>(w), reinterpret_cast<uint32_t*>(w + key_bytes),
                                                            idx_a, idx_b, vout, iout);
  return check_launch("b200_sort_rows");
}

b200Status b200_cumsum(const b200Tensor* out, const b200Tensor* in, int64_t dim, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(in) && same_shape(out, in) && out->dtype == in->dtype, B200_BAD_PARAM,
               "b200_cumsum: out and in must agree in shape and dtype");
  B200_REQUIRE(is_contiguous(out) && is_contiguous(in), B200_NOT_SUPPORTED, "b200_cumsum: contiguous operands");
  B200_REQUIRE(in->ndim == 0 || (dim >= 0 && dim < in->ndim), B200_BAD_PARAM, "b200_cumsum: dim");
  const int64_t total = numel(in);
  if (total == 0) return B200_OK;
  int64_t outer = 1, n = in->ndim ? in->sizes[dim] : 1, inner = 1;
  for (int d = 0; d < dim; ++d) outer *= in->sizes[d];
  for (int d = static_cast<int>(dim) + 1; d < in->ndim; ++d) inner *= in->sizes[d];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int sms = sm_count_current_device();
  B200_DISPATCH_ARITH(in->dtype, T, {
    if (inner == 1) {
      const int grid = static_cast<int>(outer < 8 * sms ? outer : 8 * sms);
      cumsum_rows_kernel<T><<<grid, kScanThreads, 0, s>>>(static_cast<T*>(out->data), static_cast<const T*>(in->data), outer, n);
    } else {
      const int grid = grid_for(outer * inner, kScanThreads, 8);
      cumsum_columns_kernel<T><<<grid, kScanThreads, 0, s>>>(static_cast<T*>(out->data), static_cast<const T*>(in->data), outer,
                                                            n, inner);
    }
  });
  return check_launch("b200_cumsum");
}

}  // extern "C"
