// Device-to-device copy with optional dtype cast and restriding.
//
//  * same dtype, both contiguous      -> cudaMemcpyAsync (copy engine / SM copy)
//  * same dtype, strided              -> indexed kernel over the widest unit
//                                        (16/8/4/2 bytes) the views allow
//  * f32/bf16/f16 casts, contiguous   -> streaming kernel, 8 elements per thread
//                                        step with 128-bit accesses on the wide side
//  * any other dtype pair or layout   -> indexed kernel, one element per step
//
// Conversion rules are those of c10: float->integer truncates toward zero,
// anything->bool is (x != 0), fp32->bf16/f16 rounds to nearest even (NaN stays
// NaN), wider floats go through fp32.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;

struct bool_t { uint8_t v; };

template <typename S> struct Wide { using type = int64_t; };
template <> struct Wide<float> { using type = double; };
template <> struct Wide<double> { using type = double; };
template <> struct Wide<bf16_t> { using type = double; };
template <> struct Wide<f16_t> { using type = double; };

template <typename S> __device__ __forceinline__ typename Wide<S>::type widen(S v) {
  return static_cast<typename Wide<S>::type>(v);
}
template <> __device__ __forceinline__ double widen<bf16_t>(bf16_t v) { return bf16_bits_to_f32(v.bits); }
template <> __device__ __forceinline__ double widen<f16_t>(f16_t v) { return f16_bits_to_f32(v.bits); }
template <> __device__ __forceinline__ int64_t widen<bool_t>(bool_t v) { return v.v != 0; }

template <typename D, typename W> __device__ __forceinline__ D narrow(W w) { return static_cast<D>(w); }
template <> __device__ __forceinline__ bf16_t narrow<bf16_t, double>(double w) { return bf16_t{f32_to_bf16_bits(static_cast<float>(w))}; }
template <> __device__ __forceinline__ bf16_t narrow<bf16_t, int64_t>(int64_t w) { return bf16_t{f32_to_bf16_bits(static_cast<float>(w))}; }
template <> __device__ __forceinline__ f16_t narrow<f16_t, double>(double w) { return f16_t{f32_to_f16_bits(static_cast<float>(w))}; }
template <> __device__ __forceinline__ f16_t narrow<f16_t, int64_t>(int64_t w) { return f16_t{f32_to_f16_bits(static_cast<float>(w))}; }
template <> __device__ __forceinline__ bool_t narrow<bool_t, double>(double w) { return bool_t{static_cast<uint8_t>(w != 0.0)}; }
template <> __device__ __forceinline__ bool_t narrow<bool_t, int64_t>(int64_t w) { return bool_t{static_cast<uint8_t>(w != 0)}; }

template <typename S, typename D>
__global__ void __launch_bounds__(kThreads)
cast_indexed_kernel(D* dst, const S* src, int64_t n, StridedIndexer<2> ix, bool contig) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t off[2] = {i, i};
    if (!contig) ix.offsets(i, off);
    dst[off[0]] = narrow<D>(widen<S>(src[off[1]]));
  }
}

template <typename U>
__global__ void __launch_bounds__(kThreads)
copy_indexed_kernel(U* dst, const U* src, int64_t n, StridedIndexer<2> ix) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t off[2];
    ix.offsets(i, off);
    dst[off[0]] = src[off[1]];
  }
}

// Streaming cast between f32 / bf16 / f16. E elements per thread step, chosen so
// that the wider side moves 128 bits and every warp access is contiguous on
// both sides (f32<->16-bit: 4 elements = 16 B + 8 B; 16-bit<->16-bit: 8 elements).
template <typename T, int E> struct alignas(sizeof(T) * E) PackE { T v[E]; };

template <typename P> __device__ __forceinline__ P load_stream_pack(const P* p) {
  static_assert(sizeof(P) == 16 || sizeof(P) == 8, "pack size");
  P r;
  if constexpr (sizeof(P) == 16) {
    int4 t = __ldcs(reinterpret_cast<const int4*>(p));
    r = *reinterpret_cast<P*>(&t);
  } else {
    int2 t = __ldcs(reinterpret_cast<const int2*>(p));
    r = *reinterpret_cast<P*>(&t);
  }
  return r;
}
template <typename P> __device__ __forceinline__ void store_stream_pack(P* p, const P& v) {
  if constexpr (sizeof(P) == 16) __stcs(reinterpret_cast<int4*>(p), *reinterpret_cast<const int4*>(&v));
  else __stcs(reinterpret_cast<int2*>(p), *reinterpret_cast<const int2*>(&v));
}

template <typename S, typename D>
__global__ void __launch_bounds__(kThreads)
cast_stream_kernel(D* __restrict__ dst, const S* __restrict__ src, int64_t n) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int E = 16 / (sizeof(S) > sizeof(D) ? sizeof(S) : sizeof(D));
  constexpr int U = 8;
  const int64_t nv = n / E;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  const PackE<S, E>* in = reinterpret_cast<const PackE<S, E>*>(src);
  PackE<D, E>* out = reinterpret_cast<PackE<D, E>*>(dst);
  auto convert = [](const PackE<S, E>& p) {
    PackE<D, E> o;
#pragma unroll
    for (int k = 0; k < E; ++k) o.v[k] = store_from_math<D>(load_as_math(p.v[k]));
    return o;
  };
  int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (U - 1) * stride < nv; i += U * stride) {
    PackE<S, E> p[U];
#pragma unroll
    for (int u = 0; u < U; ++u) p[u] = load_stream_pack(in + i + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u) store_stream_pack(out + i + u * stride, convert(p[u]));
  }
  if (i < nv) {  // last, partial batch: every slot predicated, loads still issued together
    PackE<S, E> p[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < nv) p[u] = load_stream_pack(in + i + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (i + u * stride < nv) store_stream_pack(out + i + u * stride, convert(p[u]));
  }
  if (blockIdx.x == 0) {
    int64_t t = nv * E + threadIdx.x;
    if (t < n) dst[t] = store_from_math<D>(load_as_math(src[t]));
  }
}

template <typename S, typename D>
b200Status launch_cast(const b200Tensor* dst, const b200Tensor* src, cudaStream_t s) {
  const int64_t n = numel(dst);
  const b200Tensor* ts[2] = {dst, src};
  auto ix = make_indexer<2>(ts);
  bool contig = is_contiguous(dst) && is_contiguous(src);
  int grid = grid_for(n, kThreads, 8);
  launch_pdl(cast_indexed_kernel<S, D>, grid, kThreads, 0, s, static_cast<D*>(dst->data),
             static_cast<const S*>(src->data), n, ix, contig);
  return check_launch("b200_copy(cast)");
}

template <typename S>
b200Status dispatch_dst(const b200Tensor* dst, const b200Tensor* src, cudaStream_t s) {
  switch (dst->dtype) {
    case B200_F32: return launch_cast<S, float>(dst, src, s);
    case B200_BF16: return launch_cast<S, bf16_t>(dst, src, s);
    case B200_F16: return launch_cast<S, f16_t>(dst, src, s);
    case B200_F64: return launch_cast<S, double>(dst, src, s);
    case B200_I64: return launch_cast<S, int64_t>(dst, src, s);
    case B200_I32: return launch_cast<S, int32_t>(dst, src, s);
    case B200_I16: return launch_cast<S, int16_t>(dst, src, s);
    case B200_I8: return launch_cast<S, int8_t>(dst, src, s);
    case B200_U8: return launch_cast<S, uint8_t>(dst, src, s);
    case B200_BOOL: return launch_cast<S, bool_t>(dst, src, s);
    default: return fail(B200_NOT_SUPPORTED, "b200_copy: dst dtype %d", dst->dtype);
  }
}

template <typename S, typename D>
b200Status launch_stream_cast(const b200Tensor* dst, const b200Tensor* src, cudaStream_t s) {
  const int64_t n = numel(dst);
  constexpr int E = 16 / (sizeof(S) > sizeof(D) ? sizeof(S) : sizeof(D));
  int grid = wave_grid<cast_stream_kernel<S, D>>((n / E + 8 * kThreads - 1) / (8 * kThreads), kThreads, kStreamWaves);
  launch_pdl(cast_stream_kernel<S, D>, grid, kThreads, 0, s, static_cast<D*>(dst->data),
             static_cast<const S*>(src->data), n);
  return check_launch("b200_copy(cast)");
}

// Same-dtype strided copy over the widest unit both views permit.
b200Status strided_same_dtype(const b200Tensor* dst, const b200Tensor* src, cudaStream_t s) {
  const b200Tensor* ts[2] = {dst, src};
  auto ix = make_indexer<2>(ts);
  const int64_t es = static_cast<int64_t>(dtype_size(dst->dtype));
  int64_t unit = es;
  if (ix.strides[0][0] == 1 && ix.strides[1][0] == 1) {
    for (int64_t w = 16; w > es; w >>= 1) {
      bool ok = (ix.sizes[0] * es) % w == 0 &&
                reinterpret_cast<uintptr_t>(dst->data) % w == 0 &&
                reinterpret_cast<uintptr_t>(src->data) % w == 0;
      for (int d = 1; d < ix.ndim && ok; ++d)
        ok = (ix.strides[0][d] * es) % w == 0 && (ix.strides[1][d] * es) % w == 0;
      if (ok) { unit = w; break; }
    }
  }
  const int64_t ratio = unit / es;
  if (ratio > 1) {
    ix.sizes[0] /= ratio;
    for (int d = 1; d < ix.ndim; ++d) {
      ix.strides[0][d] /= ratio;
      ix.strides[1][d] /= ratio;
    }
  }
  const int64_t n = numel(dst) / ratio;
  int grid = grid_for(n, kThreads, 8);
  switch (unit) {
    case 16: launch_pdl(copy_indexed_kernel<int4>, grid, kThreads, 0, s, (int4*)dst->data, (const int4*)src->data, n, ix); break;
    case 8: launch_pdl(copy_indexed_kernel<uint64_t>, grid, kThreads, 0, s, (uint64_t*)dst->data, (const uint64_t*)src->data, n, ix); break;
    case 4: launch_pdl(copy_indexed_kernel<uint32_t>, grid, kThreads, 0, s, (uint32_t*)dst->data, (const uint32_t*)src->data, n, ix); break;
    case 2: launch_pdl(copy_indexed_kernel<uint16_t>, grid, kThreads, 0, s, (uint16_t*)dst->data, (const uint16_t*)src->data, n, ix); break;
    default: launch_pdl(copy_indexed_kernel<uint8_t>, grid, kThreads, 0, s, (uint8_t*)dst->data, (const uint8_t*)src->data, n, ix); break;
  }
  return check_launch("b200_copy(strided)");
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" b200Status b200_copy(const b200Tensor* dst, const b200Tensor* src, b200Stream stream) {
  B200_REQUIRE(valid(dst) && valid(src), B200_BAD_PARAM, "b200_copy: invalid tensor view");
  B200_REQUIRE(same_shape(dst, src), B200_BAD_PARAM, "b200_copy: src must be expanded to dst's shape");
  const int64_t n = numel(dst);
  if (n == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool contig = is_contiguous(dst) && is_contiguous(src);
  if (dst->dtype == src->dtype) {
    if (dst->data == src->data && contig) return B200_OK;
    if (contig) {
      cudaError_t e = cudaMemcpyAsync(dst->data, src->data, n * dtype_size(dst->dtype),
                                      cudaMemcpyDeviceToDevice, s);
      if (e != cudaSuccess) return fail(B200_LAUNCH_FAILED, "b200_copy: %s", cudaGetErrorString(e));
      return B200_OK;
    }
    return strided_same_dtype(dst, src, s);
  }
  if (contig && aligned16(dst->data) && aligned16(src->data)) {
    const int sd = src->dtype, dd = dst->dtype;
    if (sd == B200_F32 && dd == B200_BF16) return launch_stream_cast<float, bf16_t>(dst, src, s);
    if (sd == B200_BF16 && dd == B200_F32) return launch_stream_cast<bf16_t, float>(dst, src, s);
    if (sd == B200_F32 && dd == B200_F16) return launch_stream_cast<float, f16_t>(dst, src, s);
    if (sd == B200_F16 && dd == B200_F32) return launch_stream_cast<f16_t, float>(dst, src, s);
    if (sd == B200_BF16 && dd == B200_F16) return launch_stream_cast<bf16_t, f16_t>(dst, src, s);
    if (sd == B200_F16 && dd == B200_BF16) return launch_stream_cast<f16_t, bf16_t>(dst, src, s);
  }
  switch (src->dtype) {
    case B200_F32: return dispatch_dst<float>(dst, src, s);
    case B200_BF16: return dispatch_dst<bf16_t>(dst, src, s);
    case B200_F16: return dispatch_dst<f16_t>(dst, src, s);
    case B200_F64: return dispatch_dst<double>(dst, src, s);
    case B200_I64: return dispatch_dst<int64_t>(dst, src, s);
    case B200_I32: return dispatch_dst<int32_t>(dst, src, s);
    case B200_I16: return dispatch_dst<int16_t>(dst, src, s);
    case B200_I8: return dispatch_dst<int8_t>(dst, src, s);
    case B200_U8: return dispatch_dst<uint8_t>(dst, src, s);
    case B200_BOOL: return dispatch_dst<bool_t>(dst, src, s);
    default: return fail(B200_NOT_SUPPORTED, "b200_copy: src dtype %d", src->dtype);
  }
}
