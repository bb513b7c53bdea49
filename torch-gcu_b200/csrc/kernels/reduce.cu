// Reductions over one dimension: sum / mean, softmax and layer norm.
//
// The hot layout is a contiguous (rows, N) matrix reduced along N. A row is
// read from HBM exactly once with 128-bit loads, kept in registers as fp32
// (up to 8 vectors per thread), reduced with warp shuffles plus one shared
// memory exchange, and -- for softmax and layer norm -- written back from the
// same registers, so traffic is the compulsory read (+ write). Short rows put
// several rows in one block. Anything else (reduction over an inner-strided
// dimension, rows that do not fit registers, unaligned rows, integer or fp64
// sums) takes the generic kernels at the bottom.
#include "common.cuh"

#include <math_constants.h>

namespace b200 {
namespace {

// Sum / max across the BX threads that share a row. BX <= 32: shuffles only.
template <int BX, bool IS_MAX>
__device__ __forceinline__ float row_reduce(float v, float* smem /* [rows][BX/32] */, int ty) {
  constexpr int W = BX < 32 ? BX : 32;
#pragma unroll
  for (int o = W / 2; o > 0; o >>= 1) {
    float other = __shfl_xor_sync(0xffffffffu, v, o);
    v = IS_MAX ? fmaxf(v, other) : v + other;
  }
  if constexpr (BX > 32) {
    constexpr int NW = BX / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();  // protects smem reuse between consecutive reductions
    if (lane == 0) smem[ty * NW + warp] = v;
    __syncthreads();
    float acc = smem[ty * NW];
#pragma unroll
    for (int w = 1; w < NW; ++w) acc = IS_MAX ? fmaxf(acc, smem[ty * NW + w]) : acc + smem[ty * NW + w];
    v = acc;
  }
  return v;
}

__device__ __forceinline__ void store_scalar(void* p, int32_t dtype, int64_t idx, float v) {
  switch (dtype) {
    case B200_F32: static_cast<float*>(p)[idx] = v; break;
    case B200_BF16: static_cast<uint16_t*>(p)[idx] = f32_to_bf16_bits(v); break;
    case B200_F16: static_cast<uint16_t*>(p)[idx] = f32_to_f16_bits(v); break;
    case B200_F64: static_cast<double*>(p)[idx] = v; break;
    default: break;
  }
}

// Rounds V fp32 values to TO and writes them with 128-bit streaming stores.
template <typename TO, int V>
__device__ __forceinline__ void store_vec(TO* p, const float (&y)[V]) {
  struct alignas(16) Pack { TO v[V]; } pk;
#pragma unroll
  for (int e = 0; e < V; ++e) pk.v[e] = store_from_math<TO>(y[e]);
  constexpr int NV = sizeof(Pack) / 16;
#pragma unroll
  for (int k = 0; k < NV; ++k)
    __stcs(reinterpret_cast<int4*>(p) + k, reinterpret_cast<const int4*>(&pk)[k]);
}

enum RowOp { kSum = 0, kSoftmax = 1, kLayerNorm = 2 };

struct RowArgs {
  const void* in;
  void* out;        // sum: (rows) values; softmax / layer norm: (rows, N)
  int32_t out_dtype;
  int64_t rows, N;
  float scale;      // sum: 1 or 1/N
  // layer norm
  const void* weight;
  const void* bias;
  void* mean;
  void* rstd;
  int32_t stat_dtype;
  float eps;
};

// T: input element type; TO: element type of the (rows, N) output.
template <typename T, typename TO, int BX, int VPT, int OP>
__global__ void __launch_bounds__(BX < 256 ? 256 : BX)
row_kernel(RowArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = 16 / sizeof(T);
  constexpr int ROWS = BX < 256 ? 256 / BX : 1;
  __shared__ float smem[ROWS * (BX > 32 ? BX / 32 : 1)];
  const int tx = threadIdx.x % BX, ty = threadIdx.x / BX;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * ROWS + ty;
  const bool live = row < a.rows;
  const int64_t nvec = a.N / V;
  const T* in = static_cast<const T*>(a.in) + (live ? row : 0) * a.N;

  float x[VPT][V];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int64_t vi = tx + static_cast<int64_t>(k) * BX;
    if (live && vi < nvec) {
      Vec16<T> v = load_stream16(in + vi * V);
#pragma unroll
      for (int e = 0; e < V; ++e) x[k][e] = load_as_math(v.v[e]);
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) x[k][e] = (OP == kSoftmax) ? -CUDART_INF_F : 0.0f;
    }
  }

  if constexpr (OP == kSum) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
#pragma unroll
      for (int e = 0; e < V; ++e) s += x[k][e];
    s = row_reduce<BX, false>(s, smem, ty);
    if (live && tx == 0) store_scalar(a.out, a.out_dtype, row, s * a.scale);
  } else if constexpr (OP == kSoftmax) {
    float m = -CUDART_INF_F;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
#pragma unroll
      for (int e = 0; e < V; ++e) m = fmaxf(m, x[k][e]);
    m = row_reduce<BX, true>(m, smem, ty);
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
#pragma unroll
      for (int e = 0; e < V; ++e) {
        x[k][e] = expf(x[k][e] - m);  // padding lanes: exp(-inf) = 0
        s += x[k][e];
      }
    s = row_reduce<BX, false>(s, smem, ty);
    TO* out = static_cast<TO*>(a.out) + (live ? row : 0) * a.N;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int64_t vi = tx + static_cast<int64_t>(k) * BX;
      if (live && vi < nvec) {
        float y[V];
#pragma unroll
        for (int e = 0; e < V; ++e) y[e] = x[k][e] / s;
        store_vec<TO, V>(out + vi * V, y);
      }
    }
  } else {  // layer norm
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
#pragma unroll
      for (int e = 0; e < V; ++e) s += x[k][e];
    s = row_reduce<BX, false>(s, smem, ty);
    const float mean = s / static_cast<float>(a.N);
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int64_t vi = tx + static_cast<int64_t>(k) * BX;
      if (vi < nvec) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
          float d = x[k][e] - mean;
          q += d * d;
        }
      }
    }
    q = row_reduce<BX, false>(q, smem, ty);
    const float rstd = 1.0f / sqrtf(q / static_cast<float>(a.N) + a.eps);
    TO* out = static_cast<TO*>(a.out) + (live ? row : 0) * a.N;
    const T* w = static_cast<const T*>(a.weight);
    const T* b = static_cast<const T*>(a.bias);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int64_t vi = tx + static_cast<int64_t>(k) * BX;
      if (live && vi < nvec) {
        Vec16<T> wv, bv;
        if (w) wv = load16(w + vi * V);
        if (b) bv = load16(b + vi * V);
        float y[V];
#pragma unroll
        for (int e = 0; e < V; ++e) {
          y[e] = (x[k][e] - mean) * rstd;
          if (w) y[e] *= load_as_math(wv.v[e]);
          if (b) y[e] += load_as_math(bv.v[e]);
        }
        store_vec<TO, V>(out + vi * V, y);
      }
    }
    if (live && tx == 0) {
      if (a.mean) store_scalar(a.mean, a.stat_dtype, row, mean);
      if (a.rstd) store_scalar(a.rstd, a.stat_dtype, row, rstd);
    }
  }
}

template <typename T, typename TO, int OP, int BX>
b200Status launch_row_vpt(const RowArgs& a, int vpt, cudaStream_t s) {
  constexpr int ROWS = BX < 256 ? 256 / BX : 1;
  const int threads = BX < 256 ? 256 : BX;
  const int64_t blocks = (a.rows + ROWS - 1) / ROWS;
  B200_REQUIRE(blocks <= 0x7fffffff, B200_NOT_SUPPORTED, "row kernel: too many rows");
  switch (vpt) {
    case 1: launch_pdl(row_kernel<T, TO, BX, 1, OP>, (unsigned)blocks, threads, 0, s, a); break;
    case 2: launch_pdl(row_kernel<T, TO, BX, 2, OP>, (unsigned)blocks, threads, 0, s, a); break;
    case 4: launch_pdl(row_kernel<T, TO, BX, 4, OP>, (unsigned)blocks, threads, 0, s, a); break;
    default: launch_pdl(row_kernel<T, TO, BX, 8, OP>, (unsigned)blocks, threads, 0, s, a); break;
  }
  return check_launch("row kernel");
}

// Returns false when the row shape cannot use the register-resident kernels.
template <typename T>
bool row_fast_ok(const RowArgs& a) {
  constexpr int V = 16 / sizeof(T);
  if (a.N % V != 0 || a.N == 0) return false;
  if (!aligned16(a.in)) return false;
  return a.N / V <= 1024 * 8;
}

template <typename T, typename TO, int OP>
b200Status launch_row(const RowArgs& a, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  const int64_t nvec = a.N / V;
  auto pick = [](int64_t nvec, int bx) {
    int64_t need = (nvec + bx - 1) / bx;
    return need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
  };
  if (nvec <= 32 * 2) return launch_row_vpt<T, TO, OP, 32>(a, pick(nvec, 32), s);
  if (nvec <= 256 * 8) return launch_row_vpt<T, TO, OP, 256>(a, pick(nvec, 256), s);
  return launch_row_vpt<T, TO, OP, 1024>(a, pick(nvec, 1024), s);
}

// ------------------------------------------------------------ generic paths --
template <typename T> struct AccOf { using type = int64_t; };
template <> struct AccOf<float> { using type = float; };
template <> struct AccOf<bf16_t> { using type = float; };
template <> struct AccOf<f16_t> { using type = float; };
template <> struct AccOf<double> { using type = double; };

template <typename T> __device__ __forceinline__ typename AccOf<T>::type to_acc(T v) { return v; }
template <> __device__ __forceinline__ float to_acc<bf16_t>(bf16_t v) { return bf16_bits_to_f32(v.bits); }
template <> __device__ __forceinline__ float to_acc<f16_t>(f16_t v) { return f16_bits_to_f32(v.bits); }

template <typename A>
__device__ __forceinline__ void store_acc(void* p, int32_t dtype, int64_t idx, A v) {
  switch (dtype) {
    case B200_F32: static_cast<float*>(p)[idx] = static_cast<float>(v); break;
    case B200_BF16: static_cast<uint16_t*>(p)[idx] = f32_to_bf16_bits(static_cast<float>(v)); break;
    case B200_F16: static_cast<uint16_t*>(p)[idx] = f32_to_f16_bits(static_cast<float>(v)); break;
    case B200_F64: static_cast<double*>(p)[idx] = static_cast<double>(v); break;
    case B200_I64: static_cast<int64_t*>(p)[idx] = static_cast<int64_t>(v); break;
    case B200_I32: static_cast<int32_t*>(p)[idx] = static_cast<int32_t>(v); break;
    case B200_I16: static_cast<int16_t*>(p)[idx] = static_cast<int16_t>(v); break;
    case B200_I8: static_cast<int8_t*>(p)[idx] = static_cast<int8_t>(v); break;
    case B200_U8: static_cast<uint8_t*>(p)[idx] = static_cast<uint8_t>(v); break;
    default: break;
  }
}

// in viewed as (outer, R, inner) contiguous. inner == 1: one warp per output,
// lanes stride over R. inner > 1: one thread per output, coalesced over inner.
template <typename T>
__global__ void sum_generic_kernel(const T* in, void* out, int32_t out_dtype, int64_t outer,
                                   int64_t R, int64_t inner, double scale) {
  using A = typename AccOf<T>::type;
  if (inner == 1) {
    const int lane = threadIdx.x & 31;
    const int64_t warps_per_grid = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
    for (int64_t o = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
         o < outer; o += warps_per_grid) {
      A acc = 0;
      for (int64_t r = lane; r < R; r += 32) acc += to_acc(in[o * R + r]);
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
      if (lane == 0) {
        if (scale != 1.0) acc = static_cast<A>(acc * scale);
        store_acc<A>(out, out_dtype, o, acc);
      }
    }
  } else {
    const int64_t total = outer * inner;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int64_t o = i / inner, j = i - o * inner;
      A acc = 0;
      for (int64_t r = 0; r < R; ++r) acc += to_acc(in[(o * R + r) * inner + j]);
      if (scale != 1.0) acc = static_cast<A>(acc * scale);
      store_acc<A>(out, out_dtype, i, acc);
    }
  }
}

// Full reduction to one value in two stages through a caller workspace.
template <typename T>
__global__ void __launch_bounds__(256)
sum_partial_kernel(const T* in, int64_t n, typename AccOf<T>::type* partial) {
  using A = typename AccOf<T>::type;
  __shared__ A sm[8];
  A acc = 0;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < n; i += stride)
    acc += to_acc(in[i]);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    A t = sm[0];
    for (int w = 1; w < 8; ++w) t += sm[w];
    partial[blockIdx.x] = t;
  }
}
template <typename A>
__global__ void sum_final_kernel(const A* partial, int count, void* out, int32_t out_dtype, double scale) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    A t = 0;
    for (int i = 0; i < count; ++i) t += partial[i];  // fixed order: reproducible
    if (scale != 1.0) t = static_cast<A>(t * scale);
    store_acc<A>(out, out_dtype, 0, t);
  }
}

// softmax / layer norm fallbacks over (outer, R, inner); three passes from memory.
template <typename T, typename TO>
__global__ void softmax_generic_kernel(const T* in, TO* out, int64_t outer, int64_t R, int64_t inner) {
  const int64_t total = outer * inner;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t o = i / inner, j = i - o * inner;
    const T* p = in + o * R * inner + j;
    TO* q = out + o * R * inner + j;
    float m = -CUDART_INF_F;
    for (int64_t r = 0; r < R; ++r) m = fmaxf(m, load_as_math(p[r * inner]));
    float s = 0.f;
    for (int64_t r = 0; r < R; ++r) s += expf(load_as_math(p[r * inner]) - m);
    for (int64_t r = 0; r < R; ++r) q[r * inner] = store_from_math<TO>(expf(load_as_math(p[r * inner]) - m) / s);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
layer_norm_generic_kernel(RowArgs a) {
  __shared__ float smem[8];
  const int64_t row = blockIdx.x;
  const T* in = static_cast<const T*>(a.in) + row * a.N;
  T* out = static_cast<T*>(a.out) + row * a.N;
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < a.N; i += 256) s += load_as_math(in[i]);
  s = row_reduce<256, false>(s, smem, 0);
  const float mean = s / static_cast<float>(a.N);
  float q = 0.f;
  for (int64_t i = threadIdx.x; i < a.N; i += 256) {
    float d = load_as_math(in[i]) - mean;
    q += d * d;
  }
  q = row_reduce<256, false>(q, smem, 0);
  const float rstd = 1.0f / sqrtf(q / static_cast<float>(a.N) + a.eps);
  const T* w = static_cast<const T*>(a.weight);
  const T* b = static_cast<const T*>(a.bias);
  for (int64_t i = threadIdx.x; i < a.N; i += 256) {
    float y = (load_as_math(in[i]) - mean) * rstd;
    if (w) y *= load_as_math(w[i]);
    if (b) y += load_as_math(b[i]);
    out[i] = store_from_math<T>(y);
  }
  if (threadIdx.x == 0) {
    if (a.mean) store_scalar(a.mean, a.stat_dtype, row, mean);
    if (a.rstd) store_scalar(a.rstd, a.stat_dtype, row, rstd);
  }
}

// Splits a contiguous `in` into (outer, R, inner) for the reduced dims, which
// must form one adjacent block.
bool split_dims(const b200Tensor* in, const int64_t* dims, int32_t nd, int64_t* outer, int64_t* R,
                int64_t* inner) {
  bool red[B200_MAX_DIMS] = {false};
  for (int i = 0; i < nd; ++i) {
    if (dims[i] < 0 || dims[i] >= in->ndim || red[dims[i]]) return false;
    red[dims[i]] = true;
  }
  int first = -1, last = -1;
  for (int d = 0; d < in->ndim; ++d)
    if (red[d] && in->sizes[d] != 1) {
      if (first < 0) first = d;
      last = d;
    }
  *outer = *R = *inner = 1;
  if (first < 0) {  // nothing (or only size-1 dims) reduced
    *outer = numel(in);
    return true;
  }
  for (int d = first; d <= last; ++d)
    if (!red[d] && in->sizes[d] != 1) return false;
  for (int d = 0; d < first; ++d) *outer *= in->sizes[d];
  for (int d = first; d <= last; ++d) *R *= in->sizes[d];
  for (int d = last + 1; d < in->ndim; ++d) *inner *= in->sizes[d];
  return true;
}

constexpr int64_t kFullReduceMin = 1 << 16;
constexpr int kPartialBlocks = 1184;

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

size_t b200_sum_workspace_size(const b200Tensor* in, const int64_t* dims, int32_t ndims) {
  if (!in || !valid(in)) return 0;
  int64_t outer, R, inner;
  if (!split_dims(in, dims, ndims, &outer, &R, &inner)) return 0;
  if (outer * inner == 1 && R >= kFullReduceMin) return kPartialBlocks * 8;
  return 0;
}

b200Status b200_sum(const b200Tensor* out, const b200Tensor* in, const int64_t* dims, int32_t ndims,
                    int32_t mean, void* workspace, size_t workspace_bytes, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(in), B200_BAD_PARAM, "b200_sum: invalid tensor view");
  B200_REQUIRE(ndims == 0 || dims, B200_BAD_PARAM, "b200_sum: dims is null");
  B200_REQUIRE(is_contiguous(in) && is_contiguous(out), B200_NOT_SUPPORTED,
               "b200_sum: operands must be contiguous");
  int64_t outer, R, inner;
  B200_REQUIRE(split_dims(in, dims, ndims, &outer, &R, &inner), B200_NOT_SUPPORTED,
               "b200_sum: reduced dims must be valid, unique and adjacent");
  B200_REQUIRE(numel(out) == outer * inner, B200_BAD_PARAM, "b200_sum: out has %lld elements, expected %lld",
               (long long)numel(out), (long long)(outer * inner));
  if (outer * inner == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const double scale = mean ? 1.0 / static_cast<double>(R) : 1.0;
  const bool float_in = in->dtype == B200_F32 || in->dtype == B200_BF16 || in->dtype == B200_F16;
  const bool float_out = out->dtype == B200_F32 || out->dtype == B200_BF16 || out->dtype == B200_F16;

  if (R == 0) return b200_fill(out, mean ? NAN : 0.0, stream);

  if (outer * inner == 1 && R >= kFullReduceMin) {
    B200_REQUIRE(workspace && workspace_bytes >= (size_t)kPartialBlocks * 8, B200_WORKSPACE_TOO_SMALL,
                 "b200_sum: workspace of %d bytes needed", kPartialBlocks * 8);
    int grid = grid_for(R, 256, 8);
    if (grid > kPartialBlocks) grid = kPartialBlocks;
    B200_DISPATCH_ARITH(in->dtype, T, {
      using A = typename AccOf<T>::type;
      sum_partial_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(in->data), R, static_cast<A*>(workspace));
      sum_final_kernel<A><<<1, 32, 0, s>>>(static_cast<const A*>(workspace), grid, out->data, out->dtype, scale);
    });
    return check_launch("b200_sum");
  }

  if (inner == 1 && float_in && float_out) {
    RowArgs a{};
    a.in = in->data; a.out = out->data; a.out_dtype = out->dtype;
    a.rows = outer; a.N = R; a.scale = static_cast<float>(scale);
    switch (in->dtype) {
      case B200_F32: if (row_fast_ok<float>(a)) return launch_row<float, float, kSum>(a, s); break;
      case B200_BF16: if (row_fast_ok<bf16_t>(a)) return launch_row<bf16_t, bf16_t, kSum>(a, s); break;
      default: if (row_fast_ok<f16_t>(a)) return launch_row<f16_t, f16_t, kSum>(a, s); break;
    }
  }
  B200_DISPATCH_ARITH(in->dtype, T, {
    const int64_t work = inner == 1 ? outer * 32 : outer * inner;
    int grid = grid_for(work, 256, 8);
    sum_generic_kernel<T><<<grid, 256, 0, s>>>(static_cast<const T*>(in->data), out->data, out->dtype,
                                               outer, R, inner, scale);
  });
  return check_launch("b200_sum");
}

b200Status b200_softmax(const b200Tensor* out, const b200Tensor* in, int64_t dim, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(in), B200_BAD_PARAM, "b200_softmax: invalid tensor view");
  B200_REQUIRE(same_shape(out, in), B200_BAD_PARAM, "b200_softmax: shape mismatch");
  B200_REQUIRE(is_contiguous(in) && is_contiguous(out), B200_NOT_SUPPORTED,
               "b200_softmax: operands must be contiguous");
  if (numel(in) == 0) return B200_OK;
  if (in->ndim == 0) dim = 0;
  B200_REQUIRE(in->ndim == 0 || (dim >= 0 && dim < in->ndim), B200_BAD_PARAM, "b200_softmax: dim %lld", (long long)dim);
  int64_t outer = 1, R = in->ndim ? in->sizes[dim] : 1, inner = 1;
  for (int d = 0; d < dim; ++d) outer *= in->sizes[d];
  for (int d = (int)dim + 1; d < in->ndim; ++d) inner *= in->sizes[d];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool widen_out = out->dtype == B200_F32 && in->dtype != B200_F32;
  B200_REQUIRE(out->dtype == in->dtype || widen_out, B200_BAD_PARAM,
               "b200_softmax: out dtype must equal in dtype or be f32");
  RowArgs a{};
  a.in = in->data; a.out = out->data; a.out_dtype = out->dtype; a.rows = outer; a.N = R;
  const bool out_al = aligned16(out->data);
  const int grid = grid_for(outer * inner, 128, 16);
  switch (in->dtype) {
    case B200_F32:
      if (inner == 1 && out_al && row_fast_ok<float>(a)) return launch_row<float, float, kSoftmax>(a, s);
      softmax_generic_kernel<float, float><<<grid, 128, 0, s>>>((const float*)in->data, (float*)out->data, outer, R, inner);
      break;
    case B200_BF16:
      if (widen_out) {
        if (inner == 1 && out_al && row_fast_ok<bf16_t>(a)) return launch_row<bf16_t, float, kSoftmax>(a, s);
        softmax_generic_kernel<bf16_t, float><<<grid, 128, 0, s>>>((const bf16_t*)in->data, (float*)out->data, outer, R, inner);
      } else {
        if (inner == 1 && out_al && row_fast_ok<bf16_t>(a)) return launch_row<bf16_t, bf16_t, kSoftmax>(a, s);
        softmax_generic_kernel<bf16_t, bf16_t><<<grid, 128, 0, s>>>((const bf16_t*)in->data, (bf16_t*)out->data, outer, R, inner);
      }
      break;
    case B200_F16:
      if (widen_out) {
        if (inner == 1 && out_al && row_fast_ok<f16_t>(a)) return launch_row<f16_t, float, kSoftmax>(a, s);
        softmax_generic_kernel<f16_t, float><<<grid, 128, 0, s>>>((const f16_t*)in->data, (float*)out->data, outer, R, inner);
      } else {
        if (inner == 1 && out_al && row_fast_ok<f16_t>(a)) return launch_row<f16_t, f16_t, kSoftmax>(a, s);
        softmax_generic_kernel<f16_t, f16_t><<<grid, 128, 0, s>>>((const f16_t*)in->data, (f16_t*)out->data, outer, R, inner);
      }
      break;
    default:
      return fail(B200_NOT_SUPPORTED, "b200_softmax: dtype %d", in->dtype);
  }
  return check_launch("b200_softmax");
}

b200Status b200_native_layer_norm(const b200Tensor* out, const b200Tensor* mean, const b200Tensor* rstd,
                                  const b200Tensor* in, int64_t M, int64_t N, const b200Tensor* weight,
                                  const b200Tensor* bias, double eps, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(in), B200_BAD_PARAM, "b200_native_layer_norm: invalid tensor view");
  B200_REQUIRE(is_contiguous(in) && is_contiguous(out), B200_NOT_SUPPORTED,
               "b200_native_layer_norm: in/out must be contiguous");
  B200_REQUIRE(out->dtype == in->dtype, B200_BAD_PARAM, "b200_native_layer_norm: out dtype");
  B200_REQUIRE(M >= 0 && N >= 0 && numel(in) == M * N && numel(out) == M * N, B200_BAD_PARAM,
               "b200_native_layer_norm: M*N does not match the tensors");
  if (weight) B200_REQUIRE(valid(weight) && numel(weight) == N && is_contiguous(weight) && weight->dtype == in->dtype,
                           B200_BAD_PARAM, "b200_native_layer_norm: weight must be N contiguous elements of in's dtype");
  if (bias) B200_REQUIRE(valid(bias) && numel(bias) == N && is_contiguous(bias) && bias->dtype == in->dtype,
                         B200_BAD_PARAM, "b200_native_layer_norm: bias must be N contiguous elements of in's dtype");
  RowArgs a{};
  a.in = in->data; a.out = out->data; a.out_dtype = out->dtype; a.rows = M; a.N = N;
  a.weight = weight ? weight->data : nullptr;
  a.bias = bias ? bias->data : nullptr;
  a.eps = static_cast<float>(eps);
  if (mean) {
    B200_REQUIRE(valid(mean) && numel(mean) == M && is_contiguous(mean), B200_BAD_PARAM, "b200_native_layer_norm: mean");
    a.mean = mean->data; a.stat_dtype = mean->dtype;
  }
  if (rstd) {
    B200_REQUIRE(valid(rstd) && numel(rstd) == M && is_contiguous(rstd), B200_BAD_PARAM, "b200_native_layer_norm: rstd");
    B200_REQUIRE(!mean || mean->dtype == rstd->dtype, B200_BAD_PARAM, "b200_native_layer_norm: mean/rstd dtype differ");
    a.rstd = rstd->data; a.stat_dtype = rstd->dtype;
  }
  if (M == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (N == 0) {  // CPU ATen: mean = 0 is not defined; it writes nan mean / rstd of eps. Keep ATen's: mean nan.
    if (mean) { b200Status st = b200_fill(mean, NAN, stream); if (st) return st; }
    if (rstd) { b200Status st = b200_fill(rstd, NAN, stream); if (st) return st; }
    return B200_OK;
  }
  const bool al = aligned16(out->data) && (!a.weight || aligned16(a.weight)) && (!a.bias || aligned16(a.bias));
  B200_REQUIRE(M <= 0x7fffffff, B200_NOT_SUPPORTED, "b200_native_layer_norm: M too large");
  switch (in->dtype) {
    case B200_F32:
      if (al && row_fast_ok<float>(a)) return launch_row<float, float, kLayerNorm>(a, s);
      layer_norm_generic_kernel<float><<<(unsigned)M, 256, 0, s>>>(a);
      break;
    case B200_BF16:
      if (al && row_fast_ok<bf16_t>(a)) return launch_row<bf16_t, bf16_t, kLayerNorm>(a, s);
      layer_norm_generic_kernel<bf16_t><<<(unsigned)M, 256, 0, s>>>(a);
      break;
    case B200_F16:
      if (al && row_fast_ok<f16_t>(a)) return launch_row<f16_t, f16_t, kLayerNorm>(a, s);
      layer_norm_generic_kernel<f16_t><<<(unsigned)M, 256, 0, s>>>(a);
      break;
    default:
      return fail(B200_NOT_SUPPORTED, "b200_native_layer_norm: dtype %d", in->dtype);
  }
  return check_launch("b200_native_layer_norm");
}

}  // extern "C"
