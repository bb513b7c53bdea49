// Comparison, selection, clamping, index-of-extreme and generator kernels: the
// operators model code needs around the hot path (masks, sampling, position
// ids). All follow CPU ATen's semantics: comparisons with NaN are false (ne:
// true), maximum / minimum / clamp propagate NaN, argmax / argmin return the
// first extreme and the first NaN if there is one.
// (reference: generated aotops::eq_out / where / clamp_out / argmax_out /
// max_dim / arange_out / triu_out rows of codegen/gcu_native_functions.yaml:198-617.)
#include "common.cuh"

#include <math_constants.h>

namespace b200 {
namespace {

constexpr int kThreads = 256;

// ------------------------------------------------------------ generic map ----
// out[i] = f(a[i], b[i], c[i]) over operands of different element types, any strides.
template <typename TO, typename TA, typename TB, typename TC, typename F>
__global__ void __launch_bounds__(kThreads)
map3_kernel(TO* out, const TA* a, const TB* b, const TC* c, int64_t n, StridedIndexer<4> ix, bool contig, F f) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    if (contig) {
      out[i] = f(a[i], b ? b[i] : TB{}, c ? c[i] : TC{});
    } else {
      int64_t off[4];
      ix.offsets(i, off);
      out[off[0]] = f(a[off[1]], b ? b[off[2]] : TB{}, c ? c[off[3]] : TC{});
    }
  }
}

template <typename TO, typename TA, typename TB, typename TC, typename F>
b200Status launch_map3(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, const b200Tensor* c, F f,
                       cudaStream_t s, const char* name) {
  const int64_t n = numel(out);
  if (n == 0) return B200_OK;
  const b200Tensor* tb = b ? b : a;
  const b200Tensor* tc = c ? c : a;
  const b200Tensor* ts[4] = {out, a, tb, tc};
  auto ix = make_indexer<4>(ts);
  const bool contig = is_contiguous(out) && is_contiguous(a) && is_contiguous(tb) && is_contiguous(tc);
  map3_kernel<TO, TA, TB, TC, F><<<grid_for(n, kThreads, 16), kThreads, 0, s>>>(
      static_cast<TO*>(out->data), static_cast<const TA*>(a->data), b ? static_cast<const TB*>(b->data) : nullptr,
      c ? static_cast<const TC*>(c->data) : nullptr, n, ix, contig, f);
  return check_launch(name);
}

template <typename T> __device__ __forceinline__ typename OpMath<T>::type as_math(T v) { return load_as_math(v); }

// -------------------------------------------------------------- compare ----
template <typename T> struct CompareOp {
  int op;
  typename OpMath<T>::type scalar;
  bool use_scalar;
  __device__ uint8_t operator()(T av, T bv, T) const {
    const auto x = as_math(av);
    const auto y = use_scalar ? scalar : as_math(bv);
    switch (op) {
      case B200_CMP_EQ: return x == y;
      case B200_CMP_NE: return x != y;
      case B200_CMP_LT: return x < y;
      case B200_CMP_LE: return x <= y;
      case B200_CMP_GT: return x > y;
      case B200_CMP_GE: return x >= y;
      case B200_CMP_AND: return (x != 0) && (y != 0);
      case B200_CMP_OR: return (x != 0) || (y != 0);
      default: return (x != 0) != (y != 0);  // XOR
    }
  }
};

template <typename T>
b200Status compare_typed(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, double scalar, int op,
                         cudaStream_t s) {
  using M = typename OpMath<T>::type;
  CompareOp<T> f{op, static_cast<M>(scalar), b == nullptr};
  return launch_map3<uint8_t, T, T, T>(out, a, b, nullptr, f, s, "b200_compare");
}

b200Status compare_impl(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, double scalar, int op,
                        cudaStream_t s) {
  B200_REQUIRE(valid(out) && valid(a) && (!b || valid(b)), B200_BAD_PARAM, "b200_compare: invalid tensor view");
  B200_REQUIRE(out->dtype == B200_BOOL || out->dtype == B200_U8, B200_BAD_PARAM, "b200_compare: the output must be bool");
  B200_REQUIRE(same_shape(out, a) && (!b || (same_shape(out, b) && b->dtype == a->dtype)), B200_BAD_PARAM,
               "b200_compare: operands must be expanded to the output shape and share a dtype");
  B200_REQUIRE(op >= B200_CMP_EQ && op <= B200_CMP_XOR, B200_BAD_PARAM, "b200_compare: unknown operator %d", op);
  if (a->dtype == B200_BOOL) return compare_typed<uint8_t>(out, a, b, scalar, op, s);
  B200_DISPATCH_ARITH(a->dtype, T, { return compare_typed<T>(out, a, b, scalar, op, s); });
  return B200_OK;
}

// ---------------------------------------------------- where / masked_fill ----
template <typename U> struct SelectOp {
  __device__ U operator()(uint8_t c, U x, U y) const { return c ? x : y; }
};
template <typename U> struct MaskedFillOp {
  U value;
  __device__ U operator()(U x, uint8_t m, U) const { return m ? value : x; }
};

// The bit pattern of `v` in dtype `dt`, in the low bytes of the result.
uint64_t scalar_bits(double v, int32_t dt) {
  switch (dt) {
    case B200_F32: { float f = static_cast<float>(v); uint32_t u; memcpy(&u, &f, 4); return u; }
    case B200_F64: { uint64_t u; memcpy(&u, &v, 8); return u; }
    case B200_BF16: {
      float f = static_cast<float>(round_scalar_to_dtype(v, B200_BF16));
      uint32_t u; memcpy(&u, &f, 4);
      return (v != v) ? 0x7FC0u : (u >> 16);
    }
    case B200_F16: { __half h = __float2half_rn(static_cast<float>(v)); uint16_t u; memcpy(&u, &h, 2); return u; }
    case B200_I64: return static_cast<uint64_t>(static_cast<int64_t>(v));
    case B200_I32: return static_cast<uint32_t>(static_cast<int32_t>(v));
    case B200_I16: return static_cast<uint16_t>(static_cast<int16_t>(v));
    case B200_I8: return static_cast<uint8_t>(static_cast<int8_t>(v));
    case B200_U8: return static_cast<uint8_t>(v);
    default: return v != 0.0 ? 1u : 0u;  // bool
  }
}

// ------------------------------------------------ maximum / minimum / clamp ----
template <typename T> struct MinMaxOp {
  bool is_max;
  __device__ T operator()(T av, T bv, T) const {
    const auto x = as_math(av), y = as_math(bv);
    if (x != x) return av;   // NaN propagates
    if (y != y) return bv;
    return is_max ? (x >= y ? av : bv) : (x <= y ? av : bv);
  }
};
template <typename T> struct ClampOp {
  bool has_lo, has_hi;
  typename OpMath<T>::type lo, hi;
  __device__ T operator()(T av, T, T) const {
    auto x = as_math(av);
    if (x != x) return av;
    if (has_lo && x < lo) x = lo;
    if (has_hi && x > hi) x = hi;
    return store_from_math<T>(x);
  }
};

// ----------------------------------------------------- extreme along a dim ----
// in viewed as (outer, len, inner), contiguous; one thread per (outer, inner) when
// inner > 1, one warp per row when inner == 1.
template <typename T> struct Extreme {
  using M = typename OpMath<T>::type;
  M val;
  int64_t idx;
  bool nan;
  __device__ void init() { idx = 0; nan = false; }
  // candidate x at position j (positions visited in increasing order per thread)
  __device__ void feed(M x, int64_t j, bool is_max, bool first) {
    if (nan) return;
    if (x != x) { val = x; idx = j; nan = true; return; }
    if (first || (is_max ? x > val : x < val)) { val = x; idx = j; }
  }
  // merge another partial result; the smaller index wins ties and among NaNs
  __device__ void merge(M ov, int64_t oi, bool onan, bool is_max) {
    if (onan) {
      if (!nan || oi < idx) { val = ov; idx = oi; nan = true; }
      return;
    }
    if (nan) return;
    if ((is_max ? ov > val : ov < val) || (ov == val && oi < idx)) { val = ov; idx = oi; }
  }
};

template <typename T>
__global__ void __launch_bounds__(kThreads)
extreme_inner_kernel(T* values, int64_t* indices, const T* in, int64_t outer, int64_t len, int64_t inner, bool is_max) {
  const int64_t n = outer * inner;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    const int64_t o = i / inner, k = i - o * inner;
    const T* p = in + o * len * inner + k;
    Extreme<T> e;
    e.init();
    for (int64_t j = 0; j < len; ++j) e.feed(as_math(p[j * inner]), j, is_max, j == 0);
    if (values) values[i] = p[e.idx * inner];
    if (indices) indices[i] = e.idx;
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
extreme_row_kernel(T* values, int64_t* indices, const T* in, int64_t rows, int64_t len, bool is_max) {
  using M = typename OpMath<T>::type;
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); r < rows; r += warps) {
    const T* p = in + r * len;
    Extreme<T> e;
    e.init();
    bool any = false;
    for (int64_t j = lane; j < len; j += 32) {
      e.feed(as_math(p[j]), j, is_max, !any);
      any = true;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const M ov = __shfl_xor_sync(0xffffffffu, e.val, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, e.idx, o);
      const bool onan = __shfl_xor_sync(0xffffffffu, static_cast<int>(e.nan), o) != 0;
      const bool oany = __shfl_xor_sync(0xffffffffu, static_cast<int>(any), o) != 0;
      if (oany) {
        if (!any) { e.val = ov; e.idx = oi; e.nan = onan; any = true; }
        else e.merge(ov, oi, onan, is_max);
      }
    }
    if (lane == 0) {
      if (values) values[r] = p[e.idx];
      if (indices) indices[r] = e.idx;
    }
  }
}

// ------------------------------------------------------------ generators ----
template <typename T>
__global__ void __launch_bounds__(kThreads)
arange_kernel(T* out, int64_t n, double start, double step) {
  using M = typename OpMath<T>::type;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride)
    out[i] = store_from_math<T>(static_cast<M>(start + step * static_cast<double>(i)));
}
__global__ void __launch_bounds__(kThreads)
arange_i64_kernel(int64_t* out, int64_t n, int64_t start, int64_t step) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) out[i] = start + step * i;
}

// out = in where the element is on the kept side of the diagonal, else 0 (byte-wise).
template <typename U>
__global__ void __launch_bounds__(kThreads)
tri_kernel(U* out, const U* in, int64_t n, int64_t rows, int64_t cols, int64_t diagonal, bool upper) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    const int64_t c = i % cols, r = (i / cols) % rows;
    const bool keep = upper ? (c - r >= diagonal) : (c - r <= diagonal);
    out[i] = keep ? in[i] : U(0);
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

b200Status b200_compare(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, int32_t op, b200Stream stream) {
  B200_REQUIRE(b != nullptr, B200_BAD_PARAM, "b200_compare: second operand missing");
  return compare_impl(out, a, b, 0.0, op, static_cast<cudaStream_t>(stream));
}

b200Status b200_compare_scalar(const b200Tensor* out, const b200Tensor* a, double b, int32_t op, b200Stream stream) {
  const double bs = a && valid(a) ? round_scalar_to_dtype(b, a->dtype) : b;
  return compare_impl(out, a, nullptr, bs, op, static_cast<cudaStream_t>(stream));
}

b200Status b200_where(const b200Tensor* out, const b200Tensor* cond, const b200Tensor* a, const b200Tensor* b,
                      b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(cond) && valid(a) && valid(b), B200_BAD_PARAM, "b200_where: invalid tensor view");
  B200_REQUIRE(cond->dtype == B200_BOOL || cond->dtype == B200_U8, B200_BAD_PARAM, "b200_where: the condition must be bool");
  B200_REQUIRE(same_shape(out, cond) && same_shape(out, a) && same_shape(out, b) && a->dtype == out->dtype &&
               b->dtype == out->dtype, B200_BAD_PARAM, "b200_where: operands must be expanded to the output shape and share its dtype");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_BYTES(dtype_size(out->dtype), U, {
    return launch_map3<U, uint8_t, U, U>(out, cond, a, b, SelectOp<U>{}, s, "b200_where");
  });
  return B200_OK;
}

b200Status b200_masked_fill(const b200Tensor* out, const b200Tensor* self, const b200Tensor* mask, double value,
                            b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(self) && valid(mask), B200_BAD_PARAM, "b200_masked_fill: invalid tensor view");
  B200_REQUIRE(mask->dtype == B200_BOOL || mask->dtype == B200_U8, B200_BAD_PARAM, "b200_masked_fill: the mask must be bool");
  B200_REQUIRE(same_shape(out, self) && same_shape(out, mask) && self->dtype == out->dtype, B200_BAD_PARAM,
               "b200_masked_fill: operands must be expanded to the output shape");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint64_t bits = scalar_bits(value, out->dtype);
  B200_DISPATCH_BYTES(dtype_size(out->dtype), U, {
    return launch_map3<U, U, uint8_t, U>(out, self, mask, nullptr, MaskedFillOp<U>{static_cast<U>(bits)}, s, "b200_masked_fill");
  });
  return B200_OK;
}

b200Status b200_minmax(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, int32_t is_max, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(a) && valid(b), B200_BAD_PARAM, "b200_minmax: invalid tensor view");
  B200_REQUIRE(same_shape(out, a) && same_shape(out, b) && a->dtype == out->dtype && b->dtype == out->dtype, B200_BAD_PARAM,
               "b200_minmax: operands must be expanded to the output shape and share its dtype");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_ARITH(out->dtype, T, {
    return launch_map3<T, T, T, T>(out, a, b, nullptr, MinMaxOp<T>{is_max != 0}, s, "b200_minmax");
  });
  return B200_OK;
}

b200Status b200_clamp(const b200Tensor* out, const b200Tensor* a, int32_t has_min, double min_value, int32_t has_max,
                      double max_value, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(a), B200_BAD_PARAM, "b200_clamp: invalid tensor view");
  B200_REQUIRE(same_shape(out, a) && a->dtype == out->dtype, B200_BAD_PARAM, "b200_clamp: shape or dtype mismatch");
  B200_REQUIRE(has_min || has_max, B200_BAD_PARAM, "b200_clamp: at least one bound is required");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_ARITH(out->dtype, T, {
    using M = typename OpMath<T>::type;
    ClampOp<T> f{has_min != 0, has_max != 0, static_cast<M>(round_scalar_to_dtype(min_value, out->dtype)),
                 static_cast<M>(round_scalar_to_dtype(max_value, out->dtype))};
    return launch_map3<T, T, T, T>(out, a, nullptr, nullptr, f, s, "b200_clamp");
  });
  return B200_OK;
}

b200Status b200_extreme_dim(const b200Tensor* values, const b200Tensor* indices, const b200Tensor* in, int64_t dim,
                            int32_t is_max, b200Stream stream) {
  B200_REQUIRE(valid(in) && (values || indices), B200_BAD_PARAM, "b200_extreme_dim: invalid arguments");
  B200_REQUIRE(in->ndim >= 1 && dim >= 0 && dim < in->ndim, B200_BAD_PARAM, "b200_extreme_dim: dim out of range");
  B200_REQUIRE(is_contiguous(in), B200_NOT_SUPPORTED, "b200_extreme_dim: the input must be contiguous");
  int64_t outer = 1, inner = 1;
  const int64_t len = in->sizes[dim];
  for (int i = 0; i < dim; ++i) outer *= in->sizes[i];
  for (int i = static_cast<int>(dim) + 1; i < in->ndim; ++i) inner *= in->sizes[i];
  const int64_t n_out = outer * inner;
  B200_REQUIRE(len > 0 || n_out == 0, B200_BAD_PARAM, "b200_extreme_dim: cannot reduce over an empty dimension");
  if (values)
    B200_REQUIRE(valid(values) && values->dtype == in->dtype && numel(values) == n_out && is_contiguous(values), B200_BAD_PARAM,
                 "b200_extreme_dim: values must be contiguous, of the input's dtype, one per reduced slice");
  if (indices)
    B200_REQUIRE(valid(indices) && indices->dtype == B200_I64 && numel(indices) == n_out && is_contiguous(indices), B200_BAD_PARAM,
                 "b200_extreme_dim: indices must be contiguous int64, one per reduced slice");
  if (n_out == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int64_t* pi = indices ? static_cast<int64_t*>(indices->data) : nullptr;
  B200_DISPATCH_ARITH(in->dtype, T, {
    T* pv = values ? static_cast<T*>(values->data) : nullptr;
    const T* pin = static_cast<const T*>(in->data);
    if (inner == 1)
      extreme_row_kernel<T><<<grid_for(outer * 32, kThreads, 8), kThreads, 0, s>>>(pv, pi, pin, outer, len, is_max != 0);
    else
      extreme_inner_kernel<T><<<grid_for(n_out, kThreads, 8), kThreads, 0, s>>>(pv, pi, pin, outer, len, inner, is_max != 0);
  });
  return check_launch("b200_extreme_dim");
}

b200Status b200_arange(const b200Tensor* out, double start, double step, b200Stream stream) {
  B200_REQUIRE(valid(out) && out->ndim == 1 && is_contiguous(out), B200_BAD_PARAM, "b200_arange: the output must be 1-D contiguous");
  const int64_t n = numel(out);
  if (n == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n, kThreads, 8);
  if (out->dtype == B200_I64) {
    arange_i64_kernel<<<grid, kThreads, 0, s>>>(static_cast<int64_t*>(out->data), n, static_cast<int64_t>(start),
                                               static_cast<int64_t>(step));
    return check_launch("b200_arange");
  }
  B200_DISPATCH_ARITH(out->dtype, T, { arange_kernel<T><<<grid, kThreads, 0, s>>>(static_cast<T*>(out->data), n, start, step); });
  return check_launch("b200_arange");
}

b200Status b200_tri(const b200Tensor* out, const b200Tensor* in, int64_t diagonal, int32_t upper, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(in) && same_shape(out, in) && out->dtype == in->dtype, B200_BAD_PARAM,
               "b200_tri: shape or dtype mismatch");
  B200_REQUIRE(in->ndim >= 2 && is_contiguous(in) && is_contiguous(out), B200_NOT_SUPPORTED,
               "b200_tri: contiguous tensors of at least two dimensions");
  const int64_t n = numel(out);
  if (n == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t rows = in->sizes[in->ndim - 2], cols = in->sizes[in->ndim - 1];
  B200_DISPATCH_BYTES(dtype_size(out->dtype), U, {
    tri_kernel<U><<<grid_for(n, kThreads, 8), kThreads, 0, s>>>(static_cast<U*>(out->data), static_cast<const U*>(in->data), n,
                                                                 rows, cols, diagonal, upper != 0);
  });
  return check_launch("b200_tri");
}

}  // extern "C"
