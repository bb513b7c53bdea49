// Elementwise kernels: add / sub / mul / div (tensor and scalar operand forms),
// silu and the unary helpers an unfused decoder layer reaches.
//
// Contiguous operands take the streaming path: every thread moves 128-bit
// vectors, four per operand in flight before the first use, grid-stride over a
// whole number of waves. bf16/f16 compute in fp32 and round once on store
// (the "opmath" rule of ATen's CPU kernels). Broadcast or strided operands
// take the indexed path over the collapsed shape.
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

// ----------------------------------------------------------------- functors --
template <typename M> struct AddAlpha {
  M alpha;
  __device__ __forceinline__ M operator()(M a, M b) const { return a + alpha * b; }
};
template <> struct AddAlpha<float> {
  float alpha;
  // CPU ATen's vectorised add computes fmadd(b, alpha, a).
  __device__ __forceinline__ float operator()(float a, float b) const { return fmaf(alpha, b, a); }
};
template <> struct AddAlpha<double> {
  double alpha;
  __device__ __forceinline__ double operator()(double a, double b) const { return fma(alpha, b, a); }
};
template <typename M> struct AddPlain {
  __device__ __forceinline__ M operator()(M a, M b) const { return a + b; }
};
template <typename M> struct SubPlain {
  __device__ __forceinline__ M operator()(M a, M b) const { return a - b; }
};
template <typename M> struct Mul {
  __device__ __forceinline__ M operator()(M a, M b) const { return a * b; }
};
template <typename M> struct Div {
  __device__ __forceinline__ M operator()(M a, M b) const { return a / b; }
};
template <typename M> struct AddConst {  // a + c, c = alpha*b folded on the host
  M c;
  __device__ __forceinline__ M operator()(M a) const { return a + c; }
};
template <typename M> struct MulConst {
  M c;
  __device__ __forceinline__ M operator()(M a) const { return a * c; }
};
template <typename M> struct Silu {
  __device__ __forceinline__ M operator()(M x) const { return x / (M(1) + exp(-x)); }
};
// fp32: accurate expf (2 ulp) and the approximate division (2 ulp): within 1e-6 relative of the CPU's
// x / (1 + exp(-x)); the IEEE division it replaces made the kernel issue-bound (57 % SM throughput beside 60 %
// DRAM throughput in the profiler).
template <> struct Silu<float> {
  __device__ __forceinline__ float operator()(float x) const { return __fdividef(x, 1.0f + expf(-x)); }
};
// 16-bit I/O: fast exp / reciprocal, error far below half an output ulp.
struct SiluFast {
  __device__ __forceinline__ float operator()(float x) const { return __fdividef(x, 1.0f + __expf(-x)); }
};

template <typename M, int OP> struct Unary {
  __device__ __forceinline__ M operator()(M x) const {
    if constexpr (OP == B200_UNARY_NEG) return -x;
    else if constexpr (OP == B200_UNARY_RSQRT) return M(1) / sqrt(x);
    else if constexpr (OP == B200_UNARY_SQRT) return sqrt(x);
    else if constexpr (OP == B200_UNARY_EXP) return exp(x);
    else if constexpr (OP == B200_UNARY_SIGMOID) return M(1) / (M(1) + exp(-x));
    else if constexpr (OP == B200_UNARY_TANH) return tanh(x);
    else if constexpr (OP == B200_UNARY_RELU) return x > M(0) ? x : (x != x ? x : M(0));
    else if constexpr (OP == B200_UNARY_ABS) return fabs(x);
    else if constexpr (OP == B200_UNARY_RECIPROCAL) return M(1) / x;
    else if constexpr (OP == B200_UNARY_COS) return cos(x);
    else if constexpr (OP == B200_UNARY_SIN) return sin(x);
    else if constexpr (OP == B200_UNARY_LOG) return log(x);
    else return M(0.5) * x * (M(1) + erf(x * M(0.70710678118654752440)));
  }
};

template <typename M> struct PowConst {
  M e;
  int mode;  // 0 generic, 1 square, 2 cube, 3 sqrt, 4 rsqrt, 5 reciprocal, 6 1/x^2
  __device__ __forceinline__ M operator()(M x) const {
    switch (mode) {
      case 1: return x * x;
      case 2: return x * x * x;
      case 3: return sqrt(x);
      case 4: return M(1) / sqrt(x);
      case 5: return M(1) / x;
      case 6: return M(1) / (x * x);
      default: return pow(x, e);
    }
  }
};

// ------------------------------------------------------------------ kernels --
template <typename T, int NIN, typename F>
__global__ void __launch_bounds__(kThreads)
ew_contig_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b,
                 int64_t n, F f) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = 16 / sizeof(T);
  const int64_t nvec = n / V;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
    Vec16<T> va[kUnroll], vb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      va[u] = load_stream16(a + (i + u * stride) * V);
      if constexpr (NIN == 2) vb[u] = load_stream16(b + (i + u * stride) * V);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      Vec16<T> r;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        if constexpr (NIN == 2)
          r.v[k] = store_from_math<T>(f(load_as_math(va[u].v[k]), load_as_math(vb[u].v[k])));
        else
          r.v[k] = store_from_math<T>(f(load_as_math(va[u].v[k])));
      }
      store_stream16(out + (i + u * stride) * V, r);
    }
  }
  // last, partial batch: the same loads-then-stores shape with each slot predicated, so the
  // remainder keeps kUnroll loads in flight per thread instead of one
  if (i < nvec) {
    Vec16<T> va[kUnroll], vb[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (i + u * stride < nvec) {
        va[u] = load_stream16(a + (i + u * stride) * V);
        if constexpr (NIN == 2) vb[u] = load_stream16(b + (i + u * stride) * V);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      if (i + u * stride < nvec) {
        Vec16<T> r;
#pragma unroll
        for (int k = 0; k < V; ++k) {
          if constexpr (NIN == 2)
            r.v[k] = store_from_math<T>(f(load_as_math(va[u].v[k]), load_as_math(vb[u].v[k])));
          else
            r.v[k] = store_from_math<T>(f(load_as_math(va[u].v[k])));
        }
        store_stream16(out + (i + u * stride) * V, r);
      }
    }
  }
  // ragged tail (fewer than one vector)
  if (blockIdx.x == 0) {
    int64_t t = nvec * V + threadIdx.x;
    if (t < n) {
      if constexpr (NIN == 2) out[t] = store_from_math<T>(f(load_as_math(a[t]), load_as_math(b[t])));
      else out[t] = store_from_math<T>(f(load_as_math(a[t])));
    }
  }
}

template <typename T, int NIN, typename F>
__global__ void __launch_bounds__(kThreads)
ew_strided_kernel(T* out, const T* a, const T* b, int64_t n, StridedIndexer<NIN + 1> ix, F f) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t off[NIN + 1];
    ix.offsets(i, off);
    if constexpr (NIN == 2)
      out[off[0]] = store_from_math<T>(f(load_as_math(a[off[1]]), load_as_math(b[off[2]])));
    else
      out[off[0]] = store_from_math<T>(f(load_as_math(a[off[1]])));
  }
}

template <typename T, typename F>
b200Status launch_binary(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, F f,
                         cudaStream_t s, const char* name) {
  const int64_t n = numel(out);
  if (n == 0) return B200_OK;
  T* po = static_cast<T*>(out->data);
  const T* pa = static_cast<const T*>(a->data);
  const T* pb = static_cast<const T*>(b->data);
  if (is_contiguous(out) && is_contiguous(a) && is_contiguous(b) && aligned16(po) &&
      aligned16(pa) && aligned16(pb)) {
    constexpr int V = 16 / sizeof(T);
    int grid = wave_grid<ew_contig_kernel<T, 2, F>>((n / V + kUnroll * kThreads - 1) / (kUnroll * kThreads), kThreads, kStreamWaves);
    launch_pdl(ew_contig_kernel<T, 2, F>, grid, kThreads, 0, s, po, pa, pb, n, f);
  } else {
    const b200Tensor* ts[3] = {out, a, b};
    auto ix = make_indexer<3>(ts);
    int grid = grid_for(n, kThreads, 8);
    ew_strided_kernel<T, 2, F><<<grid, kThreads, 0, s>>>(po, pa, pb, n, ix, f);
  }
  return check_launch(name);
}

template <typename T, typename F>
b200Status launch_unary(const b200Tensor* out, const b200Tensor* a, F f, cudaStream_t s,
                        const char* name) {
  const int64_t n = numel(out);
  if (n == 0) return B200_OK;
  T* po = static_cast<T*>(out->data);
  const T* pa = static_cast<const T*>(a->data);
  if (is_contiguous(out) && is_contiguous(a) && aligned16(po) && aligned16(pa)) {
    constexpr int V = 16 / sizeof(T);
    int grid = wave_grid<ew_contig_kernel<T, 1, F>>((n / V + kUnroll * kThreads - 1) / (kUnroll * kThreads), kThreads, kStreamWaves);
    launch_pdl(ew_contig_kernel<T, 1, F>, grid, kThreads, 0, s, po, pa, static_cast<const T*>(nullptr), n, f);
  } else {
    const b200Tensor* ts[2] = {out, a};
    auto ix = make_indexer<2>(ts);
    int grid = grid_for(n, kThreads, 8);
    ew_strided_kernel<T, 1, F><<<grid, kThreads, 0, s>>>(po, pa, nullptr, n, ix, f);
  }
  return check_launch(name);
}

b200Status check_binary(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b,
                        const char* name) {
  B200_REQUIRE(valid(out) && valid(a) && valid(b), B200_BAD_PARAM, "%s: invalid tensor view", name);
  B200_REQUIRE(same_shape(out, a) && same_shape(out, b), B200_BAD_PARAM,
               "%s: operands must be expanded to the output shape", name);
  B200_REQUIRE(out->dtype == a->dtype && out->dtype == b->dtype, B200_BAD_PARAM,
               "%s: operands must share the output dtype", name);
  return B200_OK;
}
b200Status check_unary(const b200Tensor* out, const b200Tensor* a, const char* name) {
  B200_REQUIRE(valid(out) && valid(a), B200_BAD_PARAM, "%s: invalid tensor view", name);
  B200_REQUIRE(same_shape(out, a), B200_BAD_PARAM, "%s: shape mismatch", name);
  B200_REQUIRE(out->dtype == a->dtype, B200_BAD_PARAM, "%s: dtype mismatch", name);
  return B200_OK;
}

template <typename T>
__global__ void fill_kernel(T* out, int64_t n, StridedIndexer<1> ix, T value, bool contig) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
    if (contig) {
      out[i] = value;
    } else {
      int64_t off[1];
      ix.offsets(i, off);
      out[off[0]] = value;
    }
  }
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

b200Status b200_add(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, double alpha,
                    b200Stream stream) {
  b200Status st = check_binary(out, a, b, "b200_add");
  if (st != B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  alpha = round_scalar_to_dtype(alpha, out->dtype);  // ATen: alpha.to<scalar_t>()
  B200_DISPATCH_ARITH(out->dtype, T, {
    using M = typename OpMath<T>::type;
    if (alpha == 1.0) return launch_binary<T>(out, a, b, AddPlain<M>{}, s, "b200_add");
    return launch_binary<T>(out, a, b, AddAlpha<M>{static_cast<M>(alpha)}, s, "b200_add");
  });
  return B200_OK;
}

b200Status b200_sub(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, double alpha,
                    b200Stream stream) {
  b200Status st = check_binary(out, a, b, "b200_sub");
  if (st != B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  alpha = round_scalar_to_dtype(alpha, out->dtype);
  B200_DISPATCH_ARITH(out->dtype, T, {
    using M = typename OpMath<T>::type;
    if (alpha == 1.0) return launch_binary<T>(out, a, b, SubPlain<M>{}, s, "b200_sub");
    return launch_binary<T>(out, a, b, AddAlpha<M>{static_cast<M>(-alpha)}, s, "b200_sub");
  });
  return B200_OK;
}

b200Status b200_mul(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b,
                    b200Stream stream) {
  b200Status st = check_binary(out, a, b, "b200_mul");
  if (st != B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_ARITH(out->dtype, T, {
    using M = typename OpMath<T>::type;
    return launch_binary<T>(out, a, b, Mul<M>{}, s, "b200_mul");
  });
  return B200_OK;
}

b200Status b200_div(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b,
                    b200Stream stream) {
  b200Status st = check_binary(out, a, b, "b200_div");
  if (st != B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_FLOAT(out->dtype, T, {
    using M = typename OpMath<T>::type;
    return launch_binary<T>(out, a, b, Div<M>{}, s, "b200_div");
  });
  return B200_OK;
}

b200Status b200_add_scalar(const b200Tensor* out, const b200Tensor* a, double b, double alpha,
                           b200Stream stream) {
  b200Status st = check_unary(out, a, "b200_add_scalar");
  if (st != B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_ARITH(out->dtype, T, {
    using M = typename OpMath<T>::type;
    // ATen casts the wrapped scalar and alpha to the tensor's dtype, then
    // evaluates a + alpha*b in the compute type.
    M c = static_cast<M>(round_scalar_to_dtype(alpha, out->dtype)) * static_cast<M>(round_scalar_to_dtype(b, out->dtype));
    return launch_unary<T>(out, a, AddConst<M>{c}, s, "b200_add_scalar");
  });
  return B200_OK;
}

b200Status b200_mul_scalar(const b200Tensor* out, const b200Tensor* a, double b, b200Stream stream) {
  b200Status st = check_unary(out, a, "b200_mul_scalar");
  if (st != B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_ARITH(out->dtype, T, {
    using M = typename OpMath<T>::type;
    return launch_unary<T>(out, a, MulConst<M>{static_cast<M>(round_scalar_to_dtype(b, out->dtype))}, s, "b200_mul_scalar");
  });
  return B200_OK;
}

b200Status b200_silu(const b200Tensor* out, const b200Tensor* a, b200Stream stream) {
  b200Status st = check_unary(out, a, "b200_silu");
  if (st != B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_FLOAT(out->dtype, T, {
    using M = typename OpMath<T>::type;
    if constexpr (sizeof(T) == 2) return launch_unary<T>(out, a, SiluFast{}, s, "b200_silu");
    else return launch_unary<T>(out, a, Silu<M>{}, s, "b200_silu");
  });
  return B200_OK;
}

b200Status b200_unary(const b200Tensor* out, const b200Tensor* a, int32_t op, b200Stream stream) {
  b200Status st = check_unary(out, a, "b200_unary");
  if (st != B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define B200_UNARY_CASE(OP) \
  case OP: return launch_unary<T>(out, a, Unary<M, OP>{}, s, "b200_unary");
  B200_DISPATCH_FLOAT(out->dtype, T, {
    using M = typename OpMath<T>::type;
    switch (op) {
      B200_UNARY_CASE(B200_UNARY_NEG)
      B200_UNARY_CASE(B200_UNARY_RSQRT)
      B200_UNARY_CASE(B200_UNARY_SQRT)
      B200_UNARY_CASE(B200_UNARY_EXP)
      B200_UNARY_CASE(B200_UNARY_SIGMOID)
      B200_UNARY_CASE(B200_UNARY_TANH)
      B200_UNARY_CASE(B200_UNARY_RELU)
      B200_UNARY_CASE(B200_UNARY_ABS)
      B200_UNARY_CASE(B200_UNARY_RECIPROCAL)
      B200_UNARY_CASE(B200_UNARY_COS)
      B200_UNARY_CASE(B200_UNARY_SIN)
      B200_UNARY_CASE(B200_UNARY_LOG)
      B200_UNARY_CASE(B200_UNARY_GELU)
      default: return fail(B200_BAD_PARAM, "b200_unary: unknown op %d", op);
    }
  });
#undef B200_UNARY_CASE
  return B200_OK;
}

b200Status b200_pow_scalar(const b200Tensor* out, const b200Tensor* a, double e, b200Stream stream) {
  b200Status st = check_unary(out, a, "b200_pow_scalar");
  if (st != B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int mode = e == 2.0 ? 1 : e == 3.0 ? 2 : e == 0.5 ? 3 : e == -0.5 ? 4 : e == -1.0 ? 5 : e == -2.0 ? 6 : 0;
  B200_DISPATCH_FLOAT(out->dtype, T, {
    using M = typename OpMath<T>::type;
    return launch_unary<T>(out, a, PowConst<M>{static_cast<M>(e), mode}, s, "b200_pow_scalar");
  });
  return B200_OK;
}

b200Status b200_fill(const b200Tensor* out, double value, b200Stream stream) {
  B200_REQUIRE(valid(out), B200_BAD_PARAM, "b200_fill: invalid tensor view");
  const int64_t n = numel(out);
  if (n == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const b200Tensor* ts[1] = {out};
  auto ix = make_indexer<1>(ts);
  bool contig = is_contiguous(out);
  int grid = grid_for(n, 256, 8);
  switch (out->dtype) {
    case B200_F32: fill_kernel<float><<<grid, 256, 0, s>>>((float*)out->data, n, ix, (float)value, contig); break;
    case B200_F64: fill_kernel<double><<<grid, 256, 0, s>>>((double*)out->data, n, ix, value, contig); break;
    case B200_BF16: case B200_F16: {
      // round on the host exactly as the device conversion does
      float f = (float)value;
      uint32_t u;
      memcpy(&u, &f, 4);
      uint16_t bits;
      if (out->dtype == B200_BF16) {
        if ((u & 0x7fffffffu) > 0x7f800000u) bits = 0x7FC0;
        else { u += 0x7FFFu + ((u >> 16) & 1u); bits = (uint16_t)(u >> 16); }
      } else {
        __half h = __float2half_rn(f);
        memcpy(&bits, &h, 2);
      }
      fill_kernel<uint16_t><<<grid, 256, 0, s>>>((uint16_t*)out->data, n, ix, bits, contig);
      break;
    }
    case B200_I64: fill_kernel<int64_t><<<grid, 256, 0, s>>>((int64_t*)out->data, n, ix, (int64_t)value, contig); break;
    case B200_I32: fill_kernel<int32_t><<<grid, 256, 0, s>>>((int32_t*)out->data, n, ix, (int32_t)value, contig); break;
    case B200_I16: fill_kernel<int16_t><<<grid, 256, 0, s>>>((int16_t*)out->data, n, ix, (int16_t)value, contig); break;
    case B200_I8: fill_kernel<int8_t><<<grid, 256, 0, s>>>((int8_t*)out->data, n, ix, (int8_t)value, contig); break;
    case B200_U8: fill_kernel<uint8_t><<<grid, 256, 0, s>>>((uint8_t*)out->data, n, ix, (uint8_t)value, contig); break;
    case B200_BOOL: fill_kernel<uint8_t><<<grid, 256, 0, s>>>((uint8_t*)out->data, n, ix, (uint8_t)(value != 0.0), contig); break;
    default: return fail(B200_NOT_SUPPORTED, "b200_fill: dtype %d", out->dtype);
  }
  return check_launch("b200_fill");
}

b200Status b200_fill_i64(const b200Tensor* out, int64_t value, b200Stream stream) {
  B200_REQUIRE(valid(out), B200_BAD_PARAM, "b200_fill_i64: invalid tensor view");
  B200_REQUIRE(out->dtype == B200_I64, B200_BAD_PARAM, "b200_fill_i64: an int64 tensor is expected");
  const int64_t n = numel(out);
  if (n == 0) return B200_OK;
  const b200Tensor* ts[1] = {out};
  auto ix = make_indexer<1>(ts);
  fill_kernel<int64_t><<<grid_for(n, 256, 8), 256, 0, static_cast<cudaStream_t>(stream)>>>((int64_t*)out->data, n, ix, value,
                                                                                         is_contiguous(out));
  return check_launch("b200_fill_i64");
}

}  // extern "C"
