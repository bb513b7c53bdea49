// Backward kernels of the decoder layer's pointwise and row operators:
// silu_backward, _softmax_backward_data, native_layer_norm_backward (the
// embedding backward is the ordered scatter of index.cu). fp32 math, one rounding
// per output; reductions over rows are taken in a fixed order, so results do not
// depend on timing. (reference: yaml rows silu_backward.grad_input,
// _softmax_backward_data.out, native_layer_norm_backward of
// codegen/gcu_native_functions.yaml, which the reference's S60 build sends to the
// CPU: codegen/gcu_op_fallback.yaml:8-50.)
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) t += sh[w];
  return t;
}

// ------------------------------------------------------------ silu backward ----
template <typename T>
__global__ void __launch_bounds__(kThreads)
silu_backward_kernel(T* dx, const T* g, const T* x, int64_t n, StridedIndexer<3> ix, bool contig) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < n; i += stride) {
    int64_t off[3] = {i, i, i};
    if (!contig) ix.offsets(i, off);
    const float xv = static_cast<float>(load_as_math(x[off[2]])), gv = static_cast<float>(load_as_math(g[off[1]]));
    const float s = 1.0f / (1.0f + expf(-xv));
    dx[off[0]] = store_from_math<T>(static_cast<typename OpMath<T>::type>(gv * s * (1.0f + xv * (1.0f - s))));
  }
}

// --------------------------------------------------------- softmax backward ----
// dx = y * (g - sum_r(g * y)) over (outer, R, inner); one block per (outer, inner) slice.
template <typename T>
__global__ void __launch_bounds__(kThreads)
softmax_backward_kernel(T* dx, const T* g, const T* y, int64_t R, int64_t inner) {
  __shared__ float sh[kThreads / 32];
  const int64_t o = blockIdx.x / inner, k = blockIdx.x - o * inner;
  const int64_t base = o * R * inner + k;
  float acc = 0.f;
  for (int64_t r = threadIdx.x; r < R; r += kThreads)
    acc += static_cast<float>(load_as_math(g[base + r * inner])) * static_cast<float>(load_as_math(y[base + r * inner]));
  const float dot = block_sum(acc, sh);
  for (int64_t r = threadIdx.x; r < R; r += kThreads) {
    const float gv = static_cast<float>(load_as_math(g[base + r * inner])), yv = static_cast<float>(load_as_math(y[base + r * inner]));
    dx[base + r * inner] = store_from_math<T>(static_cast<typename OpMath<T>::type>(yv * (gv - dot)));
  }
}

// ------------------------------------------------------ layer norm backward ----
// dx row r: xhat = (x - mean) * rstd, gw = g * w:
//   dx = rstd * (gw - mean_N(gw) - xhat * mean_N(gw * xhat))
template <typename T>
__global__ void __launch_bounds__(kThreads)
layer_norm_dx_kernel(T* dx, const T* g, const T* x, const float* mean, const float* rstd, const T* w, int64_t N) {
  __shared__ float sh[kThreads / 32];
  const int64_t r = blockIdx.x;
  const float mu = mean[r], rs = rstd[r];
  const T* gr = g + r * N;
  const T* xr = x + r * N;
  float s1 = 0.f, s2 = 0.f;
  for (int64_t c = threadIdx.x; c < N; c += kThreads) {
    const float gw = static_cast<float>(load_as_math(gr[c])) * (w ? static_cast<float>(load_as_math(w[c])) : 1.0f);
    const float xh = (static_cast<float>(load_as_math(xr[c])) - mu) * rs;
    s1 += gw;
    s2 += gw * xh;
  }
  const float m1 = block_sum(s1, sh) / static_cast<float>(N);
  const float m2 = block_sum(s2, sh) / static_cast<float>(N);
  for (int64_t c = threadIdx.x; c < N; c += kThreads) {
    const float gw = static_cast<float>(load_as_math(gr[c])) * (w ? static_cast<float>(load_as_math(w[c])) : 1.0f);
    const float xh = (static_cast<float>(load_as_math(xr[c])) - mu) * rs;
    dx[r * N + c] = store_from_math<T>(static_cast<typename OpMath<T>::type>(rs * (gw - m1 - xh * m2)));
  }
}

// Column sums in two ordered stages: partial[chunk][c] over a band of rows, then over the chunks.
constexpr int kRowsPerChunk = 256;
template <typename T>
__global__ void __launch_bounds__(kThreads)
layer_norm_dwdb_partial_kernel(float* pw, float* pb, const T* g, const T* x, const float* mean, const float* rstd,
                               int64_t M, int64_t N) {
  // block: 32 columns x 8 row lanes
  __shared__ float sw[8][33], sb[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int64_t c = static_cast<int64_t>(blockIdx.x) * 32 + cx;
  const int64_t r0 = static_cast<int64_t>(blockIdx.y) * kRowsPerChunk;
  const int64_t r1 = min(M, r0 + kRowsPerChunk);
  float aw = 0.f, ab = 0.f;
  if (c < N) {
    for (int64_t r = r0 + ry; r < r1; r += 8) {
      const float gv = static_cast<float>(load_as_math(g[r * N + c]));
      const float xh = (static_cast<float>(load_as_math(x[r * N + c])) - mean[r]) * rstd[r];
      aw += gv * xh;
      ab += gv;
    }
  }
  sw[ry][cx] = aw;
  sb[ry][cx] = ab;
  __syncthreads();
  if (ry == 0 && c < N) {
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { tw += sw[k][cx]; tb += sb[k][cx]; }
    pw[static_cast<int64_t>(blockIdx.y) * N + c] = tw;
    pb[static_cast<int64_t>(blockIdx.y) * N + c] = tb;
  }
}
template <typename T>
__global__ void __launch_bounds__(kThreads)
layer_norm_dwdb_final_kernel(T* dw, T* db, const float* pw, const float* pb, int64_t chunks, int64_t N) {
  const int64_t c = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (c >= N) return;
  float tw = 0.f, tb = 0.f;
  for (int64_t k = 0; k < chunks; ++k) { tw += pw[k * N + c]; tb += pb[k * N + c]; }
  using M = typename OpMath<T>::type;
  if (dw) dw[c] = store_from_math<T>(static_cast<M>(tw));
  if (db) db[c] = store_from_math<T>(static_cast<M>(tb));
}

// ----------------------------------------------- log-softmax and NLL loss ----
// y = x - max - log(sum exp(x - max)) over (outer, R, inner); one block per slice.
template <typename T>
__global__ void __launch_bounds__(kThreads)
log_softmax_kernel(T* y, const T* x, int64_t R, int64_t inner) {
  __shared__ float sh[kThreads / 32];
  const int64_t o = blockIdx.x / inner, k = blockIdx.x - o * inner;
  const int64_t base = o * R * inner + k;
  float mx = -INFINITY;
  for (int64_t r = threadIdx.x; r < R; r += kThreads) mx = fmaxf(mx, static_cast<float>(load_as_math(x[base + r * inner])));
  mx = warp_max(mx);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = sh[0];
#pragma unroll
  for (int w = 1; w < kThreads / 32; ++w) mx = fmaxf(mx, sh[w]);
  const float m0 = mx == -INFINITY ? 0.f : mx;
  float acc = 0.f;
  for (int64_t r = threadIdx.x; r < R; r += kThreads) acc += expf(static_cast<float>(load_as_math(x[base + r * inner])) - m0);
  const float lse = m0 + logf(block_sum(acc, sh));
  for (int64_t r = threadIdx.x; r < R; r += kThreads)
    y[base + r * inner] = store_from_math<T>(static_cast<typename OpMath<T>::type>(static_cast<float>(load_as_math(x[base + r * inner])) - lse));
}

// dx = g - exp(y) * sum_r(g)
template <typename T>
__global__ void __launch_bounds__(kThreads)
log_softmax_backward_kernel(T* dx, const T* g, const T* y, int64_t R, int64_t inner) {
  __shared__ float sh[kThreads / 32];
  const int64_t o = blockIdx.x / inner, k = blockIdx.x - o * inner;
  const int64_t base = o * R * inner + k;
  float acc = 0.f;
  for (int64_t r = threadIdx.x; r < R; r += kThreads) acc += static_cast<float>(load_as_math(g[base + r * inner]));
  const float tot = block_sum(acc, sh);
  for (int64_t r = threadIdx.x; r < R; r += kThreads) {
    const float gv = static_cast<float>(load_as_math(g[base + r * inner])), yv = static_cast<float>(load_as_math(y[base + r * inner]));
    dx[base + r * inner] = store_from_math<T>(static_cast<typename OpMath<T>::type>(gv - expf(yv) * tot));
  }
}

// Negative log-likelihood over (N, C) log-probabilities: one block, rows added in a fixed order.
// reduction: 0 none (loss per row), 1 mean, 2 sum. total_weight (1 element) always written.
template <typename T>
__global__ void __launch_bounds__(1024)
nll_loss_kernel(T* out, T* total_weight, const T* logp, const int64_t* target, const T* weight, int64_t N, int64_t C,
                int reduction, int64_t ignore_index, unsigned int* error_word) {
  __shared__ float s_loss[32], s_w[32];
  float loss = 0.f, wsum = 0.f;
  for (int64_t i = threadIdx.x; i < N; i += 1024) {
    const int64_t t = target[i];
    float li = 0.f, wi = 0.f;
    if (t != ignore_index) {
      if (t < 0 || t >= C) {
        atomicOr(error_word, 1u);
      } else {
        wi = weight ? static_cast<float>(load_as_math(weight[t])) : 1.f;
        li = -wi * static_cast<float>(load_as_math(logp[i * C + t]));
      }
    }
    if (reduction == 0) out[i] = store_from_math<T>(static_cast<typename OpMath<T>::type>(li));
    loss += li;
    wsum += wi;
  }
  loss = warp_sum(loss);
  wsum = warp_sum(wsum);
  if ((threadIdx.x & 31) == 0) { s_loss[threadIdx.x >> 5] = loss; s_w[threadIdx.x >> 5] = wsum; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float l = 0.f, w = 0.f;
    for (int k = 0; k < 32; ++k) { l += s_loss[k]; w += s_w[k]; }
    using M = typename OpMath<T>::type;
    *total_weight = store_from_math<T>(static_cast<M>(w));
    if (reduction == 1) out[0] = store_from_math<T>(static_cast<M>(l / w));
    else if (reduction == 2) out[0] = store_from_math<T>(static_cast<M>(l));
  }
}

// grad_input (N, C), zero-filled by the caller: entry (i, target[i]) = -w * g (/ total_weight for mean)
template <typename T>
__global__ void __launch_bounds__(kThreads)
nll_loss_backward_kernel(T* grad_in, const T* grad_out, const int64_t* target, const T* weight, const T* total_weight, int64_t N,
                         int64_t C, int reduction, int64_t ignore_index) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; i < N; i += stride) {
    const int64_t t = target[i];
    if (t == ignore_index || t < 0 || t >= C) continue;
    const float w = weight ? static_cast<float>(load_as_math(weight[t])) : 1.f;
    float g = static_cast<float>(load_as_math(grad_out[reduction == 0 ? i : 0]));
    if (reduction == 1) g /= static_cast<float>(load_as_math(total_weight[0]));
    grad_in[i * C + t] = store_from_math<T>(static_cast<typename OpMath<T>::type>(-w * g));
  }
}

inline bool float_dtype(int32_t d) { return d == B200_F32 || d == B200_BF16 || d == B200_F16; }

}  // namespace

unsigned int* device_error_word();
}  // namespace b200

using namespace b200;

#define B200_DISPATCH_F3(DT, T, ...)                                   \
  switch (DT) {                                                        \
    case B200_F32: { using T = float; __VA_ARGS__; break; }            \
    case B200_BF16: { using T = ::b200::bf16_t; __VA_ARGS__; break; }  \
    default: { using T = ::b200::f16_t; __VA_ARGS__; break; }          \
  }

extern "C" {

b200Status b200_silu_backward(const b200Tensor* grad_in, const b200Tensor* grad_out, const b200Tensor* x, b200Stream stream) {
  B200_REQUIRE(valid(grad_in) && valid(grad_out) && valid(x), B200_BAD_PARAM, "b200_silu_backward: invalid tensor view");
  B200_REQUIRE(same_shape(grad_in, grad_out) && same_shape(grad_in, x) && grad_out->dtype == grad_in->dtype &&
               x->dtype == grad_in->dtype, B200_BAD_PARAM, "b200_silu_backward: operands must share shape and dtype");
  B200_REQUIRE(float_dtype(grad_in->dtype), B200_NOT_SUPPORTED, "b200_silu_backward: f32, bf16 or f16");
  const int64_t n = numel(grad_in);
  if (n == 0) return B200_OK;
  const b200Tensor* ts[3] = {grad_in, grad_out, x};
  auto ix = make_indexer<3>(ts);
  const bool contig = is_contiguous(grad_in) && is_contiguous(grad_out) && is_contiguous(x);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_F3(grad_in->dtype, T, {
    silu_backward_kernel<T><<<grid_for(n, kThreads, 16), kThreads, 0, s>>>(static_cast<T*>(grad_in->data),
        static_cast<const T*>(grad_out->data), static_cast<const T*>(x->data), n, ix, contig);
  });
  return check_launch("b200_silu_backward");
}

b200Status b200_softmax_backward(const b200Tensor* grad_in, const b200Tensor* grad_out, const b200Tensor* output, int64_t dim,
                                 b200Stream stream) {
  B200_REQUIRE(valid(grad_in) && valid(grad_out) && valid(output), B200_BAD_PARAM, "b200_softmax_backward: invalid tensor view");
  B200_REQUIRE(same_shape(grad_in, grad_out) && same_shape(grad_in, output) && grad_out->dtype == grad_in->dtype &&
               output->dtype == grad_in->dtype, B200_BAD_PARAM, "b200_softmax_backward: operands must share shape and dtype");
  B200_REQUIRE(float_dtype(grad_in->dtype), B200_NOT_SUPPORTED, "b200_softmax_backward: f32, bf16 or f16");
  B200_REQUIRE(is_contiguous(grad_in) && is_contiguous(grad_out) && is_contiguous(output), B200_NOT_SUPPORTED,
               "b200_softmax_backward: operands must be contiguous");
  if (numel(grad_in) == 0) return B200_OK;
  if (grad_in->ndim == 0) dim = 0;
  B200_REQUIRE(grad_in->ndim == 0 || (dim >= 0 && dim < grad_in->ndim), B200_BAD_PARAM, "b200_softmax_backward: dim out of range");
  int64_t outer = 1, R = grad_in->ndim ? grad_in->sizes[dim] : 1, inner = 1;
  for (int d = 0; d < dim; ++d) outer *= grad_in->sizes[d];
  for (int d = static_cast<int>(dim) + 1; d < grad_in->ndim; ++d) inner *= grad_in->sizes[d];
  B200_REQUIRE(outer * inner <= 0x7fffffff, B200_NOT_SUPPORTED, "b200_softmax_backward: too many slices");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_F3(grad_in->dtype, T, {
    softmax_backward_kernel<T><<<static_cast<unsigned>(outer * inner), kThreads, 0, s>>>(
        static_cast<T*>(grad_in->data), static_cast<const T*>(grad_out->data), static_cast<const T*>(output->data), R, inner);
  });
  return check_launch("b200_softmax_backward");
}

static b200Status log_softmax_common(const b200Tensor* out, const b200Tensor* a, const b200Tensor* b, int64_t dim, bool backward,
                                     cudaStream_t s, const char* name) {
  B200_REQUIRE(valid(out) && valid(a) && (!b || valid(b)), B200_BAD_PARAM, "%s: invalid tensor view", name);
  B200_REQUIRE(same_shape(out, a) && a->dtype == out->dtype && (!b || (same_shape(out, b) && b->dtype == out->dtype)), B200_BAD_PARAM,
               "%s: operands must share shape and dtype", name);
  B200_REQUIRE(float_dtype(out->dtype), B200_NOT_SUPPORTED, "%s: f32, bf16 or f16", name);
  B200_REQUIRE(is_contiguous(out) && is_contiguous(a) && (!b || is_contiguous(b)), B200_NOT_SUPPORTED, "%s: operands must be contiguous", name);
  if (numel(out) == 0) return B200_OK;
  if (out->ndim == 0) dim = 0;
  B200_REQUIRE(out->ndim == 0 || (dim >= 0 && dim < out->ndim), B200_BAD_PARAM, "%s: dim out of range", name);
  int64_t outer = 1, R = out->ndim ? out->sizes[dim] : 1, inner = 1;
  for (int d = 0; d < dim; ++d) outer *= out->sizes[d];
  for (int d = static_cast<int>(dim) + 1; d < out->ndim; ++d) inner *= out->sizes[d];
  B200_REQUIRE(outer * inner <= 0x7fffffff, B200_NOT_SUPPORTED, "%s: too many slices", name);
  B200_DISPATCH_F3(out->dtype, T, {
    if (backward)
      log_softmax_backward_kernel<T><<<static_cast<unsigned>(outer * inner), kThreads, 0, s>>>(
          static_cast<T*>(out->data), static_cast<const T*>(a->data), static_cast<const T*>(b->data), R, inner);
    else
      log_softmax_kernel<T><<<static_cast<unsigned>(outer * inner), kThreads, 0, s>>>(static_cast<T*>(out->data),
                                                                                       static_cast<const T*>(a->data), R, inner);
  });
  return check_launch(name);
}

b200Status b200_log_softmax(const b200Tensor* out, const b200Tensor* in, int64_t dim, b200Stream stream) {
  return log_softmax_common(out, in, nullptr, dim, false, static_cast<cudaStream_t>(stream), "b200_log_softmax");
}

b200Status b200_log_softmax_backward(const b200Tensor* grad_in, const b200Tensor* grad_out, const b200Tensor* output, int64_t dim,
                                     b200Stream stream) {
  B200_REQUIRE(output != nullptr, B200_BAD_PARAM, "b200_log_softmax_backward: output missing");
  return log_softmax_common(grad_in, grad_out, output, dim, true, static_cast<cudaStream_t>(stream), "b200_log_softmax_backward");
}

b200Status b200_nll_loss(const b200Tensor* out, const b200Tensor* total_weight, const b200Tensor* logp, const b200Tensor* target,
                         const b200Tensor* weight, int32_t reduction, int64_t ignore_index, b200Stream stream) {
  const char* name = "b200_nll_loss";
  B200_REQUIRE(valid(out) && valid(total_weight) && valid(logp) && valid(target), B200_BAD_PARAM, "%s: invalid tensor view", name);
  B200_REQUIRE(logp->ndim == 2 && target->ndim == 1 && target->sizes[0] == logp->sizes[0] && target->dtype == B200_I64, B200_BAD_PARAM,
               "%s: log-probabilities (N, C) and int64 targets (N) expected", name);
  B200_REQUIRE(float_dtype(logp->dtype) && out->dtype == logp->dtype && total_weight->dtype == logp->dtype, B200_BAD_PARAM,
               "%s: out and total_weight must have the input's floating dtype", name);
  B200_REQUIRE(is_contiguous(logp) && is_contiguous(target) && is_contiguous(out), B200_NOT_SUPPORTED, "%s: operands must be contiguous", name);
  B200_REQUIRE(reduction >= 0 && reduction <= 2, B200_BAD_PARAM, "%s: reduction must be 0 (none), 1 (mean) or 2 (sum)", name);
  const int64_t N = logp->sizes[0], C = logp->sizes[1];
  B200_REQUIRE(numel(out) == (reduction == 0 ? N : 1) && numel(total_weight) == 1, B200_BAD_PARAM, "%s: output sizes", name);
  if (weight) B200_REQUIRE(valid(weight) && weight->dtype == logp->dtype && numel(weight) == C && is_contiguous(weight), B200_BAD_PARAM,
                           "%s: weight must be C contiguous elements of the input's dtype", name);
  unsigned int* ew = device_error_word();
  B200_REQUIRE(ew, B200_LAUNCH_FAILED, "%s: device error word unavailable", name);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_F3(logp->dtype, T, {
    nll_loss_kernel<T><<<1, 1024, 0, s>>>(static_cast<T*>(out->data), static_cast<T*>(total_weight->data),
                                          static_cast<const T*>(logp->data), static_cast<const int64_t*>(target->data),
                                          weight ? static_cast<const T*>(weight->data) : nullptr, N, C, reduction, ignore_index, ew);
  });
  return check_launch(name);
}

b200Status b200_nll_loss_backward(const b200Tensor* grad_in, const b200Tensor* grad_out, const b200Tensor* target,
                                  const b200Tensor* weight, const b200Tensor* total_weight, int32_t reduction, int64_t ignore_index,
                                  b200Stream stream) {
  const char* name = "b200_nll_loss_backward";
  B200_REQUIRE(valid(grad_in) && valid(grad_out) && valid(target) && valid(total_weight), B200_BAD_PARAM, "%s: invalid tensor view", name);
  B200_REQUIRE(grad_in->ndim == 2 && target->ndim == 1 && target->sizes[0] == grad_in->sizes[0] && target->dtype == B200_I64,
               B200_BAD_PARAM, "%s: grad_input (N, C) and int64 targets (N) expected", name);
  B200_REQUIRE(float_dtype(grad_in->dtype) && grad_out->dtype == grad_in->dtype && total_weight->dtype == grad_in->dtype, B200_BAD_PARAM,
               "%s: operands must share one floating dtype", name);
  B200_REQUIRE(is_contiguous(grad_in) && is_contiguous(target) && is_contiguous(grad_out), B200_NOT_SUPPORTED, "%s: operands must be contiguous", name);
  const int64_t N = grad_in->sizes[0], C = grad_in->sizes[1];
  B200_REQUIRE(numel(grad_out) == (reduction == 0 ? N : 1), B200_BAD_PARAM, "%s: grad_output size", name);
  if (weight) B200_REQUIRE(valid(weight) && weight->dtype == grad_in->dtype && numel(weight) == C && is_contiguous(weight), B200_BAD_PARAM,
                           "%s: weight must be C contiguous elements", name);
  if (N == 0 || C == 0) return B200_OK;
  b200Status st = b200_fill(grad_in, 0.0, stream);
  if (st != B200_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_F3(grad_in->dtype, T, {
    nll_loss_backward_kernel<T><<<grid_for(N, kThreads, 8), kThreads, 0, s>>>(
        static_cast<T*>(grad_in->data), static_cast<const T*>(grad_out->data), static_cast<const int64_t*>(target->data),
        weight ? static_cast<const T*>(weight->data) : nullptr, static_cast<const T*>(total_weight->data), N, C, reduction, ignore_index);
  });
  return check_launch(name);
}

size_t b200_layer_norm_backward_workspace_size(int64_t M, int64_t N) {
  const int64_t chunks = (M + kRowsPerChunk - 1) / kRowsPerChunk;
  return static_cast<size_t>(2 * chunks * N) * sizeof(float) + 256;
}

b200Status b200_layer_norm_backward(const b200Tensor* dx, const b200Tensor* dweight, const b200Tensor* dbias,
                                    const b200Tensor* grad_out, const b200Tensor* x, const b200Tensor* mean,
                                    const b200Tensor* rstd, const b200Tensor* weight, int64_t M, int64_t N,
                                    void* workspace, size_t workspace_bytes, b200Stream stream) {
  B200_REQUIRE(valid(grad_out) && valid(x) && valid(mean) && valid(rstd), B200_BAD_PARAM, "b200_layer_norm_backward: invalid tensor view");
  B200_REQUIRE(float_dtype(x->dtype) && grad_out->dtype == x->dtype, B200_NOT_SUPPORTED, "b200_layer_norm_backward: f32, bf16 or f16");
  B200_REQUIRE(is_contiguous(grad_out) && is_contiguous(x) && numel(grad_out) == M * N && numel(x) == M * N, B200_BAD_PARAM,
               "b200_layer_norm_backward: grad_out and x must be contiguous M x N");
  B200_REQUIRE(mean->dtype == B200_F32 && rstd->dtype == B200_F32 && numel(mean) == M && numel(rstd) == M && is_contiguous(mean) &&
               is_contiguous(rstd), B200_BAD_PARAM, "b200_layer_norm_backward: mean and rstd must be contiguous f32 of M elements");
  if (weight) B200_REQUIRE(valid(weight) && weight->dtype == x->dtype && numel(weight) == N && is_contiguous(weight), B200_BAD_PARAM,
                           "b200_layer_norm_backward: weight must be N contiguous elements of x's dtype");
  for (const b200Tensor* t : {dweight, dbias})
    if (t) B200_REQUIRE(valid(t) && t->dtype == x->dtype && numel(t) == N && is_contiguous(t), B200_BAD_PARAM,
                        "b200_layer_norm_backward: dweight / dbias must be N contiguous elements of x's dtype");
  if (dx) B200_REQUIRE(valid(dx) && dx->dtype == x->dtype && numel(dx) == M * N && is_contiguous(dx), B200_BAD_PARAM,
                       "b200_layer_norm_backward: dx must be contiguous M x N of x's dtype");
  B200_REQUIRE(M <= 0x7fffffff, B200_NOT_SUPPORTED, "b200_layer_norm_backward: M too large");
  if (N == 0) return B200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float* pm = static_cast<const float*>(mean->data);
  const float* pr = static_cast<const float*>(rstd->data);
  if (M == 0) {
    if (dweight) { b200Status st = b200_fill(dweight, 0.0, stream); if (st) return st; }
    if (dbias) { b200Status st = b200_fill(dbias, 0.0, stream); if (st) return st; }
    return B200_OK;
  }
  B200_DISPATCH_F3(x->dtype, T, {
    if (dx)
      layer_norm_dx_kernel<T><<<static_cast<unsigned>(M), kThreads, 0, s>>>(static_cast<T*>(dx->data),
          static_cast<const T*>(grad_out->data), static_cast<const T*>(x->data), pm, pr,
          weight ? static_cast<const T*>(weight->data) : nullptr, N);
    if (dweight || dbias) {
      const int64_t chunks = (M + kRowsPerChunk - 1) / kRowsPerChunk;
      B200_REQUIRE(workspace && workspace_bytes >= b200_layer_norm_backward_workspace_size(M, N) &&
                   reinterpret_cast<uintptr_t>(workspace) % 256 == 0, B200_WORKSPACE_TOO_SMALL,
                   "b200_layer_norm_backward: workspace of %zu bytes (256-byte aligned) required",
                   b200_layer_norm_backward_workspace_size(M, N));
      B200_REQUIRE(chunks <= 65535, B200_NOT_SUPPORTED, "b200_layer_norm_backward: M too large for the column reduction");
      float* pw = static_cast<float*>(workspace);
      float* pb = pw + chunks * N;
      layer_norm_dwdb_partial_kernel<T><<<dim3(static_cast<unsigned>((N + 31) / 32), static_cast<unsigned>(chunks)), kThreads, 0, s>>>(
          pw, pb, static_cast<const T*>(grad_out->data), static_cast<const T*>(x->data), pm, pr, M, N);
      layer_norm_dwdb_final_kernel<T><<<static_cast<unsigned>((N + kThreads - 1) / kThreads), kThreads, 0, s>>>(
          dweight ? static_cast<T*>(dweight->data) : nullptr, dbias ? static_cast<T*>(dbias->data) : nullptr, pw, pb, chunks, N);
      note_launches(dx ? 2 : 1);
    }
  });
  return check_launch("b200_layer_norm_backward");
}

}  // extern "C"
