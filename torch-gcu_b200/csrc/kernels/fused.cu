// Single-pass fused inference kernels: RMSNorm with residual add, rotate-half
// rotary embedding and SwiGLU. Each reads its operands from HBM once with
// 128-bit loads, computes in fp32 and rounds once on store.
#include "common.cuh"

namespace b200 {
unsigned int* device_error_word();  // index.cu: address of the device error word

namespace {

// ------------------------------------------------------ RMSNorm + residual --
template <typename T, int BX, int VPT>
__global__ void __launch_bounds__(BX)
rms_norm_residual_kernel(T* __restrict__ y, T* res_out, const T* x, const T* res,
                         const T* __restrict__ w, int64_t N, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = 16 / sizeof(T);
  __shared__ float smem[BX / 32];
  const int64_t row = blockIdx.x;
  const int64_t nvec = N / V;
  const T* xr = x + row * N;
  const T* rr = res ? res + row * N : nullptr;
  float h[VPT][V];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int64_t vi = threadIdx.x + static_cast<int64_t>(k) * BX;
    if (vi < nvec) {
      Vec16<T> xv = load_stream16(xr + vi * V);
      if (rr) {
        Vec16<T> rv = load_stream16(rr + vi * V);
        Vec16<T> hv;
#pragma unroll
        for (int e = 0; e < V; ++e) {
          hv.v[e] = store_from_math<T>(load_as_math(xv.v[e]) + load_as_math(rv.v[e]));
          h[k][e] = load_as_math(hv.v[e]);  // the norm sees the rounded sum
        }
        if (res_out) store_stream16(res_out + row * N + vi * V, hv);
      } else {
#pragma unroll
        for (int e = 0; e < V; ++e) h[k][e] = load_as_math(xv.v[e]);
        if (res_out) store_stream16(res_out + row * N + vi * V, xv);
      }
#pragma unroll
      for (int e = 0; e < V; ++e) ss += h[k][e] * h[k][e];
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) h[k][e] = 0.f;
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < BX / 32; ++i) tot += smem[i];
  const float rstd = 1.0f / sqrtf(tot / static_cast<float>(N) + eps);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int64_t vi = threadIdx.x + static_cast<int64_t>(k) * BX;
    if (vi < nvec) {
      Vec16<T> wv = load16(w + vi * V), o;
#pragma unroll
      for (int e = 0; e < V; ++e) o.v[e] = store_from_math<T>(h[k][e] * rstd * load_as_math(wv.v[e]));
      store_stream16(y + row * N + vi * V, o);
    }
  }
}

// generic row (any N, any alignment): block strides over the row three times
template <typename T>
__global__ void __launch_bounds__(256)
rms_norm_residual_generic_kernel(T* y, T* res_out, const T* x, const T* res, const T* w, int64_t N, float eps) {
  __shared__ float smem[8];
  const int64_t row = blockIdx.x;
  float ss = 0.f;
  for (int64_t i = threadIdx.x; i < N; i += 256) {
    T hv = res ? store_from_math<T>(load_as_math(x[row * N + i]) + load_as_math(res[row * N + i])) : x[row * N + i];
    float h = load_as_math(hv);
    ss += h * h;
    if (res_out) res_out[row * N + i] = hv;
    else if (res) y[row * N + i] = hv;  // parked in y until the second sweep
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < 8; ++i) tot += smem[i];
  const float rstd = 1.0f / sqrtf(tot / static_cast<float>(N) + eps);
  for (int64_t i = threadIdx.x; i < N; i += 256) {
    // each thread re-reads only elements it wrote itself
    T hv = res_out ? res_out[row * N + i] : (res ? y[row * N + i] : x[row * N + i]);
    y[row * N + i] = store_from_math<T>(load_as_math(hv) * rstd * load_as_math(w[i]));
  }
}

template <typename T>
b200Status launch_rms(void* y, void* res_out, const void* x, const void* res, const void* w, int64_t M,
                      int64_t N, float eps, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  const bool al = aligned16(y) && aligned16(x) && aligned16(w) && (!res || aligned16(res)) &&
                  (!res_out || aligned16(res_out)) && N % V == 0;
  const int64_t nvec = N / V;
  T* py = static_cast<T*>(y);
  T* pro = static_cast<T*>(res_out);
  const T* px = static_cast<const T*>(x);
  const T* pr = static_cast<const T*>(res);
  const T* pw = static_cast<const T*>(w);
  const unsigned grid = static_cast<unsigned>(M);
  if (al && nvec <= 128) launch_pdl(rms_norm_residual_kernel<T, 128, 1>, grid, 128, 0, s, py, pro, px, pr, pw, N, eps);
  else if (al && nvec <= 256) launch_pdl(rms_norm_residual_kernel<T, 256, 1>, grid, 256, 0, s, py, pro, px, pr, pw, N, eps);
  else if (al && nvec <= 512) launch_pdl(rms_norm_residual_kernel<T, 256, 2>, grid, 256, 0, s, py, pro, px, pr, pw, N, eps);
  else if (al && nvec <= 1024) launch_pdl(rms_norm_residual_kernel<T, 256, 4>, grid, 256, 0, s, py, pro, px, pr, pw, N, eps);
  else if (al && nvec <= 2048) launch_pdl(rms_norm_residual_kernel<T, 512, 4>, grid, 512, 0, s, py, pro, px, pr, pw, N, eps);
  else if (al && nvec <= 4096) launch_pdl(rms_norm_residual_kernel<T, 1024, 4>, grid, 1024, 0, s, py, pro, px, pr, pw, N, eps);
  else rms_norm_residual_generic_kernel<T><<<grid, 256, 0, s>>>(py, pro, px, pr, pw, N, eps);
  return check_launch("b200_rms_norm_residual");
}

// ------------------------------------------------------------------- RoPE --
struct RopeArgs {
  const void* x;
  void* out;
  const float* cos_t;
  const float* sin_t;
  const int64_t* positions;  // (B, S) or null
  int64_t pos_stride_b, pos_stride_s;
  int64_t B, S, H, D;
  int64_t xs[3], os[3];  // element strides of (b, s, h)
  int64_t P;             // rows of the tables
};

// W: index arithmetic type (uint32_t when the element count allows).
template <typename T, typename W>
__global__ void __launch_bounds__(256)
rope_kernel(RopeArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = 16 / sizeof(T);
  const int64_t half = a.D / 2;
  const W vph = static_cast<W>(half / V);  // vectors per half row
  const W total = static_cast<W>(a.B * a.S * a.H) * vph;
  const W stride = static_cast<W>(gridDim.x) * 256;
  const W H = static_cast<W>(a.H), S = static_cast<W>(a.S);
  for (W i = static_cast<W>(blockIdx.x) * 256 + threadIdx.x; i < total; i += stride) {
    W t = i / vph;
    const int v = static_cast<int>(i - t * vph);
    const W th = t / H;
    const int64_t h = t - th * H;
    const W tb = th / S;
    const int64_t s = th - tb * S;
    const int64_t b = tb;
    int64_t p = a.positions ? a.positions[b * a.pos_stride_b + s * a.pos_stride_s] : s;
    if (p < 0 || p >= a.P) p = 0;  // caller guarantees range; keep reads in bounds
    const T* xr = static_cast<const T*>(a.x) + b * a.xs[0] + s * a.xs[1] + h * a.xs[2];
    T* orow = static_cast<T*>(a.out) + b * a.os[0] + s * a.os[1] + h * a.os[2];
    Vec16<T> x1 = load_stream16(xr + v * V);
    Vec16<T> x2 = load_stream16(xr + half + v * V);
    const float* c = a.cos_t + p * half + v * V;
    const float* sn = a.sin_t + p * half + v * V;
    Vec16<T> o1, o2;
#pragma unroll
    for (int q = 0; q < V / 4; ++q) {
      const float4 cv = *reinterpret_cast<const float4*>(c + q * 4);
      const float4 sv = *reinterpret_cast<const float4*>(sn + q * 4);
      const float cc[4] = {cv.x, cv.y, cv.z, cv.w};
      const float sc[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float a1 = load_as_math(x1.v[q * 4 + e]);
        const float a2 = load_as_math(x2.v[q * 4 + e]);
        // separate roundings (no fma) so the fp32 value equals the unfused chain
        o1.v[q * 4 + e] = store_from_math<T>(__fadd_rn(__fmul_rn(a1, cc[e]), __fmul_rn(-a2, sc[e])));
        o2.v[q * 4 + e] = store_from_math<T>(__fadd_rn(__fmul_rn(a2, cc[e]), __fmul_rn(a1, sc[e])));
      }
    }
    store_stream16(orow + v * V, o1);
    store_stream16(orow + half + v * V, o2);
  }
}

// ------------------------------------------- RoPE + write into the KV cache --
// One pass over a fused projection output qkv (B, S, q_heads + 2 k_heads, D): query heads are rotated in place, key
// heads are rotated and written to k_cache[b, head, position, :], value heads are copied to v_cache[b, head,
// position, :]; position = positions[b, s] is both the row of the tables and the slot of the caches. The key and
// value parts of qkv stay as they were. A position outside the caches or the tables sets the index-out-of-range
// bit of the device error word and writes nothing.
struct RopeAppendArgs {
  void* qkv;
  void* kc;
  void* vc;
  const float* cos_t;
  const float* sin_t;
  const int64_t* positions;
  int64_t pos_stride_b, pos_stride_s;
  int64_t B, S, Hq, Hk, D;
  int64_t xs[3];          // element strides of qkv (b, s, h)
  int64_t ks[3], vs[3];   // element strides of the caches (b, h, t)
  int64_t P, T;           // rows of the tables, slots of the caches
  unsigned int* error_word;
};

template <typename T>
__global__ void __launch_bounds__(256)
rope_kv_append_kernel(RopeAppendArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = 16 / sizeof(T);
  const int64_t half = a.D / 2;
  const int64_t vph = half / V;  // vectors per half row
  const int64_t H = a.Hq + 2 * a.Hk;
  const int64_t total = a.B * a.S * H * vph;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += stride) {
    int64_t t = i / vph;
    const int v = static_cast<int>(i - t * vph);
    const int64_t th = t / H;
    const int64_t h = t - th * H;
    const int64_t b = th / a.S;
    const int64_t s = th - b * a.S;
    const int64_t p = a.positions[b * a.pos_stride_b + s * a.pos_stride_s];
    if (p < 0 || p >= a.P || p >= a.T) {
      if (v == 0 && h == 0) atomicOr(a.error_word, 1u);   // bit 0: index out of range
      continue;
    }
    T* xr = static_cast<T*>(a.qkv) + b * a.xs[0] + s * a.xs[1] + h * a.xs[2];
    Vec16<T> x1 = load_stream16(xr + v * V);
    Vec16<T> x2 = load_stream16(xr + half + v * V);
    T* orow = xr;
    if (h >= a.Hq + a.Hk) {   // value head: copied as it is
      orow = static_cast<T*>(a.vc) + b * a.vs[0] + (h - a.Hq - a.Hk) * a.vs[1] + p * a.vs[2];
      store_stream16(orow + v * V, x1);
      store_stream16(orow + half + v * V, x2);
      continue;
    }
    if (h >= a.Hq) orow = static_cast<T*>(a.kc) + b * a.ks[0] + (h - a.Hq) * a.ks[1] + p * a.ks[2];
    const float* c = a.cos_t + p * half + v * V;
    const float* sn = a.sin_t + p * half + v * V;
    Vec16<T> o1, o2;
#pragma unroll
    for (int q = 0; q < V / 4; ++q) {
      const float4 cv = *reinterpret_cast<const float4*>(c + q * 4);
      const float4 sv = *reinterpret_cast<const float4*>(sn + q * 4);
      const float cc[4] = {cv.x, cv.y, cv.z, cv.w};
      const float sc[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float a1 = load_as_math(x1.v[q * 4 + e]);
        const float a2 = load_as_math(x2.v[q * 4 + e]);
        // the arithmetic of rope_kernel: separate roundings, so both paths give the same bits
        o1.v[q * 4 + e] = store_from_math<T>(__fadd_rn(__fmul_rn(a1, cc[e]), __fmul_rn(-a2, sc[e])));
        o2.v[q * 4 + e] = store_from_math<T>(__fadd_rn(__fmul_rn(a2, cc[e]), __fmul_rn(a1, sc[e])));
      }
    }
    store_stream16(orow + v * V, o1);
    store_stream16(orow + half + v * V, o2);
  }
}

// ----------------------------------------------------------------- SwiGLU --
template <typename T>
__device__ __forceinline__ Vec16<T> swiglu_vec(const Vec16<T>& g, const Vec16<T>& u) {
  constexpr int V = 16 / sizeof(T);
  Vec16<T> o;
#pragma unroll
  for (int e = 0; e < V; ++e) {
    const float x = load_as_math(g.v[e]);
    if constexpr (sizeof(T) == 2) {
      // 16-bit output: the fast exp / reciprocal (a few fp32 ulp) are far below
      // half an output ulp, and keep the kernel off the instruction-issue limit
      o.v[e] = store_from_math<T>(__fdividef(x, 1.0f + __expf(-x)) * load_as_math(u.v[e]));
    } else {
      o.v[e] = store_from_math<T>(x / (1.0f + expf(-x)) * load_as_math(u.v[e]));
    }
  }
  return o;
}

// rows x (vectors per row); row strides in elements; flat when all rows abut.
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_kernel(T* __restrict__ out, const T* __restrict__ gate, const T* __restrict__ up, int64_t rows,
              int64_t vpr, int64_t so, int64_t sg, int64_t su) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = 16 / sizeof(T);
  constexpr int U = 4;
  const int64_t total = rows * vpr;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * 256;
  int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
  auto offs = [&](int64_t idx, int64_t& oo, int64_t& og, int64_t& ou) {
    const int64_t r = idx / vpr, c = (idx - r * vpr) * V;
    oo = r * so + c; og = r * sg + c; ou = r * su + c;
  };
  for (; i + (U - 1) * stride < total; i += U * stride) {
    Vec16<T> g[U], u[U];
    int64_t oo[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      int64_t og, ou;
      offs(i + k * stride, oo[k], og, ou);
      g[k] = load_stream16(gate + og);
      u[k] = load_stream16(up + ou);
    }
#pragma unroll
    for (int k = 0; k < U; ++k) store_stream16(out + oo[k], swiglu_vec<T>(g[k], u[k]));
  }
  for (; i < total; i += stride) {
    int64_t oo, og, ou;
    offs(i, oo, og, ou);
    store_stream16(out + oo, swiglu_vec<T>(load_stream16(gate + og), load_stream16(up + ou)));
  }
}

template <typename T>
__global__ void swiglu_scalar_kernel(T* out, const T* gate, const T* up, int64_t rows, int64_t cols,
                                     int64_t so, int64_t sg, int64_t su) {
  const int64_t total = rows * cols;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / cols, c = i - r * cols;
    const float x = load_as_math(gate[r * sg + c]);
    out[r * so + c] = store_from_math<T>(x / (1.0f + expf(-x)) * load_as_math(up[r * su + c]));
  }
}

#define B200_DISPATCH_HALF_FLOAT(DT, T, ...)                                     \
  switch (DT) {                                                                  \
    case B200_F32: { using T = float; __VA_ARGS__; break; }                      \
    case B200_BF16: { using T = ::b200::bf16_t; __VA_ARGS__; break; }            \
    case B200_F16: { using T = ::b200::f16_t; __VA_ARGS__; break; }              \
    default: return ::b200::fail(B200_NOT_SUPPORTED, "%s: dtype %d not supported", __func__, (int)(DT)); \
  }

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

b200Status b200_rms_norm_residual(const b200Tensor* y, const b200Tensor* residual_out, const b200Tensor* x,
                                  const b200Tensor* residual, const b200Tensor* weight, double eps,
                                  b200Stream stream) {
  B200_REQUIRE(valid(y) && valid(x) && valid(weight), B200_BAD_PARAM, "b200_rms_norm_residual: invalid tensor view");
  B200_REQUIRE(x->ndim >= 1, B200_BAD_PARAM, "b200_rms_norm_residual: x must have rank >= 1");
  const int64_t N = x->sizes[x->ndim - 1];
  const int64_t M = N ? numel(x) / N : 0;
  B200_REQUIRE(same_shape(y, x) && y->dtype == x->dtype && is_contiguous(x) && is_contiguous(y), B200_BAD_PARAM,
               "b200_rms_norm_residual: x and y must be contiguous, same shape and dtype");
  B200_REQUIRE(numel(weight) == N && weight->dtype == x->dtype && is_contiguous(weight), B200_BAD_PARAM,
               "b200_rms_norm_residual: weight must be N contiguous elements of x's dtype");
  if (residual)
    B200_REQUIRE(valid(residual) && same_shape(residual, x) && residual->dtype == x->dtype && is_contiguous(residual),
                 B200_BAD_PARAM, "b200_rms_norm_residual: residual must match x");
  if (residual_out)
    B200_REQUIRE(valid(residual_out) && same_shape(residual_out, x) && residual_out->dtype == x->dtype &&
                 is_contiguous(residual_out), B200_BAD_PARAM, "b200_rms_norm_residual: residual_out must match x");
  if (M == 0 || N == 0) return B200_OK;
  B200_REQUIRE(M <= 0x7fffffff, B200_NOT_SUPPORTED, "b200_rms_norm_residual: too many rows");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  B200_DISPATCH_HALF_FLOAT(x->dtype, T, {
    return launch_rms<T>(y->data, residual_out ? residual_out->data : nullptr, x->data,
                         residual ? residual->data : nullptr, weight->data, M, N, static_cast<float>(eps), s);
  });
  return B200_OK;
}

b200Status b200_rope(const b200Tensor* out, const b200Tensor* x, const b200Tensor* cos_table,
                     const b200Tensor* sin_table, const b200Tensor* positions, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(x) && valid(cos_table) && valid(sin_table), B200_BAD_PARAM,
               "b200_rope: invalid tensor view");
  B200_REQUIRE(x->ndim == 4 && same_shape(out, x) && out->dtype == x->dtype, B200_BAD_PARAM,
               "b200_rope: x and out must be (B,S,H,D) of one dtype");
  RopeArgs a{};
  a.B = x->sizes[0]; a.S = x->sizes[1]; a.H = x->sizes[2]; a.D = x->sizes[3];
  if (numel(x) == 0) return B200_OK;
  B200_REQUIRE(a.D % 2 == 0 && (a.D == 1 || (x->strides[3] == 1 && out->strides[3] == 1)), B200_BAD_PARAM,
               "b200_rope: head dim must be even and contiguous");
  const int64_t es = static_cast<int64_t>(dtype_size(x->dtype));
  const int64_t V = 16 / es;
  B200_REQUIRE((a.D / 2) % V == 0 && V >= 4, B200_NOT_SUPPORTED,
               "b200_rope: D/2 must be a multiple of %lld elements", (long long)V);
  B200_REQUIRE(cos_table->dtype == B200_F32 && sin_table->dtype == B200_F32 && cos_table->ndim == 2 &&
               same_shape(cos_table, sin_table) && cos_table->sizes[1] == a.D / 2 &&
               is_contiguous(cos_table) && is_contiguous(sin_table), B200_BAD_PARAM,
               "b200_rope: cos/sin must be contiguous f32 (P, D/2) tables");
  a.P = cos_table->sizes[0];
  B200_REQUIRE(aligned16(cos_table->data) && aligned16(sin_table->data) && aligned16(x->data) &&
               aligned16(out->data), B200_NOT_SUPPORTED, "b200_rope: 16-byte aligned operands needed");
  for (int d = 0; d < 3; ++d) {
    a.xs[d] = x->strides[d]; a.os[d] = out->strides[d];
    B200_REQUIRE(x->sizes[d] == 1 || ((a.xs[d] * es) % 16 == 0 && (a.os[d] * es) % 16 == 0), B200_NOT_SUPPORTED,
                 "b200_rope: strides must keep rows 16-byte aligned");
  }
  if (positions) {
    B200_REQUIRE(valid(positions) && positions->dtype == B200_I64 && positions->ndim == 2 &&
                 positions->sizes[0] == a.B && positions->sizes[1] == a.S, B200_BAD_PARAM,
                 "b200_rope: positions must be int64 (B,S)");
    a.positions = static_cast<const int64_t*>(positions->data);
    a.pos_stride_b = positions->strides[0]; a.pos_stride_s = positions->strides[1];
  } else {
    B200_REQUIRE(a.P >= a.S, B200_BAD_PARAM, "b200_rope: tables shorter than the sequence");
  }
  a.x = x->data; a.out = out->data;
  a.cos_t = static_cast<const float*>(cos_table->data);
  a.sin_t = static_cast<const float*>(sin_table->data);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t total = a.B * a.S * a.H * (a.D / 2 / V);
  const int64_t need = (total + 255) / 256;
  // 32-bit item arithmetic needs total + one grid stride below 2^32; bound the stride by 64 waves of 8 blocks
  const bool small = total + static_cast<int64_t>(sm_count_current_device()) * 8 * 64 * 256 < (int64_t(1) << 32);
  B200_DISPATCH_HALF_FLOAT(x->dtype, T, {
    if (small) launch_pdl(rope_kernel<T, uint32_t>, wave_grid<rope_kernel<T, uint32_t>>(need, 256, 4), 256, 0, s, a);
    else launch_pdl(rope_kernel<T, int64_t>, wave_grid<rope_kernel<T, int64_t>>(need, 256, 4), 256, 0, s, a);
  });
  return check_launch("b200_rope");
}

b200Status b200_rope_kv_append(const b200Tensor* qkv, const b200Tensor* cos_table, const b200Tensor* sin_table,
                               const b200Tensor* positions, int64_t q_heads, int64_t k_heads, const b200Tensor* k_cache,
                               const b200Tensor* v_cache, b200Stream stream) {
  const char* name = "b200_rope_kv_append";
  B200_REQUIRE(valid(qkv) && valid(cos_table) && valid(sin_table) && valid(positions) && valid(k_cache) && valid(v_cache),
               B200_BAD_PARAM, "%s: invalid tensor view", name);
  B200_REQUIRE(qkv->ndim == 4 && k_cache->ndim == 4 && v_cache->ndim == 4 && q_heads >= 0 && k_heads >= 0 &&
               qkv->sizes[2] == q_heads + 2 * k_heads, B200_BAD_PARAM,
               "%s: qkv must be (B, S, q_heads + 2 k_heads, D), the caches (B, k_heads, T, D)", name);
  RopeAppendArgs a{};
  a.B = qkv->sizes[0]; a.S = qkv->sizes[1]; a.Hq = q_heads; a.Hk = k_heads; a.D = qkv->sizes[3];
  B200_REQUIRE(same_shape(k_cache, v_cache) && k_cache->sizes[0] == a.B && k_cache->sizes[1] == a.Hk &&
               k_cache->sizes[3] == a.D && k_cache->dtype == qkv->dtype && v_cache->dtype == qkv->dtype, B200_BAD_PARAM,
               "%s: the caches must be (B, k_heads, T, D) of qkv's dtype", name);
  if (numel(qkv) == 0) return B200_OK;
  a.T = k_cache->sizes[2];
  const int64_t es = static_cast<int64_t>(dtype_size(qkv->dtype));
  const int64_t V = 16 / es;
  B200_REQUIRE(a.D % 2 == 0 && qkv->strides[3] == 1 && k_cache->strides[3] == 1 && v_cache->strides[3] == 1, B200_BAD_PARAM,
               "%s: head dim must be even and contiguous", name);
  B200_REQUIRE((a.D / 2) % V == 0 && V >= 4, B200_NOT_SUPPORTED, "%s: D/2 must be a multiple of %lld elements", name, (long long)V);
  B200_REQUIRE(cos_table->dtype == B200_F32 && sin_table->dtype == B200_F32 && cos_table->ndim == 2 &&
               same_shape(cos_table, sin_table) && cos_table->sizes[1] == a.D / 2 && is_contiguous(cos_table) &&
               is_contiguous(sin_table), B200_BAD_PARAM, "%s: cos/sin must be contiguous f32 (P, D/2) tables", name);
  a.P = cos_table->sizes[0];
  B200_REQUIRE(positions->dtype == B200_I64 && positions->ndim == 2 && positions->sizes[0] == a.B && positions->sizes[1] == a.S,
               B200_BAD_PARAM, "%s: positions must be int64 (B,S)", name);
  B200_REQUIRE(aligned16(cos_table->data) && aligned16(sin_table->data) && aligned16(qkv->data) && aligned16(k_cache->data) &&
               aligned16(v_cache->data), B200_NOT_SUPPORTED, "%s: 16-byte aligned operands needed", name);
  for (int d = 0; d < 3; ++d) {
    a.xs[d] = qkv->strides[d]; a.ks[d] = k_cache->strides[d]; a.vs[d] = v_cache->strides[d];
    B200_REQUIRE((qkv->sizes[d] == 1 || (a.xs[d] * es) % 16 == 0) &&
                 (k_cache->sizes[d] == 1 || ((a.ks[d] * es) % 16 == 0 && (a.vs[d] * es) % 16 == 0)), B200_NOT_SUPPORTED,
                 "%s: strides must keep rows 16-byte aligned", name);
  }
  a.qkv = qkv->data; a.kc = k_cache->data; a.vc = v_cache->data;
  a.cos_t = static_cast<const float*>(cos_table->data);
  a.sin_t = static_cast<const float*>(sin_table->data);
  a.positions = static_cast<const int64_t*>(positions->data);
  a.pos_stride_b = positions->strides[0]; a.pos_stride_s = positions->strides[1];
  a.error_word = device_error_word();
  B200_REQUIRE(a.error_word, B200_LAUNCH_FAILED, "%s: device error word unavailable", name);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t total = a.B * a.S * (a.Hq + 2 * a.Hk) * (a.D / 2 / V);
  const int64_t need = (total + 255) / 256;
  B200_DISPATCH_HALF_FLOAT(qkv->dtype, T, {
    launch_pdl(rope_kv_append_kernel<T>, wave_grid<rope_kv_append_kernel<T>>(need, 256, 4), 256, 0, s, a);
  });
  return check_launch(name);
}

b200Status b200_swiglu(const b200Tensor* out, const b200Tensor* gate, const b200Tensor* up, b200Stream stream) {
  B200_REQUIRE(valid(out) && valid(gate) && valid(up), B200_BAD_PARAM, "b200_swiglu: invalid tensor view");
  B200_REQUIRE(same_shape(out, gate) && same_shape(out, up) && out->dtype == gate->dtype && out->dtype == up->dtype,
               B200_BAD_PARAM, "b200_swiglu: operands must agree in shape and dtype");
  B200_REQUIRE(out->ndim == 2, B200_BAD_PARAM, "b200_swiglu: operands must be 2-D (fold leading dims)");
  const int64_t rows = out->sizes[0], cols = out->sizes[1];
  if (rows * cols == 0) return B200_OK;
  B200_REQUIRE(cols == 1 || (out->strides[1] == 1 && gate->strides[1] == 1 && up->strides[1] == 1), B200_NOT_SUPPORTED,
               "b200_swiglu: last dim must be contiguous");
  int64_t so = rows > 1 ? out->strides[0] : cols, sg = rows > 1 ? gate->strides[0] : cols,
          su = rows > 1 ? up->strides[0] : cols;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t es = static_cast<int64_t>(dtype_size(out->dtype));
  const int64_t V = 16 / es;
  const bool vec = cols % V == 0 && so % V == 0 && sg % V == 0 && su % V == 0 && aligned16(out->data) &&
                   aligned16(gate->data) && aligned16(up->data);
  B200_DISPATCH_HALF_FLOAT(out->dtype, T, {
    if (vec) {
      int64_t r = rows, vpr = cols / V;
      if (so == cols && sg == cols && su == cols) {  // flat
        vpr = rows * vpr; r = 1;
      }
      const int grid = wave_grid<swiglu_kernel<T>>((r * vpr + 1023) / 1024, 256, kStreamWaves);
      launch_pdl(swiglu_kernel<T>, grid, 256, 0, s, (T*)out->data, (const T*)gate->data, (const T*)up->data, r, vpr, so, sg, su);
    } else {
      const int grid = grid_for(rows * cols, 256, 8);
      swiglu_scalar_kernel<T><<<grid, 256, 0, s>>>((T*)out->data, (const T*)gate->data, (const T*)up->data, rows, cols, so, sg, su);
    }
  });
  return check_launch("b200_swiglu");
}

}  // extern "C"
