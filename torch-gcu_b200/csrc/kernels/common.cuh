// Shared helpers of the sm_100a kernel library: status/error plumbing, tensor
// view inspection, dtype dispatch, 128-bit vector access and the bf16/f16
// conversions (round to nearest even, bit-identical to c10::BFloat16 / c10::Half
// for every non-NaN value).
#pragma once

#include <cuda_runtime.h>
#include <cstdlib>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>
#include <string.h>

#include "b200ops.h"

namespace b200 {

// ---------------------------------------------------------------- errors ----
char* error_buffer();  // thread-local, 512 bytes (runtime.cu)

inline b200Status fail(b200Status st, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return st;
}

#define B200_REQUIRE(cond, status, ...)                \
  do {                                                 \
    if (!(cond)) return ::b200::fail((status), __VA_ARGS__); \
  } while (0)

// Kernel launches issued by this library in this process (b200_launch_count): one per checked
// launch; entry points that launch several kernels before one check add the rest themselves.
void note_launches(int n);

inline b200Status check_launch(const char* what) {
  note_launches(1);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(B200_LAUNCH_FAILED, "%s: %s", what, cudaGetErrorString(e));
  return B200_OK;
}

int sm_count_current_device();
int gemm_sm_budget();   // SM count minus the SMs reserved through b200_set_reserved_sms  // cached per device (runtime.cu)

// ------------------------------------------------------------ tensor view ----
inline int64_t numel(const b200Tensor* t) {
  int64_t n = 1;
  for (int i = 0; i < t->ndim; ++i) n *= t->sizes[i];
  return n;
}

inline bool valid(const b200Tensor* t) {
  if (!t || t->ndim < 0 || t->ndim > B200_MAX_DIMS) return false;
  for (int i = 0; i < t->ndim; ++i)
    if (t->sizes[i] < 0) return false;
  if (t->dtype < 0 || t->dtype > B200_BOOL) return false;
  return numel(t) == 0 || t->data != nullptr;
}

inline bool is_contiguous(const b200Tensor* t) {
  int64_t expect = 1;
  for (int i = t->ndim - 1; i >= 0; --i) {
    if (t->sizes[i] == 1) continue;
    if (t->strides[i] != expect) return false;
    expect *= t->sizes[i];
  }
  return true;
}

inline bool same_shape(const b200Tensor* a, const b200Tensor* b) {
  if (a->ndim != b->ndim) return false;
  for (int i = 0; i < a->ndim; ++i)
    if (a->sizes[i] != b->sizes[i]) return false;
  return true;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline size_t dtype_size(int32_t dt) {
  switch (dt) {
    case B200_F32: case B200_I32: return 4;
    case B200_BF16: case B200_F16: case B200_I16: return 2;
    case B200_F64: case B200_I64: return 8;
    case B200_I8: case B200_U8: case B200_BOOL: return 1;
    default: return 0;
  }
}

// Strided addressing of up to three operands over a common (collapsed) shape.
// Dimension 0 is the fastest-varying one.
template <int NARGS>
struct StridedIndexer {
  int ndim;
  int64_t sizes[B200_MAX_DIMS];
  int64_t strides[NARGS][B200_MAX_DIMS];

  __host__ __device__ void offsets(int64_t linear, int64_t (&off)[NARGS]) const {
#pragma unroll
    for (int a = 0; a < NARGS; ++a) off[a] = 0;
#pragma unroll 1
    for (int d = 0; d < ndim; ++d) {
      int64_t q = linear / sizes[d];
      int64_t r = linear - q * sizes[d];
      linear = q;
#pragma unroll
      for (int a = 0; a < NARGS; ++a) off[a] += r * strides[a][d];
    }
  }
};

// Builds an indexer over `ts[0..NARGS)` (all of the same shape) and merges
// neighbouring dimensions that every operand walks contiguously.
template <int NARGS>
inline StridedIndexer<NARGS> make_indexer(const b200Tensor* const (&ts)[NARGS]) {
  StridedIndexer<NARGS> ix;
  int nd = 0;
  const b200Tensor* t0 = ts[0];
  for (int i = t0->ndim - 1; i >= 0; --i) {  // innermost first
    int64_t sz = t0->sizes[i];
    if (sz == 1) continue;
    bool merged = false;
    if (nd > 0) {
      bool can = true;
      for (int a = 0; a < NARGS; ++a)
        if (ts[a]->strides[i] != ix.strides[a][nd - 1] * ix.sizes[nd - 1]) can = false;
      if (can) {
        ix.sizes[nd - 1] *= sz;
        merged = true;
      }
    }
    if (!merged) {
      ix.sizes[nd] = sz;
      for (int a = 0; a < NARGS; ++a) ix.strides[a][nd] = ts[a]->strides[i];
      ++nd;
    }
  }
  if (nd == 0) {
    ix.sizes[0] = 1;
    for (int a = 0; a < NARGS; ++a) ix.strides[a][0] = 0;
    nd = 1;
  }
  ix.ndim = nd;
  return ix;
}

// ------------------------------------------------------------- conversions ----
// fp32 -> bf16, round to nearest even, one hardware conversion (cvt.rn.bf16.f32).
// NaN stays NaN; its payload is not part of the contract (c10::BFloat16 gives
// 0x7FC0, ATen's vectorised CPU cast 0xFFFF, the hardware 0x7FFF).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
// Two at once: cvt.rn.bf16x2.f32 (lo in the low half).
__device__ __forceinline__ uint32_t f32x2_to_bf16x2_bits(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) {
  return __uint_as_float(static_cast<uint32_t>(b) << 16);
}
// fp32 -> fp16, round to nearest even (cvt.rn.f16.f32); NaN stays NaN.
__device__ __forceinline__ uint16_t f32_to_f16_bits(float f) {
  return __half_as_ushort(__float2half_rn(f));
}
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
  return __half2float(__ushort_as_half(h));
}

// Host-side rounding of a scalar operand to the tensor's element type: ATen
// converts `alpha` and wrapped-number operands to the op's dtype before use.
inline double round_scalar_to_dtype(double v, int32_t dtype) {
  if (dtype == B200_F32) return static_cast<double>(static_cast<float>(v));
  if (dtype == B200_BF16) {
    float f = static_cast<float>(v);
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return v;
    u += 0x7FFFu + ((u >> 16) & 1u);
    u &= 0xFFFF0000u;
    memcpy(&f, &u, 4);
    return f;
  }
  if (dtype == B200_F16) return static_cast<double>(__half2float(__float2half_rn(static_cast<float>(v))));
  return v;
}

// Storage types: bf16 and f16 are carried as tagged 16-bit integers so that all
// arithmetic goes through the conversions above.
struct bf16_t { uint16_t bits; };
struct f16_t { uint16_t bits; };

template <typename T> struct OpMath { using type = T; };
template <> struct OpMath<bf16_t> { using type = float; };
template <> struct OpMath<f16_t> { using type = float; };

template <typename T> __device__ __forceinline__ typename OpMath<T>::type load_as_math(T v) { return v; }
template <> __device__ __forceinline__ float load_as_math<bf16_t>(bf16_t v) { return bf16_bits_to_f32(v.bits); }
template <> __device__ __forceinline__ float load_as_math<f16_t>(f16_t v) { return f16_bits_to_f32(v.bits); }

template <typename T> __device__ __forceinline__ T store_from_math(typename OpMath<T>::type v) { return v; }
template <> __device__ __forceinline__ bf16_t store_from_math<bf16_t>(float v) { return bf16_t{f32_to_bf16_bits(v)}; }
template <> __device__ __forceinline__ f16_t store_from_math<f16_t>(float v) { return f16_t{f32_to_f16_bits(v)}; }

// ------------------------------------------------------- 128-bit accessors ----
template <typename T> struct alignas(16) Vec16 { T v[16 / sizeof(T)]; };

template <typename T>
__device__ __forceinline__ Vec16<T> load_stream16(const T* p) {
  int4 r = __ldcs(reinterpret_cast<const int4*>(p));
  return *reinterpret_cast<Vec16<T>*>(&r);
}
template <typename T>
__device__ __forceinline__ Vec16<T> load16(const T* p) {
  int4 r = *reinterpret_cast<const int4*>(p);
  return *reinterpret_cast<Vec16<T>*>(&r);
}
template <typename T>
__device__ __forceinline__ void store_stream16(T* p, const Vec16<T>& v) {
  __stcs(reinterpret_cast<int4*>(p), *reinterpret_cast<const int4*>(&v));
}
template <typename T>
__device__ __forceinline__ void store16(T* p, const Vec16<T>& v) {
  *reinterpret_cast<int4*>(p) = *reinterpret_cast<const int4*>(&v);
}

// --------------------------------------------------------------- dispatch ----
#define B200_DISPATCH_FLOAT(DT, T, ...)                                          \
  switch (DT) {                                                                  \
    case B200_F32: { using T = float; __VA_ARGS__; break; }                      \
    case B200_BF16: { using T = ::b200::bf16_t; __VA_ARGS__; break; }            \
    case B200_F16: { using T = ::b200::f16_t; __VA_ARGS__; break; }              \
    case B200_F64: { using T = double; __VA_ARGS__; break; }                     \
    default: return ::b200::fail(B200_NOT_SUPPORTED, "%s: dtype %d not supported", __func__, (int)(DT)); \
  }

#define B200_DISPATCH_ARITH(DT, T, ...)                                          \
  switch (DT) {                                                                  \
    case B200_F32: { using T = float; __VA_ARGS__; break; }                      \
    case B200_BF16: { using T = ::b200::bf16_t; __VA_ARGS__; break; }            \
    case B200_F16: { using T = ::b200::f16_t; __VA_ARGS__; break; }              \
    case B200_F64: { using T = double; __VA_ARGS__; break; }                     \
    case B200_I64: { using T = int64_t; __VA_ARGS__; break; }                    \
    case B200_I32: { using T = int32_t; __VA_ARGS__; break; }                    \
    case B200_I16: { using T = int16_t; __VA_ARGS__; break; }                    \
    case B200_I8: { using T = int8_t; __VA_ARGS__; break; }                      \
    case B200_U8: { using T = uint8_t; __VA_ARGS__; break; }                     \
    default: return ::b200::fail(B200_NOT_SUPPORTED, "%s: dtype %d not supported", __func__, (int)(DT)); \
  }

// Byte-width dispatch for pure data movement (bit-exact by construction).
#define B200_DISPATCH_BYTES(NBYTES, T, ...)                                      \
  switch (NBYTES) {                                                              \
    case 1: { using T = uint8_t; __VA_ARGS__; break; }                           \
    case 2: { using T = uint16_t; __VA_ARGS__; break; }                          \
    case 4: { using T = uint32_t; __VA_ARGS__; break; }                          \
    case 8: { using T = uint64_t; __VA_ARGS__; break; }                          \
    default: return ::b200::fail(B200_NOT_SUPPORTED, "%s: element size %d", __func__, (int)(NBYTES)); \
  }

// Grid size for grid-stride kernels: a whole number of waves of the device.
inline int grid_for(int64_t work_items, int threads, int blocks_per_sm) {
  int64_t need = (work_items + threads - 1) / threads;
  int64_t cap = static_cast<int64_t>(sm_count_current_device()) * blocks_per_sm;
  if (need < 1) need = 1;
  return static_cast<int>(need < cap ? need : cap);
}

// Grid size for a grid-stride kernel: at most `waves` resident waves, a wave taken from the
// occupancy the compiled kernel really gets (its register count decides; a grid sized for 8
// blocks per SM runs as 1.6 waves when only 5 fit). One wave is a static partition of the
// work; several let the block scheduler even out SMs that stream at different speeds. The
// occupancy is cached per kernel instantiation (all devices of a box are alike);
// B200_GRID_WAVES overrides every call site's `waves` (tuning aid).
inline int grid_waves_override() {
  static int v = -1;
  if (v < 0) {
    const char* e = std::getenv("B200_GRID_WAVES");
    v = e ? std::atoi(e) : 0;
    if (v < 0) v = 0;
    if (v > 64) v = 64;
  }
  return v;
}
// Streaming kernels whose blocks each move one batch of 128-bit accesses: measured on the (4096,4096)
// and table workloads, many short blocks beat one persistent wave by 2-10 %.
constexpr int kStreamWaves = 64;

template <auto Kernel>
inline int wave_grid(int64_t need_blocks, int threads, int waves = 1, size_t dyn_smem = 0) {
  static int per_sm = 0;
  if (per_sm == 0) {
    int v = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, Kernel, threads, dyn_smem) != cudaSuccess || v < 1) v = 1;
    per_sm = v;
  }
  if (grid_waves_override() > 0) waves = grid_waves_override();
  int64_t cap = static_cast<int64_t>(sm_count_current_device()) * per_sm * waves;
  if (need_blocks < 1) need_blocks = 1;
  return static_cast<int>(need_blocks < cap ? need_blocks : cap);
}

// ------------------------------------------------- programmatic dependent launch --
// A kernel launched through launch_pdl may become resident while its predecessor on the stream
// is still draining (its blocks are scheduled as soon as every block of the predecessor has
// called pdl_launch_dependents() or exited), which hides the launch latency and the ramp of a
// short kernel under the predecessor's tail. The contract of such a kernel: pdl_wait() before
// its first access to global memory (the wait returns once the predecessor has completed and
// its writes are visible; it is a no-op for a kernel launched without the attribute).
// B200_PDL=0 launches everything fully serialised.
inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = std::getenv("B200_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                              Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace b200
