// The one hop between ATen and the kernel library: at::Tensor -> b200Tensor view,
// status -> exception, current stream lookup. It plays the part of the
// reference's bridge macros and topsaten_variable<T> marshallers
// (reference: torch_gcu/csrc/aten/aot_ops/topsaten_bridge_define.h:21-427,
// createTopsatenTensor torch_gcu/csrc/gcu/gcu_utils.cpp:79-108), minus the
// std::function op-info lambda and the extra wrapper layers.
#pragma once

#include <ATen/ATen.h>
#include <ATen/record_function.h>

#include "b200ops.h"
#include "runtime/gcu_allocator.h"
#include "runtime/gcu_runtime.h"

namespace torch_gcu {

inline int32_t to_b200_dtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return B200_F32;
    case at::kBFloat16: return B200_BF16;
    case at::kHalf: return B200_F16;
    case at::kDouble: return B200_F64;
    case at::kLong: return B200_I64;
    case at::kInt: return B200_I32;
    case at::kShort: return B200_I16;
    case at::kChar: return B200_I8;
    case at::kByte: return B200_U8;
    case at::kBool: return B200_BOOL;
    default: TORCH_CHECK(false, "dtype ", t, " is not supported on the gcu backend");
  }
}

inline b200Tensor to_b200(const at::Tensor& t) {
  TORCH_CHECK(t.defined(), "undefined tensor passed to a gcu kernel");
  TORCH_CHECK(t.device().is_privateuseone(), "expected a gcu tensor but got one on ", t.device(),
              " (a device kernel must never dereference a host pointer)");
  TORCH_CHECK(t.dim() <= B200_MAX_DIMS, "gcu kernels support at most ", B200_MAX_DIMS, " dimensions");
  b200Tensor v;
  v.data = t.data_ptr();
  v.dtype = to_b200_dtype(t.scalar_type());
  v.ndim = static_cast<int32_t>(t.dim());
  for (int i = 0; i < v.ndim; ++i) {
    v.sizes[i] = t.size(i);
    v.strides[i] = t.stride(i);
  }
  return v;
}

// Mirrors CHECK_TOPSATEN_CALL (reference: gcu_utils.cpp:64-77): a non-OK status
// becomes a c10::Error carrying the library's message. There is no CPU fallback.
inline void check_status(b200Status st, const char* op) {
  if (st == B200_OK) return;
  static const char* names[] = {"OK", "BAD_PARAM", "NOT_SUPPORTED", "LAUNCH_FAILED", "WORKSPACE_TOO_SMALL", "TIMEOUT"};
  TORCH_CHECK(false, "gcu kernel ", op, " failed with ", names[st <= B200_TIMEOUT ? st : 1], ": ", b200_last_error());
}

inline cudaStream_t current_stream(const at::Tensor& t) {
  return getCurrentGCUStream(t.device().index()).stream();
}

// Runs a kernel call, checks it, and honours op_sync_mode.
#define GCU_KERNEL_CALL(NAME, STREAM, ...)                       \
  do {                                                           \
    RECORD_FUNCTION("GCU::" #NAME, std::vector<c10::IValue>()); \
    ::torch_gcu::check_status(NAME(__VA_ARGS__, (STREAM)), #NAME); \
    ::torch_gcu::maybe_stream_synchronize(STREAM);               \
  } while (0)

// Scratch memory for kernels that need it: a byte tensor from the caching
// allocator on the current stream (freed, stream-ordered, when it goes out of scope).
inline at::Tensor alloc_workspace(size_t bytes, const at::Tensor& like) {
  return at::empty({static_cast<int64_t>(bytes ? bytes : 1)}, like.options().dtype(at::kByte));
}

}  // namespace torch_gcu
