// Output handling for structured kernels: what torchgen's generated
// resize_out / maybe_create_proxy helpers do for in-tree backends
// (reference: torch_gcu/csrc/aten/shape_inference/gcu_structured.cpp:17-52,
// aot_ops/gcu_resize.cpp:99-130). Meta's advisory strides are applied only when a
// resize actually happened, the same rule ATen follows.
#pragma once

#include <ATen/ATen.h>
#include <ATen/native/Resize.h>

#include <optional>

namespace torch_gcu {

inline void resize_out(const at::Tensor& out, at::IntArrayRef sizes, at::IntArrayRef strides,
                       const at::TensorOptions& options) {
  TORCH_CHECK(options.dtype() == out.dtype(), "Expected out tensor to have dtype ", options.dtype(), ", but got ",
              out.dtype(), " instead");
  TORCH_CHECK(options.device() == out.device(), "Expected out tensor to have device ", options.device(),
              ", but got ", out.device(), " instead");
  const bool resized = at::native::resize_output(out, sizes);
  if (resized) {
    if (!strides.empty()) {
      TORCH_INTERNAL_ASSERT(!options.memory_format_opt().has_value());
      out.as_strided_(sizes, strides);
    } else if (options.memory_format_opt().has_value()) {
      out.unsafeGetTensorImpl()->empty_tensor_restride(*options.memory_format_opt());
    }
  }
}

inline std::optional<at::Tensor> maybe_create_proxy(const at::Tensor& out, at::IntArrayRef sizes,
                                                    at::IntArrayRef strides, const at::TensorOptions& options) {
  if (out.strides() != strides) return at::empty_strided(sizes, strides, options);
  return std::nullopt;
}

}  // namespace torch_gcu
