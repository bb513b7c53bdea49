// Dispatcher plumbing around the operator kernels: the autocast policy table for
// AutocastPrivateUse1 (reference: torch_gcu/csrc/aten/gcu_autocast_ops.cpp:28-72),
// the AutogradPrivateUse1 fallthrough (VariableFallbackKernel.cpp:33-35) and the
// boxed PrivateUse1 fallback. Where the reference falls back to the CPU for an
// operator without a kernel (aten_cpu_fallback.cpp:342-451), this backend raises:
// there is no CPU fallback.
#include <ATen/autocast_mode.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <torch/library.h>

namespace {

void not_implemented_fallback(const c10::OperatorHandle& op, torch::jit::Stack*) {
  TORCH_CHECK_NOT_IMPLEMENTED(false, "operator '", op.schema().operator_name(),
                              "' is not implemented for the gcu (B200) backend; this backend has no CPU fallback. "
                              "Supported operators are listed in codegen/gcu_native_functions.yaml.");
}

at::Tensor binary_cross_entropy_banned(const at::Tensor&, const at::Tensor&, const std::optional<at::Tensor>&, int64_t) {
  TORCH_CHECK(false, "torch.nn.functional.binary_cross_entropy and torch.nn.BCELoss are unsafe to autocast.\n"
                     "Use torch.nn.functional.binary_cross_entropy_with_logits or torch.nn.BCEWithLogitsLoss instead.");
}

bool has_compatible_shallow_copy_type(const at::Tensor& self, const at::Tensor& from) {
  // lets `param.data = device_tensor` swap a CPU parameter for a device one
  // (reference: aten_cpu_fallback.cpp:432-446)
  auto is_dense = [](c10::DispatchKeySet ks) {
    return ks.has(c10::DispatchKey::CPU) || ks.has(c10::DispatchKey::PrivateUse1) || ks.has(c10::DispatchKey::CUDA);
  };
  return (self.is_sparse() && from.is_sparse()) || (is_dense(self.key_set()) && is_dense(from.key_set()));
}

}  // namespace

TORCH_LIBRARY_IMPL(_, PrivateUse1, m) { m.fallback(torch::CppFunction::makeFromBoxedFunction<&not_implemented_fallback>()); }

TORCH_LIBRARY_IMPL(_, AutogradPrivateUse1, m) { m.fallback(torch::CppFunction::makeFallthrough()); }

TORCH_LIBRARY_IMPL(aten, CatchAll, m) { m.impl("_has_compatible_shallow_copy_type", TORCH_FN(has_compatible_shallow_copy_type)); }

TORCH_LIBRARY_IMPL(_, AutocastPrivateUse1, m) { m.fallback(torch::CppFunction::makeFallthrough()); }

namespace at::autocast {
namespace {
TORCH_LIBRARY_IMPL(aten, AutocastPrivateUse1, m) {
#define GCU_KERNEL_LOW_PRECISION_FP(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, lower_precision_fp)
  AT_FORALL_LOWER_PRECISION_FP(GCU_KERNEL_LOW_PRECISION_FP)
#define GCU_KERNEL_FP32(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, fp32)
  AT_FORALL_FP32(GCU_KERNEL_FP32)
#define GCU_KERNEL_FP32_SET_OPT_DTYPE(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, fp32_set_opt_dtype)
  AT_FORALL_FP32_SET_OPT_DTYPE(GCU_KERNEL_FP32_SET_OPT_DTYPE)
  AT_FORALL_DIFFERENT_REDISPATCH_SIGNATURE(KERNEL_DIFFERENT_REDISPATCH_SIGNATURE_PRIVATEUSEONE)
#define GCU_KERNEL_PROMOTE(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, promote)
  AT_FORALL_PROMOTE(GCU_KERNEL_PROMOTE)
  m.impl(TORCH_SELECTIVE_NAME("aten::binary_cross_entropy"), TORCH_FN((&binary_cross_entropy_banned)));
}
}  // namespace
}  // namespace at::autocast
