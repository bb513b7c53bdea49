// Declarations of the host-side operator implementations (`torch_gcu::aotops`).
// The list itself is generated from gcu_native_functions.yaml; hand-written
// helpers shared between the implementation files are declared here.
#pragma once

#include "aten/generated/gcu_aot_ops_gen.h"

namespace torch_gcu {
namespace aotops {

// y, h = rms_norm(x + residual): the fused efficient op (also used by the SDPA /
// decoder harness); declared here because python/ binds it directly.
std::tuple<at::Tensor, at::Tensor> rms_norm_residual(const at::Tensor& x, const std::optional<at::Tensor>& residual,
                                                     const at::Tensor& weight, double eps);
at::Tensor rope(const at::Tensor& x, const at::Tensor& cos, const at::Tensor& sin,
                const std::optional<at::Tensor>& positions, bool inplace);
at::Tensor swiglu(const at::Tensor& gate, const at::Tensor& up);
at::Tensor swiglu_packed(const at::Tensor& gate_up);
at::Tensor linear_swiglu(const at::Tensor& x, const at::Tensor& w_gate_up);
at::Tensor linear_rope(const at::Tensor& x, const at::Tensor& w, const at::Tensor& cos, const at::Tensor& sin, int64_t rope_heads);
void rope_kv_append(const at::Tensor& qkv, const at::Tensor& cos, const at::Tensor& sin, const at::Tensor& positions,
                    int64_t q_heads, const at::Tensor& k_cache, const at::Tensor& v_cache);
at::Tensor int32_indices_index(const at::Tensor& self, const c10::List<std::optional<at::Tensor>>& indices);
// (out, logsumexp) of the flash kernel for q (B,Hq,Sq,D), k/v (B,Hkv,Sk,D)
std::tuple<at::Tensor, at::Tensor> sdpa_flash(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                              bool is_causal, std::optional<double> scale);

}  // namespace aotops
}  // namespace torch_gcu
