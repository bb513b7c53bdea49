// Flash attention forward, the SDPA backend choice, and the fused efficient ops
// (reference: aot_ops/gcu_attention.cpp:21-80, shape_inference/attention.cpp:
// 67-192,424-446, RegisterSPDA.cpp:137-178,223-275; the fused RMSNorm+residual,
// RoPE and SwiGLU entries have no reference kernel -- the reference runs them as
// chains of pointwise ops -- and sit beside its one efficient op,
// efficient_ops/ops.cpp:335-342).
#include <ATen/native/DispatchStub.h>
#include <ATen/native/transformers/attention.h>
#include <ATen/native/transformers/sdp_utils_cpp.h>
#include <torch/library.h>

#include "aten/aot_ops.h"
#include "aten/bridge.h"

namespace torch_gcu {
namespace aotops {

std::tuple<at::Tensor, at::Tensor> sdpa_flash(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v, bool is_causal,
                                              std::optional<double> scale) {
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "flash attention expects (B,H,S,D) query, key and value");
  const int64_t B = q.size(0), H = q.size(1), S = q.size(2), D = q.size(3);
  // allocated (B,S,H,D) and returned transposed, as the reference's shape inference does
  at::Tensor out = at::empty({B, S, H, D}, q.options()).transpose(1, 2);
  at::Tensor lse = at::empty({B, H, S}, q.options().dtype(at::kFloat));
  if (q.numel() == 0) return std::make_tuple(out, lse);
  auto last_contig = [](const at::Tensor& t) { return t.stride(-1) == 1 ? t : t.contiguous(); };
  at::Tensor qc = last_contig(q), kc = last_contig(k), vc = last_contig(v);
  b200Tensor vo = to_b200(out), vl = to_b200(lse), vq = to_b200(qc), vk = to_b200(kc), vv = to_b200(vc);
  const double sc = scale.has_value() ? *scale : 1.0 / std::sqrt(static_cast<double>(D));
  cudaStream_t stream = current_stream(q);
  GCU_KERNEL_CALL(b200_sdpa_flash_fwd, stream, &vo, &vl, &vq, &vk, &vv, is_causal ? 1 : 0, sc);
  return std::make_tuple(out, lse);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, c10::SymInt, c10::SymInt, at::Tensor, at::Tensor, at::Tensor>
_scaled_dot_product_flash_attention(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, double dropout_p,
                                    bool is_causal, bool return_debug_mask, std::optional<double> scale) {
  TORCH_CHECK(dropout_p == 0.0, "flash attention on the gcu backend does not implement dropout");
  TORCH_CHECK(!return_debug_mask, "flash attention on the gcu backend has no debug mask");
  auto [out, lse] = sdpa_flash(query, key, value, is_causal, scale);
  at::Tensor empty_long = at::empty({0}, query.options().dtype(at::kLong));
  at::Tensor none;
  return std::make_tuple(out, lse, at::Tensor(), at::Tensor(), c10::SymInt(query.size(2)), c10::SymInt(key.size(2)),
                         empty_long, empty_long.clone(), at::empty({0}, query.options()));
}

// What PyTorch's composite scaled_dot_product_attention calls for a PrivateUse1
// device when the backend choice is "overrideable": the same flash kernel.
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, c10::SymInt, c10::SymInt, at::Tensor, at::Tensor, at::Tensor>
_scaled_dot_product_fused_attention_overrideable(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value,
                                                 const std::optional<at::Tensor>& attn_bias, double dropout_p, bool is_causal,
                                                 bool return_debug_mask, std::optional<double> scale) {
  TORCH_CHECK(!(attn_bias.has_value() && attn_bias->defined()), "flash attention on the gcu backend takes no attention bias");
  return aotops::_scaled_dot_product_flash_attention(query, key, value, dropout_p, is_causal, return_debug_mask, scale);
}

// Backward of the flash kernel: dq, dk, dv (reference: aot_ops/gcu_attention.cpp:135-203).
static std::tuple<at::Tensor, at::Tensor, at::Tensor> sdpa_flash_backward(const at::Tensor& grad_out, const at::Tensor& q,
                                                                          const at::Tensor& k, const at::Tensor& v,
                                                                          const at::Tensor& out, const at::Tensor& lse, bool is_causal,
                                                                          std::optional<double> scale) {
  TORCH_CHECK(q.dim() == 4 && q.size(3) == 128, "flash attention backward on the gcu backend supports head dim 128");
  auto last_contig = [](const at::Tensor& t) { return t.stride(-1) == 1 ? t : t.contiguous(); };
  at::Tensor go = last_contig(grad_out), qc = last_contig(q), kc = last_contig(k), vc = last_contig(v), oc = last_contig(out);
  at::Tensor l = lse.contiguous();
  // gradients in the layout the forward uses for its output: (B,S,H,D) storage viewed (B,H,S,D)
  at::Tensor dq = at::empty({q.size(0), q.size(2), q.size(1), q.size(3)}, q.options()).transpose(1, 2);
  at::Tensor dk = at::empty({k.size(0), k.size(2), k.size(1), k.size(3)}, k.options()).transpose(1, 2);
  at::Tensor dv = at::empty({v.size(0), v.size(2), v.size(1), v.size(3)}, v.options()).transpose(1, 2);
  if (q.numel() == 0 || k.numel() == 0) return std::make_tuple(dq.zero_(), dk.zero_(), dv.zero_());
  b200Tensor vdq = to_b200(dq), vdk = to_b200(dk), vdv = to_b200(dv), vgo = to_b200(go), vq = to_b200(qc), vk = to_b200(kc),
             vv = to_b200(vc), vo = to_b200(oc), vl = to_b200(l);
  const size_t ws_bytes = b200_sdpa_flash_bwd_workspace_size(&vq);
  at::Tensor ws = at::empty({static_cast<int64_t>(ws_bytes)}, q.options().dtype(at::kByte));
  const double sc = scale.has_value() ? *scale : 1.0 / std::sqrt(static_cast<double>(q.size(3)));
  const c10::OptionalDeviceGuard guard(q.device());
  cudaStream_t stream = current_stream(q);
  GCU_KERNEL_CALL(b200_sdpa_flash_bwd, stream, &vdq, &vdk, &vdv, &vgo, &vq, &vk, &vv, &vo, &vl, is_causal ? 1 : 0, sc, ws.data_ptr(),
                  ws_bytes);
  return std::make_tuple(dq, dk, dv);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> _scaled_dot_product_flash_attention_backward(
    const at::Tensor& grad_out, const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, const at::Tensor& out,
    const at::Tensor& logsumexp, const at::Tensor&, const at::Tensor&, int64_t, int64_t, double dropout_p, bool is_causal,
    const at::Tensor&, const at::Tensor&, std::optional<double> scale) {
  TORCH_CHECK(dropout_p == 0.0, "flash attention on the gcu backend does not implement dropout");
  return sdpa_flash_backward(grad_out, query, key, value, out, logsumexp, is_causal, scale);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> _scaled_dot_product_fused_attention_overrideable_backward(
    const at::Tensor& grad_out, const at::Tensor& query, const at::Tensor& key, const at::Tensor& value, const at::Tensor& attn_bias,
    std::array<bool, 4> grad_input_mask, const at::Tensor& out, const at::Tensor& logsumexp, const at::Tensor&, const at::Tensor&, int64_t,
    int64_t, double dropout_p, bool is_causal, const at::Tensor&, const at::Tensor&, std::optional<double> scale) {
  TORCH_CHECK(dropout_p == 0.0, "flash attention on the gcu backend does not implement dropout");
  TORCH_CHECK(!attn_bias.defined() || attn_bias.numel() == 0, "flash attention on the gcu backend takes no attention bias");
  (void)grad_input_mask;
  auto [dq, dk, dv] = sdpa_flash_backward(grad_out, query, key, value, out, logsumexp, is_causal, scale);
  return std::make_tuple(dq, dk, dv, at::Tensor());
}

// --------------------------------------------------------------- fused ops --
std::tuple<at::Tensor, at::Tensor> rms_norm_residual(const at::Tensor& x, const std::optional<at::Tensor>& residual,
                                                     const at::Tensor& weight, double eps) {
  TORCH_CHECK(x.dim() >= 1 && weight.dim() == 1 && weight.size(0) == x.size(-1), "rms_norm_residual: weight must be (hidden,)");
  at::Tensor xc = x.contiguous();
  at::Tensor w = weight.scalar_type() == x.scalar_type() ? weight.contiguous() : weight.to(x.scalar_type()).contiguous();
  at::Tensor y = at::empty_like(xc);
  const c10::OptionalDeviceGuard guard(x.device());
  cudaStream_t stream = current_stream(x);
  b200Tensor vy = to_b200(y), vx = to_b200(xc), vw = to_b200(w);
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->sizes() == x.sizes() && residual->scalar_type() == x.scalar_type(),
                "rms_norm_residual: residual must match x");
    at::Tensor rc = residual->contiguous();
    at::Tensor h = at::empty_like(xc);
    b200Tensor vr = to_b200(rc), vh = to_b200(h);
    GCU_KERNEL_CALL(b200_rms_norm_residual, stream, &vy, &vh, &vx, &vr, &vw, eps);
    return std::make_tuple(y, h);
  }
  GCU_KERNEL_CALL(b200_rms_norm_residual, stream, &vy, static_cast<const b200Tensor*>(nullptr), &vx,
                  static_cast<const b200Tensor*>(nullptr), &vw, eps);
  return std::make_tuple(y, xc);
}

at::Tensor rope(const at::Tensor& x, const at::Tensor& cos, const at::Tensor& sin, const std::optional<at::Tensor>& positions,
                bool inplace) {
  TORCH_CHECK(x.dim() == 4, "rope: x must be (B,S,H,D)");
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat, "rope: cos/sin tables must be float32 (P, D/2)");
  const c10::OptionalDeviceGuard guard(x.device());
  at::Tensor src = x.stride(-1) == 1 ? x : x.contiguous();
  at::Tensor out = inplace && src.is_same(x) ? x : at::empty_like(src, at::MemoryFormat::Contiguous);
  at::Tensor c = cos.contiguous(), s = sin.contiguous();
  b200Tensor vo = to_b200(out), vx = to_b200(src), vc = to_b200(c), vs = to_b200(s), vp;
  at::Tensor pos;
  if (positions.has_value() && positions->defined()) {
    pos = positions->to(x.device(), at::kLong);
    vp = to_b200(pos);
  }
  cudaStream_t stream = current_stream(x);
  GCU_KERNEL_CALL(b200_rope, stream, &vo, &vx, &vc, &vs, pos.defined() ? &vp : static_cast<const b200Tensor*>(nullptr));
  return out;
}

// Decode step: rotate the query heads of qkv (B, S, q_heads + 2 k_heads, D) in place and write the rotated key
// heads and the value heads into the caches (B, k_heads, T, D) at positions (B, S), in one launch.
void rope_kv_append(const at::Tensor& qkv, const at::Tensor& cos, const at::Tensor& sin, const at::Tensor& positions,
                    int64_t q_heads, const at::Tensor& k_cache, const at::Tensor& v_cache) {
  TORCH_CHECK(qkv.dim() == 4 && k_cache.dim() == 4 && v_cache.dim() == 4, "rope_kv_append: qkv (B,S,H,D) and caches (B,Hk,T,D) expected");
  TORCH_CHECK(qkv.stride(-1) == 1 && k_cache.stride(-1) == 1 && v_cache.stride(-1) == 1, "rope_kv_append: head dim must be contiguous");
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat, "rope_kv_append: cos/sin tables must be float32 (P, D/2)");
  TORCH_CHECK(k_cache.device() == qkv.device() && v_cache.device() == qkv.device(), "rope_kv_append: operands on one device");
  const c10::OptionalDeviceGuard guard(qkv.device());
  at::Tensor c = cos.contiguous(), s = sin.contiguous();
  at::Tensor pos = positions.to(qkv.device(), at::kLong);
  b200Tensor vq = to_b200(qkv), vc = to_b200(c), vs = to_b200(s), vp = to_b200(pos), vk = to_b200(k_cache), vv = to_b200(v_cache);
  cudaStream_t stream = current_stream(qkv);
  GCU_KERNEL_CALL(b200_rope_kv_append, stream, &vq, &vc, &vs, &vp, q_heads, k_cache.size(1), &vk, &vv);
}

static at::Tensor swiglu_2d(const at::Tensor& gate, const at::Tensor& up, at::IntArrayRef out_shape) {
  at::Tensor out = at::empty(out_shape, gate.options());
  if (out.numel() == 0) return out;
  const int64_t cols = out_shape.back();
  at::Tensor o2 = out.view({-1, cols});
  b200Tensor vo = to_b200(o2), vg = to_b200(gate), vu = to_b200(up);
  const c10::OptionalDeviceGuard guard(gate.device());
  cudaStream_t stream = current_stream(gate);
  GCU_KERNEL_CALL(b200_swiglu, stream, &vo, &vg, &vu);
  return out;
}

at::Tensor swiglu(const at::Tensor& gate, const at::Tensor& up) {
  TORCH_CHECK(gate.sizes() == up.sizes() && gate.scalar_type() == up.scalar_type() && gate.dim() >= 1,
              "swiglu: gate and up must agree in shape and dtype");
  const int64_t cols = gate.size(-1);
  at::Tensor g = gate.contiguous().view({-1, cols}), u = up.contiguous().view({-1, cols});
  return swiglu_2d(g, u, gate.sizes());
}

// gate and up as the two halves of one projection output (..., 2F)
at::Tensor swiglu_packed(const at::Tensor& gate_up) {
  TORCH_CHECK(gate_up.dim() >= 1 && gate_up.size(-1) % 2 == 0, "swiglu_packed: last dim must be even");
  const int64_t f = gate_up.size(-1) / 2;
  at::Tensor gu = gate_up.contiguous().view({-1, 2 * f});
  std::vector<int64_t> shape = gate_up.sizes().vec();
  shape.back() = f;
  return swiglu_2d(gu.narrow(1, 0, f), gu.narrow(1, f, f), shape);
}

// x (..., K) times a fused gate/up weight (2F, K): large row counts run the GEMM whose
// epilogue applies silu(gate) * up, and so do few rows (a decode step) whenever the kernel
// library has a few-row form for the weight (one equal tile per SM, or K split over clusters);
// otherwise mm followed by the activation kernel.
at::Tensor linear_swiglu(const at::Tensor& x, const at::Tensor& w_gate_up) {
  TORCH_CHECK(x.dim() >= 1 && w_gate_up.dim() == 2 && w_gate_up.size(0) % 2 == 0 && w_gate_up.size(1) == x.size(-1),
              "linear_swiglu: x (..., K) and w (2F, K) expected");
  TORCH_CHECK(x.scalar_type() == w_gate_up.scalar_type(), "linear_swiglu: x and w must share a dtype");
  const int64_t k = x.size(-1), f = w_gate_up.size(0) / 2;
  at::Tensor x2 = x.contiguous().view({-1, k});
  std::vector<int64_t> shape = x.sizes().vec();
  shape.back() = f;
  const c10::OptionalDeviceGuard guard(x.device());
  const bool fused = (x2.size(0) >= 512 || b200_mm_swiglu_few_rows(x2.size(0), f, k) != 0) &&
                     (x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf) && k % 8 == 0;
  if (!fused) return swiglu_packed(at::mm(x2, w_gate_up.t())).view(shape);
  at::Tensor w = w_gate_up.contiguous();
  at::Tensor out = at::empty({x2.size(0), f}, x.options());
  cudaStream_t stream = current_stream(x);
  b200Tensor vo = to_b200(out), va = to_b200(x2), vw = to_b200(w);
  GCU_KERNEL_CALL(b200_mm_swiglu, stream, &vo, &va, &vw);
  return out.view(shape);
}

// x (B, S, K) times a fused qkv weight (N, K), RoPE (heads of 128, position = index along S) on the first
// rope_heads heads: one GEMM whose epilogue rotates; small or odd problems run mm followed by the rope kernel.
at::Tensor linear_rope(const at::Tensor& x, const at::Tensor& w, const at::Tensor& cos, const at::Tensor& sin, int64_t rope_heads) {
  TORCH_CHECK(x.dim() == 3 && w.dim() == 2 && w.size(1) == x.size(2) && w.size(0) % 128 == 0,
              "linear_rope: x (B, S, K) and w (heads * 128, K) expected");
  TORCH_CHECK(x.scalar_type() == w.scalar_type(), "linear_rope: x and w must share a dtype");
  TORCH_CHECK(cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat && cos.dim() == 2 && cos.size(1) == 64 &&
              cos.sizes() == sin.sizes() && cos.size(0) >= x.size(1), "linear_rope: cos / sin must be float32 (positions >= S, 64)");
  const int64_t B = x.size(0), S = x.size(1), K = x.size(2), N = w.size(0), heads = N / 128;
  TORCH_CHECK(rope_heads >= 0 && rope_heads <= heads, "linear_rope: rope_heads out of range");
  at::Tensor x2 = x.contiguous().view({B * S, K});
  const bool fused = B * S >= 512 && (x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kHalf) && K % 8 == 0;
  if (!fused) {
    at::Tensor out = at::mm(x2, w.t()).view({B, S, heads, 128});
    if (rope_heads > 0) rope(out.narrow(2, 0, rope_heads), cos, sin, std::nullopt, true);
    return out;
  }
  at::Tensor wc = w.contiguous(), c = cos.contiguous(), s = sin.contiguous();
  at::Tensor out = at::empty({B * S, N}, x.options());
  const c10::OptionalDeviceGuard guard(x.device());
  cudaStream_t stream = current_stream(x);
  b200Tensor vo = to_b200(out), va = to_b200(x2), vw = to_b200(wc), vc = to_b200(c), vs = to_b200(s);
  GCU_KERNEL_CALL(b200_mm_rope, stream, &vo, &va, &vw, &vc, &vs, S, rope_heads * 128);
  return out.view({B, S, heads, 128});
}

// ------------------------------------------------------ SDPA backend choice --
// flash (reported as "overrideable", the slot PyTorch gives PrivateUse1 backends)
// when the kernel can take the problem, otherwise the math composite
// (reference priority flash -> mem-efficient -> math, RegisterSPDA.cpp:223-275;
// flash gate :137-178).
int64_t fused_sdp_choice(const at::Tensor& query, const at::Tensor& key, const at::Tensor& value,
                                const std::optional<at::Tensor>& attn_mask, double dropout_p, bool is_causal,
                                std::optional<double>, bool) {
  const bool has_mask = attn_mask.has_value() && attn_mask->defined();
  const auto dt = query.scalar_type();
  const bool flash_ok = !has_mask && dropout_p == 0.0 && query.dim() == 4 && key.dim() == 4 && value.dim() == 4 &&
                        (dt == at::kBFloat16 || dt == at::kHalf) && key.scalar_type() == dt && value.scalar_type() == dt &&
                        (query.size(-1) == 64 || query.size(-1) == 128) && key.size(-1) == query.size(-1) &&
                        value.size(-1) == query.size(-1) && key.size(1) > 0 && query.size(1) % key.size(1) == 0 &&
                        (!is_causal || query.size(2) == key.size(2)) && key.size(2) > 0 &&
                        // the backward kernel exists for head dim 128; other sizes train through the math path
                        (query.size(-1) == 128 || !(query.requires_grad() || key.requires_grad() || value.requires_grad()));
  return static_cast<int64_t>(flash_ok ? sdp::SDPBackend::overrideable : sdp::SDPBackend::math);
}

}  // namespace aotops
}  // namespace torch_gcu

// The composite scaled_dot_product_attention asks the per-device dispatch stub;
// the operator form is registered too for callers that go through the dispatcher.
namespace at::native {
REGISTER_PRIVATEUSE1_DISPATCH(_fused_sdp_choice_stub, &torch_gcu::aotops::fused_sdp_choice)
}  // namespace at::native

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("_fused_sdp_choice", TORCH_FN(torch_gcu::aotops::fused_sdp_choice));
}
