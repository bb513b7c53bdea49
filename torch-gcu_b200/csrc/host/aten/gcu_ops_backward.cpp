// Backward operators of the decoder layer's pointwise / row ops and of the
// embedding (reference: yaml rows silu_backward.grad_input,
// _softmax_backward_data.out, native_layer_norm_backward, embedding_dense_backward,
// which the reference's S60 build routes to the CPU, codegen/gcu_op_fallback.yaml:8-50).
#include <ATen/native/Resize.h>

#include "aten/aot_ops.h"
#include "aten/bridge.h"

namespace torch_gcu {
namespace aotops {

void silu_backward_grad_input(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor&, const at::Tensor& grad_input) {
  if (grad_input.numel() == 0) return;
  const at::ScalarType common = iter.common_dtype();
  auto prep = [&](const at::Tensor& t) {
    at::Tensor x = t.scalar_type() == common ? t : t.to(common);
    return x.sizes() == grad_input.sizes() ? x : x.expand(grad_input.sizes());
  };
  at::Tensor g = prep(iter.tensor(1)), x = prep(iter.tensor(2));
  at::Tensor work = grad_input.scalar_type() == common ? grad_input : at::empty(grad_input.sizes(), grad_input.options().dtype(common));
  b200Tensor vo = to_b200(work), vg = to_b200(g), vx = to_b200(x);
  cudaStream_t stream = current_stream(grad_input);
  GCU_KERNEL_CALL(b200_silu_backward, stream, &vo, &vg, &vx);
  if (!work.is_same(grad_input)) grad_input.copy_(work);
}

void _softmax_backward_data_out(const at::Tensor& grad_output, const at::Tensor& output, int64_t dim, at::ScalarType input_dtype,
                                const at::Tensor& grad_input) {
  if (grad_input.numel() == 0) return;
  // half_to_float forward: the gradient arrives in fp32 and leaves in the input's type
  const at::ScalarType math = grad_output.scalar_type();
  at::Tensor g = grad_output.contiguous();
  at::Tensor y = (output.scalar_type() == math ? output : output.to(math)).contiguous();
  at::Tensor work = (grad_input.scalar_type() == math && grad_input.is_contiguous())
                        ? grad_input : at::empty(grad_input.sizes(), grad_input.options().dtype(math));
  b200Tensor vo = to_b200(work), vg = to_b200(g), vy = to_b200(y);
  cudaStream_t stream = current_stream(grad_input);
  GCU_KERNEL_CALL(b200_softmax_backward, stream, &vo, &vg, &vy, at::maybe_wrap_dim(dim, grad_output.dim()));
  if (!work.is_same(grad_input)) grad_input.copy_(work);
  (void)input_dtype;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor> native_layer_norm_backward(const at::Tensor& grad_out, const at::Tensor& input,
                                                                          at::IntArrayRef normalized_shape, const at::Tensor& mean,
                                                                          const at::Tensor& rstd,
                                                                          const std::optional<at::Tensor>& weight_opt,
                                                                          const std::optional<at::Tensor>& bias_opt,
                                                                          std::array<bool, 3> output_mask) {
  int64_t N = 1;
  for (int64_t s : normalized_shape) N *= s;
  const int64_t M = N ? input.numel() / N : 0;
  at::Tensor x = input.contiguous();
  at::Tensor g = (grad_out.scalar_type() == x.scalar_type() ? grad_out : grad_out.to(x.scalar_type())).contiguous();
  at::Tensor mu = mean.to(at::kFloat).contiguous().view({-1}), rs = rstd.to(at::kFloat).contiguous().view({-1});
  at::Tensor w;
  if (weight_opt.has_value() && weight_opt->defined()) w = weight_opt->to(x.scalar_type()).contiguous();
  at::Tensor dx, dw, db;
  if (output_mask[0]) dx = at::empty_like(x);
  if (output_mask[1]) dw = w.defined() ? at::empty_like(w) : at::empty(normalized_shape, x.options());
  if (output_mask[2]) {
    if (bias_opt.has_value() && bias_opt->defined()) db = at::empty(bias_opt->sizes(), x.options());
    else db = at::empty(normalized_shape, x.options());
  }
  if (M == 0 || N == 0) {
    if (dw.defined()) dw.zero_();
    if (db.defined()) db.zero_();
    return std::make_tuple(dx, dw, db);
  }
  const size_t ws_bytes = (dw.defined() || db.defined()) ? b200_layer_norm_backward_workspace_size(M, N) : 0;
  at::Tensor ws = at::empty({static_cast<int64_t>(ws_bytes)}, x.options().dtype(at::kByte));
  b200Tensor vg = to_b200(g), vx = to_b200(x), vm = to_b200(mu), vr = to_b200(rs), vdx, vdw, vdb, vw;
  if (dx.defined()) vdx = to_b200(dx);
  if (dw.defined()) vdw = to_b200(dw);
  if (db.defined()) vdb = to_b200(db);
  if (w.defined()) vw = to_b200(w);
  cudaStream_t stream = current_stream(input);
  const b200Tensor* none = nullptr;
  GCU_KERNEL_CALL(b200_layer_norm_backward, stream, dx.defined() ? &vdx : none, dw.defined() ? &vdw : none,
                  db.defined() ? &vdb : none, &vg, &vx, &vm, &vr, w.defined() ? &vw : none, M, N,
                  ws_bytes ? ws.data_ptr() : nullptr, ws_bytes);
  if (dw.defined() && weight_opt.has_value() && weight_opt->defined() && dw.scalar_type() != weight_opt->scalar_type())
    dw = dw.to(weight_opt->scalar_type());
  if (db.defined() && bias_opt.has_value() && bias_opt->defined() && db.scalar_type() != bias_opt->scalar_type())
    db = db.to(bias_opt->scalar_type());
  return std::make_tuple(dx, dw, db);
}

// grad_weight[k] = sum of the grad rows whose index is k, added in ascending position
// order (what the CPU kernel does), through the ordered scatter of index_put.
at::Tensor embedding_dense_backward(const at::Tensor& grad_output, const at::Tensor& indices, int64_t num_weights, int64_t padding_idx,
                                    bool scale_grad_by_freq) {
  TORCH_CHECK(!scale_grad_by_freq, "embedding_dense_backward on the gcu backend does not implement scale_grad_by_freq");
  TORCH_CHECK(indices.scalar_type() == at::kLong || indices.scalar_type() == at::kInt, "embedding_dense_backward: indices must be int64 or int32");
  const int64_t D = grad_output.size(-1);
  at::Tensor gw = at::zeros({num_weights, D}, grad_output.options());
  if (indices.numel() == 0) return gw;
  at::Tensor idx = indices.reshape({-1}).to(at::kLong);
  at::Tensor g2 = grad_output.reshape({-1, D});
  if (padding_idx >= 0) g2 = g2.masked_fill(idx.eq(padding_idx).unsqueeze(1), 0);
  c10::List<std::optional<at::Tensor>> ind;
  ind.push_back(idx);
  aotops::_index_put_impl_(gw, ind, g2, /*accumulate=*/true, /*unsafe=*/false);
  return gw;
}

}  // namespace aotops
}  // namespace torch_gcu

// ------------------------------------------------- log-softmax and NLL loss --
namespace torch_gcu {
namespace aotops {

void _log_softmax_out(const at::Tensor& self, int64_t dim, bool half_to_float, const at::Tensor& out) {
  if (out.numel() == 0) return;
  at::Tensor in = (half_to_float ? self.to(at::kFloat) : self).contiguous();
  at::Tensor work = (out.is_contiguous() && out.scalar_type() == in.scalar_type()) ? out : at::empty(out.sizes(), in.options());
  b200Tensor vo = to_b200(work), vi = to_b200(in);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_log_softmax, stream, &vo, &vi, at::maybe_wrap_dim(dim, self.dim()));
  if (!work.is_same(out)) out.copy_(work);
}

void _log_softmax_backward_data_out(const at::Tensor& grad_output, const at::Tensor& output, int64_t dim, at::ScalarType,
                                    const at::Tensor& out) {
  if (out.numel() == 0) return;
  const at::ScalarType math = grad_output.scalar_type();
  at::Tensor g = grad_output.contiguous();
  at::Tensor y = (output.scalar_type() == math ? output : output.to(math)).contiguous();
  at::Tensor work = (out.is_contiguous() && out.scalar_type() == math) ? out : at::empty(out.sizes(), g.options());
  b200Tensor vo = to_b200(work), vg = to_b200(g), vy = to_b200(y);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_log_softmax_backward, stream, &vo, &vg, &vy, at::maybe_wrap_dim(dim, grad_output.dim()));
  if (!work.is_same(out)) out.copy_(work);
}

void nll_loss_forward_output(const at::Tensor& self, const at::Tensor& target, const std::optional<at::Tensor>& weight_opt,
                             int64_t reduction, int64_t ignore_index, const at::Tensor& output, const at::Tensor& total_weight) {
  // ATen's reduction codes: 0 none, 1 mean, 2 sum
  at::Tensor x = (self.dim() == 1 ? self.unsqueeze(0) : self).contiguous();
  at::Tensor t = (target.dim() == 0 ? target.unsqueeze(0) : target).to(at::kLong).contiguous();
  at::Tensor w;
  if (weight_opt.has_value() && weight_opt->defined()) w = weight_opt->to(x.scalar_type()).contiguous();
  if (x.size(0) == 0) {
    if (reduction != 0) output.fill_(reduction == 1 ? std::numeric_limits<double>::quiet_NaN() : 0.0);
    total_weight.zero_();
    return;
  }
  at::Tensor out_work = output.is_contiguous() ? output : at::empty(output.sizes(), output.options());
  b200Tensor vo = to_b200(out_work), vt = to_b200(total_weight), vx = to_b200(x), vtg = to_b200(t), vw;
  if (w.defined()) vw = to_b200(w);
  cudaStream_t stream = current_stream(self);
  GCU_KERNEL_CALL(b200_nll_loss, stream, &vo, &vt, &vx, &vtg, w.defined() ? &vw : static_cast<const b200Tensor*>(nullptr),
                  static_cast<int32_t>(reduction), ignore_index);
  if (!out_work.is_same(output)) output.copy_(out_work);
}

void nll_loss_backward_grad_input(const at::Tensor& grad_output, const at::Tensor& self, const at::Tensor& target,
                                  const std::optional<at::Tensor>& weight_opt, int64_t reduction, int64_t ignore_index,
                                  const at::Tensor& total_weight, const at::Tensor& grad_input) {
  if (grad_input.numel() == 0) return;
  at::Tensor gi = grad_input.is_contiguous() ? grad_input : at::empty(grad_input.sizes(), grad_input.options());
  at::Tensor gi2 = gi.dim() == 1 ? gi.unsqueeze(0) : gi;
  at::Tensor t = (target.dim() == 0 ? target.unsqueeze(0) : target).to(at::kLong).contiguous();
  at::Tensor go = grad_output.to(gi.scalar_type()).contiguous();
  at::Tensor tw = total_weight.to(gi.scalar_type()).contiguous();
  at::Tensor w;
  if (weight_opt.has_value() && weight_opt->defined()) w = weight_opt->to(gi.scalar_type()).contiguous();
  b200Tensor vgi = to_b200(gi2), vgo = to_b200(go), vtg = to_b200(t), vtw = to_b200(tw), vw;
  if (w.defined()) vw = to_b200(w);
  cudaStream_t stream = current_stream(self);
  GCU_KERNEL_CALL(b200_nll_loss_backward, stream, &vgi, &vgo, &vtg, w.defined() ? &vw : static_cast<const b200Tensor*>(nullptr), &vtw,
                  static_cast<int32_t>(reduction), ignore_index);
  if (!gi.is_same(grad_input)) grad_input.copy_(gi);
}

}  // namespace aotops
}  // namespace torch_gcu
