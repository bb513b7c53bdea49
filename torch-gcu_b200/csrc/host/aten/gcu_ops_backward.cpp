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
