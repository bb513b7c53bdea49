// Elementwise, reduction and normalisation operators: shape / dtype / stride
// inference is ATen's own structured meta (run by the generated wrapper); this
// file is the single hop from there into the kernel library's C ABI
// (reference: generated aotops::add_out / mul_out / silu_out / sum_out /
// _softmax_out from codegen/gen_aot_ops.py:902-1063, scalar-operand peeling
// codegen/gen_backend_stubs.py:1061-1078, aot_ops/gcu_layer_norm.cpp:17-86).
#include <ATen/AccumulateType.h>
#include <ATen/WrapDimUtilsMulti.h>
#include <ATen/native/Resize.h>

#include "aten/aot_ops.h"
#include "aten/bridge.h"

namespace torch_gcu {
namespace aotops {
namespace {

// An input as the kernel wants it: common dtype, expanded to the output shape.
at::Tensor prep_input(const at::Tensor& t, at::ScalarType common, at::IntArrayRef shape) {
  at::Tensor x = t;
  if (x.scalar_type() != common) x = x.to(common);
  if (x.sizes() != shape) x = x.expand(shape);
  return x;
}

// Output staging: kernels write `common`; a different out dtype gets a copy.
struct OutStage {
  const at::Tensor& out;
  at::Tensor work;
  OutStage(const at::Tensor& o, at::ScalarType common) : out(o) {
    work = o.scalar_type() == common ? o : at::empty(o.sizes(), o.options().dtype(common));
  }
  void finish() {
    if (!work.is_same(out)) out.copy_(work);
  }
};

bool cpu_scalar(at::TensorIteratorBase& iter, int arg) { return iter.is_cpu_scalar(arg); }

enum class Bin { Add, Sub, Mul, Div };

void binary_impl(at::TensorIteratorBase& iter, Bin kind, const at::Scalar& alpha_s, const at::Tensor& out) {
  if (out.numel() == 0) return;
  const at::ScalarType common = iter.common_dtype();
  const at::Tensor& ta = iter.tensor(1);
  const at::Tensor& tb = iter.tensor(2);
  const double alpha = alpha_s.isBoolean() ? static_cast<double>(alpha_s.toBool()) : alpha_s.toDouble();
  OutStage st(out, common);
  b200Tensor vo = to_b200(st.work);
  cudaStream_t stream = current_stream(out);
  bool sa = cpu_scalar(iter, 1), sb = cpu_scalar(iter, 2);
  // the scalar entry points carry the operand as a double: an int64 operand beyond 2^53 would be rounded, so
  // such a scalar goes to the device as a 0-d tensor instead (filled exactly) and takes the tensor kernel
  auto too_big = [&](const at::Tensor& t) {
    if (common != at::kLong || !c10::isIntegralType(t.scalar_type(), false)) return false;
    const int64_t v = t.item().toLong();
    return v > (int64_t(1) << 53) || v < -(int64_t(1) << 53);
  };
  if (sa && too_big(ta)) sa = false;
  if (sb && too_big(tb)) sb = false;
  if (sb && !sa && (kind == Bin::Add || kind == Bin::Sub || kind == Bin::Mul)) {
    // tensor (op) host scalar: scalar kernel, the device never sees the host pointer
    at::Tensor a = prep_input(ta, common, out.sizes());
    b200Tensor va = to_b200(a);
    const double b = tb.item().toDouble();
    if (kind == Bin::Mul) GCU_KERNEL_CALL(b200_mul_scalar, stream, &vo, &va, b);
    else GCU_KERNEL_CALL(b200_add_scalar, stream, &vo, &va, b, kind == Bin::Add ? alpha : -alpha);
    st.finish();
    return;
  }
  if (sa && !sb && kind == Bin::Mul) {
    at::Tensor b = prep_input(tb, common, out.sizes());
    b200Tensor vb = to_b200(b);
    GCU_KERNEL_CALL(b200_mul_scalar, stream, &vo, &vb, ta.item().toDouble());
    st.finish();
    return;
  }
  // general case; a remaining host scalar is materialised on the device first
  auto on_device = [&](const at::Tensor& t) {
    return t.device().is_privateuseone() ? t : at::full({}, t.item(), out.options().dtype(common));
  };
  at::Tensor a = prep_input(on_device(ta), common, out.sizes());
  at::Tensor b = prep_input(on_device(tb), common, out.sizes());
  b200Tensor va = to_b200(a), vb = to_b200(b);
  switch (kind) {
    case Bin::Add: GCU_KERNEL_CALL(b200_add, stream, &vo, &va, &vb, alpha); break;
    case Bin::Sub: GCU_KERNEL_CALL(b200_sub, stream, &vo, &va, &vb, alpha); break;
    case Bin::Mul: GCU_KERNEL_CALL(b200_mul, stream, &vo, &va, &vb); break;
    case Bin::Div: GCU_KERNEL_CALL(b200_div, stream, &vo, &va, &vb); break;
  }
  st.finish();
}

void unary_impl(at::TensorIteratorBase& iter, int32_t op, const at::Tensor& out) {
  if (out.numel() == 0) return;
  const at::ScalarType common = iter.common_dtype();
  at::Tensor a = prep_input(iter.tensor(1), common, out.sizes());
  OutStage st(out, common);
  b200Tensor vo = to_b200(st.work), va = to_b200(a);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_unary, stream, &vo, &va, op);
  st.finish();
}

}  // namespace

void add_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor&, const at::Scalar& alpha, const at::Tensor& out) {
  binary_impl(iter, Bin::Add, alpha, out);
}
void sub_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor&, const at::Scalar& alpha, const at::Tensor& out) {
  binary_impl(iter, Bin::Sub, alpha, out);
}
void mul_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor&, const at::Tensor& out) {
  binary_impl(iter, Bin::Mul, 1, out);
}
void div_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor&, const at::Tensor& out) {
  binary_impl(iter, Bin::Div, 1, out);
}

void silu_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor& out) {
  if (out.numel() == 0) return;
  const at::ScalarType common = iter.common_dtype();
  at::Tensor a = prep_input(iter.tensor(1), common, out.sizes());
  OutStage st(out, common);
  b200Tensor vo = to_b200(st.work), va = to_b200(a);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_silu, stream, &vo, &va);
  st.finish();
}

#define GCU_UNARY(NAME, OP) \
  void NAME(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor& out) { unary_impl(iter, OP, out); }
GCU_UNARY(neg_out, B200_UNARY_NEG)
GCU_UNARY(rsqrt_out, B200_UNARY_RSQRT)
GCU_UNARY(sqrt_out, B200_UNARY_SQRT)
GCU_UNARY(exp_out, B200_UNARY_EXP)
GCU_UNARY(sigmoid_out, B200_UNARY_SIGMOID)
GCU_UNARY(tanh_out, B200_UNARY_TANH)
GCU_UNARY(reciprocal_out, B200_UNARY_RECIPROCAL)
GCU_UNARY(cos_out, B200_UNARY_COS)
GCU_UNARY(sin_out, B200_UNARY_SIN)
GCU_UNARY(log_out, B200_UNARY_LOG)
#undef GCU_UNARY

void gelu_out(at::TensorIteratorBase& iter, const at::Tensor&, c10::string_view approximate, const at::Tensor& out) {
  TORCH_CHECK(approximate == "none", "gelu on the gcu backend implements the erf form (approximate='none'), as CPU ATen's default");
  unary_impl(iter, B200_UNARY_GELU, out);
}

at::Tensor& abs_out(const at::Tensor& self, at::Tensor& out) {
  TORCH_CHECK(at::isFloatingType(self.scalar_type()), "abs on the gcu backend supports floating types");
  at::native::resize_output(out, self.sizes());
  if (self.numel() == 0) return out;
  at::Tensor a = self.scalar_type() == out.scalar_type() ? self : self.to(out.scalar_type());
  b200Tensor vo = to_b200(out), va = to_b200(a);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_unary, stream, &vo, &va, static_cast<int32_t>(B200_UNARY_ABS));
  return out;
}

at::Tensor relu(const at::Tensor& self) {
  at::Tensor out = at::empty_like(self);
  if (self.numel() == 0) return out;
  b200Tensor vo = to_b200(out), va = to_b200(self);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_unary, stream, &vo, &va, static_cast<int32_t>(B200_UNARY_RELU));
  return out;
}

void pow_Tensor_Scalar_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Scalar& exponent, const at::Tensor& out) {
  if (out.numel() == 0) return;
  const at::ScalarType common = iter.common_dtype();
  TORCH_CHECK(at::isFloatingType(common), "pow on the gcu backend supports floating types");
  at::Tensor a = prep_input(iter.tensor(1), common, out.sizes());
  OutStage st(out, common);
  b200Tensor vo = to_b200(st.work), va = to_b200(a);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_pow_scalar, stream, &vo, &va, exponent.toDouble());
  st.finish();
}

// ------------------------------------------------------------- reductions --
namespace {

void reduce_impl(const at::Tensor& self, at::OptionalIntArrayRef dim, const at::Tensor& out, bool mean) {
  if (out.numel() == 0) return;
  const int64_t nd = self.dim();
  std::vector<int64_t> dims;
  if (!dim.has_value() || dim->empty()) {
    for (int64_t d = 0; d < nd; ++d) dims.push_back(d);
  } else {
    auto mask = at::dim_list_to_bitset(dim, nd);
    for (int64_t d = 0; d < nd; ++d)
      if (mask[d]) dims.push_back(d);
  }
  at::Tensor in = self;
  if (mean && in.scalar_type() != out.scalar_type()) in = in.to(out.scalar_type());
  // integer and bool inputs are summed in the output's type (int64 by default), as ATen promotes them
  if (!mean && at::isIntegralType(in.scalar_type(), /*includeBool=*/true) && in.scalar_type() != out.scalar_type())
    in = in.to(out.scalar_type());
  // the kernel wants the reduced dimensions adjacent: permute them to the end otherwise
  bool adjacent = true;
  for (size_t i = 1; i < dims.size(); ++i) adjacent = adjacent && dims[i] == dims[i - 1] + 1;
  if (!adjacent) {
    std::vector<int64_t> perm;
    std::vector<bool> red(nd, false);
    for (int64_t d : dims) red[d] = true;
    for (int64_t d = 0; d < nd; ++d)
      if (!red[d]) perm.push_back(d);
    const int64_t kept = static_cast<int64_t>(perm.size());
    for (int64_t d : dims) perm.push_back(d);
    in = in.permute(perm);
    for (size_t i = 0; i < dims.size(); ++i) dims[i] = kept + static_cast<int64_t>(i);
  }
  in = in.contiguous();
  at::Tensor work = out.is_contiguous() ? out : at::empty(out.sizes(), out.options());
  b200Tensor vo = to_b200(work), vi = to_b200(in);
  cudaStream_t stream = current_stream(out);
  const size_t ws_bytes = b200_sum_workspace_size(&vi, dims.data(), static_cast<int32_t>(dims.size()));
  at::Tensor ws;
  void* ws_ptr = nullptr;
  if (ws_bytes) {
    ws = alloc_workspace(ws_bytes, out);
    ws_ptr = ws.data_ptr();
  }
  GCU_KERNEL_CALL(b200_sum, stream, &vo, &vi, dims.data(), static_cast<int32_t>(dims.size()), mean ? 1 : 0, ws_ptr, ws_bytes);
  if (!work.is_same(out)) out.copy_(work);
}

}  // namespace

void sum_IntList_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool, std::optional<at::ScalarType>, const at::Tensor& out) {
  reduce_impl(self, dim, out, false);
}
void mean_out(const at::Tensor& self, at::OptionalIntArrayRef dim, bool, std::optional<at::ScalarType>, const at::Tensor& out) {
  reduce_impl(self, dim, out, true);
}

void _softmax_out(const at::Tensor& self, int64_t dim, bool half_to_float, const at::Tensor& out) {
  if (out.numel() == 0) return;
  if (half_to_float) TORCH_CHECK(out.scalar_type() == at::kFloat, "softmax half_to_float needs a float output");
  at::Tensor in = self.contiguous();
  at::Tensor work = out.is_contiguous() ? out : at::empty(out.sizes(), out.options());
  b200Tensor vo = to_b200(work), vi = to_b200(in);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_softmax, stream, &vo, &vi, at::maybe_wrap_dim(dim, self.dim()));
  if (!work.is_same(out)) out.copy_(work);
}

// y, mean, rstd; statistics in the accumulate type and shaped
// input.shape[:axis] + [1]*len(normalized_shape) (reference: gcu_layer_norm.cpp:43-47,79-85)
std::tuple<at::Tensor, at::Tensor, at::Tensor> native_layer_norm(const at::Tensor& input, at::IntArrayRef normalized_shape,
                                                                 const std::optional<at::Tensor>& weight_opt,
                                                                 const std::optional<at::Tensor>& bias_opt, double eps) {
  const int64_t nnd = static_cast<int64_t>(normalized_shape.size());
  TORCH_CHECK(nnd >= 1 && input.dim() >= nnd, "normalized_shape does not match the input");
  const int64_t axis = input.dim() - nnd;
  for (int64_t i = 0; i < nnd; ++i)
    TORCH_CHECK(input.size(axis + i) == normalized_shape[i], "Given normalized_shape=", normalized_shape,
                ", expected input with shape [*, ", normalized_shape, "], but got input of size", input.sizes());
  int64_t N = 1;
  for (int64_t s : normalized_shape) N *= s;
  const int64_t M = N ? input.numel() / N : 0;
  at::Tensor x = input.contiguous();
  at::Tensor w, b;
  if (weight_opt.has_value() && weight_opt->defined()) {
    TORCH_CHECK(weight_opt->sizes().equals(normalized_shape), "weight shape must equal normalized_shape");
    w = weight_opt->to(x.scalar_type()).contiguous();
  }
  if (bias_opt.has_value() && bias_opt->defined()) {
    TORCH_CHECK(bias_opt->sizes().equals(normalized_shape), "bias shape must equal normalized_shape");
    b = bias_opt->to(x.scalar_type()).contiguous();
  }
  at::Tensor y = at::empty_like(x, at::MemoryFormat::Contiguous);
  const at::ScalarType acc = at::toAccumulateType(x.scalar_type(), /*is_cuda=*/true);
  at::Tensor mean = at::empty({M}, x.options().dtype(acc));
  at::Tensor rstd = at::empty({M}, x.options().dtype(acc));
  if (M > 0) {
    b200Tensor vy = to_b200(y), vm = to_b200(mean), vr = to_b200(rstd), vx = to_b200(x), vw, vb;
    if (w.defined()) vw = to_b200(w);
    if (b.defined()) vb = to_b200(b);
    cudaStream_t stream = current_stream(x);
    GCU_KERNEL_CALL(b200_native_layer_norm, stream, &vy, &vm, &vr, &vx, M, N, w.defined() ? &vw : nullptr,
                    b.defined() ? &vb : nullptr, eps);
  }
  std::vector<int64_t> stat_shape;
  for (int64_t i = 0; i < axis; ++i) stat_shape.push_back(input.size(i));
  for (int64_t i = 0; i < nnd; ++i) stat_shape.push_back(1);
  return std::make_tuple(std::move(y), mean.view(stat_shape), rstd.view(stat_shape));
}

}  // namespace aotops
}  // namespace torch_gcu
