// Comparison, selection, clamping, extreme and generator operators: ATen's meta
// functions do shape / dtype inference, this file marshals into the kernel
// library (reference: the generated aotops::eq_out … ge_out, where, masked_fill_,
// maximum_out, clamp_out, argmax_out, max_dim, amax_out, arange_out, triu_out rows
// of codegen/gcu_native_functions.yaml:198-617 and their topsaten calls).
#include <ATen/ExpandUtils.h>
#include <ATen/WrapDimUtilsMulti.h>
#include <ATen/native/Resize.h>
#include <ATen/ops/sort.h>

#include "aten/aot_ops.h"
#include "aten/bridge.h"

namespace torch_gcu {
namespace aotops {
namespace {

at::Tensor as_common(const at::Tensor& t, at::ScalarType common, at::IntArrayRef shape, const at::TensorOptions& dev_opts) {
  at::Tensor x = t;
  if (!x.device().is_privateuseone()) x = at::full({}, x.item(), dev_opts.dtype(common));  // a wrapped host scalar
  if (x.scalar_type() != common) x = x.to(common);
  if (x.sizes() != shape) x = x.expand(shape);
  return x;
}

// A bool (or other dtype) result computed into `work`, copied to `out` when they differ.
struct Staged {
  const at::Tensor& out;
  at::Tensor work;
  Staged(const at::Tensor& o, at::ScalarType want) : out(o) {
    work = (o.scalar_type() == want) ? o : at::empty(o.sizes(), o.options().dtype(want));
  }
  void finish() {
    if (!work.is_same(out)) out.copy_(work);
  }
};

void compare_tensor(at::TensorIteratorBase& iter, int32_t op, const at::Tensor& out) {
  if (out.numel() == 0) return;
  const at::ScalarType common = iter.common_dtype();
  Staged st(out, at::kBool);
  b200Tensor vo = to_b200(st.work);
  cudaStream_t stream = current_stream(out);
  const at::Tensor& ta = iter.tensor(1);
  const at::Tensor& tb = iter.tensor(2);
  if (iter.is_cpu_scalar(2) && !iter.is_cpu_scalar(1)) {
    at::Tensor a = as_common(ta, common, out.sizes(), out.options());
    b200Tensor va = to_b200(a);
    GCU_KERNEL_CALL(b200_compare_scalar, stream, &vo, &va, tb.item().toDouble(), op);
  } else {
    at::Tensor a = as_common(ta, common, out.sizes(), out.options()), b = as_common(tb, common, out.sizes(), out.options());
    b200Tensor va = to_b200(a), vb = to_b200(b);
    GCU_KERNEL_CALL(b200_compare, stream, &vo, &va, &vb, op);
  }
  st.finish();
}

void logical_binary(const at::Tensor& self, const at::Tensor& other, int32_t op, at::Tensor& out) {
  const auto shape = at::infer_size(self.sizes(), other.sizes());
  at::native::resize_output(out, shape);
  if (out.numel() == 0) return;
  const at::ScalarType common = at::result_type(self, other);
  Staged st(out, at::kBool);
  at::Tensor a = as_common(self, common, shape, out.options()), b = as_common(other, common, shape, out.options());
  b200Tensor vo = to_b200(st.work), va = to_b200(a), vb = to_b200(b);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_compare, stream, &vo, &va, &vb, op);
  st.finish();
}

void minmax_tensor(at::TensorIteratorBase& iter, bool is_max, const at::Tensor& out) {
  if (out.numel() == 0) return;
  const at::ScalarType common = iter.common_dtype();
  Staged st(out, common);
  at::Tensor a = as_common(iter.tensor(1), common, out.sizes(), out.options());
  at::Tensor b = as_common(iter.tensor(2), common, out.sizes(), out.options());
  b200Tensor vo = to_b200(st.work), va = to_b200(a), vb = to_b200(b);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_minmax, stream, &vo, &va, &vb, is_max ? 1 : 0);
  st.finish();
}

void clamp_impl(at::TensorIteratorBase& iter, const std::optional<at::Scalar>& lo, const std::optional<at::Scalar>& hi,
                const at::Tensor& out) {
  if (out.numel() == 0) return;
  const at::ScalarType common = iter.common_dtype();
  Staged st(out, common);
  at::Tensor a = as_common(iter.tensor(1), common, out.sizes(), out.options());
  b200Tensor vo = to_b200(st.work), va = to_b200(a);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_clamp, stream, &vo, &va, lo.has_value() ? 1 : 0, lo.has_value() ? lo->toDouble() : 0.0,
                  hi.has_value() ? 1 : 0, hi.has_value() ? hi->toDouble() : 0.0);
  st.finish();
}

// Values and / or indices of the extreme along `dim` of `self`, written to outputs that ATen's
// meta sized (with or without the kept dim: same element order either way).
void extreme_dim(const at::Tensor& self, int64_t dim, bool is_max, const at::Tensor* values, const at::Tensor* indices) {
  const at::Tensor src = self.dim() == 0 ? self.reshape({1}).contiguous() : self.contiguous();
  const int64_t d = self.dim() == 0 ? 0 : at::maybe_wrap_dim(dim, self.dim());
  const int64_t n_out = src.size(d) == 0 ? 0 : src.numel() / src.size(d);
  TORCH_CHECK(src.size(d) > 0 || src.numel() == 0, "max/min/argmax/argmin: cannot reduce over an empty dimension");
  if (n_out == 0) return;
  at::Tensor vwork, iwork;
  if (values) vwork = (values->is_contiguous() && values->scalar_type() == src.scalar_type()) ? *values
                                                                                                : at::empty({n_out}, src.options());
  if (indices) iwork = (indices->is_contiguous() && indices->scalar_type() == at::kLong) ? *indices
                                                                                          : at::empty({n_out}, src.options().dtype(at::kLong));
  b200Tensor vs = to_b200(src), vv, vi;
  if (values) vv = to_b200(vwork.view({n_out}));
  if (indices) vi = to_b200(iwork.view({n_out}));
  cudaStream_t stream = current_stream(self);
  GCU_KERNEL_CALL(b200_extreme_dim, stream, values ? &vv : static_cast<const b200Tensor*>(nullptr),
                  indices ? &vi : static_cast<const b200Tensor*>(nullptr), &vs, d, is_max ? 1 : 0);
  if (values && !vwork.is_same(*values)) values->copy_(vwork.view(values->sizes()));
  if (indices && !iwork.is_same(*indices)) indices->copy_(iwork.view(indices->sizes()));
}

at::Tensor extreme_all(const at::Tensor& self, bool is_max) {
  TORCH_CHECK(self.numel() > 0, is_max ? "max" : "min", "(): expected a non-empty tensor");
  at::Tensor flat = self.contiguous().view({-1});
  // two stages so that a large tensor is not reduced by a single warp
  int64_t rows = 1;
  for (int64_t r = 4096; r > 1; r >>= 1)
    if (flat.numel() % r == 0 && flat.numel() / r >= 32) { rows = r; break; }
  at::Tensor out = at::empty({}, self.options());
  if (rows > 1) {
    at::Tensor part = at::empty({rows}, self.options());
    extreme_dim(flat.view({rows, flat.numel() / rows}), 1, is_max, &part, nullptr);
    flat = part;
  }
  at::Tensor o1 = out.view({1});
  extreme_dim(flat.view({1, flat.numel()}), 1, is_max, &o1, nullptr);
  return out;
}

void amax_impl(const at::Tensor& self, at::IntArrayRef dim, bool keepdim, bool is_max, const at::Tensor& out) {
  if (out.numel() == 0) return;
  if (self.dim() == 0) { out.copy_(self); return; }
  std::vector<int64_t> dims;
  if (dim.empty()) for (int64_t i = 0; i < self.dim(); ++i) dims.push_back(i);
  else for (int64_t d : dim) dims.push_back(at::maybe_wrap_dim(d, self.dim()));
  std::sort(dims.begin(), dims.end(), std::greater<int64_t>());
  at::Tensor cur = self;
  for (size_t k = 0; k < dims.size(); ++k) {   // one dim at a time, innermost first, keeping the dim
    std::vector<int64_t> shape = cur.sizes().vec();
    shape[dims[k]] = 1;
    const bool last = k + 1 == dims.size();
    at::Tensor nxt = (last && out.is_contiguous()) ? out.view(shape) : at::empty(shape, cur.options());
    extreme_dim(cur, dims[k], is_max, &nxt, nullptr);
    cur = nxt;
  }
  (void)keepdim;
  if (cur.data_ptr() != out.data_ptr()) out.copy_(cur.view(out.sizes()));
}

void tri_impl(const at::Tensor& self, int64_t diagonal, bool upper, const at::Tensor& out) {
  if (out.numel() == 0) return;
  at::Tensor src = self.contiguous();
  at::Tensor work = out.is_contiguous() ? out : at::empty(out.sizes(), out.options());
  b200Tensor vo = to_b200(work), vs = to_b200(src);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_tri, stream, &vo, &vs, diagonal, upper ? 1 : 0);
  if (!work.is_same(out)) out.copy_(work);
}

}  // namespace

#define GCU_COMPARE(NAME, OP)                                                                                              \
  void NAME##_Tensor_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor&, const at::Tensor& out) {     \
    compare_tensor(iter, OP, out);                                                                                         \
  }                                                                                                                        \
  void NAME##_Scalar_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Scalar&, const at::Tensor& out) {     \
    compare_tensor(iter, OP, out);                                                                                         \
  }
GCU_COMPARE(eq, B200_CMP_EQ)
GCU_COMPARE(ne, B200_CMP_NE)
GCU_COMPARE(lt, B200_CMP_LT)
GCU_COMPARE(le, B200_CMP_LE)
GCU_COMPARE(gt, B200_CMP_GT)
GCU_COMPARE(ge, B200_CMP_GE)
#undef GCU_COMPARE

at::Tensor& where_self_out(const at::Tensor& condition, const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
  TORCH_CHECK(condition.scalar_type() == at::kBool, "where expected condition to be a boolean tensor, but got a tensor with dtype ",
              condition.scalar_type());
  const at::ScalarType common = at::result_type(self, other);
  const auto shape = at::infer_size(at::infer_size(condition.sizes(), self.sizes()), other.sizes());
  at::native::resize_output(out, shape);
  if (out.numel() == 0) return out;
  Staged st(out, common);
  at::Tensor c = condition.device().is_privateuseone() ? condition : condition.to(out.device());
  if (c.sizes() != at::IntArrayRef(shape)) c = c.expand(shape);
  at::Tensor a = as_common(self, common, shape, out.options()), b = as_common(other, common, shape, out.options());
  b200Tensor vo = to_b200(st.work), vc = to_b200(c), va = to_b200(a), vb = to_b200(b);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_where, stream, &vo, &vc, &va, &vb);
  st.finish();
  return out;
}

at::Tensor where_self(const at::Tensor& condition, const at::Tensor& self, const at::Tensor& other) {
  const at::Tensor& on_dev = self.device().is_privateuseone() ? self : (other.device().is_privateuseone() ? other : condition);
  at::Tensor out = at::empty({0}, on_dev.options().dtype(at::result_type(self, other)));
  return where_self_out(condition, self, other, out);
}

at::Tensor& masked_fill__Scalar(at::Tensor& self, const at::Tensor& mask, const at::Scalar& value) {
  TORCH_CHECK(mask.scalar_type() == at::kBool, "masked_fill_ only supports boolean masks, but got mask with dtype ", mask.scalar_type());
  if (self.numel() == 0) return self;
  at::Tensor m = mask.device().is_privateuseone() ? mask : mask.to(self.device());
  TORCH_CHECK(at::is_expandable_to(m.sizes(), self.sizes()), "masked_fill_: the mask must be broadcastable to self");
  m = m.expand(self.sizes());
  b200Tensor vs = to_b200(self), vm = to_b200(m);
  cudaStream_t stream = current_stream(self);
  const double v = value.isBoolean() ? static_cast<double>(value.toBool()) : value.toDouble();
  GCU_KERNEL_CALL(b200_masked_fill, stream, &vs, &vs, &vm, v);
  return self;
}

void maximum_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor&, const at::Tensor& out) {
  minmax_tensor(iter, true, out);
}
void minimum_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor&, const at::Tensor& out) {
  minmax_tensor(iter, false, out);
}
void clamp_out(at::TensorIteratorBase& iter, const at::Tensor&, const std::optional<at::Scalar>& min,
               const std::optional<at::Scalar>& max, const at::Tensor& out) {
  clamp_impl(iter, min, max, out);
}
void clamp_min_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Scalar& min, const at::Tensor& out) {
  clamp_impl(iter, min, std::nullopt, out);
}
void clamp_max_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Scalar& max, const at::Tensor& out) {
  clamp_impl(iter, std::nullopt, max, out);
}

at::Tensor& logical_not_out(const at::Tensor& self, at::Tensor& out) {
  at::native::resize_output(out, self.sizes());
  if (out.numel() == 0) return out;
  Staged st(out, at::kBool);
  b200Tensor vo = to_b200(st.work), va = to_b200(self);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_compare_scalar, stream, &vo, &va, 0.0, static_cast<int32_t>(B200_CMP_EQ));
  st.finish();
  return out;
}
at::Tensor& logical_and_out(const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
  logical_binary(self, other, B200_CMP_AND, out);
  return out;
}
at::Tensor& logical_or_out(const at::Tensor& self, const at::Tensor& other, at::Tensor& out) {
  logical_binary(self, other, B200_CMP_OR, out);
  return out;
}

// Bitwise operators are provided for boolean masks (~m, m1 & m2, m1 | m2).
void bitwise_not_out(at::TensorIteratorBase& iter, const at::Tensor& self, const at::Tensor& out) {
  TORCH_CHECK(self.scalar_type() == at::kBool, "bitwise_not on the gcu backend supports boolean tensors");
  if (out.numel() == 0) return;
  at::Tensor a = as_common(iter.tensor(1), at::kBool, out.sizes(), out.options());
  b200Tensor vo = to_b200(out), va = to_b200(a);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_compare_scalar, stream, &vo, &va, 0.0, static_cast<int32_t>(B200_CMP_EQ));
}
void bitwise_and_Tensor_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor&, const at::Tensor& out) {
  TORCH_CHECK(iter.common_dtype() == at::kBool, "bitwise_and on the gcu backend supports boolean tensors");
  compare_tensor(iter, B200_CMP_AND, out);
}
void bitwise_or_Tensor_out(at::TensorIteratorBase& iter, const at::Tensor&, const at::Tensor&, const at::Tensor& out) {
  TORCH_CHECK(iter.common_dtype() == at::kBool, "bitwise_or on the gcu backend supports boolean tensors");
  compare_tensor(iter, B200_CMP_OR, out);
}

at::Tensor isnan(const at::Tensor& self) {
  at::Tensor out = at::empty(self.sizes(), self.options().dtype(at::kBool));
  if (out.numel() == 0) return out;
  if (!at::isFloatingType(self.scalar_type())) return out.zero_();
  b200Tensor vo = to_b200(out), va = to_b200(self);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_compare, stream, &vo, &va, &va, static_cast<int32_t>(B200_CMP_NE));
  return out;
}

void argmax_out(const at::Tensor& self, std::optional<int64_t> dim, bool, const at::Tensor& out) {
  if (out.numel() == 0) return;
  if (dim.has_value()) extreme_dim(self, *dim, true, nullptr, &out);
  else extreme_dim(self.contiguous().view({1, -1}), 1, true, nullptr, &out);
}
void argmin_out(const at::Tensor& self, std::optional<int64_t> dim, bool, const at::Tensor& out) {
  if (out.numel() == 0) return;
  if (dim.has_value()) extreme_dim(self, *dim, false, nullptr, &out);
  else extreme_dim(self.contiguous().view({1, -1}), 1, false, nullptr, &out);
}
void max_dim_max(const at::meta::structured_max_dim::meta_return_ty& precompute, const at::Tensor& self, int64_t, bool,
                 const at::Tensor& max, const at::Tensor& max_values) {
  if (max.numel() == 0) return;
  extreme_dim(self, precompute.dim, true, &max, &max_values);
}
void min_dim_min(const at::meta::structured_min_dim::meta_return_ty& precompute, const at::Tensor& self, int64_t, bool,
                 const at::Tensor& min, const at::Tensor& min_indices) {
  if (min.numel() == 0) return;
  extreme_dim(self, precompute.dim, false, &min, &min_indices);
}
void amax_out(const at::Tensor& self, at::IntArrayRef dim, bool keepdim, const at::Tensor& out) {
  amax_impl(self, dim, keepdim, true, out);
}
void amin_out(const at::Tensor& self, at::IntArrayRef dim, bool keepdim, const at::Tensor& out) {
  amax_impl(self, dim, keepdim, false, out);
}
at::Tensor max(const at::Tensor& self) { return extreme_all(self, true); }
at::Tensor min(const at::Tensor& self) { return extreme_all(self, false); }

at::Tensor& arange_start_out(const at::Scalar& start, const at::Scalar& end, const at::Scalar& step, at::Tensor& out) {
  const double s = start.toDouble(), e = end.toDouble(), st = step.toDouble();
  TORCH_CHECK(st != 0.0, "arange: step must be nonzero");
  TORCH_CHECK((st > 0 && e >= s) || (st < 0 && e <= s), "arange: upper bound and lower bound inconsistent with step sign");
  int64_t n;
  if (start.isIntegral(false) && end.isIntegral(false) && step.isIntegral(false)) {
    const int64_t si = start.toLong(), ei = end.toLong(), sti = step.toLong();
    n = sti > 0 ? (ei - si + sti - 1) / sti : (si - ei + (-sti) - 1) / (-sti);
  } else {
    n = static_cast<int64_t>(std::ceil((e - s) / st));
  }
  if (n < 0) n = 0;
  at::native::resize_output(out, {n});
  if (n == 0) return out;
  at::Tensor work = out.is_contiguous() ? out : at::empty({n}, out.options());
  b200Tensor vo = to_b200(work);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_arange, stream, &vo, s, st);
  if (!work.is_same(out)) out.copy_(work);
  return out;
}

namespace {

// The first k entries of every slice of `self` along `dim`, sorted (stable) ascending or descending,
// into `values` and `indices` (shaped by ATen's meta: self's shape with k along dim). The kernel
// sorts the rows of a contiguous (rows, n) view, so the dimension is moved last first; the results
// are written straight into the outputs when those are the matching contiguous views.
void sort_rows_impl(const at::Tensor& self, int64_t dim, bool descending, int64_t k, const at::Tensor& values,
                    const at::Tensor& indices) {
  if (values.numel() == 0) return;
  if (self.dim() == 0) {
    values.copy_(self);
    indices.zero_();
    return;
  }
  const int64_t d = at::maybe_wrap_dim(dim, self.dim());
  const int64_t n = self.size(d);
  const bool last = d == self.dim() - 1;
  at::Tensor src = (last ? self : self.movedim(d, -1)).contiguous();
  const int64_t rows = src.numel() / n;
  const bool direct = last && values.is_contiguous() && indices.is_contiguous();
  at::Tensor v2 = direct ? values.view({rows, k}) : at::empty({rows, k}, self.options());
  at::Tensor i2 = direct ? indices.view({rows, k}) : at::empty({rows, k}, self.options().dtype(at::kLong));
  at::Tensor s2 = src.view({rows, n});
  b200Tensor vin = to_b200(s2), vv = to_b200(v2), vi = to_b200(i2);
  const size_t ws_bytes = b200_sort_rows_workspace_size(&vin);
  at::Tensor ws = alloc_workspace(ws_bytes, self);
  cudaStream_t stream = current_stream(self);
  GCU_KERNEL_CALL(b200_sort_rows, stream, &vv, &vi, &vin, descending ? 1 : 0, ws.data_ptr(), ws_bytes);
  if (!direct) {
    std::vector<int64_t> moved = src.sizes().vec();
    moved.back() = k;
    (last ? values : values.movedim(d, -1)).copy_(v2.view(moved));
    (last ? indices : indices.movedim(d, -1)).copy_(i2.view(moved));
  }
}

}  // namespace

// Always the stable algorithm: a stable sort is a valid answer to a request that does not ask for one.
void sort_values_stable(const at::Tensor& self, std::optional<bool>, int64_t dim, bool descending, const at::Tensor& values,
                        const at::Tensor& indices) {
  sort_rows_impl(self, dim, descending, self.dim() ? self.size(at::maybe_wrap_dim(dim, self.dim())) : 1, values, indices);
}

at::Tensor argsort_stable(const at::Tensor& self, bool stable, int64_t dim, bool descending) {
  return std::get<1>(at::sort(self, stable, dim, descending));
}

// Largest (or smallest) k along dim, always returned sorted (a sorted answer is valid for sorted = false);
// among equal elements the lowest index comes first.
void topk_values(const at::Tensor& self, int64_t k, int64_t dim, bool largest, bool, const at::Tensor& values,
                 const at::Tensor& indices) {
  sort_rows_impl(self, dim, largest, k, values, indices);
}

void cumsum_out(const at::Tensor& self, int64_t dim, std::optional<at::ScalarType>, const at::Tensor& out) {
  if (out.numel() == 0) return;
  // ATen's meta fixed out's dtype (the dtype argument, or int64 for integer inputs): the sum runs in it
  at::Tensor src = self.scalar_type() == out.scalar_type() ? self : self.to(out.scalar_type());
  src = src.contiguous();
  at::Tensor work = out.is_contiguous() ? out : at::empty(out.sizes(), out.options());
  b200Tensor vo = to_b200(work), vs = to_b200(src);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_cumsum, stream, &vo, &vs, self.dim() ? at::maybe_wrap_dim(dim, self.dim()) : 0);
  if (!work.is_same(out)) out.copy_(work);
}

void triu_out(const at::Tensor& self, int64_t diagonal, const at::Tensor& out) { tri_impl(self, diagonal, true, out); }
void tril_out(const at::Tensor& self, int64_t diagonal, const at::Tensor& out) { tri_impl(self, diagonal, false, out); }

}  // namespace aotops
}  // namespace torch_gcu
