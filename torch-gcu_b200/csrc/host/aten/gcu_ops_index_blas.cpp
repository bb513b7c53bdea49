// Index operators, concatenation and the contractions (reference: generated
// aotops::index_select / gather_out / scatter_add_out with the deterministic
// flag of codegen/gen_aot_ops.py:833-841, aot_ops/gcu_tensor_advanced_indexing.cpp
// :40-90, generated aotops::mm_out / addmm_out / bmm_out).
#include <ATen/ExpandUtils.h>
#include <ATen/WrapDimUtils.h>
#include <ATen/native/Resize.h>

#include "aten/aot_ops.h"
#include "aten/bridge.h"

namespace torch_gcu {
namespace aotops {
namespace {

at::Tensor index_on_device(const at::Tensor& index, const at::Tensor& like) {
  TORCH_CHECK(index.scalar_type() == at::kLong || index.scalar_type() == at::kInt,
              "index tensors must be int32 or int64, got ", index.scalar_type());
  return index.device() == like.device() ? index : index.to(like.device());
}

}  // namespace

// ----------------------------------------------------------- index_select --
at::Tensor& index_select_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, at::Tensor& out) {
  dim = at::maybe_wrap_dim(dim, self.dim());
  TORCH_CHECK(index.dim() <= 1, "index_select(): Index is supposed to be a vector, but got dim: ", index.dim());
  TORCH_CHECK(self.scalar_type() == out.scalar_type(), "index_select(): self and result must have the same scalar type");
  at::Tensor idx = index_on_device(index, self);
  std::vector<int64_t> shape = self.sizes().vec();
  if (self.dim() > 0) shape[dim] = idx.numel();
  at::native::resize_output(out, shape);
  if (out.numel() == 0) return out;
  at::Tensor src = self.contiguous();
  at::Tensor work = out.is_contiguous() ? out : at::empty(shape, out.options());
  at::Tensor idx1 = idx.dim() == 0 ? idx.reshape({1}) : idx;
  b200Tensor vo = to_b200(work), vs = to_b200(src), vi = to_b200(idx1);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_index_select, stream, &vo, &vs, dim, &vi);
  if (!work.is_same(out)) out.copy_(work);
  return out;
}

at::Tensor index_select(const at::Tensor& self, int64_t dim, const at::Tensor& index) {
  at::Tensor out = at::empty({0}, self.options());
  return index_select_out(self, dim, index, out);
}

// ----------------------------------------------------------------- gather --
void gather_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, bool, const at::Tensor& out) {
  if (out.numel() == 0) return;
  dim = at::maybe_wrap_dim(dim, self.dim());
  at::Tensor idx = index_on_device(index, self);
  at::Tensor work = out.is_contiguous() ? out : at::empty(out.sizes(), out.options());
  b200Tensor vo = to_b200(work), vs = to_b200(self), vi = to_b200(idx);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_gather, stream, &vo, &vs, dim, &vi);
  if (!work.is_same(out)) out.copy_(work);
}

// ------------------------------------------------------------ scatter_add --
void scatter_add_out(const at::Tensor& self, int64_t dim, const at::Tensor& index, const at::Tensor& src,
                     const at::Tensor& out) {
  dim = at::maybe_wrap_dim(dim, self.dim());
  if (out.numel() == 0) return;
  if (index.numel() == 0) {
    if (!out.is_same(self)) out.copy_(self);
    return;
  }
  at::Tensor idx = index_on_device(index, self);
  // only index.size(d) entries of src take part in every dimension
  at::Tensor s = src;
  for (int64_t d = 0; d < idx.dim(); ++d)
    if (s.size(d) != idx.size(d)) s = s.narrow(d, 0, idx.size(d));
  s = s.contiguous();
  at::Tensor base = self.contiguous();
  at::Tensor work = out.is_contiguous() ? out : at::empty(out.sizes(), out.options());
  b200Tensor vo = to_b200(work), vb = to_b200(base), vi = to_b200(idx), vs = to_b200(s);
  cudaStream_t stream = current_stream(out);
  const size_t ws_bytes = b200_scatter_add_workspace_size(&vb, dim, &vi, &vs);
  at::Tensor ws = alloc_workspace(ws_bytes, out);
  GCU_KERNEL_CALL(b200_scatter_add, stream, &vo, &vb, dim, &vi, &vs, ws.data_ptr(), ws_bytes);
  if (!work.is_same(out)) out.copy_(work);
}

// ------------------------------------------------------- advanced indexing --
static void index_with_info(at::TensorIteratorBase& iter, at::IntArrayRef indexed_sizes, at::IntArrayRef indexed_strides_bytes,
                            const at::Tensor& out) {
  if (out.numel() == 0) return;
  const int n = iter.ntensors() - 2;
  TORCH_CHECK(n >= 1 && n <= 4, "index on the gcu backend supports 1 to 4 index tensors, got ", n);
  const at::Tensor& src = iter.tensor(1);  // self restrided to the result shape, stride 0 on indexed dims
  const int64_t es = static_cast<int64_t>(src.element_size());
  std::vector<at::Tensor> idx_keep;
  std::vector<b200Tensor> idx_views(n);
  std::vector<const b200Tensor*> idx_ptrs(n);
  std::vector<int64_t> sizes(n), strides(n);
  for (int k = 0; k < n; ++k) {
    at::Tensor t = index_on_device(iter.tensor(2 + k), out);
    idx_keep.push_back(t.sizes() == out.sizes() ? t : t.expand(out.sizes()));
    idx_views[k] = to_b200(idx_keep.back());
    idx_ptrs[k] = &idx_views[k];
    sizes[k] = indexed_sizes[k];
    strides[k] = indexed_strides_bytes[k] / es;
  }
  at::Tensor src_view = src.sizes() == out.sizes() ? src : src.expand(out.sizes());
  b200Tensor vo = to_b200(out), vs = to_b200(src_view);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_index, stream, &vo, &vs, idx_ptrs.data(), n, sizes.data(), strides.data());
}

void index_Tensor_out(at::TensorIteratorBase& iter, const at::meta::structured_index_Tensor::meta_return_ty& precompute,
                      const at::Tensor&, const c10::List<std::optional<at::Tensor>>&, const at::Tensor& out) {
  index_with_info(iter, precompute.sizes, precompute.strides, out);
}

// `aten::index` that accepts int32 device indices without widening them
// (reference: efficient::device_int32_indices_index, efficient_ops/ops.cpp:221-342):
// same argument checks -- indices on self's device, int32 only.
at::Tensor int32_indices_index(const at::Tensor& self, const c10::List<std::optional<at::Tensor>>& indices) {
  TORCH_CHECK_INDEX(indices.size() <= static_cast<size_t>(self.dim()), "too many indices for tensor of dimension ",
                    self.dim(), " (got ", indices.size(), ")");
  std::vector<at::Tensor> defined;
  for (size_t i = 0; i < indices.size(); ++i) {
    std::optional<at::Tensor> t = indices.get(i);
    TORCH_CHECK_INDEX(t.has_value() && t->defined(), "gcu_index supports leading index tensors only (no None entries)");
    TORCH_CHECK_INDEX(t->device() == self.device(), "indice error, indice should be in the same device as self but got self: ",
                      self.device(), " indice: ", t->device());
    TORCH_CHECK_INDEX(t->scalar_type() == at::kInt, "indice error, should be int in gcu_index but got ", t->dtype());
    defined.push_back(*t);
  }
  TORCH_CHECK_INDEX(!defined.empty() && defined.size() <= 4, "gcu_index takes 1 to 4 index tensors");
  std::vector<at::Tensor> bidx;
  try {
    bidx = at::expand_outplace(defined);
  } catch (std::exception&) {
    TORCH_CHECK_INDEX(false, "shape mismatch: indexing tensors could not be broadcast together");
  }
  const int64_t n = static_cast<int64_t>(bidx.size());
  std::vector<int64_t> shape = bidx[0].sizes().vec();
  const size_t idx_nd = shape.size();
  for (int64_t d = n; d < self.dim(); ++d) shape.push_back(self.size(d));
  at::Tensor out = at::empty(shape, self.options());
  if (out.numel() == 0) return out;
  // src: self restrided to the result shape, stride 0 over the index dims
  std::vector<int64_t> sstrides(idx_nd, 0);
  for (int64_t d = n; d < self.dim(); ++d) sstrides.push_back(self.stride(d));
  at::Tensor src = self.as_strided(shape, sstrides);
  std::vector<at::Tensor> keep;
  std::vector<b200Tensor> views(n);
  std::vector<const b200Tensor*> ptrs(n);
  std::vector<int64_t> isz(n), ist(n);
  for (int64_t k = 0; k < n; ++k) {
    std::vector<int64_t> vshape = bidx[k].sizes().vec();
    vshape.resize(shape.size(), 1);
    keep.push_back(bidx[k].reshape(vshape).expand(shape));
    views[k] = to_b200(keep.back());
    ptrs[k] = &views[k];
    isz[k] = self.size(k);
    ist[k] = self.stride(k);
  }
  b200Tensor vo = to_b200(out), vs = to_b200(src);
  cudaStream_t stream = current_stream(out);
  GCU_KERNEL_CALL(b200_index, stream, &vo, &vs, ptrs.data(), static_cast<int32_t>(n), isz.data(), ist.data());
  return out;
}

// self[indices] (+)= values. The kernel takes one index over the leading
// dimension; several leading index tensors are linearised first.
at::Tensor& _index_put_impl_(at::Tensor& self, const c10::List<std::optional<at::Tensor>>& indices, const at::Tensor& values,
                             bool accumulate, bool) {
  std::vector<at::Tensor> idx;
  bool tail_none = false;
  for (size_t i = 0; i < indices.size(); ++i) {
    std::optional<at::Tensor> t = indices.get(i);
    if (t.has_value() && t->defined()) {
      TORCH_CHECK(!tail_none, "index_put on the gcu backend supports index tensors on the leading dimensions only");
      TORCH_CHECK(t->scalar_type() == at::kLong || t->scalar_type() == at::kInt,
                  "index_put on the gcu backend takes int32/int64 index tensors (no masks)");
      idx.push_back(*t);
    } else {
      tail_none = true;
    }
  }
  TORCH_CHECK(!idx.empty(), "index_put needs at least one index tensor");
  TORCH_CHECK(static_cast<int64_t>(idx.size()) <= self.dim(), "too many indices for tensor of dimension ", self.dim());
  const int64_t k = static_cast<int64_t>(idx.size());
  at::Tensor lin;
  int64_t rows = 1;
  for (int64_t d = 0; d < k; ++d) rows *= self.size(d);
  if (k == 1) {
    lin = index_on_device(idx[0], self);
  } else {
    // several index tensors: wrap, range-check and linearise on the host (small), one upload. The
    // copies of the indices to the host synchronise with the device, so this form cannot be recorded
    // into a graph; the one-index form stays on the device.
    std::vector<at::Tensor> host;
    for (auto& t : idx) host.push_back(t.to(at::kCPU, at::kLong));
    host = at::expand_outplace(host);
    at::Tensor acc = at::zeros_like(host[0]);
    for (int64_t d = 0; d < k; ++d) {
      at::Tensor w = at::where(host[d] < 0, host[d] + self.size(d), host[d]);
      // checked per dimension, as ATen does: once linearised, an index one past the end of a
      // trailing dimension would name a valid element of the next row
      if (w.numel() > 0) {
        const int64_t lo = w.min().item<int64_t>(), hi = w.max().item<int64_t>();
        const int64_t bad = lo < 0 ? lo - self.size(d) : hi;
        TORCH_CHECK_INDEX(lo >= 0 && hi < self.size(d), "index ", bad, " is out of bounds for dimension ", d, " with size ",
                          self.size(d));
      }
      acc = acc * self.size(d) + w;
    }
    lin = acc.to(self.device());
  }
  const std::vector<int64_t> idx_shape = lin.sizes().vec();
  std::vector<int64_t> vshape = idx_shape, row_shape = {rows};
  for (int64_t d = k; d < self.dim(); ++d) {
    vshape.push_back(self.size(d));
    row_shape.push_back(self.size(d));
  }
  if (lin.numel() == 0 || self.numel() == 0) return self;
  at::Tensor target = self.is_contiguous() ? self : self.contiguous();
  at::Tensor vals = values.device() == self.device() ? values : values.to(self.device());
  if (vals.scalar_type() != self.scalar_type()) vals = vals.to(self.scalar_type());
  vals = vals.expand(vshape).contiguous();
  at::Tensor flat_idx = lin.reshape({-1}).contiguous();
  at::Tensor tview = target.view(row_shape);
  std::vector<int64_t> flat_vshape = row_shape;
  flat_vshape[0] = flat_idx.numel();
  at::Tensor vview = vals.view(flat_vshape);
  b200Tensor vt = to_b200(tview), vi = to_b200(flat_idx), vv = to_b200(vview);
  cudaStream_t stream = current_stream(self);
  const size_t ws_bytes = b200_index_put_workspace_size(&vt, &vi, &vv);
  at::Tensor ws = alloc_workspace(ws_bytes, self);
  GCU_KERNEL_CALL(b200_index_put, stream, &vt, &vi, &vv, accumulate ? 1 : 0, ws.data_ptr(), ws_bytes);
  if (!target.is_same(self)) self.copy_(target);
  return self;
}

// ------------------------------------------------------------------- cat --
void cat_out(const at::meta::structured_cat::meta_return_ty& precompute, const at::ITensorListRef& tensors, int64_t,
             const at::Tensor& out) {
  if (out.numel() == 0) return;
  const int64_t dim = precompute.dim;
  int64_t offset = 0;
  for (const at::Tensor& t : tensors) {
    if (t.numel() == 0 && t.dim() == 1) continue;  // legacy empty tensors are skipped
    const int64_t n = t.size(dim);
    if (n > 0) out.narrow(dim, offset, n).copy_(t);
    offset += n;
  }
}

// ------------------------------------------------------------ contractions --
namespace {

void matmul_impl(const at::Tensor& out, const at::Tensor* self, const at::Tensor& a, const at::Tensor& b,
                 const at::Scalar& beta, const at::Scalar& alpha, bool batched) {
  if (out.numel() == 0) return;
  TORCH_CHECK(a.scalar_type() == b.scalar_type() && a.scalar_type() == out.scalar_type(),
              "expected both matrices and the output to share one dtype, got ", a.scalar_type(), ", ", b.scalar_type(),
              " and ", out.scalar_type());
  at::Tensor work = out.stride(-1) == 1 || out.size(-1) == 1 ? out : at::empty(out.sizes(), out.options());
  b200Tensor vo = to_b200(work), va = to_b200(a), vb = to_b200(b);
  cudaStream_t stream = current_stream(out);
  if (self) {
    at::Tensor c = self->scalar_type() == out.scalar_type() ? *self : self->to(out.scalar_type());
    if (c.sizes() != out.sizes()) c = c.expand(out.sizes());
    b200Tensor vc = to_b200(c);
    if (batched) GCU_KERNEL_CALL(b200_baddbmm, stream, &vo, &vc, &va, &vb, beta.toDouble(), alpha.toDouble());
    else GCU_KERNEL_CALL(b200_addmm, stream, &vo, &vc, &va, &vb, beta.toDouble(), alpha.toDouble());
  } else {
    if (batched) GCU_KERNEL_CALL(b200_bmm, stream, &vo, &va, &vb);
    else GCU_KERNEL_CALL(b200_mm, stream, &vo, &va, &vb);
  }
  if (!work.is_same(out)) out.copy_(work);
}

}  // namespace

void mm_out(const at::Tensor& self, const at::Tensor& mat2, const at::Tensor& out) {
  matmul_impl(out, nullptr, self, mat2, 0, 1, false);
}
void addmm_out(const at::Tensor& self, const at::Tensor& mat1, const at::Tensor& mat2, const at::Scalar& beta,
               const at::Scalar& alpha, const at::Tensor& out) {
  matmul_impl(out, &self, mat1, mat2, beta, alpha, false);
}
void bmm_out(const at::Tensor& self, const at::Tensor& mat2, const at::Tensor& out) {
  matmul_impl(out, nullptr, self, mat2, 0, 1, true);
}
void baddbmm_out(const at::Tensor& self, const at::Tensor& batch1, const at::Tensor& batch2, const at::Scalar& beta,
                 const at::Scalar& alpha, const at::Tensor& out) {
  matmul_impl(out, &self, batch1, batch2, beta, alpha, true);
}

}  // namespace aotops
}  // namespace torch_gcu
