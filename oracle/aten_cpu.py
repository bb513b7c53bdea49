"""PyTorch CPU ATen evaluation of every operator on the path (the oracle).

Each function takes CPU tensors and returns CPU tensors. The reference call
site each one stands for is cited; the computation is the CPU kernel of the
same ATen operator, which is what the reference compares itself against
(torch_gcu/csrc/aten/aot_ops/gcu_op_check.cpp:202-230).
"""
import contextlib

import torch
import torch.nn.functional as F

# Tolerances: reference defaults fp32 1e-6, fp16/bf16 1e-3, integers exact
# (torch_gcu/csrc/aten/op_debug_config.h:144-149). Reductions use 1e-5 because
# their association order differs from the CPU's vectorised order.
TOL = {
    "fp32_elementwise": dict(rtol=1e-6, atol=1e-6),
    "fp32_reduction": dict(rtol=1e-5, atol=1e-5),
    "bf16_elementwise": dict(rtol=2 ** -8, atol=1e-3),
    "bf16_contraction": dict(rtol=1.6e-2, atol=1e-2),
}


# -- elementwise: generated aotops::add_out / mul_out / silu_out ---------------
def add(a, b, alpha=1):
    return torch.ops.aten.add(a, b, alpha=alpha)


def mul(a, b):
    return torch.ops.aten.mul(a, b)


def silu(a):
    return torch.ops.aten.silu(a)


# -- cast: aotops::_copy_from (aot_ops/gcu_copy.cpp:402-442) -------------------
def cast(a, dtype):
    return a.to(dtype)


# -- reductions ----------------------------------------------------------------
def sum_dim(a, dims, keepdim=False, dtype=None):
    return torch.ops.aten.sum.dim_IntList(a, dims, keepdim, dtype=dtype)


def mean_dim(a, dims, keepdim=False):
    return torch.ops.aten.mean.dim(a, dims, keepdim)


def softmax(a, dim, half_to_float=False):
    if half_to_float:  # the CPU kernel has no half_to_float form: widen first, same result
        return torch.ops.aten._softmax(a.float(), dim, False)
    return torch.ops.aten._softmax(a, dim, False)


def native_layer_norm(a, normalized_shape, weight, bias, eps):
    # aot_ops/gcu_layer_norm.cpp:17-86 returns (y, mean, rstd)
    return torch.ops.aten.native_layer_norm(a, list(normalized_shape), weight, bias, eps)


# -- index ops -----------------------------------------------------------------
def index_select(a, dim, index):
    return torch.ops.aten.index_select(a, dim, index.long())


def embedding(table, ids):
    return F.embedding(ids, table)


def gather(a, dim, index):
    return torch.ops.aten.gather(a, dim, index.long())


def scatter_add(self, dim, index, src):
    return torch.ops.aten.scatter_add(self, dim, index.long(), src)


@contextlib.contextmanager
def _deterministic():
    prev = torch.are_deterministic_algorithms_enabled()
    torch.use_deterministic_algorithms(True)
    try:
        yield
    finally:
        torch.use_deterministic_algorithms(prev)


def index_put(self, indices, values, accumulate):
    """CPU index_put; with accumulate the multi-threaded CPU kernel is not
    reproducible, so it runs under deterministic algorithms, which gives
    ascending-source-order sequential accumulation."""
    out = self.clone()
    with _deterministic():
        torch.ops.aten.index_put_(out, [None if i is None else i.long() for i in indices], values, accumulate)
    return out


def index(self, indices):
    """aten::index; the int32-index entry point of the reference
    (efficient_ops/ops.cpp:335-342) has the same result as int64 indexing."""
    return torch.ops.aten.index(self, [None if i is None else i.long() for i in indices])


# -- fused ops: compositions of CPU ATen ops -----------------------------------
def rms_norm_residual(x, residual, weight, eps):
    """h = x + residual (in x's dtype); y = rms_norm(h) computed in fp32."""
    h = x + residual if residual is not None else x
    hf = h.float()
    y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return y.to(x.dtype), h


def rotate_half(x):
    d = x.shape[-1] // 2
    return torch.cat((-x[..., d:], x[..., :d]), dim=-1)


def rope(x, cos_half, sin_half, positions=None):
    """x: (B,S,H,D); cos/sin: fp32 (P, D/2). fp32 math, one rounding."""
    B, S = x.shape[0], x.shape[1]
    if positions is None:
        positions = torch.arange(S).expand(B, S)
    cos = torch.cat((cos_half, cos_half), -1)[positions][:, :, None, :]
    sin = torch.cat((sin_half, sin_half), -1)[positions][:, :, None, :]
    xf = x.float()
    return (xf * cos + rotate_half(xf) * sin).to(x.dtype)


def swiglu(gate, up):
    return (F.silu(gate.float()) * up.float()).to(gate.dtype)


# -- contractions --------------------------------------------------------------
def mm(a, b):
    return torch.ops.aten.mm(a, b)


def addmm(c, a, b, beta=1, alpha=1):
    return torch.ops.aten.addmm(c, a, b, beta=beta, alpha=alpha)


def bmm(a, b):
    return torch.ops.aten.bmm(a, b)


def mm_fp32_rounded(a, b):
    """fp32-accumulated product of bf16 operands, rounded once to bf16."""
    return (a.float() @ b.float()).to(a.dtype)


def sdpa_causal(q, k, v, scale=None):
    """q (B,Hq,S,D), k/v (B,Hkv,S,D): causal GQA attention computed in fp32
    from the given operands; returns (out in q's dtype, logsumexp fp32)."""
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    qf, kf, vf = q.float(), k.float(), v.float()
    if Hkv != Hq:
        kf = kf.repeat_interleave(Hq // Hkv, dim=1)
        vf = vf.repeat_interleave(Hq // Hkv, dim=1)
    scale = scale if scale is not None else D ** -0.5
    s = (qf @ kf.transpose(-1, -2)) * scale
    Sk = kf.shape[2]
    mask = torch.ones(S, Sk, dtype=torch.bool).tril(diagonal=Sk - S)
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    out = torch.softmax(s, dim=-1) @ vf
    return out.to(q.dtype), lse
