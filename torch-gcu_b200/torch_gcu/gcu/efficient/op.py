"""Fused / efficient operators.

`gcu_index` keeps the reference's signature and argument checks (reference:
torch_gcu/gcu/efficient/op.py:9-16, csrc/efficient_ops/ops.cpp:221-342). The fused
RMSNorm+residual, RoPE and SwiGLU entries are additions: the reference runs them
as chains of pointwise operators."""
from typing import List, Optional

import torch
from torch import Tensor

from torch_gcu import _C


def gcu_index(self: Tensor, indices: Optional[List[Tensor]]):
    """index op for int32 indices which will not convert int32 indices to int64.

    Args:
      self: tensor to be selected.
      indices: list of int32 indices (on self's device).
    """
    return _C._int32_indices_index(self, indices)


def rms_norm_residual(x: Tensor, residual: Optional[Tensor], weight: Tensor, eps: float = 1e-6):
    """h = x + residual (rounded to x's dtype); y = h * rsqrt(mean(h^2) + eps) * weight in fp32,
    rounded once. Returns (y, h); with residual=None it is plain RMSNorm and h is x."""
    return _C._rms_norm_residual(x, residual, weight, eps)


def rope_tables(positions: int, head_dim: int, theta: float = 10000.0, device="gcu"):
    """fp32 cos/sin tables (positions, head_dim/2) of pos * theta^(-2i/head_dim), built on the
    host exactly as the CPU reference computes them, then copied to the device."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = torch.outer(torch.arange(positions, dtype=torch.float32), inv_freq)
    return freqs.cos().to(device), freqs.sin().to(device)


def rope(x: Tensor, cos: Tensor, sin: Tensor, positions: Optional[Tensor] = None, inplace: bool = False):
    """Rotate-half rotary embedding (the Llama / HF convention) of x (B,S,H,D):
    out = x*cos + rotate_half(x)*sin with rotate_half(x) = cat(-x[..., D/2:], x[..., :D/2]),
    cos/sin the fp32 (P, D/2) tables, positions int64 (B,S) or None for 0..S-1."""
    return _C._rope(x, cos, sin, positions, inplace)


def swiglu(gate: Tensor, up: Tensor):
    """silu(gate) * up, fp32 internally, one rounding."""
    return _C._swiglu(gate, up)


def swiglu_packed(gate_up: Tensor):
    """silu(gate) * up with gate, up the two halves of the last dimension."""
    return _C._swiglu_packed(gate_up)


def linear_swiglu(x: Tensor, w_gate_up: Tensor):
    """silu(x @ w[:F].T) * (x @ w[F:].T) for a fused gate/up weight (2F, K): one GEMM whose
    epilogue applies the activation, so the (…, 2F) projection output is never materialised."""
    return _C._linear_swiglu(x, w_gate_up)


def linear_rope(x: Tensor, w: Tensor, cos: Tensor, sin: Tensor, rope_heads: int):
    """Fused qkv projection of x (B, S, K) with weight (heads*128, K): returns (B, S, heads, 128) with the
    rotate-half rotary embedding (tables as for `rope`, position = index along S) applied to the first
    `rope_heads` heads in the GEMM's epilogue."""
    return _C._linear_rope(x, w, cos, sin, rope_heads)


def rope_kv_append(qkv: Tensor, cos: Tensor, sin: Tensor, positions: Tensor, q_heads: int, k_cache: Tensor, v_cache: Tensor):
    """One decode step's rotary embedding and cache update in one launch: the first `q_heads` heads of qkv
    (B, S, q_heads + 2 k_heads, D) are rotated in place; the next k_heads heads are rotated and written to
    k_cache[b, head, positions[b, s]], the last k_heads heads copied to v_cache[b, head, positions[b, s]];
    caches (B, k_heads, T, D). Same arithmetic as `rope`."""
    _C._rope_kv_append(qkv, cos, sin, positions, q_heads, k_cache, v_cache)


def sdpa_flash(q: Tensor, k: Tensor, v: Tensor, is_causal: bool, scale: Optional[float] = None):
    """Flash attention forward for q (B,Hq,Sq,D), k/v (B,Hkv,Sk,D); returns (out, logsumexp)."""
    return _C._sdpa_flash(q, k, v, is_causal, scale)
