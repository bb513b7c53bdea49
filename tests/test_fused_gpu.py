"""Fused RMSNorm+residual, RoPE and SwiGLU against their CPU ATen compositions."""
import pytest
import torch

from oracle import aten_cpu
from test_ops_gpu import DEV, close, dev, exact
import workloads

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def bf16_close(a, b):
    # reference tolerance for bf16 is 1e-3 absolute/relative; one bf16 ulp is up to
    # 2^-7 relative at the bottom of a binade, which a different summation order
    # of the row statistics can flip, so allow exactly one ulp
    close(a, b, 2 ** -7, 1e-3)


@pytest.mark.parametrize("rows,n", [(9, 64), (33, 4096), (4, 8192), (3, 1000), (2, 24576), (5, 40), (0, 64)])
@pytest.mark.parametrize("dtype", [BF, torch.float32, torch.float16])
def test_rms_norm_residual(ops, rows, n, dtype):
    g = torch.Generator().manual_seed(31)
    x, res = torch.randn(rows, n, generator=g).to(dtype), torch.randn(rows, n, generator=g).to(dtype)
    w = (torch.randn(n, generator=g) * 0.02 + 1).to(dtype)
    ry, rh = aten_cpu.rms_norm_residual(x, res, w, 1e-6)
    y, h = torch.empty_like(dev(x)), torch.empty_like(dev(x))
    ops.rms_norm_residual(y, h, dev(x), dev(res), dev(w), 1e-6)
    exact(h, rh)
    if dtype == torch.float32:
        close(y, ry, 1e-5, 1e-5)
    else:
        bf16_close(y, ry)
    # in place on both inputs, and without a residual
    dx, dr = dev(x).clone(), dev(res).clone()
    ops.rms_norm_residual(dx, dr, dx, dr, dev(w), 1e-6)
    exact(dr, rh)
    exact(dx, y.cpu())
    ry2, _ = aten_cpu.rms_norm_residual(x, None, w, 1e-6)
    ops.rms_norm_residual(y, None, dev(x), None, dev(w), 1e-6)
    if dtype == torch.float32:
        close(y, ry2, 1e-5, 1e-5)
    else:
        bf16_close(y, ry2)


def test_rms_norm_golden(ops, golden):
    r = golden("op_small")["rms_norm_residual"]
    y, h = torch.empty_like(dev(r["x"])), torch.empty_like(dev(r["x"]))
    ops.rms_norm_residual(y, h, dev(r["x"]), dev(r["res"]), dev(r["w"]), r["eps"])
    exact(h, r["h"])
    bf16_close(y, r["y"])


@pytest.mark.parametrize("B,S,H,D", [(2, 7, 3, 32), (1, 33, 8, 128), (3, 16, 2, 64), (2, 5, 1, 256)])
@pytest.mark.parametrize("dtype", [BF, torch.float32])
def test_rope_bit_exact(ops, B, S, H, D, dtype):
    g = torch.Generator().manual_seed(32)
    q = torch.randn(B, S, H, D, generator=g).to(dtype)
    cos, sin = workloads.rope_tables(S + 10, D)
    ref = aten_cpu.rope(q, cos, sin)
    out = torch.empty_like(dev(q))
    ops.rope(out, dev(q), dev(cos), dev(sin))
    exact(out, ref)  # same fp32 operations, separately rounded: identical bits
    pos = torch.randint(0, S + 10, (B, S), generator=g)
    ops.rope(out, dev(q), dev(cos), dev(sin), dev(pos))
    exact(out, aten_cpu.rope(q, cos, sin, pos))
    # in place on a strided view: q inside a fused qkv projection output
    qkv = torch.randn(B, S, H + 2, D, generator=g).to(dtype)
    dq = dev(qkv)
    view = dq[:, :, :H]
    ops.rope(view, view, dev(cos), dev(sin))
    exact(dq[:, :, :H].contiguous(), aten_cpu.rope(qkv[:, :, :H], cos, sin))
    exact(dq[:, :, H:].contiguous(), qkv[:, :, H:].contiguous())


@pytest.mark.parametrize("B,S,Hq,Hk,D,T", [(4, 1, 8, 2, 128, 40), (2, 3, 3, 1, 64, 16), (64, 1, 32, 8, 128, 64), (1, 1, 1, 1, 32, 8)])
@pytest.mark.parametrize("dtype", [BF, torch.float32])
def test_rope_kv_append(ops, B, S, Hq, Hk, D, T, dtype):
    """The decode step's rotary embedding fused with the cache write, against rope + two copies on the CPU:
    query heads rotated in place, rotated keys and plain values in the caches' slots, everything else untouched."""
    g = torch.Generator().manual_seed(34)
    qkv = torch.randn(B, S, Hq + 2 * Hk, D, generator=g).to(dtype)
    cos, sin = workloads.rope_tables(T, D)
    pos = torch.stack([torch.randperm(T, generator=g)[:S] for _ in range(B)])   # distinct slots per sequence
    # caches as views of a larger allocation (a cache with room to grow), filled with a marker
    kc_full = torch.full((B, Hk, T + 5, D), 7.0).to(dtype)
    vc_full = torch.full((B, Hk, T + 5, D), -3.0).to(dtype)
    dq, dk, dv = dev(qkv), dev(kc_full), dev(vc_full)
    ops.rope_kv_append(dq, dev(cos), dev(sin), dev(pos), Hq, Hk, dk[:, :, :T], dv[:, :, :T])
    assert ops.device_error_fetch() == 0
    rot = aten_cpu.rope(qkv[:, :, :Hq + Hk], cos, sin, pos)
    want_q = qkv.clone()
    want_q[:, :, :Hq] = rot[:, :, :Hq]
    exact(dq, want_q)                       # k and v parts of qkv unchanged
    want_k, want_v = kc_full.clone(), vc_full.clone()
    for b in range(B):
        for s in range(S):
            want_k[b, :, pos[b, s]] = rot[b, s, Hq:]
            want_v[b, :, pos[b, s]] = qkv[b, s, Hq + Hk:]
    exact(dk, want_k)
    exact(dv, want_v)
    # a position outside the cache writes nothing and raises the index bit of the error word
    bad = pos.clone()
    bad[0, 0] = T
    before = dk.clone()
    ops.rope_kv_append(dev(qkv), dev(cos), dev(sin), dev(bad), Hq, Hk, dk[:, :, :T], dv[:, :, :T])
    assert ops.device_error_fetch() & 1
    assert torch.equal(dk[0], before[0])


def test_rope_golden(ops, golden):
    r = golden("op_small")["rope"]
    out = torch.empty_like(dev(r["q"]))
    ops.rope(out, dev(r["q"]), dev(r["cos"]), dev(r["sin"]))
    exact(out, r["out"])


@pytest.mark.parametrize("rows,cols", [(5, 48), (16, 14336), (3, 1001), (1, 8), (0, 16), (257, 64)])
@pytest.mark.parametrize("dtype", [BF, torch.float32])
def test_swiglu(ops, rows, cols, dtype):
    g = torch.Generator().manual_seed(33)
    gate, up = torch.randn(rows, cols, generator=g).to(dtype), torch.randn(rows, cols, generator=g).to(dtype)
    out = torch.empty_like(dev(gate))
    ops.swiglu(out, dev(gate), dev(up))
    ref = aten_cpu.swiglu(gate, up)
    if dtype == torch.float32:
        close(out, ref, 1e-6, 1e-6)
    else:
        bf16_close(out, ref)
    # gate and up as the two halves of one projection output
    both = dev(torch.cat([gate, up], 1))
    ops.swiglu(out, both[:, :cols], both[:, cols:])
    if dtype == torch.float32:
        close(out, ref, 1e-6, 1e-6)
    else:
        bf16_close(out, ref)


def test_swiglu_golden(ops, golden):
    r = golden("op_small")["swiglu"]
    out = torch.empty_like(dev(r["gate"]))
    ops.swiglu(out, dev(r["gate"]), dev(r["up"]))
    bf16_close(out, r["out"])
