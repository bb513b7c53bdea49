"""Flash-attention forward through the C ABI against an fp32 CPU evaluation of
softmax(scale*QK^T + mask)V on the same bf16 operands."""
import pytest
import torch

from oracle import aten_cpu
from test_ops_gpu import DEV, close, dev

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def cpu_ref(q, k, v, causal):
    if causal:
        return aten_cpu.sdpa_causal(q, k, v)
    B, Hq, S, D = q.shape
    G = Hq // k.shape[1]
    kf, vf = k.float().repeat_interleave(G, 1), v.float().repeat_interleave(G, 1)
    s = (q.float() @ kf.transpose(-1, -2)) * D ** -0.5
    return (torch.softmax(s, -1) @ vf).to(q.dtype), torch.logsumexp(s, -1)


def run(ops, q, k, v, causal):
    B, Hq, S, D = q.shape
    out = torch.empty(B, S, Hq, D, dtype=q.dtype, device=DEV).transpose(1, 2)  # allocated (B,S,H,D) like the reference
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=DEV)
    ops.sdpa_flash_fwd(out, lse, dev(q), dev(k), dev(v), causal)
    assert ops.device_error_fetch() == 0
    return out, lse


@pytest.mark.parametrize("B,Hq,Hkv,S,D", [(1, 4, 2, 16, 32 * 2), (1, 2, 2, 128, 128), (2, 8, 2, 256, 128),
                                          (1, 4, 1, 384, 64), (1, 2, 1, 200, 128), (1, 4, 4, 77, 64),
                                          (1, 8, 2, 1024, 128)])
@pytest.mark.parametrize("causal", [True, False])
def test_sdpa_prefill(ops, B, Hq, Hkv, S, D, causal):
    g = torch.Generator().manual_seed(51)
    q = torch.randn(B, Hq, S, D, generator=g).to(BF)
    k = torch.randn(B, Hkv, S, D, generator=g).to(BF)
    v = torch.randn(B, Hkv, S, D, generator=g).to(BF)
    out, lse = run(ops, q, k, v, causal)
    ro, rl = cpu_ref(q, k, v, causal)
    close(out, ro, 1.6e-2, 1e-2)   # bf16 contraction tolerance
    close(lse, rl, 1e-3, 1e-3)


def test_sdpa_golden_and_strided_inputs(ops, golden):
    g = torch.Generator().manual_seed(52)
    B, S, Hq, Hkv, D = 2, 160, 8, 2, 128
    # q/k/v as views into one fused projection output (B,S,(Hq+2Hkv)*D), as the decoder layer produces
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, generator=g).to(BF)
    dq = dev(qkv)
    def heads(t, lo, n):
        return t[:, :, lo * D:(lo + n) * D].view(B, S, n, D).transpose(1, 2)
    q, k, v = heads(qkv, 0, Hq), heads(qkv, Hq, Hkv), heads(qkv, Hq + Hkv, Hkv)
    out = torch.empty(B, S, Hq, D, dtype=BF, device=DEV).transpose(1, 2)
    lse = torch.empty(B, Hq, S, device=DEV)
    ops.sdpa_flash_fwd(out, lse, heads(dq, 0, Hq), heads(dq, Hq, Hkv), heads(dq, Hq + Hkv, Hkv), True)
    ro, rl = aten_cpu.sdpa_causal(q, k, v)
    close(out, ro, 1.6e-2, 1e-2)
    close(lse, rl, 1e-3, 1e-3)


@pytest.mark.parametrize("B,Hq,Hkv,Sk,D,Sq", [(3, 8, 2, 300, 128, 1), (2, 4, 4, 128, 64, 1), (2, 32, 8, 1000, 128, 1),
                                              (1, 8, 2, 513, 128, 5), (2, 8, 2, 50, 128, 3), (1, 16, 2, 1147, 128, 2),
                                              (2, 4, 1, 4096, 128, 4), (1, 4, 4, 2500, 128, 1), (1, 16, 1, 700, 128, 1)])
def test_sdpa_decode_packed_heads(ops, B, Hq, Hkv, Sk, D, Sq):
    """A few query positions against a long KV cache, is_causal=False: the query
    heads of one KV group share a tile."""
    g = torch.Generator().manual_seed(53)
    q = torch.randn(B, Hq, Sq, D, generator=g).to(BF)
    k = torch.randn(B, Hkv, Sk, D, generator=g).to(BF)
    v = torch.randn(B, Hkv, Sk, D, generator=g).to(BF)
    out = torch.empty(B, Sq, Hq, D, dtype=BF, device=DEV).transpose(1, 2)
    lse = torch.empty(B, Hq, Sq, device=DEV)
    # KV cache longer than the valid length: a strided slice
    cache_k = torch.zeros(B, Hkv, Sk + 24, D, dtype=BF, device=DEV)
    cache_v = torch.zeros(B, Hkv, Sk + 24, D, dtype=BF, device=DEV)
    cache_k[:, :, :Sk] = dev(k)
    cache_v[:, :, :Sk] = dev(v)
    ops.sdpa_flash_fwd(out, lse, dev(q), cache_k[:, :, :Sk], cache_v[:, :, :Sk], False)
    assert ops.device_error_fetch() == 0
    ro, rl = cpu_ref(q, k, v, False)
    close(out, ro, 1.6e-2, 1e-2)
    close(lse, rl, 1e-3, 1e-3)


def test_sdpa_golden(ops, golden):
    s = golden("op_small")["sdpa"]
    q = s["q"]
    out = torch.empty(1, 16, 4, 32, dtype=BF, device=DEV).transpose(1, 2)
    with pytest.raises(ops.B200Error):  # head dim 32: not a tensor-core shape of this kernel
        ops.sdpa_flash_fwd(out, None, dev(q), dev(s["k"]), dev(s["v"]), True)


@pytest.mark.parametrize("dtype", [torch.float16, BF])
@pytest.mark.parametrize("Sq,Sk,causal", [(640, 640, True), (300, 300, False), (1, 900, False), (2, 2000, False)])
def test_sdpa_growing_maximum(ops, dtype, Sq, Sk, causal):
    """Scores that keep growing along the key axis, so the running maximum moves in
    every key tile and the accumulator has to be rescaled again and again; both
    16-bit dtypes."""
    g = torch.Generator().manual_seed(54)
    B, Hq, Hkv, D = 1, 4, 1, 128
    q = torch.randn(B, Hq, Sq, D, generator=g)
    k = torch.randn(B, Hkv, Sk, D, generator=g)
    v = torch.randn(B, Hkv, Sk, D, generator=g)
    # add a component along q's mean direction that grows with the key position
    ramp = torch.linspace(0, 6, Sk).view(1, 1, Sk, 1)
    k = k + ramp * q.mean((1, 2), keepdim=True).sign() * 0.5
    q = q.abs() * q.mean((1, 2), keepdim=True).sign()
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    out = torch.empty(B, Sq, Hq, D, dtype=dtype, device=DEV).transpose(1, 2)
    lse = torch.empty(B, Hq, Sq, device=DEV)
    ops.sdpa_flash_fwd(out, lse, dev(q), dev(k), dev(v), causal)
    assert ops.device_error_fetch() == 0
    G = Hq // Hkv
    kf, vf = k.float().repeat_interleave(G, 1), v.float().repeat_interleave(G, 1)
    s = (q.float() @ kf.transpose(-1, -2)) * D ** -0.5
    if causal:
        s = s.masked_fill(torch.ones(Sq, Sk, dtype=torch.bool).triu(1), float("-inf"))
    assert (s.max(-1).values - s[..., :128].max(-1).values).max() > 20   # the maximum really moves
    close(out, (torch.softmax(s, -1) @ vf).to(dtype), 1.6e-2, 1e-2)
    close(lse, torch.logsumexp(s, -1), 1e-3, 2e-3)


def _cpu_attention_grads(q, k, v, go, causal):
    """fp32 autograd on the CPU over the same 16-bit operands."""
    qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
    G = q.shape[1] // k.shape[1]
    ke, ve = kf.repeat_interleave(G, 1), vf.repeat_interleave(G, 1)
    s = (qf @ ke.transpose(-1, -2)) * q.shape[-1] ** -0.5
    if causal:
        S = q.shape[2]
        s = s.masked_fill(torch.ones(S, S, dtype=torch.bool).triu(1), float("-inf"))
    o = torch.softmax(s, -1) @ ve
    o.backward(go.float())
    return qf.grad, kf.grad, vf.grad


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,causal", [(1, 2, 2, 128, 128, True), (2, 4, 2, 256, 256, True), (1, 4, 1, 200, 200, True),
                                                   (1, 2, 1, 128, 384, False), (2, 8, 2, 77, 300, False), (1, 4, 4, 640, 640, True)])
@pytest.mark.parametrize("dtype", [BF, torch.float16])
def test_sdpa_backward(ops, B, Hq, Hkv, Sq, Sk, causal, dtype):
    """dq, dk, dv of the flash kernel against fp32 CPU autograd on the same operands."""
    g = torch.Generator().manual_seed(55)
    D = 128
    q = torch.randn(B, Hq, Sq, D, generator=g).to(dtype)
    k = torch.randn(B, Hkv, Sk, D, generator=g).to(dtype)
    v = torch.randn(B, Hkv, Sk, D, generator=g).to(dtype)
    go = torch.randn(B, Hq, Sq, D, generator=g).to(dtype)
    qd, kd, vd, god = dev(q), dev(k), dev(v), dev(go)
    out = torch.empty(B, Sq, Hq, D, dtype=dtype, device=DEV).transpose(1, 2)
    lse = torch.empty(B, Hq, Sq, device=DEV)
    ops.sdpa_flash_fwd(out, lse, qd, kd, vd, causal)
    dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    ops.sdpa_flash_bwd(dq, dk, dv, god, qd, kd, vd, out, lse, causal)
    assert ops.device_error_fetch() == 0
    rq, rk, rv = _cpu_attention_grads(q, k, v, go, causal)
    for got, ref, name in ((dq, rq, "dq"), (dk, rk, "dk"), (dv, rv, "dv")):
        err = (got.float().cpu() - ref).norm() / ref.norm()
        assert err < 2e-2, (name, err.item())
        close(got, ref.to(dtype), 5e-2, 5e-2 * ref.abs().max().item())
    # reproducible: no atomics anywhere in the backward
    dq2, dk2, dv2 = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    ops.sdpa_flash_bwd(dq2, dk2, dv2, god, qd, kd, vd, out, lse, causal)
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)
