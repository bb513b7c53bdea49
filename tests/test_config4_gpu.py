"""Parity at the shapes the benchmark times (workload configurations 4 and 5): the
decoder layer at batch 8 x sequence 2048, the four projections at M = 16384 with
their fused epilogues, causal attention at (8, 32 q / 8 kv heads, 2048, 128), and
decode at batch 64 against a 4096-token cache. Everything runs through the C ABI or
the registered "gcu" device and is compared with CPU ATen on the same seeded values
(the reference backend's own method: every device result against the CPU kernel of
the same operator, test/op_test/gcu_op_test.py:49-135). The CPU side is kept to
seconds by checking sampled rows / heads / sequences; the samples are taken from
every band of the GEMM tile walk and from the first and last tiles of each axis,
which is where a full-size launch differs from a small one.

Tolerances: bf16 contractions rtol 1.6e-2 (as the small-shape tests) with atol 1e-2 for
attention and 2e-2 for projection outputs of magnitude 1.3 - 2.4; a whole layer rel-norm
< 2e-2 plus an element bound of rtol 1.6e-2 / atol 8e-2 (the 16-bit roundings between its
seven launches add up).
"""
import pytest
import torch
import torch.nn.functional as F

from oracle import aten_cpu
from test_ops_gpu import DEV, close, dev
import workloads

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
CFG = dict(hidden=4096, heads=32, kv_heads=8, head_dim=128, ffn=14336)
M_FULL = 16384
# rows at both edges of every 128-row tile boundary that starts a band of the tile walk (a band is
# 16 row-tiles of 256), the last row, and rows inside the second CTA of a pair tile
EDGE_ROWS = [0, 127, 128, 255, 256, 4095, 4096, 4223, 8191, 8192, 12287, 12288, 16255, 16256, 16383]


def sample_rows(m, extra, seed):
    g = torch.Generator().manual_seed(seed)
    rows = torch.cat([torch.tensor([r for r in EDGE_ROWS if r < m]), torch.randint(0, m, (extra,), generator=g)])
    return torch.unique(rows)


@pytest.mark.parametrize("N,K,name", [(6144, 4096, "qkv"), (4096, 4096, "o_proj"), (4096, 14336, "down")])
def test_mm_at_benchmark_rows(ops, N, K, name):
    """x @ w.t() at M = 16384: every column of ~270 sampled rows against fp32 CPU arithmetic."""
    g = torch.Generator().manual_seed(401)
    a = torch.randn(M_FULL, K, generator=g).to(BF)
    w = (torch.randn(N, K, generator=g) * 0.02).to(BF)
    out = torch.empty(M_FULL, N, dtype=BF, device=DEV)
    ops.mm(out, dev(a), dev(w).t())
    assert ops.device_error_fetch() == 0
    rows = sample_rows(M_FULL, 256, 1)
    ref = a[rows].float() @ w.float().t()
    close(out[dev(rows)], ref.to(BF), 1.6e-2, 2e-2)   # |out| ~ 0.02 sqrt(K) = 1.3 .. 2.4
    # the untouched rows are finite and of the right magnitude (no tile left unwritten)
    col_norm = out.float().norm(dim=1)
    assert torch.isfinite(col_norm).all() and (col_norm > 0).all()


def test_addmm_residual_epilogue_at_benchmark_rows(ops):
    """down projection with the residual added in the epilogue (what the tp = 1 layer calls)."""
    g = torch.Generator().manual_seed(402)
    K, N = CFG["ffn"], CFG["hidden"]
    a = torch.randn(M_FULL, K, generator=g).to(BF)
    w = (torch.randn(N, K, generator=g) * 0.02).to(BF)
    r = torch.randn(M_FULL, N, generator=g).to(BF)
    out = torch.empty(M_FULL, N, dtype=BF, device=DEV)
    ops.addmm(out, dev(r), dev(a), dev(w).t())
    assert ops.device_error_fetch() == 0
    rows = sample_rows(M_FULL, 256, 2)
    ref = r[rows].float() + a[rows].float() @ w.float().t()
    close(out[dev(rows)], ref.to(BF), 1.6e-2, 4e-2)


def test_mm_swiglu_at_benchmark_rows(ops):
    """gate/up projection 16384 x (2 x 14336) x 4096 with the SwiGLU in the epilogue: the kernel the
    benchmark's roofline entry times. All 14336 columns of the sampled rows."""
    g = torch.Generator().manual_seed(403)
    K, Fd = CFG["hidden"], CFG["ffn"]
    a = torch.randn(M_FULL, K, generator=g).to(BF)
    w = (torch.randn(2 * Fd, K, generator=g) * 0.02).to(BF)
    out = torch.empty(M_FULL, Fd, dtype=BF, device=DEV)
    ops.mm_swiglu(out, dev(a), dev(w))
    assert ops.device_error_fetch() == 0
    rows = sample_rows(M_FULL, 256, 3)
    gu = a[rows].float() @ w.float().t()
    ref = F.silu(gu[:, :Fd]) * gu[:, Fd:]
    close(out[dev(rows)], ref.to(BF), 1.6e-2, 2e-2)
    nrm = out.float().norm(dim=1)
    assert torch.isfinite(nrm).all() and (nrm > 0).all()


def test_mm_rope_at_benchmark_rows(ops):
    """qkv projection of 8 x 2048 tokens with RoPE on the 32 + 8 q / k heads in the epilogue."""
    g = torch.Generator().manual_seed(404)
    B, S, K = 8, 2048, CFG["hidden"]
    heads, rope_heads = 48, 40
    a = torch.randn(B * S, K, generator=g).to(BF)
    w = (torch.randn(heads * 128, K, generator=g) * 0.02).to(BF)
    cos, sin = workloads.rope_tables(S, 128)
    out = torch.empty(B * S, heads * 128, dtype=BF, device=DEV)
    ops.mm_rope(out, dev(a), dev(w), dev(cos), dev(sin), S, rope_heads * 128)
    assert ops.device_error_fetch() == 0
    rows = sample_rows(B * S, 256, 4)
    y = (a[rows].float() @ w.float().t()).view(-1, heads, 128)
    pos = rows % S
    c = torch.cat((cos[pos], cos[pos]), -1)[:, None, :]
    s_ = torch.cat((sin[pos], sin[pos]), -1)[:, None, :]
    rot = torch.cat((-y[..., 64:], y[..., :64]), -1)
    ref = y.clone()
    ref[:, :rope_heads] = (y * c + rot * s_)[:, :rope_heads]
    close(out[dev(rows)].view(-1, heads, 128), ref.to(BF), 1.6e-2, 2e-2)


def test_sdpa_prefill_benchmark_shape_against_aten_cpu_kernel(ops):
    """Causal GQA attention at (8, 32 q / 8 kv, 2048, 128): every batch element, query heads 0-7 and
    28-31 (KV heads 0, 1 and 7; heads 0, 3, 4 and 31 among them), against ATen's own CPU kernel
    (`scaled_dot_product_attention(is_causal=True, enable_gqa=True)` -- the kernel the reference
    backend's op check compares its device result with,
    torch_gcu/csrc/aten/GCUNativeFunctions.cpp:49-102) and against the fp32 formula."""
    g = torch.Generator().manual_seed(405)
    B, Hq, Hkv, S, D = 8, 32, 8, 2048, 128
    q = torch.randn(B, Hq, S, D, generator=g).to(BF)
    k = torch.randn(B, Hkv, S, D, generator=g).to(BF)
    v = torch.randn(B, Hkv, S, D, generator=g).to(BF)
    out = torch.empty(B, S, Hq, D, dtype=BF, device=DEV).transpose(1, 2)
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=DEV)
    ops.sdpa_flash_fwd(out, lse, dev(q), dev(k), dev(v), True)
    assert ops.device_error_fetch() == 0
    qh = list(range(8)) + list(range(28, 32))
    kh = [0, 1, 7]
    got = out[:, qh].cpu()
    aten = F.scaled_dot_product_attention(q[:, qh], k[:, kh], v[:, kh], is_causal=True, enable_gqa=True)
    close(got, aten, 1.6e-2, 1e-2)
    aten32 = F.scaled_dot_product_attention(q[:, qh].float(), k[:, kh].float(), v[:, kh].float(), is_causal=True,
                                            enable_gqa=True)
    close(got, aten32, 1.6e-2, 1e-2)
    # the builder's formula oracle (logsumexp too) on two batch elements
    for b in (0, 7):
        ro, rl = aten_cpu.sdpa_causal(q[b:b + 1, qh], k[b:b + 1, kh], v[b:b + 1, kh])
        close(got[b:b + 1], ro, 1.6e-2, 1e-2)
        close(lse[b:b + 1, qh], rl, 1e-3, 1e-3)
    assert torch.isfinite(out.float()).all()


def test_sdpa_decode_benchmark_shape(ops):
    """One query position per sequence, batch 64, 32 q / 8 kv heads, against a 4096-token cache:
    every sequence and head against ATen's CPU kernel."""
    g = torch.Generator().manual_seed(406)
    B, Hq, Hkv, T, D = 64, 32, 8, 4096, 128
    q = torch.randn(B, Hq, 1, D, generator=g).to(BF)
    k = torch.randn(B, Hkv, T, D, generator=g).to(BF)
    v = torch.randn(B, Hkv, T, D, generator=g).to(BF)
    out = torch.empty(B, 1, Hq, D, dtype=BF, device=DEV).transpose(1, 2)
    ops.sdpa_flash_fwd(out, None, dev(q), dev(k), dev(v), False)
    assert ops.device_error_fetch() == 0
    ref = F.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=False, enable_gqa=True)
    close(out, ref.to(BF), 1.6e-2, 1e-2)


@pytest.fixture(scope="module")
def gcu():
    import torch_gcu  # noqa: F401
    assert torch.gcu.is_available()
    return torch.device("gcu", 0)


def test_config4_layer_full_size(gcu):
    """One decoder layer at batch 8 x sequence 2048 (hidden 4096, 32 q / 8 kv heads, FFN 14336, bf16
    weights) on the "gcu" device -- the seven launches of the benchmark's layer -- against the unsharded
    fp32 CPU layer on batch elements 0 and 7 (attention is per batch element)."""
    from tp_decoder import DecoderLayer, reference_layer_cpu
    g = torch.Generator().manual_seed(407)
    x = torch.randn(8, 2048, CFG["hidden"], generator=g).to(BF)
    w = workloads.decoder_layer_weights(seed=3, dtype=BF, **CFG)
    layer = DecoderLayer(w, tp=1, backend="gcu", device=gcu, **CFG)
    with torch.autocast("gcu", dtype=BF):
        y = layer.forward_prefill(x.to(gcu))
    torch.gcu.synchronize()
    y = y.cpu().float()
    assert torch.isfinite(y).all()
    for b in (0, 7):
        ref = reference_layer_cpu(x[b:b + 1], w, **CFG)
        rel = ((y[b:b + 1] - ref).norm() / ref.norm()).item()
        assert rel < 2e-2, (b, rel)
        # element bound: one bf16 ulp at the output's magnitude plus the accumulated 16-bit roundings inside
        close(y[b:b + 1], ref, 1.6e-2, 8e-2)


def test_config5_decode_layer_batch64_kv4096(gcu):
    """One decode step of one layer at batch 64 against a 4096-token cache (position 4095), on sampled
    sequences, against the fp32 CPU evaluation of the same step."""
    from tp_decoder import DecoderLayer, reference_decode_cpu
    g = torch.Generator().manual_seed(408)
    B, T = 64, 4096
    hk, d = CFG["kv_heads"], CFG["head_dim"]
    x = torch.randn(B, 1, CFG["hidden"], generator=g).to(BF)
    kc = torch.randn(B, hk, T, d, generator=g).to(BF)
    vc = torch.randn(B, hk, T, d, generator=g).to(BF)
    w = workloads.decoder_layer_weights(seed=4, dtype=BF, **CFG)
    layer = DecoderLayer(w, tp=1, backend="gcu", device=gcu, **CFG)
    kv = (kc.to(gcu), vc.to(gcu))
    pos = T - 1
    with torch.autocast("gcu", dtype=BF):
        y = layer.forward_decode(x.to(gcu), kv, pos)
    torch.gcu.synchronize()
    y = y.cpu().float()
    assert torch.isfinite(y).all()
    seqs = [0, 1, 31, 62, 63]
    ref, k_new, v_new = reference_decode_cpu(x[seqs], kc[seqs], vc[seqs], pos, w, **CFG)
    rel = ((y[seqs] - ref).norm() / ref.norm()).item()
    assert rel < 2e-2, rel
    close(y[seqs], ref, 1.6e-2, 8e-2)
    # the step wrote the new key / value rows into the cache at `pos`, and nothing else
    close(kv[0][seqs, :, pos].cpu(), k_new.to(BF), 1.6e-2, 2e-2)
    close(kv[1][seqs, :, pos].cpu(), v_new.to(BF), 1.6e-2, 2e-2)
    assert torch.equal(kv[0][:, :, :pos].cpu().view(torch.int16), kc[:, :, :pos].view(torch.int16))
