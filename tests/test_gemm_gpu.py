"""mm / addmm / bmm / baddbmm through the C ABI: the reference's own fp32 cases
(test/op_test/test_linear.py) and bf16 / f16 tensor-core shapes and layouts,
checked against CPU arithmetic."""
import pytest
import torch

from oracle import aten_cpu
from test_ops_gpu import DEV, close, dev

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def tc_close(out, a, b, extra=None, alpha=1.0, beta=1.0):
    """bf16/f16 contraction tolerance: fp32-accumulated CPU result rounded once;
    rtol 1.6e-2 (reference class tolerance for 16-bit contractions), atol scaled
    with sqrt(K) because |out| grows like sqrt(K) for N(0,1) operands."""
    ref = alpha * (a.float() @ b.float())
    if extra is not None:
        ref = ref + beta * extra.float()
    K = a.shape[-1]
    close(out, ref.to(out.dtype), 1.6e-2, 1e-2 * max(1.0, (K / 64) ** 0.5))


def test_reference_linear_cases_fp32(ops, golden):
    g = golden("ref_linear")
    m = g["mm"]
    out = torch.empty(2, 3, device=DEV)
    ops.mm(out, dev(m["m1"]), dev(m["m2"]))
    close(out, m["out"], 1e-5, 1e-8)  # torch.allclose defaults, as the reference test uses
    am = g["addmm"]
    ops.addmm(out, dev(am["c"]).expand(2, 3), dev(am["m1"]), dev(am["m2"]))
    close(out, am["out"], 1e-5, 1e-8)
    bm = g["bmm"]
    ob = torch.empty(4, 2, 3, device=DEV)
    ops.bmm(ob, dev(bm["b1"]), dev(bm["b2"]))
    close(ob, bm["out"], 1e-5, 1e-8)
    bb = g["baddbmm"]
    o2 = torch.empty(4, 2, 5, device=DEV)
    ops.baddbmm(o2, dev(bb["i"]), dev(bb["b1"]), dev(bb["b2"]), bb["beta"], bb["alpha"])
    close(o2, bb["out"], 1e-5, 1e-7)
    lin = g["linear"]  # linear = addmm(bias, x, w.t())
    ol = torch.empty(2, 3, device=DEV)
    ops.addmm(ol, dev(lin["b"]).expand(2, 3), dev(lin["x"]), dev(lin["w"]).t())
    close(ol, lin["out"], 1e-5, 1e-7)
    ops.mm(ol, dev(lin["x"]), dev(lin["w"]).t())
    close(ol, lin["out_nobias"], 1e-5, 1e-7)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 64, 128), (256, 512, 256), (130, 200, 72), (64, 6144, 512),
                                   (1, 8, 8), (300, 136, 40), (1024, 1024, 1024), (257, 1032, 192)])
@pytest.mark.parametrize("dtype", [BF, torch.float16])
def test_mm_weight_transposed(ops, M, N, K, dtype):
    """x @ w.t(): both operands K-contiguous (the nn.Linear layout)."""
    g = torch.Generator().manual_seed(41)
    a = torch.randn(M, K, generator=g).to(dtype)
    w = torch.randn(N, K, generator=g).to(dtype)
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    ops.mm(out, dev(a), dev(w).t())
    tc_close(out, a, w.t())
    assert ops.device_error_fetch() == 0


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (200, 136, 96), (512, 384, 320)])
def test_mm_other_layouts(ops, M, N, K):
    g = torch.Generator().manual_seed(42)
    a = torch.randn(M, K, generator=g).to(BF)
    b = torch.randn(K, N, generator=g).to(BF)
    out = torch.empty(M, N, dtype=BF, device=DEV)
    ops.mm(out, dev(a), dev(b))                  # B row-major (N contiguous)
    tc_close(out, a, b)
    at = dev(a.t().contiguous()).t()             # A column-major (M contiguous)
    ops.mm(out, at, dev(b))
    tc_close(out, a, b)
    ops.mm(out, at, dev(b.t().contiguous()).t())
    tc_close(out, a, b)
    wide = torch.zeros(M, N + 24, dtype=BF, device=DEV)   # strided output rows
    ops.mm(wide[:, 8:8 + N], dev(a), dev(b))
    tc_close(wide[:, 8:8 + N], a, b)
    assert wide[:, :8].abs().sum().item() == 0 and wide[:, 8 + N:].abs().sum().item() == 0


def test_addmm_bias_and_scaling(ops, golden):
    g = torch.Generator().manual_seed(43)
    a, w = torch.randn(160, 192, generator=g).to(BF), torch.randn(264, 192, generator=g).to(BF)
    bias = torch.randn(264, generator=g).to(BF)
    out = torch.empty(160, 264, dtype=BF, device=DEV)
    ops.addmm(out, dev(bias).expand(160, 264), dev(a), dev(w).t())
    tc_close(out, a, w.t(), bias.expand(160, 264))
    full = torch.randn(160, 264, generator=g).to(BF)
    ops.addmm(out, dev(full), dev(a), dev(w).t(), beta=-0.5, alpha=0.25)
    tc_close(out, a, w.t(), full, alpha=0.25, beta=-0.5)
    m = golden("op_small")["mm_bf16"]
    o = torch.empty(64, 80, dtype=BF, device=DEV)
    ops.mm(o, dev(m["a"]), dev(m["b"]))
    close(o, m["out"], 1.6e-2, 1e-2)


def test_bmm_batched(ops):
    g = torch.Generator().manual_seed(44)
    a = torch.randn(5, 130, 72, generator=g).to(BF)
    b = torch.randn(5, 72, 96, generator=g).to(BF)
    out = torch.empty(5, 130, 96, dtype=BF, device=DEV)
    ops.bmm(out, dev(a), dev(b))
    tc_close(out, a, b)
    ops.bmm(out, dev(a), dev(b.transpose(1, 2).contiguous()).transpose(1, 2))
    tc_close(out, a, b)
    add = torch.randn(5, 130, 96, generator=g).to(BF)
    ops.baddbmm(out, dev(add), dev(a), dev(b), beta=2.0, alpha=0.5)
    tc_close(out, a, b, add, alpha=0.5, beta=2.0)
    f = torch.randn(3, 7, 5, generator=g)
    h = torch.randn(3, 5, 9, generator=g)
    of = torch.empty(3, 7, 9, device=DEV)
    ops.bmm(of, dev(f), dev(h))
    close(of, aten_cpu.bmm(f, h), 1e-5, 1e-6)


def test_mm_unaligned_falls_back_and_empty(ops):
    g = torch.Generator().manual_seed(45)
    a, b = torch.randn(33, 21, generator=g).to(BF), torch.randn(21, 19, generator=g).to(BF)
    out = torch.empty(33, 19, dtype=BF, device=DEV)
    ops.mm(out, dev(a), dev(b))  # leading dimensions not multiples of 8: SIMT path
    tc_close(out, a, b)
    e = torch.empty(0, 19, dtype=BF, device=DEV)
    ops.mm(e, torch.empty(0, 21, dtype=BF, device=DEV), dev(b))
    z = torch.ones(4, 6, dtype=BF, device=DEV)
    ops.mm(z, torch.empty(4, 0, dtype=BF, device=DEV), torch.empty(0, 6, dtype=BF, device=DEV))
    assert z.abs().sum().item() == 0


def test_layer_projection_shapes(ops):
    """Decoder-layer GEMM shapes at a reduced token count, checked on sampled rows."""
    g = torch.Generator().manual_seed(46)
    x = torch.randn(512, 4096, generator=g).to(BF)
    for n in (6144, 4096):
        w = (torch.randn(n, 4096, generator=g) * 0.02).to(BF)
        out = torch.empty(512, n, dtype=BF, device=DEV)
        ops.mm(out, dev(x), dev(w).t())
        rows = torch.tensor([0, 1, 127, 128, 255, 300, 511])
        ref = (x[rows].float() @ w.float().t())
        close(out[rows], ref.to(BF), 1.6e-2, 1e-2)


def _sampled_close(out, a_f, b_f, rows, cols, K, extra=None, alpha=1.0, beta=1.0):
    ref = alpha * (a_f[rows] @ b_f[:, cols])
    if extra is not None:
        ref = ref + beta * extra.float()[rows][:, cols]
    close(out[dev(rows)][:, dev(cols)], ref.to(out.dtype), 1.6e-2, 1e-2 * max(1.0, (K / 64) ** 0.5))


@pytest.mark.parametrize("M,N,K", [(3000, 3500, 520), (4096, 4096, 256), (2309, 4100, 72)])
def test_mm_large_enough_for_cta_pairs(ops, M, N, K):
    """Products with at least 148 tiles of 256 x 256 run on the two-CTA kernel: ragged
    edges in M, N and K, every operand layout, scaling and an addend; checked on
    sampled rows and columns that cover both CTAs of a pair and the tile borders."""
    g = torch.Generator().manual_seed(47)
    a = torch.randn(M, K, generator=g).to(BF)
    b = torch.randn(K, N, generator=g).to(BF)
    af, bf_ = a.float(), b.float()
    rows = torch.tensor(sorted({0, 1, 127, 128, 129, 255, 256, 383, 384, 511, 512, M // 2, M - 130, M - 2, M - 1}))
    cols = torch.tensor(sorted({0, 31, 32, 127, 128, 255, 256, 257, N // 2, N - 129, N - 33, N - 1}))
    out = torch.empty(M, N, dtype=BF, device=DEV)
    layouts = [(dev(a), dev(b.t().contiguous()).t()),                      # both K-contiguous
               (dev(a), dev(b)),                                           # B N-contiguous
               (dev(a.t().contiguous()).t(), dev(b)),                      # A M-contiguous
               (dev(a.t().contiguous()).t(), dev(b.t().contiguous()).t())]
    for x, y in layouts:
        out.zero_()
        ops.mm(out, x, y)
        assert ops.device_error_fetch() == 0
        _sampled_close(out, af, bf_, rows, cols, K)
    add = torch.randn(M, N, generator=g).to(BF)
    ops.addmm(out, dev(add), layouts[0][0], layouts[0][1], beta=-0.5, alpha=0.25)
    _sampled_close(out, af, bf_, rows, cols, K, add, alpha=0.25, beta=-0.5)
    # whole-matrix check against the one fp32 product, loose: catches a misplaced tile
    ops.mm(out, layouts[0][0], layouts[0][1])
    full = (af @ bf_)
    assert (out.float().cpu() - full).abs().max().item() <= 0.02 * full.abs().max().item() + 0.5


def test_bmm_large_enough_for_cta_pairs(ops):
    g = torch.Generator().manual_seed(48)
    a = torch.randn(40, 500, 136, generator=g).to(torch.float16)
    b = torch.randn(40, 136, 520, generator=g).to(torch.float16)
    out = torch.empty(40, 500, 520, dtype=torch.float16, device=DEV)
    ops.bmm(out, dev(a), dev(b))
    tc_close(out, a, b)


@pytest.mark.parametrize("M,N,K", [(64, 4096, 14336), (100, 520, 1000), (1, 6144, 4096), (128, 1032, 2048),
                                   # the rows that exist are dealt out in bands over the cluster: bands of 8, 5
                                   # (37 = 7 x 5 + 2) and 1 row (three rows over eight CTAs: five own nothing),
                                   # ragged N and K, two / four / eight slices
                                   (64, 4096, 4096), (37, 1000, 4104), (3, 2048, 8192), (33, 136, 520), (64, 9000, 1024),
                                   (65, 4096, 4096)])
def test_mm_skinny_split_k(ops, M, N, K):
    """Few rows against a large weight matrix (the decode step): K is split over a
    cluster and the partial tiles are summed in a fixed order, so two runs agree
    bit for bit."""
    g = torch.Generator().manual_seed(49)
    a = torch.randn(M, K, generator=g).to(BF)
    w = (torch.randn(N, K, generator=g) * 0.05).to(BF)
    out = torch.empty(M, N, dtype=BF, device=DEV)
    ops.mm(out, dev(a), dev(w).t())
    assert ops.device_error_fetch() == 0
    tc_close(out, a, w.t())
    again = torch.empty_like(out)
    ops.mm(again, dev(a), dev(w).t())
    assert torch.equal(out, again)
    ops.mm(again, dev(a.t().contiguous()).t(), dev(w.t().contiguous()))      # both operands MN-contiguous
    tc_close(again, a, w.t())
    add = torch.randn(M, N, generator=g).to(BF)
    ops.addmm(again, dev(add), dev(a), dev(w).t(), beta=0.5, alpha=2.0)
    tc_close(again, a, w.t(), add, alpha=2.0, beta=0.5)
    if M <= 64:   # through the batched entry point (fewer slices per product: close, not identical)
        a3, w3 = torch.stack([a, a.flip(0)]), torch.stack([w, w.flip(0)])
        out3 = torch.empty(2, M, N, dtype=BF, device=DEV)
        ops.bmm(out3, dev(a3), dev(w3).transpose(1, 2))
        assert ops.device_error_fetch() == 0
        tc_close(out3[0], a, w.t())
        tc_close(out3[1], a3[1], w3[1].t())


def test_mm_swiglu_few_rows_rule(ops):
    """The predicate a caller uses to choose between the fused product and mm + swiglu for few rows: a weight
    wide enough for one tile of 64 to 128 gate columns per SM, or one whose K can be split over clusters."""
    assert ops.mm_swiglu_few_rows(64, 14336, 4096) and ops.mm_swiglu_few_rows(1, 9472, 512) and ops.mm_swiglu_few_rows(128, 18944, 256)
    assert ops.mm_swiglu_few_rows(64, 3584, 4096) and ops.mm_swiglu_few_rows(64, 7168, 4096) and ops.mm_swiglu_few_rows(64, 1792, 4096)
    assert not ops.mm_swiglu_few_rows(129, 14336, 4096) and not ops.mm_swiglu_few_rows(64, 3584, 256)
    assert not ops.mm_swiglu_few_rows(64, 148 * 136, 256) and not ops.mm_swiglu_few_rows(0, 14336, 4096)


@pytest.mark.parametrize("M,F,K,dtype", [(2048, 1024, 256, BF), (1000, 1100, 520, BF), (300, 136, 72, torch.float16),
                                         (4096, 3584, 512, BF),
                                         # one row-tile against a wide weight: the one-wave kernel (tile width chosen
                                         # so that the tiles fill the SMs: 104 + 104, 64 + 64, 128 + 128 rows), and
                                         # narrower weights, which stay on the pair kernel
                                         (64, 14336, 4096, BF), (1, 9472, 512, BF), (128, 9400, 256, torch.float16),
                                         (1, 7168, 512, BF), (128, 7104, 256, torch.float16),
                                         # few rows against a narrower weight: K split over clusters of 2 / 4 / 8, tiles
                                         # of 64 gate + 64 up rows, the activation applied by the CTA that sums a band
                                         (64, 7168, 4096, BF), (37, 1000, 1032, BF), (5, 100, 4096, torch.float16), (128, 1792, 2048, BF),
                                         (37, 9000, 520, BF), (64, 18944, 1024, BF), (64, 1792, 4096, BF), (64, 3584, 1024, BF),
                                         (16, 2368, 256, torch.float16), (3, 1200, 136, BF), (128, 200, 64, BF)])
def test_mm_swiglu_fused_epilogue(ops, M, F, K, dtype):
    """Gate/up projection with silu(gate) * up applied in the GEMM epilogue, against
    fp32 CPU arithmetic on the same operands; ragged M, F and K."""
    g = torch.Generator().manual_seed(50)
    a = torch.randn(M, K, generator=g).to(dtype)
    w = (torch.randn(2 * F, K, generator=g) * (2.0 / K ** 0.5)).to(dtype)
    out = torch.empty(M, F, dtype=dtype, device=DEV)
    ops.mm_swiglu(out, dev(a), dev(w))
    assert ops.device_error_fetch() == 0
    gu = a.float() @ w.float().t()
    ref = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    close(out, ref.to(dtype), 1.6e-2, 2e-2)
    # the unfused pair of calls rounds the projection to 16 bits first: close, not identical
    gu_dev = torch.empty(M, 2 * F, dtype=dtype, device=DEV)
    ops.mm(gu_dev, dev(a), dev(w).t())
    two = torch.empty_like(out)
    ops.swiglu(two, gu_dev[:, :F], gu_dev[:, F:])
    close(out, two.cpu(), 3e-2, 3e-2)


@pytest.mark.parametrize("B,S,K,heads,rope_heads,dtype", [(2, 512, 256, 6, 5, BF), (1, 600, 136, 3, 2, torch.float16),
                                                          (4, 300, 512, 8, 8, BF), (2, 256, 128, 4, 0, BF)])
def test_mm_rope_fused_epilogue(ops, B, S, K, heads, rope_heads, dtype):
    """qkv projection with rotate-half RoPE applied to the first heads in the GEMM epilogue, against fp32
    CPU arithmetic; heads past rope_heads (the v part) come out unrotated."""
    g = torch.Generator().manual_seed(56)
    N = heads * 128
    a = torch.randn(B * S, K, generator=g).to(dtype)
    w = (torch.randn(N, K, generator=g) * (1.0 / K ** 0.5)).to(dtype)
    import workloads
    cos, sin = workloads.rope_tables(S + 7, 128)
    out = torch.empty(B * S, N, dtype=dtype, device=DEV)
    ops.mm_rope(out, dev(a), dev(w), dev(cos), dev(sin), S, rope_heads * 128)
    assert ops.device_error_fetch() == 0
    y = (a.float() @ w.float().t()).view(B, S, heads, 128)
    pos = torch.arange(S)
    c = torch.cat((cos[pos], cos[pos]), -1)[None, :, None, :]
    s_ = torch.cat((sin[pos], sin[pos]), -1)[None, :, None, :]
    rot = torch.cat((-y[..., 64:], y[..., :64]), -1)
    ref = y.clone()
    ref[:, :, :rope_heads] = (y * c + rot * s_)[:, :, :rope_heads]
    close(out.view(B, S, heads, 128), ref.to(dtype), 1.6e-2, 1e-2 * max(1.0, (K / 64) ** 0.5))
