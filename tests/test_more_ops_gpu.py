"""Comparison, selection, clamping, extreme and generator operators through the
registered backend, checked bit for bit against CPU ATen on the same inputs
(NaN handling, ties, broadcasting, scalar operands, type promotion)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import torch_gcu  # noqa: F401
    return torch.device("gcu", 0)


def _inputs(dtype, shape, seed):
    g = torch.Generator().manual_seed(seed)
    if dtype.is_floating_point:
        x = torch.randn(shape, generator=g).mul(3).round().div(2).to(dtype)   # many ties
        flat = x.view(-1)
        flat[::17] = float("nan")
        flat[5::29] = float("inf")
        flat[7::31] = float("-inf")
        return x
    if dtype == torch.bool:
        return torch.rand(shape, generator=g) > 0.5
    return torch.randint(-5, 6, shape, generator=g).to(dtype)


def same(a, b):
    assert a.dtype == b.dtype and a.shape == b.shape, (a.dtype, b.dtype, a.shape, b.shape)
    if a.dtype.is_floating_point:
        assert torch.equal(a.isnan(), b.isnan())
        assert torch.equal(torch.nan_to_num(a.float(), nan=0.0), torch.nan_to_num(b.float(), nan=0.0))
    else:
        assert torch.equal(a, b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int64, torch.int32, torch.uint8])
def test_comparisons_match_cpu(dev, dtype):
    a, b = _inputs(dtype, (37, 65), 1), _inputs(dtype, (37, 65), 2)
    row = _inputs(dtype, (65,), 3)
    for op in (torch.eq, torch.ne, torch.lt, torch.le, torch.gt, torch.ge):
        same(op(a.to(dev), b.to(dev)).cpu(), op(a, b))
        same(op(a.to(dev), row.to(dev)).cpu(), op(a, row))              # broadcast
        same(op(a.to(dev), 1).cpu(), op(a, 1))                           # scalar
        same(op(a.to(dev).t(), b.to(dev).t()).cpu(), op(a.t(), b.t()))   # strided
    if dtype == torch.int64:
        same((a.to(dev) > 0.5).cpu(), a > 0.5)                           # promotion to float


def test_logical_and_mask_ops_match_cpu(dev):
    a, b = _inputs(torch.float32, (33, 40), 4), _inputs(torch.int32, (33, 40), 5)
    m1, m2 = _inputs(torch.bool, (33, 40), 6), _inputs(torch.bool, (40,), 7)
    same(torch.logical_not(a.to(dev)).cpu(), torch.logical_not(a))
    same(torch.logical_and(a.to(dev), b.to(dev)).cpu(), torch.logical_and(a, b))
    same(torch.logical_or(b.to(dev), m1.to(dev)).cpu(), torch.logical_or(b, m1))
    same((~m1.to(dev)).cpu(), ~m1)
    same((m1.to(dev) & m2.to(dev)).cpu(), m1 & m2)
    same((m1.to(dev) | m2.to(dev)).cpu(), m1 | m2)
    same(torch.isnan(a.to(dev)).cpu(), torch.isnan(a))
    same(torch.isnan(b.to(dev)).cpu(), torch.isnan(b))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64, torch.bool])
def test_where_and_masked_fill_match_cpu(dev, dtype):
    a, b = _inputs(dtype, (19, 50), 8), _inputs(dtype, (19, 50), 9)
    c = _inputs(torch.bool, (19, 50), 10)
    crow = _inputs(torch.bool, (50,), 11)
    same(torch.where(c.to(dev), a.to(dev), b.to(dev)).cpu(), torch.where(c, a, b))
    same(torch.where(crow.to(dev), a.to(dev), b.to(dev)[0]).cpu(), torch.where(crow, a, b[0]))
    if dtype != torch.bool:
        same(torch.where(c.to(dev), a.to(dev), 2).cpu(), torch.where(c, a, 2))
        fill = -1.5 if dtype.is_floating_point else -3
        same(a.to(dev).masked_fill(c.to(dev), fill).cpu(), a.masked_fill(c, fill))
        x = a.clone().to(dev)
        x.masked_fill_(crow.to(dev), fill)
        same(x.cpu(), a.masked_fill(crow, fill))
        if dtype.is_floating_point:
            same(a.to(dev).masked_fill(c.to(dev), float("-inf")).cpu(), a.masked_fill(c, float("-inf")))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32])
def test_maximum_minimum_clamp_match_cpu(dev, dtype):
    a, b = _inputs(dtype, (29, 70), 12), _inputs(dtype, (29, 70), 13)
    same(torch.maximum(a.to(dev), b.to(dev)).cpu(), torch.maximum(a, b))
    same(torch.minimum(a.to(dev), b.to(dev)).cpu(), torch.minimum(a, b))
    lo, hi = (-1, 2) if not dtype.is_floating_point else (-0.75, 1.25)
    same(torch.clamp(a.to(dev), lo, hi).cpu(), torch.clamp(a, lo, hi))
    same(torch.clamp(a.to(dev), min=lo).cpu(), torch.clamp(a, min=lo))
    same(torch.clamp(a.to(dev), max=hi).cpu(), torch.clamp(a, max=hi))
    same(a.to(dev).clamp_min(lo).cpu(), a.clamp_min(lo))
    same(a.to(dev).clamp_max(hi).cpu(), a.clamp_max(hi))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64])
@pytest.mark.parametrize("shape,dim", [((8, 1000), 1), ((8, 1000), 0), ((5, 7, 33), 1), ((3, 4, 5), -1), ((4000,), 0)])
def test_extremes_match_cpu(dev, dtype, shape, dim):
    x = _inputs(dtype, shape, 14)
    xd = x.to(dev)
    for fn in (torch.argmax, torch.argmin):
        same(fn(xd, dim).cpu(), fn(x, dim))
        same(fn(xd, dim, keepdim=True).cpu(), fn(x, dim, keepdim=True))
    for fn in (torch.max, torch.min):
        v, i = fn(xd, dim)
        rv, ri = fn(x, dim)
        same(v.cpu(), rv)
        same(i.cpu(), ri)
    same(torch.amax(xd, dim).cpu(), torch.amax(x, dim))
    same(torch.amin(xd, dim, keepdim=True).cpu(), torch.amin(x, dim, keepdim=True))
    clean = torch.nan_to_num(x.float(), nan=0.25).to(dtype) if dtype.is_floating_point else x
    same(torch.argmax(clean.to(dev)).cpu(), torch.argmax(clean))
    same(clean.to(dev).max().cpu(), clean.max())
    same(clean.to(dev).min().cpu(), clean.min())
    same(xd.max().cpu(), x.max())   # NaN wins
    if len(shape) == 3:
        same(torch.amax(xd, (0, 2)).cpu(), torch.amax(x, (0, 2)))


def test_large_full_reduction(dev):
    g = torch.Generator().manual_seed(15)
    x = torch.randn(1 << 20, generator=g)
    same(x.to(dev).max().cpu(), x.max())
    same(x.to(dev).min().cpu(), x.min())
    same(torch.argmax(x.to(dev)).cpu(), torch.argmax(x))


def test_arange_triu_tril_match_cpu(dev):
    for args, dt in (((10,), torch.int64), ((3, 50, 7), torch.int64), ((0, 1, 0.125), torch.float32), ((5, -5, -1), torch.int32),
                     ((2048,), torch.float32), ((0, 300), torch.bfloat16)):
        same(torch.arange(*args, dtype=dt, device=dev).cpu(), torch.arange(*args, dtype=dt))
    same(torch.arange(7, device=dev).cpu(), torch.arange(7))
    x = _inputs(torch.float32, (3, 17, 23), 16)
    m = _inputs(torch.bool, (40, 40), 17)
    for d in (-3, 0, 1, 5):
        same(torch.triu(x.to(dev), d).cpu(), torch.triu(x, d))
        same(torch.tril(x.to(dev), d).cpu(), torch.tril(x, d))
        same(torch.tril(m.to(dev), d).cpu(), torch.tril(m, d))
    causal = torch.ones(64, 64, dtype=torch.bool, device=dev).tril()
    same(causal.cpu(), torch.ones(64, 64, dtype=torch.bool).tril())


def test_greedy_sampling_step(dev):
    """The ops in concert: mask logits, take the arg-max token, compare with the CPU."""
    g = torch.Generator().manual_seed(18)
    logits = torch.randn(6, 32000, generator=g)
    banned = torch.rand(32000, generator=g) < 0.01
    ld = logits.to(dev).masked_fill(banned.to(dev), float("-inf"))
    tok = torch.argmax(ld, -1)
    ref = torch.argmax(logits.masked_fill(banned, float("-inf")), -1)
    same(tok.cpu(), ref)
    probs = torch.softmax(ld, -1)
    same((probs > 1e-3).sum(-1).cpu(), (torch.softmax(logits.masked_fill(banned, float("-inf")), -1) > 1e-3).sum(-1))


# ---- sort / argsort / topk / cumsum ------------------------------------------------------------
SORT_DTYPES = [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int64, torch.int32, torch.int16,
               torch.uint8]


@pytest.mark.parametrize("dtype", SORT_DTYPES)
@pytest.mark.parametrize("descending", [False, True])
def test_stable_sort_matches_cpu(dev, dtype, descending):
    """Stable sort along every dimension: values and indices bit for bit with CPU ATen's stable sort
    (many ties, NaN above every number, infinities, both zeros; rows longer than one 2048-key tile)."""
    for shape, seed in (((5, 4099), 21), ((3, 7, 33), 22), ((1,), 23), ((2, 0, 3), 24), ((70, 130), 25)):
        x = _inputs(dtype, shape, seed)
        if dtype.is_floating_point and x.numel() > 40:
            x.view(-1)[3::37] = -0.0
            x.view(-1)[4::41] = 0.0
        for dim in range(-1, x.dim() - 1 if x.dim() > 1 else 0):
            v, i = torch.sort(x.to(dev), dim=dim, descending=descending, stable=True)
            rv, ri = torch.sort(x, dim=dim, descending=descending, stable=True)
            same(i.cpu(), ri)
            same(v.cpu(), rv)
            if dtype.is_floating_point:   # the values are the input's own bits: zero signs survive
                assert torch.equal(torch.signbit(v.cpu()), torch.signbit(rv))
            same(torch.argsort(x.to(dev), dim=dim, descending=descending, stable=True).cpu(), ri)
    s = torch.tensor(3.5).to(dtype)
    v, i = torch.sort(s.to(dev), stable=True)
    assert v.cpu() == s and i.item() == 0


def test_sort_default_and_noncontiguous_inputs(dev):
    g = torch.Generator().manual_seed(26)
    x = torch.randn(40, 50, generator=g)           # distinct values: the unstable request has one answer
    v, i = torch.sort(x.to(dev).t(), dim=0)
    rv, ri = torch.sort(x.t(), dim=0)
    same(v.cpu(), rv)
    same(i.cpu(), ri)
    same(torch.argsort(x.to(dev), descending=True).cpu(), torch.argsort(x, descending=True))
    out_v, out_i = torch.empty(50, 40, device=dev).t(), torch.empty(50, 40, dtype=torch.int64, device=dev).t()
    torch.sort(x.to(dev), dim=1, stable=True, out=(out_v, out_i))   # non-contiguous outputs
    rv, ri = torch.sort(x, dim=1, stable=True)
    same(out_v.cpu(), rv)
    same(out_i.cpu(), ri)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int64])
def test_topk_matches_cpu(dev, dtype):
    g = torch.Generator().manual_seed(27)
    # distinct values per row (a permutation, scaled): top-k has one answer, indices included
    n = 300 if dtype == torch.bfloat16 else 5000
    x = torch.stack([torch.randperm(n, generator=g) for _ in range(6)]).sub(n // 2)
    x = (x.float() * 0.25).to(dtype) if dtype.is_floating_point else x.to(dtype)
    for k, largest in ((1, True), (50, True), (17, False), (n, True)):
        v, i = torch.topk(x.to(dev), k, dim=-1, largest=largest)
        rv, ri = torch.topk(x, k, dim=-1, largest=largest)
        same(v.cpu(), rv)
        same(i.cpu(), ri)
    v, i = torch.topk(x.to(dev), 5, dim=0)     # a column may hold equal values: the indices are checked through the values
    rv, ri = torch.topk(x, 5, dim=0)
    same(v.cpu(), rv)
    same(torch.gather(x, 0, i.cpu()), rv)
    # ties and NaN: the values are determined, and every index points at its value; among equal
    # elements this backend returns the lowest index first (NaN counts as the largest)
    y = _inputs(torch.float32, (4, 999), 28)
    v, i = torch.topk(y.to(dev), 40, dim=-1)
    rv, _ = torch.topk(y, 40, dim=-1)
    same(v.cpu(), rv)
    same(torch.gather(y, 1, i.cpu()), rv)
    sv, si = torch.sort(y, dim=-1, descending=True, stable=True)
    same(i.cpu(), si[:, :40])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64, torch.bfloat16, torch.float16, torch.int64, torch.int32,
                                   torch.uint8])
def test_cumsum_matches_cpu(dev, dtype):
    g = torch.Generator().manual_seed(29)
    for shape in ((3, 5000), (17, 9, 11), (1,), (0, 4), (2, 3, 2100)):
        if dtype.is_floating_point:
            x = torch.randn(shape, generator=g).to(dtype)
        else:
            x = torch.randint(0 if dtype == torch.uint8 else -50, 50, shape, generator=g).to(dtype)
        for dim in range(x.dim()):
            got = torch.cumsum(x.to(dev), dim).cpu()
            ref = torch.cumsum(x, dim)
            assert got.dtype == ref.dtype and got.shape == ref.shape
            if not dtype.is_floating_point or dim != x.dim() - 1:
                same(got, ref)   # integers, and the serial order of a non-last dimension: identical
            else:
                # a row is scanned in parallel: fp32 / fp64 within 1e-6 relative, 16-bit types within one ulp
                rtol = 1e-6 if dtype in (torch.float32, torch.float64) else 2 ** -7
                scale = x.float().abs().cumsum(dim).clamp_min(1.0)   # error grows with the running magnitude
                assert ((got.float() - ref.float()).abs() <= rtol * scale).all()
    # integer inputs promote to int64, and dtype= is honoured
    xi = torch.randint(-5, 5, (4, 100), generator=g, dtype=torch.int32)
    same(torch.cumsum(xi.to(dev), 1).cpu(), torch.cumsum(xi, 1))
    same(torch.cumsum(xi.to(dev), 1, dtype=torch.float32).cpu(), torch.cumsum(xi, 1, dtype=torch.float32))


def test_top_k_top_p_sampling_step(dev):
    """A sampling step the way serving code writes it: top-k cut, softmax, descending sort, cumulative
    probability, nucleus mask, renormalise -- the kept token set and the renormalised distribution match
    the CPU."""
    g = torch.Generator().manual_seed(30)
    logits = torch.randn(8, 32000, generator=g) * 2.0

    def step(lg):
        kth = torch.topk(lg, 50, dim=-1).values[:, -1:]
        lg = lg.masked_fill(lg < kth, float("-inf"))
        probs = torch.softmax(lg, -1)
        sp, si = torch.sort(probs, dim=-1, descending=True, stable=True)
        cum = torch.cumsum(sp, -1)
        keep = (cum - sp) < 0.9                      # tokens whose preceding mass is below top-p
        sp = torch.where(keep, sp, torch.zeros_like(sp))
        sp = sp / sp.sum(-1, keepdim=True)
        return sp, si, keep
    sp, si, keep = step(logits.to(dev))
    rsp, rsi, rkeep = step(logits)
    same(si.cpu()[:, :50], rsi[:, :50])              # beyond the top-k cut every probability is an equal zero
    same(keep.cpu(), rkeep)
    assert torch.allclose(sp.cpu(), rsp, rtol=1e-5, atol=1e-7)
    # the C ABI itself: sorted probabilities and their cumulative sum
    import b200ops as ops
    p = torch.softmax(logits, -1).to("cuda:0")
    v = torch.empty_like(p)
    i = torch.empty(p.shape, dtype=torch.int64, device="cuda:0")
    ops.sort_rows(v, i, p, descending=True)
    rv, ri = torch.sort(p.cpu(), dim=-1, descending=True, stable=True)
    same(v.cpu(), rv)
    same(i.cpu(), ri)
    c = torch.empty_like(v)
    ops.cumsum(c, v, 1)
    assert torch.allclose(c.cpu(), torch.cumsum(rv, -1), rtol=1e-6, atol=1e-7)
    assert ops.device_error_fetch() == 0
