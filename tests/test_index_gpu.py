"""Bit-exact parity of the index kernels (through the C ABI) with CPU ATen."""
import pytest
import torch

from oracle import aten_cpu
from test_ops_gpu import DEV, dev, exact

pytestmark = pytest.mark.gpu


def _ws(n):
    return torch.empty(max(int(n), 1), dtype=torch.uint8, device=DEV)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.int64, torch.uint8])
@pytest.mark.parametrize("shape,dim,k", [((300, 24), 0, 50), ((300, 24), 1, 10), ((128, 4096), 0, 333),
                                         ((7, 9, 5), 1, 13), ((50, 3), 0, 0), ((1000, 1), 0, 77), ((4, 33, 7), 2, 6)])
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_index_select(ops, dtype, shape, dim, k, idt):
    g = torch.Generator().manual_seed(21)
    a = (torch.randn(shape, generator=g) * 100).to(dtype)
    idx = torch.randint(0, shape[dim], (k,), generator=g).to(idt)
    ref = aten_cpu.index_select(a, dim, idx)
    out = torch.empty(ref.shape, dtype=dtype, device=DEV)
    ops.index_select(out, dev(a), dim, dev(idx))
    exact(out, ref)


def test_embedding_golden(ops, golden):
    g = golden("op_small")["embedding"]
    out = torch.empty(3, 17, 24, dtype=torch.bfloat16, device=DEV)
    ops.index_select(out, dev(g["table"]), 0, dev(g["ids"].reshape(-1)))
    exact(out, g["out"])


@pytest.mark.parametrize("shape,cols", [((19, 40), 40), ((64, 1024), 1024), ((5, 7), 3), ((33, 128), 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64])
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_gather_last_dim(ops, shape, cols, dtype, idt):
    g = torch.Generator().manual_seed(22)
    a = torch.randn(shape, generator=g).to(dtype)
    idx = torch.randint(0, shape[1], (shape[0], cols), generator=g).to(idt)
    out = torch.empty(idx.shape, dtype=dtype, device=DEV)
    ops.gather(out, dev(a), 1, dev(idx))
    exact(out, aten_cpu.gather(a, 1, idx))


def test_gather_other_dims_and_smaller_index(ops):
    g = torch.Generator().manual_seed(23)
    a = torch.randn(9, 11, 13, generator=g)
    idx = torch.randint(0, 9, (4, 11, 13), generator=g)
    out = torch.empty(4, 11, 13, device=DEV)
    ops.gather(out, dev(a), 0, dev(idx))
    exact(out, aten_cpu.gather(a, 0, idx))
    idx = torch.randint(0, 11, (5, 6, 7), generator=g)
    out = torch.empty(5, 6, 7, device=DEV)
    ops.gather(out, dev(a), 1, dev(idx))
    exact(out, aten_cpu.gather(a, 1, idx))


@pytest.mark.parametrize("n_src,n_dst,inner", [(500, 60, 12), (5000, 300, 256), (4097, 1, 8), (10, 5000, 64),
                                               (70000, 70000, 4), (1, 1, 1), (9000, 513, 3), (0, 7, 4), (70000, 3, 4),
                                               (3000, 90, 8)])
@pytest.mark.parametrize("idt", [torch.int64, torch.int32])
def test_scatter_add_rows_bit_exact(ops, n_src, n_dst, inner, idt):
    g = torch.Generator().manual_seed(24)
    src = torch.randn(n_src, inner, generator=g)
    rows = torch.randint(0, n_dst, (n_src,), generator=g)
    base = torch.randn(n_dst, inner, generator=g)
    index = rows[:, None].expand(-1, inner)
    ref = aten_cpu.scatter_add(base, 0, index, src)
    d_index = dev(rows.to(idt))[:, None].expand(-1, inner)
    ws = _ws(ops.scatter_add_workspace_size(dev(base), 0, d_index, dev(src)))
    out = torch.empty_like(dev(base))
    ops.scatter_add(out, dev(base), 0, d_index, dev(src), ws)
    exact(out, ref)
    # twice: reproducible, and in place
    out2 = dev(base).clone()
    ops.scatter_add(out2, out2, 0, d_index, dev(src), ws)
    exact(out2, ref)
    # index_put(accumulate) is the same computation, deterministic order
    if n_src > 0:
        tgt = dev(base).clone()
        ws2 = _ws(ops.index_put_workspace_size(tgt, dev(rows.to(idt)), dev(src)))
        ops.index_put(tgt, dev(rows.to(idt)), dev(src), True, ws2)
        exact(tgt, aten_cpu.index_put(base, [rows], src, True))
        tgt = dev(base).clone()
        ops.index_put(tgt, dev(rows.to(idt)), dev(src), False, ws2)
        exact(tgt, aten_cpu.index_put(base, [rows], src, False))


def test_scatter_add_bad_index_is_dropped_and_flagged(ops):
    """An out-of-range row index never traps: that source row is dropped, bit 0 of the device error word
    is set, and every other row's sum is unaffected."""
    g = torch.Generator().manual_seed(28)
    src = torch.randn(4000, 8, generator=g)
    rows = torch.randint(0, 50, (4000,), generator=g)
    bad = rows.clone()
    bad[123], bad[3999] = 50, -7
    base = torch.randn(50, 8, generator=g)
    keep = torch.ones(4000, dtype=torch.bool)
    keep[123] = keep[3999] = False
    ref = aten_cpu.scatter_add(base, 0, rows[keep][:, None].expand(-1, 8), src[keep])
    idx = dev(bad)[:, None].expand(-1, 8)
    ws = _ws(ops.scatter_add_workspace_size(dev(base), 0, idx, dev(src)))
    out = torch.empty_like(dev(base))
    ops.scatter_add(out, dev(base), 0, idx, dev(src), ws)
    assert ops.device_error_fetch() & 1
    exact(out, ref)


def test_scatter_add_element_form_four_pass_sort_with_a_bad_index(ops):
    """Element form (a full index tensor) over more than 2^24 destination elements: the stable sort of
    (destination offset, source) takes four 8-bit passes, and its top digit reaches bit 24-30 while bit 31
    carries the out-of-range flag. One bad index must drop that element only (error word bit 0), not
    disturb the order of the rest."""
    g = torch.Generator().manual_seed(29)
    R, C = (1 << 21) + 3, 8                       # 16.8 M destination elements: 25 key bits
    base = torch.zeros(R, C)
    n = 3000
    idx = torch.randint(0, R, (n, C), generator=g)
    idx[:200] = idx[0]                             # collisions: ordered sums
    idx[:, 0] = R - 1                              # the top of the key range
    src = torch.randn(n, C, generator=g)
    ref = aten_cpu.scatter_add(base, 0, idx, src)
    bad = idx.clone()
    bad[1234, 5] = R                               # out of range
    ref_bad = ref.clone()
    ref_bad[idx[1234, 5], 5] = aten_cpu.scatter_add(torch.zeros(R, 1), 0, torch.cat([idx[:1234, 5:6], idx[1235:, 5:6]]),
                                                    torch.cat([src[:1234, 5:6], src[1235:, 5:6]]))[idx[1234, 5], 0]
    for index, want, flagged in ((idx, ref, False), (bad, ref_bad, True)):
        ws = _ws(ops.scatter_add_workspace_size(dev(base), 0, dev(index), dev(src)))
        out = torch.empty_like(dev(base))
        ops.scatter_add(out, dev(base), 0, dev(index), dev(src), ws)
        assert bool(ops.device_error_fetch() & 1) == flagged
        exact(out, want)


def test_scatter_add_all_sources_one_row(ops):
    """Worst-case collision: one destination takes every source, in order."""
    g = torch.Generator().manual_seed(25)
    src = torch.randn(20000, 16, generator=g)
    rows = torch.full((20000,), 3, dtype=torch.int64)
    base = torch.randn(8, 16, generator=g)
    ref = aten_cpu.scatter_add(base, 0, rows[:, None].expand(-1, 16), src)
    idx = dev(rows)[:, None].expand(-1, 16)
    ws = _ws(ops.scatter_add_workspace_size(dev(base), 0, idx, dev(src)))
    out = torch.empty_like(dev(base))
    ops.scatter_add(out, dev(base), 0, idx, dev(src), ws)
    exact(out, ref)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float64, torch.int64])
@pytest.mark.parametrize("inner", [24, 8])
def test_scatter_add_other_dtypes(ops, dtype, inner):
    """bf16: CPU scatter_add sums in fp32 and rounds once (index_put, checked
    below, rounds after every add); both must match bit for bit."""
    g = torch.Generator().manual_seed(26)
    src = (torch.randn(3000, inner, generator=g) * 4).to(dtype)
    rows = torch.randint(0, 100, (3000,), generator=g)
    base = (torch.randn(100, inner, generator=g) * 4).to(dtype)
    ref = aten_cpu.scatter_add(base, 0, rows[:, None].expand(-1, inner), src)
    idx = dev(rows)[:, None].expand(-1, inner)
    ws = _ws(ops.scatter_add_workspace_size(dev(base), 0, idx, dev(src)))
    out = torch.empty_like(dev(base))
    ops.scatter_add(out, dev(base), 0, idx, dev(src), ws)
    exact(out, ref)
    full = torch.randint(0, 100, (3000, inner), generator=g)
    ws = _ws(ops.scatter_add_workspace_size(dev(base), 0, dev(full), dev(src)))
    ops.scatter_add(out, dev(base), 0, dev(full), dev(src), ws)
    exact(out, aten_cpu.scatter_add(base, 0, full, src))
    tgt = dev(base).clone()
    ops.index_put(tgt, dev(rows), dev(src), True, _ws(ops.index_put_workspace_size(tgt, dev(rows), dev(src))))
    exact(tgt, aten_cpu.index_put(base, [rows], src, True))


@pytest.mark.parametrize("dim", [0, 1])
def test_scatter_add_full_index_bit_exact(ops, dim):
    g = torch.Generator().manual_seed(27)
    src = torch.randn(700, 33, generator=g)
    base = torch.randn(90, 33, generator=g) if dim == 0 else torch.randn(700, 50, generator=g)
    index = torch.randint(0, base.shape[dim], (700, 33), generator=g)
    ref = aten_cpu.scatter_add(base, dim, index, src)
    ws = _ws(ops.scatter_add_workspace_size(dev(base), dim, dev(index), dev(src)))
    out = torch.empty_like(dev(base))
    ops.scatter_add(out, dev(base), dim, dev(index), dev(src), ws)
    exact(out, ref)


def test_scatter_golden(ops, golden):
    g = golden("op_small")
    s = g["scatter_add"]
    idx = dev(s["rows"])[:, None].expand(-1, 12)
    ws = _ws(ops.scatter_add_workspace_size(dev(s["self"]), 0, idx, dev(s["src"])))
    out = torch.empty_like(dev(s["self"]))
    ops.scatter_add(out, dev(s["self"]), 0, idx, dev(s["src"]), ws)
    exact(out, s["out"])
    f = g["scatter_add_full"]
    ws = _ws(ops.scatter_add_workspace_size(dev(f["self"]), 0, dev(f["index"]), dev(f["src"])))
    ops.scatter_add(out, dev(f["self"]), 0, dev(f["index"]), dev(f["src"]), ws)
    exact(out, f["out"])


def _advanced_index_args(self_d, indices):
    """ATen's AdvancedIndex for leading-dim indices (ops.cpp:48-90 of the
    reference's efficient_ops): src restrided to the result shape, indices
    broadcast to it, plus the replaced sizes/strides."""
    idx = torch.broadcast_tensors(*indices)
    n = len(idx)
    ishape = tuple(idx[0].shape)
    rest = tuple(self_d.shape[n:])
    out_shape = ishape + rest
    src_view = self_d.as_strided(out_shape, (0,) * len(ishape) + tuple(self_d.stride()[n:]))
    views = [i.reshape(ishape + (1,) * len(rest)).expand(out_shape) for i in idx]
    return out_shape, src_view, views, list(self_d.shape[:n]), list(self_d.stride()[:n])


@pytest.mark.parametrize("idt", [torch.int32, torch.int64])
def test_index_int32_and_int64(ops, golden, idt):
    gi = golden("op_small")["index_int32"]
    base, idx = gi["self"], gi["idx"].to(idt)
    shape, sv, views, isz, ist = _advanced_index_args(dev(base), [dev(idx)])
    out = torch.empty(shape, device=DEV)
    ops.index(out, sv, views, isz, ist)
    exact(out, gi["out"])
    g = torch.Generator().manual_seed(28)
    a = torch.randn(13, 17, 40, generator=g).to(torch.bfloat16)
    i0 = torch.randint(-13, 13, (6, 1), generator=g).to(idt)
    i1 = torch.randint(-17, 17, (1, 5), generator=g).to(idt)
    shape, sv, views, isz, ist = _advanced_index_args(dev(a), [dev(i0), dev(i1)])
    out = torch.empty(shape, dtype=torch.bfloat16, device=DEV)
    ops.index(out, sv, views, isz, ist)
    exact(out, aten_cpu.index(a, [i0, i1]))


def test_out_of_range_index_sets_error_word(ops):
    a = torch.arange(12.0).reshape(4, 3)
    out = torch.empty(2, 3, device=DEV)
    ops.device_error_fetch()
    ops.index_select(out, dev(a), 0, dev(torch.tensor([1, 9])))
    assert ops.device_error_fetch() & 1
    assert ops.device_error_fetch() == 0
    exact(out[:1], a[1:2])
