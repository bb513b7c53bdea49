"""The PrivateUse1 device end to end: tensors on "gcu", operators dispatched
through the generated registrations into the kernel library, compared with the
CPU result of the same torch call -- the reference's own test method
(test/op_test/gcu_op_test.py:49-135: run on CPU, copy args to the device, run the
same op, compare)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import torch_gcu  # noqa: F401
    assert torch.gcu.is_available()
    return torch.device("gcu", 0)


def run_op_test(op, dev, *args, rtol=1e-5, atol=1e-5, exact=False, **kwargs):
    cpu_out = op(*copy.deepcopy(args), **copy.deepcopy(kwargs))
    def to_dev(x):
        if isinstance(x, torch.Tensor):
            return x.to(dev)
        if isinstance(x, (list, tuple)) and x and isinstance(x[0], torch.Tensor):
            return [t.to(dev) for t in x]
        return x
    dev_out = op(*[to_dev(a) for a in args], **{k: to_dev(v) for k, v in kwargs.items()})
    cpu_outs = cpu_out if isinstance(cpu_out, tuple) else (cpu_out,)
    dev_outs = dev_out if isinstance(dev_out, tuple) else (dev_out,)
    assert len(cpu_outs) == len(dev_outs)
    for c, d in zip(cpu_outs, dev_outs):
        assert d.device.type == "gcu"
        assert c.shape == d.shape and c.dtype == d.dtype, (c.shape, d.shape, c.dtype, d.dtype)
        d = d.cpu()
        if exact:
            assert torch.equal(c, d)
        else:
            assert torch.allclose(c.float(), d.float(), rtol=rtol, atol=atol, equal_nan=True), (c - d).abs().max()
    return dev_out


def test_roundtrip_and_metadata(dev):
    a = torch.randn(37, 19)
    d = a.to(dev)
    assert d.is_gcu and d.device == dev and d.shape == a.shape
    assert torch.equal(d.cpu(), a)
    assert torch.equal(d.t().contiguous().cpu(), a.t().contiguous())
    assert torch.equal(d[3:20, ::2].cpu(), a[3:20, ::2])
    assert torch.equal(d.view(19, 37).cpu(), a.view(19, 37))
    assert torch.equal(d.to(torch.bfloat16).cpu(), a.to(torch.bfloat16))
    assert torch.equal(a.gcu().cpu(), a)
    z = torch.zeros(5, 3, device=dev)
    assert z.cpu().abs().sum() == 0
    e = torch.empty(0, 4, device=dev)
    assert e.cpu().shape == (0, 4)
    assert abs(d.sum().item() - a.sum().item()) < 1e-3
    f = torch.full((4, 4), 2.5, device=dev)
    assert f.cpu().eq(2.5).all()
    g = torch.empty(3, device=dev)
    g.resize_(10)
    assert g.shape == (10,)


def test_reference_binary_cases(dev):
    """test/op_test/test_binary_ops.py:21-57: scalar operands on either side, alpha."""
    torch.manual_seed(1 << 11)
    a = torch.randn(3, 8)
    run_op_test(torch.ops.aten.add, dev, a, 20.0, alpha=0.8, rtol=1e-5, atol=1e-8)
    run_op_test(torch.ops.aten.sub, dev, a, 20.0, alpha=0.8, rtol=1e-5, atol=1e-8)
    h = torch.randn(3, 6).half()
    run_op_test(torch.ops.aten.add, dev, 10, h, alpha=0.8, rtol=1e-3, atol=1e-3)
    run_op_test(torch.ops.aten.mul, dev, a, 20.0, rtol=1e-5, atol=1e-8)
    run_op_test(torch.ops.aten.mul, dev, 10, h, rtol=1e-3, atol=1e-3)
    b = torch.randn(3, 8)
    run_op_test(torch.ops.aten.add, dev, a, b, alpha=0.1, rtol=1e-5, atol=1e-7)
    run_op_test(torch.ops.aten.add, dev, torch.randn(1, 8).half(), torch.randn(3, 1).half(), alpha=0.6, rtol=1e-3, atol=1e-3)
    run_op_test(torch.ops.aten.div, dev, a, b, rtol=1e-6, atol=1e-6)
    out = torch.empty(0)
    torch.add(a.to(dev), b.to(dev), out=(o := torch.empty(0, device=dev)))  # out= of size 0 is resized
    assert torch.equal(o.cpu(), a + b) and out.numel() == 0
    x = a.to(dev)
    x += b.to(dev)
    assert torch.equal(x.cpu(), a + b)
    # int + float promotes like the CPU
    i = torch.randint(-5, 5, (3, 8))
    run_op_test(torch.add, dev, i, a, exact=True)


def test_reference_linear_cases(dev):
    """test/op_test/test_linear.py:19-147 on the device."""
    torch.manual_seed(11)
    x, w, b = torch.randn(2, 5), torch.randn(3, 5), torch.randn(3)
    run_op_test(torch.ops.aten.linear, dev, x, w, b)
    run_op_test(torch.ops.aten.linear, dev, x, w)
    run_op_test(torch.ops.aten.addmm, dev, torch.randn(3), torch.randn(2, 5), torch.randn(5, 3))
    run_op_test(torch.ops.aten.mm, dev, torch.randn(2, 5), torch.randn(5, 3))
    run_op_test(torch.ops.aten.bmm, dev, torch.randn(4, 2, 5), torch.randn(4, 5, 3))
    run_op_test(torch.ops.aten.matmul, dev, torch.randn(4, 2, 5), torch.randn(4, 5, 3))
    run_op_test(torch.ops.aten.baddbmm, dev, torch.randn(4, 2, 5), torch.randn(4, 2, 6), torch.randn(4, 6, 5), beta=-0.3, alpha=0.3)


def test_config_ops_through_dispatcher(dev):
    g = torch.Generator().manual_seed(0)
    a = torch.randn(64, 4096, generator=g)
    run_op_test(torch.nn.functional.silu, dev, a, rtol=1e-6, atol=1e-6)
    run_op_test(lambda t: t.sum(-1), dev, a, rtol=1e-5, atol=1e-4)
    run_op_test(lambda t: t.sum(), dev, a, rtol=1e-5, atol=1e-2)
    run_op_test(lambda t: t.mean((0,)), dev, a, rtol=1e-5, atol=1e-5)
    run_op_test(lambda t: t.softmax(-1), dev, a, rtol=1e-5, atol=1e-7)
    w, b = torch.randn(4096, generator=g) * 0.02 + 1, torch.randn(4096, generator=g) * 0.02
    run_op_test(torch.nn.functional.layer_norm, dev, a, (4096,), w, b, 1e-5)
    y, mean, rstd = torch.ops.aten.native_layer_norm(a.to(dev), [4096], w.to(dev), b.to(dev), 1e-5)
    assert mean.shape == (64, 1) and rstd.dtype == torch.float32
    table = (torch.randn(1000, 64, generator=g) * 0.02).bfloat16()
    ids = torch.randint(0, 1000, (4, 33), generator=g)
    run_op_test(torch.nn.functional.embedding, dev, ids, table, exact=True)
    run_op_test(torch.index_select, dev, table, 0, ids[0], exact=True)
    src = torch.randn(50, 40, generator=g)
    idx = torch.randint(0, 40, (50, 40), generator=g)
    run_op_test(torch.gather, dev, src, 1, idx, exact=True)
    vals, rows = torch.randn(3000, 32, generator=g), torch.randint(0, 100, (3000,), generator=g)
    base = torch.zeros(100, 32)
    run_op_test(torch.scatter_add, dev, base, 0, rows[:, None].expand(-1, 32), vals, exact=True)
    torch.use_deterministic_algorithms(True)
    try:
        ref = base.clone().index_put_((rows,), vals, accumulate=True)
    finally:
        torch.use_deterministic_algorithms(False)
    got = base.to(dev).index_put_((rows.to(dev),), vals.to(dev), accumulate=True)
    assert torch.equal(got.cpu(), ref)
    # two index tensors: linearised on the host, every dimension range-checked as ATen does
    base2 = torch.zeros(6, 5, 4)
    i0, i1 = torch.tensor([0, 5, -1, 2, 5]), torch.tensor([4, 0, -5, 3, 0])
    v2 = torch.randn(5, 4, generator=g)
    torch.use_deterministic_algorithms(True)
    try:
        ref2 = base2.clone().index_put_((i0, i1), v2, accumulate=True)
    finally:
        torch.use_deterministic_algorithms(False)
    got2 = base2.to(dev).index_put_((i0.to(dev), i1.to(dev)), v2.to(dev), accumulate=True)
    assert torch.equal(got2.cpu(), ref2)
    for bad0, bad1 in ((torch.tensor([0]), torch.tensor([5])), (torch.tensor([0]), torch.tensor([-6])),
                       (torch.tensor([6]), torch.tensor([0]))):
        with pytest.raises(IndexError):   # not folded into a neighbouring row
            base2.to(dev).index_put_((bad0.to(dev), bad1.to(dev)), v2[:1].to(dev), accumulate=True)
        with pytest.raises(IndexError):
            base2.clone().index_put_((bad0, bad1), v2[:1], accumulate=True)
    run_op_test(lambda t, i: t[i], dev, src, rows[:7] % 50, exact=True)
    run_op_test(lambda t: torch.cat([t, t * 2], dim=-1), dev, src, exact=True)
    run_op_test(lambda t: t.pow(2).mean(-1, keepdim=True).add(1e-6).rsqrt(), dev, src, rtol=1e-5, atol=1e-6)
    run_op_test(torch.neg, dev, src, exact=True)


def test_int64_scalars_beyond_2_53_stay_exact(dev):
    """Integer scalar operands that a double cannot carry: fill, full, add, sub and mul keep them exact, as ATen does."""
    big = 2 ** 60 + 1
    assert torch.full((3,), big, dtype=torch.int64, device=dev).cpu().tolist() == [big] * 3
    x = torch.arange(5, dtype=torch.int64)
    assert torch.equal((x.to(dev) + big).cpu(), x + big)
    assert torch.equal((x.to(dev) - big).cpu(), x - big)
    assert torch.equal((big + x.to(dev)).cpu(), big + x)
    assert torch.equal((x.to(dev) * (2 ** 55 + 3)).cpu(), x * (2 ** 55 + 3))
    t = torch.zeros(4, dtype=torch.int64, device=dev)
    t.fill_(-big)
    assert t.cpu().tolist() == [-big] * 4


def test_int32_index_efficient_op(dev):
    import torch_gcu
    from torch_gcu.gcu.efficient.op import gcu_index
    base = torch.randn(60, 12)
    idx = torch.randint(-60, 60, (4, 5)).int()
    out = gcu_index(base.to(dev), [idx.to(dev)])
    assert torch.equal(out.cpu(), base[idx.long()])
    with pytest.raises(IndexError):  # int64 indices are rejected, as in the reference
        gcu_index(base.to(dev), [idx.long().to(dev)])
    with pytest.raises(IndexError):  # indices must live on self's device
        gcu_index(base.to(dev), [idx])


def test_fused_efficient_ops(dev):
    from torch_gcu.gcu import efficient
    from oracle import aten_cpu
    g = torch.Generator().manual_seed(3)
    bf = torch.bfloat16
    x, r = torch.randn(33, 4096, generator=g).to(bf), torch.randn(33, 4096, generator=g).to(bf)
    w = (torch.randn(4096, generator=g) * 0.02 + 1).to(bf)
    y, h = efficient.rms_norm_residual(x.to(dev), r.to(dev), w.to(dev), 1e-6)
    ry, rh = aten_cpu.rms_norm_residual(x, r, w, 1e-6)
    assert torch.equal(h.cpu(), rh)
    assert torch.allclose(y.cpu().float(), ry.float(), rtol=2 ** -7, atol=1e-3)
    q = torch.randn(2, 40, 8, 128, generator=g).to(bf)
    cos, sin = efficient.rope_tables(40, 128, device="cpu")
    out = efficient.rope(q.to(dev), cos.to(dev), sin.to(dev))
    assert torch.equal(out.cpu(), aten_cpu.rope(q, cos, sin))
    gate, up = torch.randn(17, 512, generator=g).to(bf), torch.randn(17, 512, generator=g).to(bf)
    s = efficient.swiglu(gate.to(dev), up.to(dev))
    assert torch.allclose(s.cpu().float(), aten_cpu.swiglu(gate, up).float(), rtol=2 ** -7, atol=1e-3)
    xs = torch.randn(2, 300, 256, generator=g).to(torch.bfloat16)
    wgu = (torch.randn(2 * 384, 256, generator=g) * 0.1).to(torch.bfloat16)
    for xin in (xs, xs[:, :4]):   # the fused-epilogue GEMM (>= 512 rows) and the few-row path
        ls = efficient.linear_swiglu(xin.to(dev), wgu.to(dev))
        gu = xin.float() @ wgu.float().t()
        ref = torch.nn.functional.silu(gu[..., :384]) * gu[..., 384:]
        assert ls.shape == ref.shape and torch.allclose(ls.cpu().float(), ref, rtol=3e-2, atol=3e-2)
    xr = torch.randn(2, 300, 256, generator=g).to(torch.bfloat16)
    wr = (torch.randn(5 * 128, 256, generator=g) * 0.06).to(torch.bfloat16)
    cr, sr = efficient.rope_tables(300, 128, device="cpu")
    for xin in (xr, xr[:, :7]):   # GEMM with the rotation in its epilogue (>= 512 rows), and mm followed by the rope kernel
        lr = efficient.linear_rope(xin.to(dev), wr.to(dev), cr.to(dev), sr.to(dev), 4)
        y = (xin.float() @ wr.float().t()).view(2, -1, 5, 128)
        ref = y.clone()
        ref[:, :, :4] = aten_cpu.rope(y[:, :, :4].contiguous(), cr, sr).float()
        assert lr.shape == ref.shape and torch.allclose(lr.cpu().float(), ref, rtol=3e-2, atol=3e-2)
    s2 = efficient.swiglu_packed(torch.cat([gate, up], -1).to(dev))
    assert torch.equal(s2.cpu(), s.cpu())


def test_sdpa_dispatch_and_autocast(dev):
    from oracle import aten_cpu
    g = torch.Generator().manual_seed(4)
    bf = torch.bfloat16
    q = torch.randn(2, 8, 256, 128, generator=g).to(bf)
    k, v = torch.randn(2, 2, 256, 128, generator=g).to(bf), torch.randn(2, 2, 256, 128, generator=g).to(bf)
    out = torch.nn.functional.scaled_dot_product_attention(q.to(dev), k.to(dev), v.to(dev), is_causal=True, enable_gqa=True)
    ref, _ = aten_cpu.sdpa_causal(q, k, v)
    assert torch.allclose(out.cpu().float(), ref.float(), rtol=1.6e-2, atol=1e-2)
    # autocast: fp32 linear runs its matmul in bf16, softmax stays fp32
    lin = torch.nn.Linear(256, 128, bias=True)
    x = torch.randn(64, 256, generator=g)
    lin_d = copy.deepcopy(lin).to(dev)
    with torch.autocast("gcu", dtype=bf):
        y = lin_d(x.to(dev))
        sm = torch.softmax(y, -1)
    assert y.dtype == bf and sm.dtype == torch.float32
    ref = lin(x)
    assert torch.allclose(y.cpu().float(), ref, rtol=1.6e-2, atol=3e-2)


def test_streams_events_and_allocator(dev):
    s = torch.gcu.Stream()
    assert s.gcu_stream != 0 and s.device == dev
    e0, e1 = torch.gcu.Event(enable_timing=True), torch.gcu.Event(enable_timing=True)
    a = torch.randn(1 << 20).to(dev)
    with torch.gcu.stream(s):
        assert torch.gcu.current_stream() == s
        e0.record()
        b = a * 2
        e1.record()
    assert torch.gcu.current_stream() == torch.gcu.default_stream()
    e1.synchronize()
    assert e0.elapsed_time(e1) >= 0
    assert e1.query()
    torch.gcu.current_stream().wait_stream(s)
    assert torch.equal(b.cpu(), (a * 2).cpu())
    torch.gcu.synchronize()
    before = torch.gcu.memory_stats()
    t = torch.empty(1 << 20, device=dev)
    p = t.data_ptr()
    del t
    t2 = torch.empty(1 << 20, device=dev)
    assert t2.data_ptr() == p  # same-stream reuse without a driver call
    after = torch.gcu.memory_stats()
    assert after["num_cache_hits"] > before["num_cache_hits"]
    assert torch.gcu.memory_allocated() > 0 and torch.gcu.max_memory_allocated() >= torch.gcu.memory_allocated()
    del t2, a, b
    torch.gcu.empty_cache()
    pin = torch.randn(1000).pin_memory()
    assert pin.is_pinned()
    d = pin.to(dev, non_blocking=True)
    torch.gcu.synchronize()
    assert torch.equal(d.cpu(), pin)


def test_unsupported_operator_raises(dev):
    a = torch.randn(4, 4).to(dev)
    with pytest.raises(NotImplementedError, match="no CPU fallback"):
        torch.linalg.inv(a)


def test_graph_capture_and_replay(dev):
    """A sequence of operators recorded once and replayed: results follow the static input,
    memory created during the capture stays private to the graph."""
    g = torch.Generator().manual_seed(7)
    bf = torch.bfloat16
    w = (torch.randn(256, 128, generator=g) * 0.1).to(bf)
    x1, x2 = torch.randn(64, 128, generator=g).to(bf), torch.randn(64, 128, generator=g).to(bf)
    wd, static_in = w.to(dev), x1.to(dev)

    def step(x):
        h = torch.mm(x, wd.t())
        h = torch.nn.functional.silu(h) + 1.0
        return torch.softmax(h.float(), -1)

    eager1 = step(static_in).cpu()          # also warms up every kernel once
    graph = torch.gcu.GCUGraph()
    with torch.gcu.graph(graph):
        static_out = step(static_in)
    assert graph.captured and graph.num_nodes >= 4
    graph.replay()
    torch.gcu.synchronize()
    assert torch.equal(static_out.cpu(), eager1)
    static_in.copy_(x2.to(dev))
    graph.replay()
    torch.gcu.synchronize()
    assert torch.equal(static_out.cpu(), step(x2.to(dev)).cpu())
    # eager allocations made after the capture never alias the graph's buffers
    junk = [torch.full((64, 256), 7.0, device=dev) for _ in range(8)]
    graph.replay()
    torch.gcu.synchronize()
    assert torch.equal(static_out.cpu(), step(x2.to(dev)).cpu())
    assert all(j.cpu().eq(7.0).all() for j in junk)
    graph.reset()
    assert not graph.captured


def test_graph_decode_step_matches_eager(dev):
    """One decode step of the decoder harness, captured and replayed."""
    import workloads
    from tp_decoder import DecoderStack
    cfg = dict(hidden=512, heads=8, kv_heads=2, head_dim=128, ffn=1024)
    stack = DecoderStack(2, 1, 0, "gcu", dev, torch.bfloat16, cfg)
    g = torch.Generator().manual_seed(8)
    B, T = 4, 300
    caches = [(torch.randn(B, 2, T, 128, generator=g).bfloat16().to(dev), torch.randn(B, 2, T, 128, generator=g).bfloat16().to(dev))
              for _ in range(2)]
    x = torch.randn(B, 1, 512, generator=g).bfloat16().to(dev)
    ref = stack.decode(x, caches, T - 1).cpu()
    graph = torch.gcu.GCUGraph()
    with torch.gcu.graph(graph):
        out = stack.decode(x, caches, T - 1)
    for _ in range(3):
        graph.replay()
    torch.gcu.synchronize()
    assert torch.equal(out.cpu(), ref)
