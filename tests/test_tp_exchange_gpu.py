"""The tensor-parallel exchange kernels through the C ABI on ONE GPU: the "ranks" are buffers of one
process, driven one after the other (a signal is always issued before the wait that needs it, so no
kernel ever waits for another launch). Checks the counting signal / wait, the bounded wait (a flag that
nothing sets: the TIMEOUT bit of the device error word, the context stays usable), and the fused
reduce-scatter + residual + RMSNorm + all-gather kernel against fp32 CPU arithmetic."""
import pytest
import torch

from test_ops_gpu import DEV, close, exact

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _controls(ops, world):
    n = ops.tp_control_bytes()
    return [torch.zeros(n, dtype=torch.uint8, device=DEV) for _ in range(world)]


def test_signal_then_wait_counts(ops):
    world = 4
    ctl = _controls(ops, world)
    tables = [ops.tp_peers(ctl, r) for r in range(world)]
    for rounds in range(3):      # counts keep running: the third round needs three signals from everyone
        for r in range(world):
            ops.tp_sync(tables[r], channel=2, signal=True, wait=False)
        for r in range(world):
            ops.tp_sync(tables[r], channel=2, signal=False, wait=True, timeout_s=0.05)
    torch.cuda.synchronize()
    assert ops.device_error_fetch() == 0
    flags = ctl[1].view(torch.int32)[2 * 8:2 * 8 + world].cpu()       # channel 2 of rank 1: one word per writer
    assert flags.tolist() == [3, 0, 3, 3]


def test_wait_is_bounded_and_reports_timeout(ops):
    ctl = _controls(ops, 2)
    table = ops.tp_peers(ctl, 0)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    ops.tp_sync(table, channel=0, signal=False, wait=True, timeout_s=0.05)   # nobody signals
    t1.record()
    torch.cuda.synchronize()
    assert 40 < t0.elapsed_time(t1) < 2000
    assert ops.device_error_fetch() & 2                                        # TIMEOUT bit, then cleared
    assert ops.device_error_fetch() == 0
    x = torch.ones(8, device=DEV)
    assert (x + x).sum().item() == 16                                          # the context is still usable
    with pytest.raises(ops.B200Error):
        ops.tp_sync(table, channel=0, signal=False, wait=True, timeout_s=0.0)  # unbounded waits are refused
    with pytest.raises(ops.B200Error):
        ops.tp_sync(table, channel=99)


@pytest.mark.parametrize("world,total_rows,N", [(2, 64, 512), (4, 256, 4096), (8, 512, 4096), (8, 64, 1024), (3, 96, 8192)])
def test_reduce_norm_scatter_mode(ops, world, total_rows, N):
    """Every rank owns total_rows / world rows: afterwards every rank's gathered buffer holds all rows,
    normalised, and each rank's residual rows are residual + the sum of all partials, rounded once."""
    g = torch.Generator().manual_seed(61)
    partial = [torch.randn(total_rows, N, generator=g).to(BF) for _ in range(world)]
    x = torch.randn(total_rows, N, generator=g).to(BF)
    w = (torch.randn(N, generator=g) * 0.02 + 1).to(BF)
    dp = [p.to(DEV) for p in partial]
    dg = [torch.zeros(total_rows, N, dtype=BF, device=DEV) for _ in range(world)]
    rows = total_rows // world
    res_out = []
    for r in range(world):
        xl = x[r * rows:(r + 1) * rows].to(DEV)
        ops.tp_reduce_norm(ops.tp_peers(dp, r), ops.tp_peers(dg, r), xl, xl, w.to(DEV), r * rows, total_rows, 1e-6)
        res_out.append(xl)
    torch.cuda.synchronize()
    acc = torch.zeros(total_rows, N)
    for p in partial:                     # rank order, fp32: the kernel's order
        acc = acc + p.float()
    h = (acc + x.float()).to(BF)
    exact(torch.cat(res_out, 0), h)
    hf = h.float()
    y = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).to(BF)
    for r in range(world):
        close(dg[r], y, 2 ** -7, 1e-3)     # one bf16 ulp: the rsqrt and the reduction order differ from the CPU's
    for r in range(1, world):
        exact(dg[r], dg[0].cpu())           # every rank received the same bits
    assert ops.device_error_fetch() == 0


def test_reduce_norm_replicated_mode_and_plain_gather(ops):
    """Decode form: every rank reduces all rows for itself (nothing gathered to the others); and the
    final form without normalisation gathers the residual rows themselves. f16 as well."""
    g = torch.Generator().manual_seed(62)
    world, B, N = 8, 64, 4096
    for dt in (BF, torch.float16):
        partial = [torch.randn(B, N, generator=g).to(dt).to(DEV) for _ in range(world)]
        x = torch.randn(B, N, generator=g).to(dt)
        w = (torch.randn(N, generator=g) * 0.02 + 1).to(dt)
        dg = [torch.zeros(B, N, dtype=dt, device=DEV) for _ in range(world)]
        out = torch.empty(B, N, dtype=dt, device=DEV)
        ops.tp_reduce_norm(ops.tp_peers(partial, 3), ops.tp_peers(dg, 3), x.to(DEV), out, w.to(DEV), 0, B, 1e-6,
                           gather_all=False)
        acc = torch.zeros(B, N)
        for p in partial:
            acc = acc + p.cpu().float()
        h = (acc + x.float()).to(dt)
        exact(out, h)
        hf = h.float()
        y = (hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).to(dt)
        close(dg[3], y, 2 ** -7 if dt == BF else 2 ** -10, 1e-3)
        assert dg[0].abs().sum().item() == 0                       # nothing was stored to the other ranks
        # no partials, no normalisation: a plain gather of the rows
        ops.tp_reduce_norm(None, ops.tp_peers(dg, 1), x.to(DEV), None, None, 0, B, normalise=False, gather_all=True)
        for r in range(world):
            exact(dg[r], x)
    with pytest.raises(ops.B200Error):
        ops.tp_reduce_norm(None, ops.tp_peers(dg, 1), None, None, None, 0, B)
