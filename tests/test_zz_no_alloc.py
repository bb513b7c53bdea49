"""The allocation-free scatter_add entry point (b200_scatter_add_static), for
callers that cannot call cudaMalloc while they run -- a serving loop that must
not serialise the device, a plugin that is handed nothing but input and output
buffers. Called through the C ABI twice in a row and compared bit for bit with
the workspace-taking entry point and with the CPU oracle (torch.scatter_add on
the same values); it must also refuse a problem whose scratch
does not fit the built-in array. This file sorts last so that a run that stops
at the first failure has already run everything else."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _reference(ops, base, rows, src):
    idx = rows[:, None].expand(-1, src.shape[1])
    ws = torch.empty(max(1, ops.scatter_add_workspace_size(base, 0, idx, src)), dtype=torch.uint8, device=DEV)
    out = torch.empty_like(base)
    ops.scatter_add(out, base, 0, idx, src, ws)
    return out


def test_static_scratch_scatter_add_matches_twice(ops):
    g = torch.Generator().manual_seed(77)
    for call, (n_src, n_dst, inner) in enumerate([(50000, 3000, 64), (20000, 9000, 32)]):
        src = torch.randn(n_src, inner, generator=g).to(DEV)
        rows = torch.randint(0, n_dst, (n_src,), generator=g).to(DEV)
        base = torch.randn(n_dst, inner, generator=g).to(DEV)
        want = _reference(ops, base, rows, src)
        got = torch.empty_like(base)
        ops.scatter_add_static(got, base, 0, rows[:, None].expand(-1, inner), src)
        torch.cuda.synchronize()
        assert torch.equal(got, want), "call %d differs" % call  # integer-ordered fp32 adds: bit exact
        from oracle import aten_cpu
        cpu = aten_cpu.scatter_add(base.cpu(), 0, rows.cpu()[:, None].expand(-1, inner), src.cpu())
        assert torch.equal(got.cpu(), cpu), "call %d differs from the CPU oracle" % call
    assert ops.device_error_fetch() == 0


def test_static_scratch_refuses_oversized_problem(ops):
    n_src = 700000  # needs more than the 8 MiB the library carries
    src = torch.zeros(n_src, 4, device=DEV)
    rows = torch.zeros(n_src, dtype=torch.int64, device=DEV)
    base = torch.zeros(8, 4, device=DEV)
    with pytest.raises(ops.B200Error) as e:
        ops.scatter_add_static(torch.empty_like(base), base, 0, rows[:, None].expand(-1, 4), src)
    assert e.value.status == ops.NOT_SUPPORTED and "scratch" in str(e.value)
