"""Full-size workload configurations 1-3 of the benchmark through the C ABI: direct comparison
with CPU ATen where the CPU finishes in seconds, plus size-independent
properties (linearity of scatter_add, gather/scatter round trip, idempotence)."""
import pytest
import torch

from oracle import aten_cpu
from test_ops_gpu import DEV, close, dev, exact
import workloads

pytestmark = pytest.mark.gpu


def _ws(n):
    return torch.empty(max(int(n), 1), dtype=torch.uint8, device=DEV)


def test_config1_op_sweep_full_size(ops):
    d = workloads.op_sweep()
    a, b = d["a"], d["b"]
    da, db = dev(a), dev(b)
    out = torch.empty_like(da)
    ops.add(out, da, db, 1.0)
    exact(out, aten_cpu.add(a, b))
    ops.mul(out, da, db)
    exact(out, aten_cpu.mul(a, b))
    ops.silu(out, da)
    close(out, aten_cpu.silu(a), 1e-6, 1e-6)
    h = torch.empty(a.shape, dtype=torch.bfloat16, device=DEV)
    ops.copy(h, da)
    exact(h, a.to(torch.bfloat16))
    ops.copy(out, h)
    exact(out, a.to(torch.bfloat16).float())
    s = torch.empty(4096, device=DEV)
    ops.sum(s, da, [1])
    close(s, aten_cpu.sum_dim(a, [-1]), 1e-5, 1e-4)  # |sum| ~ 64: atol scaled to the magnitude
    ops.softmax(out, da, 1)
    close(out, aten_cpu.softmax(a, -1), 1e-5, 1e-7)
    mean, rstd = torch.empty(4096, device=DEV), torch.empty(4096, device=DEV)
    ops.native_layer_norm(out, mean, rstd, da, 4096, 4096, dev(d["weight"]), dev(d["bias"]), 1e-5)
    y, m, r = aten_cpu.native_layer_norm(a, (4096,), d["weight"], d["bias"], 1e-5)
    close(out, y, 1e-5, 1e-5)
    close(mean, m.view(-1), 1e-5, 1e-6)
    close(rstd, r.view(-1), 1e-5, 1e-6)


def test_config2_index_ops_full_size(ops):
    d = workloads.index_ops()
    table = dev(d["table"])
    ids = d["ids"].reshape(-1)
    emb = torch.empty(ids.numel(), 4096, dtype=torch.bfloat16, device=DEV)
    ops.index_select(emb, table, 0, dev(ids))
    exact(emb, aten_cpu.embedding(d["table"], d["ids"]).reshape(-1, 4096))
    sel = torch.empty(65536, 4096, dtype=torch.bfloat16, device=DEV)
    ops.index_select(sel, table, 0, dev(d["select_idx"]))
    exact(sel, aten_cpu.index_select(d["table"], 0, d["select_idx"]))
    del table, emb, sel
    g = torch.empty(8192, 1024, device=DEV)
    ops.gather(g, dev(d["gather_src"]), 1, dev(d["gather_idx"]))
    exact(g, aten_cpu.gather(d["gather_src"], 1, d["gather_idx"]))

    vals, rows, n_dst = d["scatter_vals"], d["scatter_rows"], d["scatter_dst"]
    zeros = torch.zeros(n_dst, 256)
    dv, dr, dz = dev(vals), dev(rows), dev(zeros)
    idx = dr[:, None].expand(-1, 256)
    ws = _ws(ops.scatter_add_workspace_size(dz, 0, idx, dv))
    out = torch.empty_like(dz)
    ops.scatter_add(out, dz, 0, idx, dv, ws)
    ref = aten_cpu.scatter_add(zeros, 0, rows[:, None].expand(-1, 256), vals)
    exact(out, ref)
    tgt = dz.clone()
    ops.index_put(tgt, dr, dv, True, _ws(ops.index_put_workspace_size(tgt, dr, dv)))
    exact(tgt, aten_cpu.index_put(zeros, [rows], vals, True))
    # properties: run-to-run identical; scattering exactly-representable values
    # is order independent, so a permuted source order gives the same sums
    out2 = torch.empty_like(dz)
    ops.scatter_add(out2, dz, 0, idx, dv, ws)
    assert torch.equal(out, out2)
    ints = torch.randint(-8, 8, vals.shape, generator=torch.Generator().manual_seed(1)).float()
    perm = torch.randperm(vals.shape[0], generator=torch.Generator().manual_seed(2))
    a1, a2 = torch.empty_like(dz), torch.empty_like(dz)
    ops.scatter_add(a1, dz, 0, idx, dev(ints), ws)
    ops.scatter_add(a2, dz, 0, dev(rows[perm])[:, None].expand(-1, 256), dev(ints[perm]), ws)
    assert torch.equal(a1, a2)
    # checksum of checksums, summed in fp64: 67 M small integers add up past 2^24, where an fp32 sum depends on its order
    assert a1.double().sum().item() == ints.double().sum().item()


def test_config3_fused_full_size(ops):
    d = workloads.fused_ops()
    x, res, w = d["x"], d["res"], d["weight"]
    y, h = torch.empty_like(dev(x)), torch.empty_like(dev(x))
    ops.rms_norm_residual(y, h, dev(x), dev(res), dev(w), d["eps"])
    ry, rh = aten_cpu.rms_norm_residual(x, res, w, d["eps"])
    exact(h, rh)
    close(y, ry, 2 ** -7, 1e-3)  # bf16: one ulp
    q, k, cos, sin = d["q"], d["k"], d["cos"], d["sin"]
    qo, ko = torch.empty_like(dev(q)), torch.empty_like(dev(k))
    ops.rope(qo, dev(q), dev(cos), dev(sin))
    ops.rope(ko, dev(k), dev(cos), dev(sin))
    exact(qo, aten_cpu.rope(q, cos, sin))
    exact(ko, aten_cpu.rope(k, cos, sin))
    gate, up = d["gate"][:4096], d["up"][:4096]  # CPU checks a quarter; GPU runs the full size below
    so = torch.empty_like(dev(d["gate"]))
    ops.swiglu(so, dev(d["gate"]), dev(d["up"]))
    close(so[:4096], aten_cpu.swiglu(gate, up), 2 ** -7, 1e-3)
    close(so[-64:], aten_cpu.swiglu(d["gate"][-64:], d["up"][-64:]), 2 ** -7, 1e-3)
