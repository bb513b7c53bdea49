"""Worker of test_env_paths_gpu: the library's alternative code paths, selected by
environment variables that are read once per process (B200_PDL=0: every launch fully
serialised; B200_WALK_RING=0: the register-resident segment walk; B200_GRID_WAVES=1:
one persistent wave per streaming kernel), checked against the CPU oracle."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "torch-gcu_b200"))
import b200ops as ops  # noqa: E402
from oracle import aten_cpu  # noqa: E402

DEV = "cuda:0"
ops.lib()
g = torch.Generator().manual_seed(91)


def exact(a, b):
    a = a.cpu()
    assert a.dtype == b.dtype and a.shape == b.shape
    if a.dtype in (torch.bfloat16, torch.float16):
        a, b = a.view(torch.int16), b.view(torch.int16)
    assert torch.equal(a, b), "%d elements differ" % (a != b).sum().item()


def ws(n):
    return torch.empty(max(int(n), 1), dtype=torch.uint8, device=DEV)


# ordered accumulation: aligned rows (the ring walk's shapes), fp32 and bf16, with an empty and a crowded destination
for dtype, inner in ((torch.float32, 256), (torch.bfloat16, 64), (torch.float32, 520)):
    src = torch.randn(5000, inner, generator=g).to(dtype)
    rows = torch.randint(0, 700, (5000,), generator=g)
    rows[rows == 5] = 6
    rows[:300] = 9
    base = torch.randn(700, inner, generator=g).to(dtype)
    idx = rows.to(DEV)[:, None].expand(-1, inner)
    out = torch.empty_like(base.to(DEV))
    ops.scatter_add(out, base.to(DEV), 0, idx, src.to(DEV), ws(ops.scatter_add_workspace_size(base.to(DEV), 0, idx, src.to(DEV))))
    exact(out, aten_cpu.scatter_add(base, 0, rows[:, None].expand(-1, inner), src))
    tgt = base.to(DEV).clone()
    ops.index_put(tgt, rows.to(DEV), src.to(DEV), True, ws(ops.index_put_workspace_size(tgt, rows.to(DEV), src.to(DEV))))
    exact(tgt, aten_cpu.index_put(base, [rows], src, True))

# streaming kernels: a ragged size exercises the predicated last batch and the scalar tail
for n in (5, 4099, 1 << 20, (1 << 20) + 13):
    a, b = torch.randn(n, generator=g), torch.randn(n, generator=g)
    out = torch.empty(n, device=DEV)
    ops.add(out, a.to(DEV), b.to(DEV))
    exact(out, a + b)
    h = torch.empty(n, dtype=torch.bfloat16, device=DEV)
    ops.copy(h, a.to(DEV))
    exact(h, a.to(torch.bfloat16))

# a chain of dependent launches on one stream: each kernel reads what its predecessor wrote
x = torch.randn(2048, 1024, generator=g)
y = x.to(DEV)
t1, t2 = torch.empty_like(y), torch.empty_like(y)
ops.add(t1, y, y)
ops.softmax(t2, t1, 1)
ops.add(t1, t2, y)
sel = torch.randint(0, 2048, (4096,), generator=g)
o = torch.empty(4096, 1024, device=DEV)
ops.index_select(o, t1, 0, sel.to(DEV))
ref = (torch.softmax(x + x, 1) + x)[sel]
assert torch.allclose(o.cpu(), ref, rtol=1e-5, atol=1e-6)
torch.cuda.synchronize()
print("ENV_PATHS_OK")
