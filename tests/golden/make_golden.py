"""Generates tests/golden/*.pt from PyTorch CPU ATen (run in the build container:
`python tests/golden/make_golden.py`). The vectors are small on purpose.

Two groups:
  * `ref_*`: the reference's own unit-test cases for this path, restated from
    its test files as data (shapes, dtypes, seeds, scalar operands, tolerances):
    test/op_test/test_binary_ops.py:21-57,182-257 (add/mul with scalar operands,
    alpha, fp32 and fp16, seed 1<<11, rtol 1e-5 / atol 1e-8) and
    test/op_test/test_linear.py:19-147 (linear, addmm, mm, bmm, matmul, baddbmm
    on tiny fp32 shapes, seed 11, default allclose).
  * `op_*`: one small seeded case per remaining operator of the path, which
    the reference does not pin by any test.
Each file stores inputs and the CPU ATen outputs, so the oracle wrappers and
the CUDA path can both be checked against bits that do not depend on the
machine the tests later run on.
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import aten_cpu  # noqa: E402


def save(name, obj):
    torch.save(obj, os.path.join(HERE, name + ".pt"))


def ref_binary():
    torch.manual_seed(1 << 11)
    cases = []
    a = torch.randn(3, 8)
    cases.append(dict(op="add", lhs=a, rhs=20.0, alpha=0.8, out=torch.ops.aten.add(a, 20.0, alpha=0.8)))
    cases.append(dict(op="sub", lhs=a, rhs=20.0, alpha=0.8, out=torch.ops.aten.sub(a, 20.0, alpha=0.8)))
    h = torch.randn(3, 6).to(torch.float16)
    cases.append(dict(op="add", lhs=10, rhs=h, alpha=0.8, out=torch.ops.aten.add(10, h, alpha=0.8)))
    b = torch.randn(3, 8)
    cases.append(dict(op="mul", lhs=b, rhs=20.0, out=torch.ops.aten.mul(b, 20.0)))
    h2 = torch.randn(3, 6).to(torch.float16)
    cases.append(dict(op="mul", lhs=10, rhs=h2, out=torch.ops.aten.mul(10, h2)))
    # tensor-tensor forms with broadcasting (commented out upstream, same shapes)
    c, d = torch.randn(3, 8), torch.randn(3, 8)
    cases.append(dict(op="add", lhs=c, rhs=d, alpha=0.1, out=torch.ops.aten.add(c, d, alpha=0.1)))
    e, f = torch.randn(1, 8).half(), torch.randn(3, 1).half()
    cases.append(dict(op="add", lhs=e, rhs=f, alpha=0.6, out=torch.ops.aten.add(e, f, alpha=0.6)))
    cases.append(dict(op="mul", lhs=e, rhs=f, out=torch.ops.aten.mul(e, f)))
    save("ref_binary", dict(rtol=1e-5, atol=1e-8, cases=cases))


def ref_linear():
    torch.manual_seed(11)
    out = {}
    x, w, b = torch.randn(2, 5), torch.randn(3, 5), torch.randn(3)
    out["linear"] = dict(x=x, w=w, b=b, out=torch.ops.aten.linear(x, w, b), out_nobias=torch.ops.aten.linear(x, w))
    c, m1, m2 = torch.randn(3), torch.randn(2, 5), torch.randn(5, 3)
    out["addmm"] = dict(c=c, m1=m1, m2=m2, out=torch.ops.aten.addmm(c, m1, m2))
    out["mm"] = dict(m1=m1, m2=m2, out=torch.ops.aten.mm(m1, m2))
    b1, b2 = torch.randn(4, 2, 5), torch.randn(4, 5, 3)
    out["bmm"] = dict(b1=b1, b2=b2, out=torch.ops.aten.bmm(b1, b2), out_matmul=torch.ops.aten.matmul(b1, b2))
    i, p, q = torch.randn(4, 2, 5), torch.randn(4, 2, 6), torch.randn(4, 6, 5)
    out["baddbmm"] = dict(i=i, b1=p, b2=q, beta=-0.3, alpha=0.3,
                          out=torch.ops.aten.baddbmm(i, p, q, beta=-0.3, alpha=0.3))
    save("ref_linear", out)


def op_small():
    g = torch.Generator().manual_seed(1234)
    r = {}
    a, b = torch.randn(37, 130, generator=g), torch.randn(37, 130, generator=g)
    r["silu"] = dict(a=a, out=aten_cpu.silu(a))
    r["cast"] = dict(a=a, bf16=a.to(torch.bfloat16), back=a.to(torch.bfloat16).float(), f16=a.half())
    r["sum"] = dict(a=a, out=aten_cpu.sum_dim(a, [-1]), out0=aten_cpu.sum_dim(a, [0]))
    r["softmax"] = dict(a=a, out=aten_cpu.softmax(a, -1), out0=aten_cpu.softmax(a, 0))
    w, bias = torch.randn(130, generator=g) * 0.02 + 1, torch.randn(130, generator=g) * 0.02
    y, mean, rstd = aten_cpu.native_layer_norm(a, (130,), w, bias, 1e-5)
    r["layer_norm"] = dict(a=a, w=w, b=bias, eps=1e-5, y=y, mean=mean, rstd=rstd)
    table = (torch.randn(300, 24, generator=g) * 0.02).to(torch.bfloat16)
    ids = torch.randint(0, 300, (3, 17), generator=g)
    r["embedding"] = dict(table=table, ids=ids, out=aten_cpu.embedding(table, ids))
    sel = torch.randint(0, 300, (50,), generator=g)
    r["index_select"] = dict(table=table, idx=sel, out=aten_cpu.index_select(table, 0, sel),
                             out1=aten_cpu.index_select(table, 1, sel[:10] % 24))
    gs, gi = torch.randn(19, 40, generator=g), torch.randint(0, 40, (19, 40), generator=g)
    r["gather"] = dict(src=gs, idx=gi, out=aten_cpu.gather(gs, 1, gi))
    src, rows = torch.randn(500, 12, generator=g), torch.randint(0, 60, (500,), generator=g)
    base = torch.randn(60, 12, generator=g)
    r["scatter_add"] = dict(self=base, rows=rows, src=src,
                            out=aten_cpu.scatter_add(base, 0, rows[:, None].expand(-1, 12), src))
    full = torch.randint(0, 60, (500, 12), generator=g)
    r["scatter_add_full"] = dict(self=base, index=full, src=src, out=aten_cpu.scatter_add(base, 0, full, src))
    r["index_put"] = dict(self=base, rows=rows, src=src, out_acc=aten_cpu.index_put(base, [rows], src, True),
                          out_set=aten_cpu.index_put(base, [rows], src, False))
    i32 = torch.randint(-60, 60, (4, 5), generator=g).int()
    r["index_int32"] = dict(self=base, idx=i32, out=aten_cpu.index(base, [i32]))
    bf = torch.bfloat16
    x, res = torch.randn(9, 64, generator=g).to(bf), torch.randn(9, 64, generator=g).to(bf)
    wn = (torch.randn(64, generator=g) * 0.02 + 1).to(bf)
    yn, hn = aten_cpu.rms_norm_residual(x, res, wn, 1e-6)
    r["rms_norm_residual"] = dict(x=x, res=res, w=wn, eps=1e-6, y=yn, h=hn)
    q = torch.randn(2, 7, 3, 32, generator=g).to(bf)
    inv = 1.0 / (10000.0 ** (torch.arange(0, 32, 2, dtype=torch.float32) / 32))
    fr = torch.outer(torch.arange(7, dtype=torch.float32), inv)
    r["rope"] = dict(q=q, cos=fr.cos(), sin=fr.sin(), out=aten_cpu.rope(q, fr.cos(), fr.sin()))
    gt, up = torch.randn(5, 48, generator=g).to(bf), torch.randn(5, 48, generator=g).to(bf)
    r["swiglu"] = dict(gate=gt, up=up, out=aten_cpu.swiglu(gt, up))
    A, Bm = torch.randn(64, 96, generator=g).to(bf), torch.randn(96, 80, generator=g).to(bf)
    r["mm_bf16"] = dict(a=A, b=Bm, out=aten_cpu.mm_fp32_rounded(A, Bm))
    qq = torch.randn(1, 4, 16, 32, generator=g).to(bf)
    kk, vv = torch.randn(1, 2, 16, 32, generator=g).to(bf), torch.randn(1, 2, 16, 32, generator=g).to(bf)
    o, lse = aten_cpu.sdpa_causal(qq, kk, vv)
    r["sdpa"] = dict(q=qq, k=kk, v=vv, out=o, lse=lse)
    save("op_small", r)


if __name__ == "__main__":
    ref_binary()
    ref_linear()
    op_small()
    print("golden vectors written to", HERE)
