"""Parity of the CUDA kernels, called through the C ABI, against the CPU ATen
oracle on the same seeded inputs. Integer / index / move work must be
bit-exact; floating point within the tolerance written next to each check
(reference defaults: fp32 1e-6, bf16/fp16 1e-3, ints exact --
torch_gcu/csrc/aten/op_debug_config.h:144-149; 1e-5 for fp32 reductions whose
association order differs from the CPU's)."""
import pytest
import torch

from oracle import aten_cpu

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(t):
    return t.to(DEV)


def close(a, b, rtol, atol):
    ok = torch.isclose(a.cpu().float(), b.float(), rtol=rtol, atol=atol, equal_nan=True)
    assert ok.all(), "max abs err %g over %d mismatches" % (
        (a.cpu().float() - b.float()).abs().max().item(), (~ok).sum().item())


def exact(a, b):
    a = a.cpu()
    assert a.dtype == b.dtype and a.shape == b.shape
    if a.dtype in (torch.bfloat16, torch.float16):
        a, b = a.view(torch.int16), b.view(torch.int16)
    assert torch.equal(a, b), "%d elements differ" % (a != b).sum().item()


SHAPES = [(1,), (7,), (3, 8), (37, 130), (1024, 8, 12), (5, 4099), (0, 4), (256, 4096)]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_add_mul_silu(ops, shape, dtype):
    g = torch.Generator().manual_seed(1 << 11)
    a, b = torch.randn(shape, generator=g).to(dtype), torch.randn(shape, generator=g).to(dtype)
    da, db = dev(a), dev(b)
    out = torch.empty_like(da)
    ops.add(out, da, db, 1.0)
    exact(out, aten_cpu.add(a, b))
    ops.add(out, da, db, 0.8)
    ref = aten_cpu.add(a, b, alpha=0.8)
    if dtype == torch.float32:
        close(out, ref, 1e-6, 1e-6)
    else:
        # The kernel evaluates fma(alpha, b, a) in fp32 with alpha rounded to the
        # dtype and rounds once, like the CPU's vectorised loop. The CPU's scalar
        # tail (the last few elements of a flattened 16-bit tensor) instead rounds
        # alpha*b to 16 bits before the add, so CPU ATen disagrees with itself
        # there by up to half an ulp of the PRODUCT, whatever the size of the sum.
        # Bound the error by one ulp of the operands' magnitude.
        err = (out.cpu().float() - ref.float()).abs()
        bound = 2 ** -7 * (a.float().abs() + (0.8 * b.float()).abs()) + 1e-3
        assert (err <= bound).all(), "max excess %g" % (err - bound).max().item()
    ops.mul(out, da, db)
    exact(out, aten_cpu.mul(a, b))
    ops.silu(out, da)
    if dtype == torch.float32:
        close(out, aten_cpu.silu(a), 1e-6, 1e-6)
    else:
        close(out, aten_cpu.silu(a), 2 ** -7, 1e-3)


def test_reference_binary_cases(ops, golden):
    """The reference's own add/mul cases (test/op_test/test_binary_ops.py:21-57):
    scalar operands on either side, alpha, fp32 and fp16, its tolerances."""
    g = golden("ref_binary")
    for c in g["cases"]:
        lhs, rhs = c["lhs"], c["rhs"]
        ref = c["out"]
        if torch.is_tensor(lhs) and torch.is_tensor(rhs):
            shape = torch.broadcast_shapes(lhs.shape, rhs.shape)
            dl, dr = dev(lhs).expand(shape), dev(rhs).expand(shape)
            out = torch.empty(shape, dtype=ref.dtype, device=DEV)
            if c["op"] == "add":
                ops.add(out, dl, dr, c["alpha"])
            else:
                ops.mul(out, dl, dr)
        else:
            t, s = (lhs, rhs) if torch.is_tensor(lhs) else (rhs, lhs)
            out = torch.empty_like(dev(t))
            if c["op"] == "add":
                if torch.is_tensor(lhs):
                    ops.add_scalar(out, dev(t), s, c["alpha"])           # t + alpha*s
                else:                                                    # s + alpha*t
                    ops.mul_scalar(out, dev(t), c["alpha"])
                    ops.add_scalar(out, out, s, 1.0)
            elif c["op"] == "sub":
                ops.add_scalar(out, dev(t), s, -c["alpha"])
            else:
                ops.mul_scalar(out, dev(t), s)
        tol = dict(rtol=g["rtol"], atol=g["atol"]) if ref.dtype == torch.float32 else dict(rtol=1e-3, atol=1e-3)
        close(out, ref, **tol)


def test_broadcast_and_strided_operands(ops):
    g = torch.Generator().manual_seed(5)
    a, w = torch.randn(6, 33, 20, generator=g), torch.randn(20, generator=g)
    out = torch.empty(6, 33, 20, device=DEV)
    ops.mul(out, dev(a), dev(w).expand(6, 33, 20))
    exact(out, a * w)
    col = torch.randn(6, 33, 1, generator=g)
    ops.add(out, dev(a), dev(col).expand(6, 33, 20), 1.0)
    exact(out, a + col)
    at = dev(a).transpose(0, 2)
    out_t = torch.empty(20, 33, 6, device=DEV)
    ops.add(out_t, at, at, 1.0)
    exact(out_t, (a + a).transpose(0, 2).contiguous())
    i = torch.randint(-100, 100, (5, 7), generator=g)
    oi = torch.empty(5, 7, dtype=torch.int64, device=DEV)
    ops.add(oi, dev(i), dev(i), 3.0)
    exact(oi, i + 3 * i)


@pytest.mark.parametrize("op", ["neg", "rsqrt", "sqrt", "exp", "sigmoid", "tanh", "relu", "abs", "reciprocal",
                                "cos", "sin", "log", "gelu"])
def test_unary(ops, op):
    g = torch.Generator().manual_seed(9)
    a = torch.randn(41, 77, generator=g)
    if op in ("rsqrt", "sqrt", "log"):
        a = a.abs() + 0.1
    out = torch.empty_like(dev(a))
    ops.unary(out, dev(a), op)
    ref = getattr(torch, op)(a) if op != "gelu" else torch.nn.functional.gelu(a)
    close(out, ref, 2e-6, 1e-6)
    ops.pow_scalar(out, dev(a), 2.0)
    exact(out, a.pow(2))


@pytest.mark.parametrize("shape", [(4096,), (37, 130), (5, 4099), (3, 0), (1, 1), (64, 4096)])
def test_cast_bf16_bit_exact(ops, shape):
    g = torch.Generator().manual_seed(2)
    a = torch.randn(shape, generator=g)
    if a.numel() > 8:
        a.view(-1)[:6] = torch.tensor([float("inf"), -float("inf"), 0.0, -0.0, 1.0 + 2.0 ** -9, 1.0 + 3 * 2.0 ** -9])
    out = torch.empty(shape, dtype=torch.bfloat16, device=DEV)
    ops.copy(out, dev(a))
    exact(out, a.to(torch.bfloat16))
    back = torch.empty(shape, dtype=torch.float32, device=DEV)
    ops.copy(back, out)
    exact(back, a.to(torch.bfloat16).float())
    h = torch.empty(shape, dtype=torch.float16, device=DEV)
    ops.copy(h, dev(a))
    exact(h, a.half())


def test_cast_nan_stays_nan(ops):
    a = torch.tensor([float("nan"), 1.0, -float("nan")])
    out = torch.empty(3, dtype=torch.bfloat16, device=DEV)
    ops.copy(out, dev(a))
    assert torch.isnan(out.cpu().float()).tolist() == [True, False, True]


def test_copy_dtype_matrix_and_strides(ops):
    g = torch.Generator().manual_seed(4)
    # values in [-100, 100] with fractional parts: every conversion is defined
    base = (torch.rand(19, 23, generator=g) * 200 - 100)
    base.view(-1)[:3] = torch.tensor([0.0, -0.5, 99.5])
    dts = [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.int64, torch.int32, torch.int16,
           torch.int8, torch.uint8, torch.bool]
    for sd in dts:
        for dd in dts:
            vals = base.abs() if torch.uint8 in (sd, dd) else base
            src = (vals > 0) if sd == torch.bool else vals.to(sd)
            out = torch.empty(19, 23, dtype=dd, device=DEV)
            ops.copy(out, dev(src))
            exact(out, src.to(dd))
    # strided: transpose, slice into a larger buffer (KV-cache append shape)
    a = torch.randn(8, 16, 64, generator=g).to(torch.bfloat16)
    cache = torch.zeros(8, 40, 64, dtype=torch.bfloat16, device=DEV)
    ops.copy(cache[:, 5:21], dev(a))
    ref = torch.zeros(8, 40, 64, dtype=torch.bfloat16)
    ref[:, 5:21] = a
    exact(cache, ref)
    t = torch.empty(64, 16, 8, dtype=torch.float32, device=DEV)
    ops.copy(t, dev(a).permute(2, 1, 0))
    exact(t, a.permute(2, 1, 0).float().contiguous())


@pytest.mark.parametrize("shape", [(37, 130), (4, 4096), (3, 8192), (2, 40000), (5, 4099), (1, 1), (300, 64),
                                   (7, 24), (2, 16384)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_row_reductions(ops, shape, dtype):
    g = torch.Generator().manual_seed(11)
    a = torch.randn(shape, generator=g).to(dtype)
    rows, n = shape
    tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2 ** -7, atol=2e-2)
    out = torch.empty(rows, dtype=dtype, device=DEV)
    ops.sum(out, dev(a), [1])
    close(out, a.float().sum(-1), tol["rtol"], tol["atol"] * max(1.0, n ** 0.5 / 8))
    sm = torch.empty_like(dev(a))
    ops.softmax(sm, dev(a), 1)
    close(sm, aten_cpu.softmax(a, 1), 1e-5 if dtype == torch.float32 else 2 ** -7, 1e-6 if dtype == torch.float32 else 1e-3)
    w = (torch.randn(n, generator=g) * 0.02 + 1).to(dtype)
    b = (torch.randn(n, generator=g) * 0.02).to(dtype)
    y = torch.empty_like(dev(a))
    mean = torch.empty(rows, dtype=torch.float32, device=DEV)
    rstd = torch.empty(rows, dtype=torch.float32, device=DEV)
    ops.native_layer_norm(y, mean, rstd, dev(a), rows, n, dev(w), dev(b), 1e-5)
    ry, rm, rr = aten_cpu.native_layer_norm(a.float(), (n,), w.float(), b.float(), 1e-5)
    if dtype == torch.float32:
        close(y, ry, 1e-5, 1e-5)
    else:
        close(y, ry, 2 ** -7, 2e-2)
    close(mean, rm.view(-1), 1e-5, 1e-5)
    close(rstd, rr.view(-1), 1e-5, 1e-5)


def test_reductions_other_dims(ops):
    g = torch.Generator().manual_seed(12)
    a = torch.randn(6, 50, 33, generator=g)
    out = torch.empty(6, 33, device=DEV)
    ops.sum(out, dev(a), [1])
    close(out, a.sum(1), 1e-5, 1e-5)
    out = torch.empty(33, device=DEV)
    ops.sum(out, dev(a), [0, 1])
    close(out, a.sum((0, 1)), 1e-5, 1e-4)
    out = torch.empty(6, 50, device=DEV)
    ops.sum(out, dev(a), [2], mean=True)
    close(out, a.mean(2), 1e-5, 1e-5)
    big = torch.randn(300000, generator=g)
    ws = torch.empty(ops.sum_workspace_size(dev(big), [0]), dtype=torch.uint8, device=DEV)
    o = torch.empty((), device=DEV)
    ops.sum(o, dev(big), [0], workspace=ws)
    close(o, big.double().sum().float(), 1e-5, 1e-2)
    ints = torch.randint(-1000, 1000, (40, 70), generator=g)
    oi = torch.empty(40, dtype=torch.int64, device=DEV)
    ops.sum(oi, dev(ints), [1])
    exact(oi, ints.sum(1))
    sm = torch.empty_like(dev(a))
    ops.softmax(sm, dev(a), 1)
    close(sm, aten_cpu.softmax(a, 1), 1e-5, 1e-6)
    h = a.to(torch.bfloat16)
    smf = torch.empty(6, 50, 33, dtype=torch.float32, device=DEV)
    ops.softmax(smf, dev(h), 2)
    close(smf, aten_cpu.softmax(h, 2, True), 1e-5, 1e-6)


def test_golden_small_ops(ops, golden):
    """Against the committed CPU ATen vectors (machine independent)."""
    g = golden("op_small")
    a = g["silu"]["a"]
    out = torch.empty_like(dev(a))
    ops.silu(out, dev(a))
    close(out, g["silu"]["out"], 1e-6, 1e-6)
    o16 = torch.empty(a.shape, dtype=torch.bfloat16, device=DEV)
    ops.copy(o16, dev(a))
    exact(o16, g["cast"]["bf16"])
    s = torch.empty(37, device=DEV)
    ops.sum(s, dev(a), [1])
    close(s, g["sum"]["out"], 1e-5, 1e-5)
    s0 = torch.empty(130, device=DEV)
    ops.sum(s0, dev(a), [0])
    close(s0, g["sum"]["out0"], 1e-5, 1e-5)
    sm = torch.empty_like(dev(a))
    ops.softmax(sm, dev(a), 1)
    close(sm, g["softmax"]["out"], 1e-5, 1e-6)
    ops.softmax(sm, dev(a), 0)
    close(sm, g["softmax"]["out0"], 1e-5, 1e-6)
    ln = g["layer_norm"]
    y = torch.empty_like(dev(a)); m = torch.empty(37, device=DEV); r = torch.empty(37, device=DEV)
    ops.native_layer_norm(y, m, r, dev(ln["a"]), 37, 130, dev(ln["w"]), dev(ln["b"]), ln["eps"])
    close(y, ln["y"], 1e-5, 1e-5)
    close(m, ln["mean"].view(-1), 1e-5, 1e-5)
    close(r, ln["rstd"].view(-1), 1e-5, 1e-5)
