"""The C-ABI library loads without a GPU, exports every declared symbol and
rejects malformed arguments before touching the device."""
import ctypes

import pytest


def test_library_exports_every_declared_symbol(ops):
    L = ops.lib()
    names = ops.declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(L, n), n


def test_version_and_dtype_sizes(ops):
    L = ops.lib()
    assert b"sm_100a" in L.b200_version()
    sizes = [L.b200_dtype_size(i) for i in range(10)]
    assert sizes == [4, 2, 2, 8, 8, 4, 2, 1, 1, 1]
    assert L.b200_dtype_size(99) == 0


def test_device_count_is_non_negative(ops):
    assert ops.lib().b200_device_count() >= 0


def _fake(ops, shape, dtype, ptr=0x1000, strides=None):
    t = ops.Tensor()
    t.data, t.dtype, t.ndim = ptr, dtype, len(shape)
    st = 1
    for i in reversed(range(len(shape))):
        t.sizes[i] = shape[i]
        t.strides[i] = st if strides is None else strides[i]
        st *= shape[i]
    return t


def test_bad_arguments_return_status_without_launching(ops):
    L = ops.lib()
    a = _fake(ops, (4, 4), ops.F32)
    b = _fake(ops, (4, 5), ops.F32)
    h = _fake(ops, (4, 4), ops.BF16)
    null = ctypes.c_void_p(0)
    # shape mismatch
    assert L.b200_add(ctypes.byref(a), ctypes.byref(a), ctypes.byref(b), ctypes.c_double(1), null) == ops.BAD_PARAM
    assert b"expanded" in L.b200_last_error()
    # dtype mismatch
    assert L.b200_mul(ctypes.byref(a), ctypes.byref(a), ctypes.byref(h), null) == ops.BAD_PARAM
    # null tensor
    assert L.b200_silu(None, ctypes.byref(a), null) == ops.BAD_PARAM
    # rank too large
    bad = _fake(ops, (2, 2), ops.F32)
    bad.ndim = 9
    assert L.b200_copy(ctypes.byref(bad), ctypes.byref(a), null) == ops.BAD_PARAM
    # index dtype
    assert L.b200_gather(ctypes.byref(a), ctypes.byref(a), ctypes.c_int64(1), ctypes.byref(a), null) == ops.BAD_PARAM
    # softmax dim out of range
    assert L.b200_softmax(ctypes.byref(a), ctypes.byref(a), ctypes.c_int64(5), null) == ops.BAD_PARAM
    # scatter workspace missing
    idx = _fake(ops, (8, 4), ops.I64, strides=(1, 0))
    src = _fake(ops, (8, 4), ops.F32)
    st = L.b200_scatter_add(ctypes.byref(a), ctypes.byref(a), ctypes.c_int64(0), ctypes.byref(idx),
                            ctypes.byref(src), None, ctypes.c_size_t(0), null)
    assert st == ops.WORKSPACE_TOO_SMALL
    assert ops.scatter_add_workspace_size.__call__ is not None
    assert L.b200_scatter_add_workspace_size(ctypes.byref(a), ctypes.c_int64(0), ctypes.byref(idx),
                                             ctypes.byref(src)) > 0


def test_wrapper_raises_on_error(ops):
    import torch
    a = torch.zeros(4, 4)
    b = torch.zeros(4, 5)
    with pytest.raises(ops.B200Error):
        ops.add(a, a, b, stream=0)


def test_newer_entry_points_reject_malformed_arguments(ops):
    """Argument checks of the fused GEMMs, the comparison / selection family, the attention backward and
    the loss entries run before any device call, so they can be exercised without a GPU."""
    L = ops.lib()
    null = ctypes.c_void_p(0)
    ref = ctypes.byref
    f32 = _fake(ops, (4, 8), ops.F32)
    b16 = _fake(ops, (256, 64), ops.BF16)
    w16 = _fake(ops, (512, 64), ops.BF16)
    o16 = _fake(ops, (256, 256), ops.BF16)
    # fused gate/up GEMM: fp32 operands, then a weight whose row count is not 2F
    assert L.b200_mm_swiglu(ref(f32), ref(f32), ref(f32), null) == ops.NOT_SUPPORTED
    bad_w = _fake(ops, (500, 64), ops.BF16)
    assert L.b200_mm_swiglu(ref(o16), ref(b16), ref(bad_w), null) == ops.BAD_PARAM
    # fused qkv GEMM: rope_cols not a multiple of the head size; tables of the wrong dtype
    cos = _fake(ops, (300, 64), ops.F32)
    out_qkv = _fake(ops, (256, 512), ops.BF16)
    st = L.b200_mm_rope(ref(out_qkv), ref(b16), ref(w16), ref(cos), ref(cos), ctypes.c_int64(256), ctypes.c_int64(100), null)
    assert st == ops.BAD_PARAM and b"128" in L.b200_last_error()
    cos16 = _fake(ops, (300, 64), ops.BF16)
    st = L.b200_mm_rope(ref(out_qkv), ref(b16), ref(w16), ref(cos16), ref(cos16), ctypes.c_int64(256), ctypes.c_int64(256), null)
    assert st == ops.BAD_PARAM
    # rotary embedding + cache write: head counts that do not add up; caches of another dtype; positions not int64
    qkv = _fake(ops, (4, 1, 12, 128), ops.BF16)
    kc = _fake(ops, (4, 2, 16, 128), ops.BF16)
    kc32 = _fake(ops, (4, 2, 16, 128), ops.F32)
    pos = _fake(ops, (4, 1), ops.I64)
    posf = _fake(ops, (4, 1), ops.F32)
    tab = _fake(ops, (16, 64), ops.F32)
    call = lambda q, p_, hq, hk, k, v: L.b200_rope_kv_append(ref(q), ref(tab), ref(tab), ref(p_), ctypes.c_int64(hq),
                                                            ctypes.c_int64(hk), ref(k), ref(v), null)
    assert call(qkv, pos, 9, 2, kc, kc) == ops.BAD_PARAM          # 9 + 2 * 2 != 12
    assert call(qkv, pos, 8, 2, kc32, kc32) == ops.BAD_PARAM
    assert call(qkv, posf, 8, 2, kc, kc) == ops.BAD_PARAM
    # the rule for the few-row SwiGLU product needs no device (148 SMs assumed without one)
    L.b200_mm_swiglu_few_rows.restype = ctypes.c_int
    few = lambda m, f, k: L.b200_mm_swiglu_few_rows(ctypes.c_int64(m), ctypes.c_int64(f), ctypes.c_int64(k))
    assert few(64, 14336, 4096) == 1 and few(64, 3584, 4096) == 1 and few(64, 1792, 4096) == 1
    assert few(4096, 14336, 4096) == 0 and few(64, 3584, 64) == 0 and few(0, 3584, 4096) == 0
    # comparison: the output must be bool; unknown operator
    bool_out = _fake(ops, (4, 8), ops.BOOL)
    assert L.b200_compare(ref(f32), ref(f32), ref(f32), ctypes.c_int32(0), null) == ops.BAD_PARAM
    assert L.b200_compare(ref(bool_out), ref(f32), ref(f32), ctypes.c_int32(42), null) == ops.BAD_PARAM
    # where: the condition must be bool
    assert L.b200_where(ref(f32), ref(f32), ref(f32), ref(f32), null) == ops.BAD_PARAM
    # clamp without a bound; extreme over a dimension that does not exist
    assert L.b200_clamp(ref(f32), ref(f32), ctypes.c_int32(0), ctypes.c_double(0), ctypes.c_int32(0), ctypes.c_double(0), null) == ops.BAD_PARAM
    idx = _fake(ops, (4,), ops.I64)
    assert L.b200_extreme_dim(None, ref(idx), ref(f32), ctypes.c_int64(3), ctypes.c_int32(1), null) == ops.BAD_PARAM
    # attention backward: head dim other than 128; missing workspace
    q64 = _fake(ops, (1, 2, 128, 64), ops.BF16)
    lse = _fake(ops, (1, 2, 128), ops.F32)
    args64 = [ref(q64)] * 8
    st = L.b200_sdpa_flash_bwd(*args64, ref(lse), ctypes.c_int32(1), ctypes.c_double(0.125), None, ctypes.c_size_t(0), null)
    assert st == ops.NOT_SUPPORTED
    q128 = _fake(ops, (1, 2, 128, 128), ops.BF16)
    args128 = [ref(q128)] * 8
    st = L.b200_sdpa_flash_bwd(*args128, ref(lse), ctypes.c_int32(1), ctypes.c_double(0.09), None, ctypes.c_size_t(0), null)
    assert st == ops.WORKSPACE_TOO_SMALL
    # NLL loss: targets must be int64 of N elements
    logp = _fake(ops, (6, 10), ops.F32)
    one = _fake(ops, (1,), ops.F32)
    tgt32 = _fake(ops, (6,), ops.I32)
    st = L.b200_nll_loss(ref(one), ref(one), ref(logp), ref(tgt32), None, ctypes.c_int32(1), ctypes.c_int64(-100), null)
    assert st == ops.BAD_PARAM
    # layer-norm backward: the column sums need a workspace
    g = _fake(ops, (6, 10), ops.F32)
    stat = _fake(ops, (6,), ops.F32)
    dw = _fake(ops, (10,), ops.F32)
    L.b200_layer_norm_backward_workspace_size.restype = ctypes.c_size_t
    assert L.b200_layer_norm_backward_workspace_size(ctypes.c_int64(6), ctypes.c_int64(10)) > 0
