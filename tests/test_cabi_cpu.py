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
