"""Builds and binds oracle/seq_ref.c (plain C, gcc) -- test infrastructure only."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "seq_ref.c")
_OUT_DIR = os.path.join(_HERE, "_build")
_SO = os.path.join(_OUT_DIR, "libseqref.so")
_lib = None


def build(force=False):
    os.makedirs(_OUT_DIR, exist_ok=True)
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        # -ffp-contract=off / no fast-math: every add is a separately rounded fp32 add
        subprocess.check_call(["gcc", "-O2", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
                               _SRC, "-o", _SO])
    return _SO


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def scatter_add_rows(self_, rows, src):
    self_ = np.ascontiguousarray(self_, dtype=np.float32)
    src = np.ascontiguousarray(src, dtype=np.float32)
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    out = np.empty_like(self_)
    n_dst, inner = self_.shape[0], int(np.prod(self_.shape[1:], dtype=np.int64))
    lib().seq_scatter_add_rows_f32(_p(out), _p(self_), _p(rows), _p(src), ctypes.c_int64(rows.shape[0]),
                                   ctypes.c_int64(n_dst), ctypes.c_int64(inner))
    return out


def scatter_add_dim0(self_, index, src):
    self_ = np.ascontiguousarray(self_, dtype=np.float32)
    src = np.ascontiguousarray(src, dtype=np.float32)
    index = np.ascontiguousarray(index, dtype=np.int64)
    out = np.empty_like(self_)
    lib().seq_scatter_add_dim0_f32(_p(out), _p(self_), _p(index), _p(src), ctypes.c_int64(src.shape[0]),
                                   ctypes.c_int64(self_.shape[0]), ctypes.c_int64(self_.shape[1]))
    return out


def index_put_rows(self_, rows, src):
    out = np.array(self_, dtype=np.float32, copy=True, order="C")
    src = np.ascontiguousarray(src, dtype=np.float32)
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    inner = int(np.prod(out.shape[1:], dtype=np.int64))
    lib().seq_index_put_rows_f32(_p(out), _p(rows), _p(src), ctypes.c_int64(rows.shape[0]),
                                 ctypes.c_int64(out.shape[0]), ctypes.c_int64(inner))
    return out


def gather_rows(table, rows):
    table = np.ascontiguousarray(table)
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    row_bytes = table.strides[0]
    out = np.empty((rows.shape[0],) + table.shape[1:], dtype=table.dtype)
    lib().seq_gather_rows(_p(out), _p(table), _p(rows), ctypes.c_int64(rows.shape[0]), ctypes.c_int64(row_bytes))
    return out


def gather_lastdim(self_, index):
    self_ = np.ascontiguousarray(self_, dtype=np.float32)
    index = np.ascontiguousarray(index, dtype=np.int64)
    out = np.empty(index.shape, dtype=np.float32)
    lib().seq_gather_lastdim_f32(_p(out), _p(self_), _p(index), ctypes.c_int64(index.shape[0]),
                                 ctypes.c_int64(index.shape[1]), ctypes.c_int64(self_.shape[1]))
    return out


def f32_to_bf16_bits(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().seq_f32_to_bf16(_p(out), _p(x), ctypes.c_int64(x.size))
    return out


def bf16_bits_to_f32(b):
    b = np.ascontiguousarray(b, dtype=np.uint16)
    out = np.empty(b.shape, dtype=np.float32)
    lib().seq_bf16_to_f32(_p(out), _p(b), ctypes.c_int64(b.size))
    return out
