"""ctypes binding of the kernel library's C ABI (include/b200ops.h).

This is the thinnest possible caller of libb200ops.so: it builds `b200Tensor`
views over device memory (any object with data_ptr/shape/stride/dtype, in
practice torch CUDA tensors used purely as device buffers) and calls the
`extern "C"` entry points. The parity tests and the benchmark go through it so
that what they exercise is the C ABI itself, the same boundary the C++ host code
of the PrivateUse1 backend binds.

There is no fallback: if the library is missing or a call returns a non-OK
status an exception is raised.
"""
import ctypes
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libb200ops.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "b200ops.h")

MAX_DIMS = 8

OK, BAD_PARAM, NOT_SUPPORTED, LAUNCH_FAILED, WORKSPACE_TOO_SMALL, TIMEOUT = range(6)
STATUS_NAMES = ["OK", "BAD_PARAM", "NOT_SUPPORTED", "LAUNCH_FAILED", "WORKSPACE_TOO_SMALL", "TIMEOUT"]

F32, BF16, F16, F64, I64, I32, I16, I8, U8, BOOL = range(10)

UNARY = dict(neg=0, rsqrt=1, sqrt=2, exp=3, sigmoid=4, tanh=5, relu=6, abs=7, reciprocal=8, cos=9,
             sin=10, log=11, gelu=12)


class Tensor(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("dtype", ctypes.c_int32),
        ("ndim", ctypes.c_int32),
        ("sizes", ctypes.c_int64 * MAX_DIMS),
        ("strides", ctypes.c_int64 * MAX_DIMS),
    ]


class B200Error(RuntimeError):
    def __init__(self, status, message):
        super().__init__("b200ops status %s: %s" % (STATUS_NAMES[status] if 0 <= status < 6 else status, message))
        self.status = status


_lib = None


def declared_symbols():
    """Names of every function the public header declares."""
    text = open(HEADER_PATH).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                "libb200ops.so is not built (%s); run `python torch-gcu_b200/build.py kernels`" % LIB_PATH)
        L = ctypes.CDLL(LIB_PATH)
        L.b200_last_error.restype = ctypes.c_char_p
        L.b200_version.restype = ctypes.c_char_p
        L.b200_dtype_size.restype = ctypes.c_size_t
        for name in declared_symbols():
            fn = getattr(L, name)
            if name.endswith("_workspace_size"):
                fn.restype = ctypes.c_size_t
        _lib = L
    return _lib


def _torch_dtype_code(dt):
    import torch
    return {
        torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16, torch.float64: F64,
        torch.int64: I64, torch.int32: I32, torch.int16: I16, torch.int8: I8, torch.uint8: U8,
        torch.bool: BOOL,
    }[dt]


def view(t):
    """b200Tensor over a tensor-like object (not kept alive by the view)."""
    if t is None:
        return None
    v = Tensor()
    v.data = t.data_ptr()
    v.dtype = _torch_dtype_code(t.dtype)
    v.ndim = t.dim()
    if v.ndim > MAX_DIMS:
        raise ValueError("rank %d exceeds %d" % (v.ndim, MAX_DIMS))
    for i, (s, st) in enumerate(zip(t.shape, t.stride())):
        v.sizes[i] = s
        v.strides[i] = st
    return v


def _ref(v):
    return ctypes.byref(v) if v is not None else None


def _stream(stream):
    if stream is None:
        import torch
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    if hasattr(stream, "cuda_stream"):
        return ctypes.c_void_p(stream.cuda_stream)
    return ctypes.c_void_p(int(stream))


def check(status):
    if status != OK:
        raise B200Error(status, lib().b200_last_error().decode())


def _i64_array(values):
    arr = (ctypes.c_int64 * max(1, len(values)))(*values)
    return arr


def bind(name, *args, keep=()):
    """Pre-marshals one call: tensors become b200Tensor views once, ctypes scalars
    pass through, None is NULL. Returns a callable that enqueues the call on the
    given (or current) stream; the stream is appended as the last argument. The
    returned callable holds a reference to every tensor argument; memory passed
    as a raw pointer (a workspace) must be kept alive by the caller, e.g. through
    `keep=`. Used where per-call Python overhead matters."""
    import torch
    fn = getattr(lib(), "b200_" + name)
    keep, conv = list(keep), []
    for a in args:
        if torch.is_tensor(a):
            v = view(a)
            keep.extend([v, a])
            conv.append(ctypes.byref(v))
        elif isinstance(a, (list, tuple)) and a and torch.is_tensor(a[0]):
            views = [view(t) for t in a]
            arr = (ctypes.POINTER(Tensor) * len(views))(*[ctypes.pointer(v) for v in views])
            keep.extend([views, arr, list(a)])
            conv.append(arr)
        else:
            conv.append(a)

    def call(stream=None, _fn=fn, _conv=tuple(conv), _keep=keep):
        st = _fn(*_conv, _stream(stream))
        if st != OK:
            check(st)
    return call


def ws_args(workspace):
    """(pointer, size) ctypes pair for a workspace tensor (or NULL, 0)."""
    if workspace is None:
        return None, ctypes.c_size_t(0)
    return ctypes.c_void_p(workspace.data_ptr()), ctypes.c_size_t(workspace.numel() * workspace.element_size())


# ---- thin wrappers: one per entry point; tensors are torch tensors ----------

def add(out, a, b, alpha=1.0, stream=None):
    check(lib().b200_add(_ref(view(out)), _ref(view(a)), _ref(view(b)), ctypes.c_double(alpha), _stream(stream)))


def sub(out, a, b, alpha=1.0, stream=None):
    check(lib().b200_sub(_ref(view(out)), _ref(view(a)), _ref(view(b)), ctypes.c_double(alpha), _stream(stream)))


def mul(out, a, b, stream=None):
    check(lib().b200_mul(_ref(view(out)), _ref(view(a)), _ref(view(b)), _stream(stream)))


def div(out, a, b, stream=None):
    check(lib().b200_div(_ref(view(out)), _ref(view(a)), _ref(view(b)), _stream(stream)))


def add_scalar(out, a, b, alpha=1.0, stream=None):
    check(lib().b200_add_scalar(_ref(view(out)), _ref(view(a)), ctypes.c_double(b), ctypes.c_double(alpha),
                                _stream(stream)))


def mul_scalar(out, a, b, stream=None):
    check(lib().b200_mul_scalar(_ref(view(out)), _ref(view(a)), ctypes.c_double(b), _stream(stream)))


def silu(out, a, stream=None):
    check(lib().b200_silu(_ref(view(out)), _ref(view(a)), _stream(stream)))


def unary(out, a, op, stream=None):
    check(lib().b200_unary(_ref(view(out)), _ref(view(a)), ctypes.c_int32(UNARY[op] if isinstance(op, str) else op),
                           _stream(stream)))


def pow_scalar(out, a, exponent, stream=None):
    check(lib().b200_pow_scalar(_ref(view(out)), _ref(view(a)), ctypes.c_double(exponent), _stream(stream)))


def fill(out, value, stream=None):
    check(lib().b200_fill(_ref(view(out)), ctypes.c_double(value), _stream(stream)))


def fill_i64(out, value, stream=None):
    check(lib().b200_fill_i64(_ref(view(out)), ctypes.c_int64(value), _stream(stream)))


def copy(dst, src, stream=None):
    check(lib().b200_copy(_ref(view(dst)), _ref(view(src)), _stream(stream)))


def sum_workspace_size(inp, dims):
    return lib().b200_sum_workspace_size(_ref(view(inp)), _i64_array(dims), ctypes.c_int32(len(dims)))


def sum(out, inp, dims, mean=False, workspace=None, stream=None):  # noqa: A001
    ws_ptr = ctypes.c_void_p(workspace.data_ptr()) if workspace is not None else None
    ws_n = ctypes.c_size_t(workspace.numel() * workspace.element_size()) if workspace is not None else ctypes.c_size_t(0)
    check(lib().b200_sum(_ref(view(out)), _ref(view(inp)), _i64_array(dims), ctypes.c_int32(len(dims)),
                         ctypes.c_int32(1 if mean else 0), ws_ptr, ws_n, _stream(stream)))


def softmax(out, inp, dim, stream=None):
    check(lib().b200_softmax(_ref(view(out)), _ref(view(inp)), ctypes.c_int64(dim), _stream(stream)))


def native_layer_norm(out, mean, rstd, inp, M, N, weight, bias, eps, stream=None):
    check(lib().b200_native_layer_norm(_ref(view(out)), _ref(view(mean)), _ref(view(rstd)), _ref(view(inp)),
                                       ctypes.c_int64(M), ctypes.c_int64(N), _ref(view(weight)), _ref(view(bias)),
                                       ctypes.c_double(eps), _stream(stream)))


def index_select(out, self, dim, index, stream=None):
    check(lib().b200_index_select(_ref(view(out)), _ref(view(self)), ctypes.c_int64(dim), _ref(view(index)),
                                  _stream(stream)))


def gather(out, self, dim, index, stream=None):
    check(lib().b200_gather(_ref(view(out)), _ref(view(self)), ctypes.c_int64(dim), _ref(view(index)),
                            _stream(stream)))


def scatter_add_workspace_size(self, dim, index, src):
    return lib().b200_scatter_add_workspace_size(_ref(view(self)), ctypes.c_int64(dim), _ref(view(index)),
                                                 _ref(view(src)))


def scatter_add(out, self, dim, index, src, workspace, stream=None):
    ws_ptr = ctypes.c_void_p(workspace.data_ptr()) if workspace is not None else None
    ws_n = ctypes.c_size_t(workspace.numel() * workspace.element_size()) if workspace is not None else ctypes.c_size_t(0)
    check(lib().b200_scatter_add(_ref(view(out)), _ref(view(self)), ctypes.c_int64(dim), _ref(view(index)),
                                 _ref(view(src)), ws_ptr, ws_n, _stream(stream)))


def scatter_add_static(out, self, dim, index, src, stream=None):
    """scatter_add that allocates nothing: scratch is the library's built-in 8 MiB array."""
    check(lib().b200_scatter_add_static(_ref(view(out)), _ref(view(self)), ctypes.c_int64(dim), _ref(view(index)),
                                        _ref(view(src)), _stream(stream)))


def index_put_workspace_size(self, index, values):
    return lib().b200_index_put_workspace_size(_ref(view(self)), _ref(view(index)), _ref(view(values)))


def index_put(self, index, values, accumulate, workspace, stream=None):
    ws_ptr = ctypes.c_void_p(workspace.data_ptr()) if workspace is not None else None
    ws_n = ctypes.c_size_t(workspace.numel() * workspace.element_size()) if workspace is not None else ctypes.c_size_t(0)
    check(lib().b200_index_put(_ref(view(self)), _ref(view(index)), _ref(view(values)),
                               ctypes.c_int32(1 if accumulate else 0), ws_ptr, ws_n, _stream(stream)))


def index(out, src_view, indices, indexed_sizes, indexed_strides, stream=None):
    views = [view(i) for i in indices]
    arr = (ctypes.POINTER(Tensor) * len(views))(*[ctypes.pointer(v) for v in views])
    check(lib().b200_index(_ref(view(out)), _ref(view(src_view)), arr, ctypes.c_int32(len(views)),
                           _i64_array(indexed_sizes), _i64_array(indexed_strides), _stream(stream)))


def rms_norm_residual(y, residual_out, x, residual, weight, eps, stream=None):
    check(lib().b200_rms_norm_residual(_ref(view(y)), _ref(view(residual_out)), _ref(view(x)), _ref(view(residual)),
                                       _ref(view(weight)), ctypes.c_double(eps), _stream(stream)))


def rope(out, x, cos_table, sin_table, positions=None, stream=None):
    check(lib().b200_rope(_ref(view(out)), _ref(view(x)), _ref(view(cos_table)), _ref(view(sin_table)),
                          _ref(view(positions)), _stream(stream)))


def rope_kv_append(qkv, cos_table, sin_table, positions, q_heads, k_heads, k_cache, v_cache, stream=None):
    """Rotate the query heads of qkv (B,S,Hq+2Hk,D) in place, write the rotated key heads and the value heads
    into the caches (B,Hk,T,D) at positions (B,S)."""
    check(lib().b200_rope_kv_append(_ref(view(qkv)), _ref(view(cos_table)), _ref(view(sin_table)), _ref(view(positions)),
                                    ctypes.c_int64(q_heads), ctypes.c_int64(k_heads), _ref(view(k_cache)), _ref(view(v_cache)),
                                    _stream(stream)))


def swiglu(out, gate, up, stream=None):
    check(lib().b200_swiglu(_ref(view(out)), _ref(view(gate)), _ref(view(up)), _stream(stream)))


def mm_swiglu(out, a, w_gate_up, stream=None):
    """out (M,F) = silu(a @ w[:F].T) * (a @ w[F:].T), the SwiGLU fused into the GEMM epilogue."""
    check(lib().b200_mm_swiglu(_ref(view(out)), _ref(view(a)), _ref(view(w_gate_up)), _stream(stream)))


def mm_swiglu_few_rows(rows, f, k):
    """True when mm_swiglu has a few-row kernel (one wave of equal tiles, or split-K with the activation in the
    reduction) for rows x (2 f) x k."""
    fn = lib().b200_mm_swiglu_few_rows
    fn.restype, fn.argtypes = ctypes.c_int, [ctypes.c_int64, ctypes.c_int64, ctypes.c_int64]
    return bool(fn(rows, f, k))


def mm_rope(out, a, w, cos_table, sin_table, seq_len, rope_cols, stream=None):
    """out (M,N) = a @ w.T with rotate-half RoPE on the first rope_cols columns (heads of 128), in the GEMM epilogue."""
    check(lib().b200_mm_rope(_ref(view(out)), _ref(view(a)), _ref(view(w)), _ref(view(cos_table)), _ref(view(sin_table)),
                             ctypes.c_int64(seq_len), ctypes.c_int64(rope_cols), _stream(stream)))


def mm(out, a, b, stream=None):
    check(lib().b200_mm(_ref(view(out)), _ref(view(a)), _ref(view(b)), _stream(stream)))


def addmm(out, self, a, b, beta=1.0, alpha=1.0, stream=None):
    check(lib().b200_addmm(_ref(view(out)), _ref(view(self)), _ref(view(a)), _ref(view(b)), ctypes.c_double(beta),
                           ctypes.c_double(alpha), _stream(stream)))


def bmm(out, a, b, stream=None):
    check(lib().b200_bmm(_ref(view(out)), _ref(view(a)), _ref(view(b)), _stream(stream)))


def baddbmm(out, self, a, b, beta=1.0, alpha=1.0, stream=None):
    check(lib().b200_baddbmm(_ref(view(out)), _ref(view(self)), _ref(view(a)), _ref(view(b)), ctypes.c_double(beta),
                             ctypes.c_double(alpha), _stream(stream)))


def sdpa_flash_fwd(out, lse, q, k, v, is_causal, scale=None, stream=None):
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    check(lib().b200_sdpa_flash_fwd(_ref(view(out)), _ref(view(lse)), _ref(view(q)), _ref(view(k)), _ref(view(v)),
                                    ctypes.c_int32(1 if is_causal else 0), ctypes.c_double(scale), _stream(stream)))


def sdpa_flash_bwd(dq, dk, dv, dout, q, k, v, out, lse, is_causal, scale=None, workspace=None, stream=None):
    """Flash-attention backward: dq, dk, dv from dout and the forward's q, k, v, out, lse."""
    import torch
    sc = float(scale) if scale is not None else float(q.shape[-1]) ** -0.5
    lib().b200_sdpa_flash_bwd_workspace_size.restype = ctypes.c_size_t
    need = lib().b200_sdpa_flash_bwd_workspace_size(_ref(view(q)))
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=q.device)
    check(lib().b200_sdpa_flash_bwd(_ref(view(dq)), _ref(view(dk)), _ref(view(dv)), _ref(view(dout)), _ref(view(q)),
                                    _ref(view(k)), _ref(view(v)), _ref(view(out)), _ref(view(lse)),
                                    ctypes.c_int32(1 if is_causal else 0), ctypes.c_double(sc), *ws_args(workspace),
                                    _stream(stream)))


def sort_rows_workspace_size(inp):
    return lib().b200_sort_rows_workspace_size(_ref(view(inp)))


def sort_rows(values, indices, inp, descending=False, workspace=None, stream=None):
    """Stable sort of every row of a contiguous (rows, n) tensor; values / indices (rows, k <= n)."""
    import torch
    if workspace is None:
        workspace = torch.empty(max(1, sort_rows_workspace_size(inp)), dtype=torch.uint8, device=inp.device)
    check(lib().b200_sort_rows(_ref(view(values)), _ref(view(indices)), _ref(view(inp)),
                               ctypes.c_int32(1 if descending else 0), *ws_args(workspace), _stream(stream)))


def cumsum(out, inp, dim, stream=None):
    check(lib().b200_cumsum(_ref(view(out)), _ref(view(inp)), ctypes.c_int64(dim), _stream(stream)))


class TpPeers(ctypes.Structure):
    _fields_ = [("world", ctypes.c_int32), ("rank", ctypes.c_int32), ("base", ctypes.c_void_p * 8)]


def tp_peers(buffers, rank, offset=0):
    """b200TpPeers over one buffer per rank (tensors, or raw addresses), each at `offset` bytes."""
    t = TpPeers()
    t.world, t.rank = len(buffers), rank
    for r, b in enumerate(buffers):
        t.base[r] = (b.data_ptr() if hasattr(b, "data_ptr") else int(b)) + offset
    return t


def tp_control_bytes():
    lib().b200_tp_control_bytes.restype = ctypes.c_size_t
    return int(lib().b200_tp_control_bytes())


def tp_sync(control, channel=0, signal=True, wait=True, timeout_s=2.0, stream=None):
    check(lib().b200_tp_sync(ctypes.byref(control), ctypes.c_int32(channel), ctypes.c_int32(1 if signal else 0),
                             ctypes.c_int32(1 if wait else 0), ctypes.c_uint64(int(timeout_s * 1e9)), _stream(stream)))


def tp_reduce_norm(partial, gathered, residual, residual_out, weight, row0, total_rows, eps=1e-6, normalise=True,
                   gather_all=True, stream=None):
    check(lib().b200_tp_reduce_norm(ctypes.byref(partial) if partial is not None else None, ctypes.byref(gathered),
                                    _ref(view(residual)), _ref(view(residual_out)), _ref(view(weight)),
                                    ctypes.c_int64(row0), ctypes.c_int64(total_rows), ctypes.c_double(eps),
                                    ctypes.c_int32(1 if normalise else 0), ctypes.c_int32(1 if gather_all else 0),
                                    _stream(stream)))


def launch_count():
    """Kernel launches the library has issued in this process so far."""
    lib().b200_launch_count.restype = ctypes.c_ulonglong
    return int(lib().b200_launch_count())


def device_error_fetch():
    flags = ctypes.c_uint32(0)
    check(lib().b200_device_error_fetch(ctypes.byref(flags)))
    return flags.value
