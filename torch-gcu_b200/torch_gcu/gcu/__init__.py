"""torch.gcu: the device module of the gcu (B200) backend, a mirror of torch.cuda
for the calls the operator path needs (reference: torch_gcu/gcu/__init__.py:98-801)."""
import threading
from typing import Any, Optional, Union

import torch

import torch_gcu
from torch_gcu import _C

from . import amp  # noqa: F401
from . import efficient  # noqa: F401
from .autocast_utils import (get_amp_supported_dtype, get_autocast_dtype, is_autocast_enabled,  # noqa: F401
                             set_autocast_dtype, set_autocast_enabled)
from .memory import (empty_cache, max_memory_allocated, max_memory_reserved, mem_get_info, memory_allocated,  # noqa: F401
                     memory_reserved, memory_stats, reset_peak_memory_stats)
from .random import (get_rng_state, initial_seed, manual_seed, manual_seed_all, seed, seed_all,  # noqa: F401
                     set_rng_state)
from .streams import Event, ExternalStream, Stream  # noqa: F401
from .graphs import GCUGraph, graph, is_current_stream_capturing  # noqa: F401

_device_t = Union[torch.device, str, int, None]
_initialized = False
_init_lock = threading.Lock()


def _is_compiled() -> bool:
    return True


def is_available() -> bool:
    return _C._gcu_getDeviceCount() > 0


def is_bf16_supported() -> bool:
    return True


def _is_in_bad_fork() -> bool:
    return False


def is_initialized() -> bool:
    return _initialized


def init():
    _lazy_init()


def _lazy_init():
    """Creates the primary context of the current device on first use
    (reference: torch_gcu/gcu/__init__.py:160-216)."""
    global _initialized
    if _initialized:
        return
    with _init_lock:
        if _initialized:
            return
        if not is_available():
            raise RuntimeError("no gcu (B200) device is available; the gcu backend has no CPU fallback")
        _C._gcu_init()
        _initialized = True


def device_count() -> int:
    return _C._gcu_getDeviceCount()


def _get_device_index(device: _device_t, optional: bool = True) -> int:
    if device is None:
        return current_device() if optional else -1
    if isinstance(device, int):
        return device
    if isinstance(device, str):
        device = torch.device(device)
    if isinstance(device, torch.device):
        if device.type != "gcu":
            raise ValueError("Expected a gcu device, but got: %s" % device)
        return current_device() if device.index is None else device.index
    raise TypeError("unsupported device specification %r" % (device,))


def current_device() -> int:
    _lazy_init()
    return _C._gcu_getDevice()


def set_device(device: _device_t) -> None:
    idx = _get_device_index(device)
    if idx >= 0:
        _lazy_init()
        _C._gcu_setDevice(idx)


def _exchange_device(device: int) -> int:
    if device < 0:
        return -1
    _lazy_init()
    return _C._gcu_exchangeDevice(device)


_maybe_exchange_device = _exchange_device


class device:
    """Context manager that changes the selected device."""

    def __init__(self, device: Any):
        self.idx = _get_device_index(device, optional=True)
        self.prev_idx = -1

    def __enter__(self):
        self.prev_idx = _exchange_device(self.idx)

    def __exit__(self, *exc):
        self.idx = _exchange_device(self.prev_idx)
        return False


class device_of(device):
    def __init__(self, obj):
        super().__init__(obj.get_device() if getattr(obj, "is_gcu", False) else -1)


def set_reserved_sms(n: int) -> None:
    """Leave n SMs free of the persistent GEMM kernels, so that a collective launched on another
    stream (the process group's) can run beside them instead of after them. 0 restores the default."""
    _C._set_reserved_sms(int(n))


def get_reserved_sms() -> int:
    return _C._get_reserved_sms()


def synchronize(device: _device_t = None) -> None:
    _lazy_init()
    with torch_gcu.gcu.device(device):
        _C._gcu_synchronize()


def get_device_properties(device: _device_t = None):
    _lazy_init()
    return _C._gcu_getDeviceProperties(_get_device_index(device))


def get_device_name(device: _device_t = None) -> str:
    return get_device_properties(device)["name"]


def get_device_capability(device: _device_t = None):
    p = get_device_properties(device)
    return p["major"], p["minor"]


def current_stream(device: _device_t = None) -> Stream:
    _lazy_init()
    sid, didx, dtype = _C._gcu_getCurrentStream(_get_device_index(device))
    return Stream(stream_id=sid, device_index=didx, device_type=dtype)


def default_stream(device: _device_t = None) -> Stream:
    _lazy_init()
    sid, didx, dtype = _C._gcu_getDefaultStream(_get_device_index(device))
    return Stream(stream_id=sid, device_index=didx, device_type=dtype)


def set_stream(stream: Optional[Stream]):
    if stream is None:
        return
    _lazy_init()
    _C._gcu_setStream(stream.stream_id, stream.device_index, stream.device_type)


def _set_stream_by_id(stream_id, device_index, device_type):
    _C._gcu_setStream(stream_id, device_index, device_type)


class StreamContext:
    """Selects a stream as current inside the block (reference: gcu/__init__.py:388-443)."""

    def __init__(self, stream: Optional[Stream]):
        self.stream = stream
        self.idx = _get_device_index(None, True) if stream is not None else -1

    def __enter__(self):
        cur = self.stream
        if cur is None or self.idx == -1:
            return
        self.src_prev_stream = current_stream(None)
        if self.src_prev_stream.device != cur.device:
            with device(cur.device):
                self.dst_prev_stream = current_stream(cur.device)
        set_stream(cur)

    def __exit__(self, *exc):
        cur = self.stream
        if cur is None or self.idx == -1:
            return False
        if self.src_prev_stream.device != cur.device:
            set_stream(self.dst_prev_stream)
        set_stream(self.src_prev_stream)
        return False


def stream(stream: Optional[Stream]) -> StreamContext:
    return StreamContext(stream)


def set_sync_debug_mode(mode) -> None:
    """Per-op stream synchronisation, the op_sync_mode debug switch."""
    _C._set_op_sync_mode(bool(mode) and mode not in (0, "default"))


def get_sync_debug_mode() -> int:
    return int(_C._get_op_sync_mode())
