"""Allocator statistics and cache control (reference: torch_gcu/gcu/memory.py, subset)."""
from torch_gcu import _C


def _idx(device):
    import torch_gcu.gcu as gcu
    return gcu._get_device_index(device)


def empty_cache() -> None:
    """Returns every cached block to the driver's pool."""
    _C._gcu_emptyCache()
    _C._gcu_hostEmptyCache()


def memory_stats(device=None):
    return _C._gcu_memoryStats(_idx(device))


def memory_allocated(device=None) -> int:
    return memory_stats(device)["allocated_bytes.all.current"]


def max_memory_allocated(device=None) -> int:
    return memory_stats(device)["allocated_bytes.all.peak"]


def memory_reserved(device=None) -> int:
    return memory_stats(device)["reserved_bytes.all.current"]


def max_memory_reserved(device=None) -> int:
    return memory_stats(device)["reserved_bytes.all.peak"]


def reset_peak_memory_stats(device=None) -> None:
    _C._gcu_resetPeakMemoryStats(_idx(device))


def mem_get_info(device=None):
    import torch_gcu.gcu as gcu
    gcu._lazy_init()
    return _C._gcu_memGetInfo(_idx(device))
