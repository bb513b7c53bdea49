"""Autocast state accessors on the PrivateUse1 key (reference: torch_gcu/gcu/autocast_utils.py:8-43)."""
import torch

from torch_gcu import _C

__all__ = ["get_amp_supported_dtype", "is_autocast_enabled", "set_autocast_enabled", "get_autocast_dtype",
           "set_autocast_dtype"]


def get_amp_supported_dtype():
    return [torch.float32, torch.bfloat16, torch.float16]


def is_autocast_enabled():
    return _C.is_autocast_enabled()


def set_autocast_enabled(enable):
    _C.set_autocast_enabled(enable)


def get_autocast_dtype():
    return _C.get_autocast_dtype()


def set_autocast_dtype(dtype):
    return _C.set_autocast_dtype(dtype)
