"""`torch.gcu.amp.autocast(...)` == `torch.autocast("gcu", ...)`
(reference: torch_gcu/gcu/amp/autocast_mode.py:17-44)."""
import torch

__all__ = ["autocast"]


class autocast(torch.amp.autocast_mode.autocast):
    def __init__(self, enabled: bool = True, dtype: torch.dtype = torch.bfloat16, cache_enabled: bool = True):
        super().__init__("gcu", enabled=enabled, dtype=dtype, cache_enabled=cache_enabled)
