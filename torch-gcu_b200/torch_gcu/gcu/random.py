"""Seeding API of the device generators (reference: torch_gcu/gcu/random.py)."""
import torch

from torch_gcu import _C


def _count():
    return _C._gcu_getDeviceCount()


def manual_seed(seed: int) -> None:
    import torch_gcu.gcu as gcu
    if _count() > 0:
        _C._gcu_manualSeed(gcu.current_device(), int(seed))


def manual_seed_all(seed: int) -> None:
    for i in range(_count()):
        _C._gcu_manualSeed(i, int(seed))


def seed() -> None:
    manual_seed(torch.seed())


def seed_all() -> None:
    manual_seed_all(torch.seed())


def initial_seed() -> int:
    import torch_gcu.gcu as gcu
    return _C._gcu_initialSeed(gcu.current_device())


def get_rng_state(device="gcu"):
    import torch_gcu.gcu as gcu
    idx = gcu._get_device_index(device)
    return torch.tensor([_C._gcu_initialSeed(idx)], dtype=torch.int64).view(torch.uint8)


def set_rng_state(new_state, device="gcu") -> None:
    import torch_gcu.gcu as gcu
    idx = gcu._get_device_index(device)
    _C._gcu_manualSeed(idx, int(new_state.view(torch.int64)[0].item()))
