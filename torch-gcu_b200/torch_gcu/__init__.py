"""torch_gcu on B200: the PrivateUse1 backend "gcu" with every kernel a
hand-written sm_100a CUDA kernel behind the C ABI of libb200ops.so.

Importing this package wires the backend the way the reference's package does
(reference: torch_gcu/__init__.py:79-102): PrivateUse1 is renamed to "gcu",
`torch.gcu` becomes the device module, tensors get `.gcu()` / `.is_gcu`, and the
c10d backend "eccl" is registered for gcu devices. There is no CPU fallback: an
operator without a kernel raises.
"""
import os

# the backend is loaded explicitly, not through torch's autoload entry point
_ORG_AUTOLOAD = os.getenv("TORCH_DEVICE_BACKEND_AUTOLOAD", "1")
os.environ["TORCH_DEVICE_BACKEND_AUTOLOAD"] = "0"

import torch  # noqa: E402

try:
    from . import _C  # noqa: E402
except ImportError as e:  # pragma: no cover - a build problem, never a fallback
    raise ImportError(
        "torch_gcu._C is not built (%s); run `python torch-gcu_b200/build.py all`. "
        "The gcu backend has no CPU fallback." % e) from e

from . import gcu  # noqa: E402
from . import distributed  # noqa: E402
from .version import __version__  # noqa: E402

torch.utils.rename_privateuse1_backend("gcu")
torch._register_device_module("gcu", gcu)
torch.utils.generate_methods_for_privateuse1_backend(for_storage=True)

torch.distributed.is_eccl_available = distributed.is_available


def _new_eccl_group(store, group_rank, group_size, timeout):
    return _C._distributed_c10d.ProcessGroupECCL(store, group_rank, group_size, timeout)


if distributed.is_available() and torch.distributed.is_available():
    torch.distributed.Backend.register_backend("eccl", _new_eccl_group, devices=["gcu"])

os.environ["TORCH_DEVICE_BACKEND_AUTOLOAD"] = _ORG_AUTOLOAD


def _autoload():
    """Entry point PyTorch calls on `import torch`; importing the package is all it takes."""
