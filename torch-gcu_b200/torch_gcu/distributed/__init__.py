"""c10d backend "eccl" for gcu tensors (NCCL over NVLink underneath).
Reference: torch_gcu/distributed/__init__.py:6-15."""
import torch_gcu


def is_available():
    """True when the extension was built with the c10d bindings."""
    return hasattr(torch_gcu._C, "_c10d_gcu_init")


if is_available() and not torch_gcu._C._c10d_gcu_init():
    raise RuntimeError("Failed to initialize torch_gcu.distributed")


def all_reduce_outplace(output, input, op=None, group=None):
    """Out-of-place all-reduce through the backend's extra method
    (reference: torch_gcu/distributed/distributed_c10d.py:73-115)."""
    import torch.distributed as dist
    group = group or dist.group.WORLD
    backend = group._get_backend(input.device)
    opts = dist.AllreduceOptions()
    if op is not None:
        opts.reduceOp = op
    work = backend.allreduce_outplace(output, input, opts)
    work.wait()
    return output


def get_unique_id(group=None):
    import torch
    import torch.distributed as dist
    group = group or dist.group.WORLD
    return group._get_backend(torch.device("gcu", torch.gcu.current_device())).get_unique_id()
