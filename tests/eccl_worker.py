"""One rank of the eccl (NCCL over NVLink) tests: collectives against known
answers and the tensor-parallel decoder layer against the unsharded CPU layer."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "torch-gcu_b200"))
import torch_gcu  # noqa: E402,F401
import workloads  # noqa: E402
from tp_decoder import DecoderLayer, reference_layer_cpu  # noqa: E402

rank, world = int(sys.argv[1]), int(sys.argv[2])
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
torch.gcu.set_device(rank)
dev = torch.device("gcu", rank)
dist.init_process_group("eccl", rank=rank, world_size=world)

# every collective against its known answer
import collective_check  # noqa: E402
checked = collective_check.run(dev, rank, world)
assert "all_reduce_sum" in checked and "reduce_scatter" in checked and (world == 1 or "send_recv" in checked)

# tensor-parallel layer == unsharded layer (bf16 tolerance: summation order differs)
cfg = dict(hidden=512, heads=8, kv_heads=world if world <= 8 else 8, head_dim=64, ffn=1024)
if cfg["heads"] % world == 0 and cfg["kv_heads"] % world == 0:
    g = torch.Generator().manual_seed(0)
    xh = torch.randn(2, 128, cfg["hidden"], generator=g).bfloat16()
    full = workloads.decoder_layer_weights(seed=1, dtype=torch.bfloat16, **cfg)
    shard = workloads.decoder_layer_weights(seed=1, dtype=torch.bfloat16, tp=world, rank=rank, **cfg)
    layer = DecoderLayer(shard, tp=world, backend="gcu", device=dev, **cfg)
    y = layer.forward_prefill(xh.to(dev), group=dist.group.WORLD).cpu().float()
    ref = reference_layer_cpu(xh, full, **cfg)
    err = (y - ref).abs().max().item()
    assert err < 0.15, err
    rel = ((y - ref).norm() / ref.norm()).item()
    assert rel < 2e-2, rel
    # the two-microbatch schedule (all-reduce of one half under the other half's compute) gives the
    # same rows as the plain schedule
    from tp_decoder import DecoderStack
    stack = DecoderStack(3, world, rank, "gcu", dev, torch.bfloat16, cfg)
    x8 = torch.randn(8, 128, cfg["hidden"], generator=g).bfloat16().to(dev)   # halves of 512 rows: same kernels as the whole
    plain = stack.prefill(x8, dist.group.WORLD, overlap=False)
    piped = stack.prefill(x8, dist.group.WORLD, overlap=True)
    torch.gcu.synchronize()
    assert plain.shape == piped.shape
    if world == 2:   # a two-term sum does not depend on how the message is cut
        assert torch.equal(plain.cpu(), piped.cpu())
    else:
        assert (plain.cpu().float() - piped.cpu().float()).abs().max().item() < 0.1
dist.barrier()
torch.gcu.synchronize()
if rank == 0:
    print("ECCL_OK world", world)
dist.destroy_process_group()
