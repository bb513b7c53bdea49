"""Worker of test_tensor_parallel_sharding_gloo_world2: one CPU rank of a
world-size-2 gloo group running the decoder harness's sharding logic."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "torch-gcu_b200"))
import workloads  # noqa: E402
from tp_decoder import DecoderLayer, reference_layer_cpu  # noqa: E402

rank, world = int(sys.argv[1]), int(sys.argv[2])
dist.init_process_group("gloo", rank=rank, world_size=world)
cfg = dict(hidden=256, heads=8, kv_heads=2, head_dim=32, ffn=512)
g = torch.Generator().manual_seed(0)
x = torch.randn(2, 16, cfg["hidden"], generator=g)
full = workloads.decoder_layer_weights(seed=1, dtype=torch.float32, **cfg)
shard = workloads.decoder_layer_weights(seed=1, dtype=torch.float32, tp=world, rank=rank, **cfg)
layer = DecoderLayer(shard, tp=world, backend="cpu", **cfg)
y = layer.forward_prefill(x, group=dist.group.WORLD)
ref = reference_layer_cpu(x, full, **cfg)
err = (y - ref).abs().max().item()
assert err < 1e-4, err
dist.barrier()
if rank == 0:
    print("TP_OK", err)
dist.destroy_process_group()
