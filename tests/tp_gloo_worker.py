"""Worker of test_tensor_parallel_sharding_gloo_world2: one CPU rank of a
world-size-2 gloo group running the decoder harness's sharding logic."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "torch-gcu_b200"))
import workloads  # noqa: E402
from tp_decoder import DecoderLayer, DecoderStack, reference_layer_cpu  # noqa: E402

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
# the microbatch schedule (asynchronous all-reduces of one part under the other parts' compute) walks the
# same rows through the same arithmetic as the plain layer-by-layer pass
stack = DecoderStack(3, world, rank, "cpu", None, torch.float32, cfg)
x4 = torch.randn(4, 16, cfg["hidden"], generator=g)
plain = stack.prefill(x4, dist.group.WORLD, overlap=False)
piped = stack.prefill(x4, dist.group.WORLD, overlap=True)
assert plain.shape == piped.shape and torch.allclose(plain, piped, rtol=1e-5, atol=1e-5)
os.environ["TP_DECODER_MICROBATCHES"] = "4"
piped4 = stack.prefill(x4, dist.group.WORLD, overlap=True)
assert torch.allclose(plain, piped4, rtol=1e-5, atol=1e-5)
dist.barrier()
if rank == 0:
    print("TP_OK", err)
dist.destroy_process_group()
