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
# the exchange path's schedule on host ranks (a gloo stand-in for the peer-memory kernels): the residual stream
# sharded by rows between the projections, one reduce + residual + norm + gather step per projection pair, the
# last layer's rows gathered as they are -- against the plain pass and the unsharded reference
os.environ["TP_DECODER_MICROBATCHES"] = "2"
seq = stack.prefill_exchange(x4, dist.group.WORLD)
assert seq.shape == plain.shape and torch.allclose(plain, seq, rtol=1e-4, atol=1e-4), (plain - seq).abs().max()
os.environ["TP_DECODER_MICROBATCHES"] = "1"
seq1 = stack.prefill_exchange(x4, dist.group.WORLD)
assert torch.allclose(plain, seq1, rtol=1e-4, atol=1e-4)
ref3 = x4
for i in range(3):
    ref3 = reference_layer_cpu(ref3, workloads.decoder_layer_weights(seed=i, dtype=torch.float32, **cfg), **cfg)
assert torch.allclose(seq, ref3, rtol=1e-3, atol=1e-3), (seq - ref3).abs().max()
# decode: one token per sequence after a prefill that filled the caches; the replicated-rows form of the exchange
T = 24
hk = cfg["kv_heads"] // world
caches = [(torch.zeros(4, hk, T, cfg["head_dim"]), torch.zeros(4, hk, T, cfg["head_dim"])) for _ in range(3)]
stack.prefill_exchange(x4, dist.group.WORLD, caches)
xt = torch.randn(4, 1, cfg["hidden"], generator=g)
yd = stack.decode_exchange(xt, caches, 16, dist.group.WORLD)
full_seq = torch.cat([x4, xt], 1)          # the same step as the last row of a 17-token prefill
ref_d = full_seq
for i in range(3):
    ref_d = reference_layer_cpu(ref_d, workloads.decoder_layer_weights(seed=i, dtype=torch.float32, **cfg), **cfg)
assert torch.allclose(yd, ref_d[:, 16:17], rtol=1e-3, atol=1e-3), (yd - ref_d[:, 16:17]).abs().max()
dist.barrier()
if rank == 0:
    print("TP_OK", err)
dist.destroy_process_group()
