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

# all_reduce (sum, max), in place
t = torch.full((1000,), float(rank + 1)).to(dev)
dist.all_reduce(t)
assert torch.equal(t.cpu(), torch.full((1000,), float(sum(range(1, world + 1)))))
m = torch.tensor([float(rank)]).to(dev)
dist.all_reduce(m, op=dist.ReduceOp.MAX)
assert m.item() == world - 1
# bf16 all_reduce of exactly representable values
b = torch.full((4096,), 0.5 * (rank + 1)).bfloat16().to(dev)
dist.all_reduce(b)
assert torch.equal(b.cpu().float(), torch.full((4096,), 0.5 * sum(range(1, world + 1))))
# broadcast
x = (torch.arange(16.0) if rank == 0 else torch.zeros(16)).to(dev)
dist.broadcast(x, src=0)
assert torch.equal(x.cpu(), torch.arange(16.0))
# all_gather_into_tensor / all_gather
out = torch.empty(world * 8).to(dev)
dist.all_gather_into_tensor(out, torch.full((8,), float(rank)).to(dev))
assert torch.equal(out.cpu(), torch.arange(world).repeat_interleave(8).float())
lst = [torch.empty(3).to(dev) for _ in range(world)]
dist.all_gather(lst, torch.full((3,), float(rank * 10)).to(dev))
assert all(torch.equal(lst[r].cpu(), torch.full((3,), float(r * 10))) for r in range(world))
# reduce_scatter
inp = torch.arange(world * 4, dtype=torch.float32).to(dev)
rs = torch.empty(4).to(dev)
dist.reduce_scatter_tensor(rs, inp)
assert torch.equal(rs.cpu(), world * torch.arange(rank * 4, rank * 4 + 4, dtype=torch.float32))
# reduce_scatter, list form
ins = [torch.full((6,), float(rank + 1 + r)).to(dev) for r in range(world)]
rl = torch.empty(6).to(dev)
dist.reduce_scatter(rl, ins)
assert torch.equal(rl.cpu(), torch.full((6,), float(sum(k + 1 + rank for k in range(world)))))
# reduce to a root
rd = torch.full((7,), float(rank + 1)).to(dev)
dist.reduce(rd, dst=world - 1)
if rank == world - 1:
    assert torch.equal(rd.cpu(), torch.full((7,), float(sum(range(1, world + 1)))))
# all_to_all_single, equal splits: row block r of rank k goes to rank r
a2a_in = (torch.arange(world * 2, dtype=torch.float32).view(world, 2) + 100 * rank).reshape(-1).to(dev)
a2a_out = torch.empty(world * 2).to(dev)
dist.all_to_all_single(a2a_out, a2a_in)
exp = torch.cat([torch.arange(rank * 2, rank * 2 + 2, dtype=torch.float32) + 100 * k for k in range(world)])
assert torch.equal(a2a_out.cpu(), exp)
# send / recv around a ring
if world > 1:
    msg = torch.full((9,), float(rank)).to(dev)
    got = torch.empty(9).to(dev)
    if rank % 2 == 0:
        dist.send(msg, (rank + 1) % world)
        dist.recv(got, (rank - 1) % world)
    else:
        dist.recv(got, (rank - 1) % world)
        dist.send(msg, (rank + 1) % world)
    assert torch.equal(got.cpu(), torch.full((9,), float((rank - 1) % world)))
# coalescing: two all-reduces issued as one group
backend = dist.group.WORLD._get_backend(dev)
c1, c2 = torch.full((5,), 1.0).to(dev), torch.full((3,), float(rank)).to(dev)
backend._group_start()
w1 = dist.all_reduce(c1, async_op=True)
w2 = dist.all_reduce(c2, async_op=True)
backend._group_end()
w1.wait()
w2.wait()
assert torch.equal(c1.cpu(), torch.full((5,), float(world))) and torch.equal(c2.cpu(), torch.full((3,), float(sum(range(world)))))
# out-of-place all-reduce extra of the backend
import torch_gcu.distributed as gd  # noqa: E402
o = torch.empty(5).to(dev)
gd.all_reduce_outplace(o, torch.ones(5).to(dev))
assert torch.equal(o.cpu(), torch.full((5,), float(world)))
assert len(gd.get_unique_id()) == 256
dist.barrier()

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
