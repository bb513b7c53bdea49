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
    if world > 1:
        # the peer-memory exchange (this backend's own kernels instead of all-reduces): same rows within the
        # bf16 tolerance of a different summation order, for prefill (two microbatches and one) and for decode
        import b200ops  # noqa: E402
        fused = stack.prefill(x8, dist.group.WORLD)
        assert stack.uses_peer_exchange()
        torch.gcu.synchronize()
        ref8 = plain.cpu().float()
        rel = ((fused.cpu().float() - ref8).norm() / ref8.norm()).item()
        assert rel < 2e-2, rel
        os.environ["TP_DECODER_MICROBATCHES"] = "1"
        fused1 = stack.prefill(x8, dist.group.WORLD)
        os.environ["TP_DECODER_MICROBATCHES"] = "2"
        torch.gcu.synchronize()
        assert torch.equal(fused1.cpu(), fused.cpu())       # rows do not depend on how the batch is cut
        again = stack.prefill(x8, dist.group.WORLD)
        torch.gcu.synchronize()
        assert torch.equal(again.cpu(), fused.cpu())        # fixed summation order: reproducible
        hk = cfg["kv_heads"] // world
        T = 96
        kc = torch.randn(4, hk, T, cfg["head_dim"], generator=g).bfloat16()
        vc = torch.randn(4, hk, T, cfg["head_dim"], generator=g).bfloat16()
        xd = torch.randn(4, 1, cfg["hidden"], generator=g).bfloat16().to(dev)
        caches_a = [(kc.to(dev), vc.to(dev)) for _ in range(3)]
        caches_b = [(kc.to(dev), vc.to(dev)) for _ in range(3)]
        yd = stack.decode(xd, caches_a, T - 1, dist.group.WORLD)
        os.environ["TP_DECODER_EXCHANGE"] = "nccl"
        yn = stack.decode(xd, caches_b, T - 1, dist.group.WORLD)
        os.environ["TP_DECODER_EXCHANGE"] = "peer"
        torch.gcu.synchronize()
        rel = ((yd.cpu().float() - yn.cpu().float()).norm() / yn.cpu().float().norm()).item()
        assert rel < 2e-2, rel
        assert b200ops.device_error_fetch() == 0            # no bounded wait ran out
dist.barrier()
torch.gcu.synchronize()
if rank == 0:
    print("ECCL_OK world", world)
dist.destroy_process_group()
