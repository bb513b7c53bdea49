"""Known-answer checks of every collective of the "eccl" process group, on whatever number of ranks
the caller runs (harness code shared by the multi-rank test worker and by the benchmark, which
runs it before timing so that every multi-GPU run also proves the collectives it did not time).

Each check builds its inputs from the rank number, so the expected result is known in closed form
(reference: the collectives of torch_gcu/csrc/distributed/ProcessGroupECCL.cpp -- allreduce
2869-2926, broadcast 2967-3010, reduce 3012-3075, allgather 3077-3166, reduce_scatter 3168-3432,
alltoall_base 3464-3536, send / recv 3538-3566, coalescing 3976-4048)."""
import torch
import torch.distributed as dist


def run(dev, rank, world):
    """Runs every check on the default group; returns the names checked. Raises AssertionError on the
    first wrong answer. All ranks must call it."""
    done = []

    def ok(name, cond):
        assert cond, "eccl %s gave a wrong answer on rank %d of %d" % (name, rank, world)
        done.append(name)

    tri = float(sum(range(1, world + 1)))
    t = torch.full((1000,), float(rank + 1)).to(dev)
    dist.all_reduce(t)
    ok("all_reduce_sum", torch.equal(t.cpu(), torch.full((1000,), tri)))
    m = torch.tensor([float(rank)]).to(dev)
    dist.all_reduce(m, op=dist.ReduceOp.MAX)
    ok("all_reduce_max", m.item() == world - 1)
    b = torch.full((4096,), 0.5 * (rank + 1)).bfloat16().to(dev)   # exactly representable values
    dist.all_reduce(b)
    ok("all_reduce_bf16", torch.equal(b.cpu().float(), torch.full((4096,), 0.5 * tri)))
    x = (torch.arange(16.0) if rank == 0 else torch.zeros(16)).to(dev)
    dist.broadcast(x, src=0)
    ok("broadcast", torch.equal(x.cpu(), torch.arange(16.0)))
    out = torch.empty(world * 8).to(dev)
    dist.all_gather_into_tensor(out, torch.full((8,), float(rank)).to(dev))
    ok("all_gather_into_tensor", torch.equal(out.cpu(), torch.arange(world).repeat_interleave(8).float()))
    lst = [torch.empty(3).to(dev) for _ in range(world)]
    dist.all_gather(lst, torch.full((3,), float(rank * 10)).to(dev))
    ok("all_gather", all(torch.equal(lst[r].cpu(), torch.full((3,), float(r * 10))) for r in range(world)))
    inp = torch.arange(world * 4, dtype=torch.float32).to(dev)
    rs = torch.empty(4).to(dev)
    dist.reduce_scatter_tensor(rs, inp)
    ok("reduce_scatter_tensor", torch.equal(rs.cpu(), world * torch.arange(rank * 4, rank * 4 + 4, dtype=torch.float32)))
    ins = [torch.full((6,), float(rank + 1 + r)).to(dev) for r in range(world)]
    rl = torch.empty(6).to(dev)
    dist.reduce_scatter(rl, ins)
    ok("reduce_scatter", torch.equal(rl.cpu(), torch.full((6,), float(sum(k + 1 + rank for k in range(world))))))
    rd = torch.full((7,), float(rank + 1)).to(dev)
    dist.reduce(rd, dst=world - 1)
    ok("reduce", rank != world - 1 or torch.equal(rd.cpu(), torch.full((7,), tri)))
    # all_to_all_single, equal splits: row block r of rank k goes to rank r
    a2a_in = (torch.arange(world * 2, dtype=torch.float32).view(world, 2) + 100 * rank).reshape(-1).to(dev)
    a2a_out = torch.empty(world * 2).to(dev)
    dist.all_to_all_single(a2a_out, a2a_in)
    exp = torch.cat([torch.arange(rank * 2, rank * 2 + 2, dtype=torch.float32) + 100 * k for k in range(world)])
    ok("all_to_all_single", torch.equal(a2a_out.cpu(), exp))
    if world > 1:   # send / recv around a ring
        msg = torch.full((9,), float(rank)).to(dev)
        got = torch.empty(9).to(dev)
        if rank % 2 == 0:
            dist.send(msg, (rank + 1) % world)
            dist.recv(got, (rank - 1) % world)
        else:
            dist.recv(got, (rank - 1) % world)
            dist.send(msg, (rank + 1) % world)
        ok("send_recv", torch.equal(got.cpu(), torch.full((9,), float((rank - 1) % world))))
    # coalescing: two all-reduces issued as one group
    backend = dist.group.WORLD._get_backend(dev)
    c1, c2 = torch.full((5,), 1.0).to(dev), torch.full((3,), float(rank)).to(dev)
    backend._group_start()
    w1 = dist.all_reduce(c1, async_op=True)
    w2 = dist.all_reduce(c2, async_op=True)
    backend._group_end()
    w1.wait()
    w2.wait()
    ok("coalesced_all_reduce", torch.equal(c1.cpu(), torch.full((5,), float(world))) and
       torch.equal(c2.cpu(), torch.full((3,), float(sum(range(world))))))
    import torch_gcu.distributed as gd
    o = torch.empty(5).to(dev)
    gd.all_reduce_outplace(o, torch.ones(5).to(dev))
    ok("all_reduce_outplace", torch.equal(o.cpu(), torch.full((5,), float(world))))
    ok("get_unique_id", len(gd.get_unique_id()) == 256)
    dist.barrier()
    done.append("barrier")
    return done
