"""Tensor-parallel exchange over peer memory: the backend's own kernels in place of the
collective library for the row-parallel projections of a decoder layer.

Where the reference's tensor-parallel users call `all_reduce` on the "eccl" group after every
row-parallel projection (reference: torch_gcu/csrc/distributed/ProcessGroupECCL.cpp:2869-2926),
this class gives them the fused form: the projection writes its partial product into a
peer-visible buffer, and ONE kernel per projection does reduce-scatter + residual add + RMSNorm +
all-gather with plain peer loads and stores (`reduce_norm`), bracketed by counting signal / wait
kernels (`sync`). No collective kernel runs, so none competes with the GEMMs for SMs, and the
residual add and the normalisation run on each rank's 1 / world of the rows instead of on all of
them on every rank.

One process drives one GPU. The buffers are mapped once, when the object is made: one symmetric
allocation per rank laid out as [control block | partial 0 | partial 1 | gathered], the IPC
handles exchanged through the group's store.
"""
import itertools

import torch
import torch.distributed as dist

from torch_gcu import _C

_counter = itertools.count()


class TensorParallelExchange:
    """Buffers and kernels of the exchange for activations of shape (total_rows, hidden).

    scatter=True (prefill): rank r owns rows [r * total_rows / world, (r + 1) * total_rows / world);
    its residual stream has only those rows, and `reduce_norm` gathers the normalised rows on every
    rank. scatter=False (decode, few rows): every rank reduces all rows for itself; nothing is
    gathered and the residual stream stays replicated.
    """

    def __init__(self, total_rows, hidden, dtype=torch.bfloat16, group=None, scatter=True, timeout_s=10.0):
        group = group or dist.group.WORLD
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        assert 1 <= self.world <= 8, "the exchange kernels take up to 8 ranks"
        self.total_rows, self.hidden, self.dtype, self.scatter = total_rows, hidden, dtype, scatter
        self.timeout_s = timeout_s
        if scatter:
            assert total_rows % self.world == 0, "rows must divide by the number of ranks"
            self.rows = total_rows // self.world
            self.row0 = self.rank * self.rows
        else:
            self.rows, self.row0 = total_rows, 0
        esize = torch.empty((), dtype=dtype).element_size()
        act = (total_rows * hidden * esize + 255) // 256 * 256
        ctl = int(_C._tp_control_bytes())
        self._off_control = 0
        self._off_partial = (ctl, ctl + act)
        self._off_gathered = ctl + 2 * act
        nbytes = ctl + 3 * act
        self.device = torch.device("gcu", torch.gcu.current_device())
        local, handle = _C._symm_alloc(nbytes)
        self._buffers = [None] * self.world
        self._buffers[self.rank] = local
        if self.world > 1:
            # the IPC handles travel through the store of the default group
            store = dist.distributed_c10d._get_default_store()
            prefix = "gcu_tp_exchange/%d/" % next(_counter)
            store.set(prefix + str(dist.get_rank()), handle)
            for r in range(self.world):
                if r != self.rank:
                    peer_handle = store.get(prefix + str(dist.get_global_rank(group, r)))
                    self._buffers[r] = _C._symm_open(peer_handle, nbytes)
            # nobody signals into a control block that its owner has not zeroed yet, and ranks that
            # reach their first wait seconds apart (weights are still being built) meet here first
            dist.barrier(group)

        def view(off):
            n = total_rows * hidden * esize
            return local[off:off + n].view(dtype).view(total_rows, hidden)
        self.partial = (view(self._off_partial[0]), view(self._off_partial[1]))
        self.gathered = view(self._off_gathered)

    def sync(self, channel=0, signal=True, wait=True):
        """Counting signal and / or wait between the ranks on the current stream; both = a barrier.
        What this rank wrote earlier on the stream is visible to a peer once it has waited."""
        if self.world > 1:
            _C._tp_sync(self._buffers, self.rank, self._off_control, channel, signal, wait, self.timeout_s)

    def reduce_norm(self, partial, residual, residual_out, weight, eps=1e-6, normalise=True):
        """Sum the rows this rank owns over every rank's partial buffer `partial` (0, 1 or None for
        nothing to sum), add `residual` (rows, hidden), round once into `residual_out`, RMS-normalise
        with `weight`, and store the rows into the gathered buffer of every rank (scatter mode) or of
        this rank (replicated mode). Order it between two `sync` calls."""
        _C._tp_reduce_norm(self._buffers, self.rank, None if partial is None else self._off_partial[partial],
                           self._off_gathered, residual, residual_out, weight if normalise else None, self.row0,
                           self.total_rows, eps, normalise, self.scatter)
