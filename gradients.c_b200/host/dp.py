"""Batch-sharded data parallelism: one process per GPU, parameters replicated, parameter gradients
summed with NCCL (gdb200_dp_* entries of the backend). The reference has no multi-device code; the
hook points in its host are gd_autograd_accumulate (src/autograd/autograd.c:1072-1083: a leaf
gradient is final) and gd_optimizer_step_amp_clip_lr (src/optim/adamw.c:2163: wait before clipping).

Rendezvous (exchange of the 128-byte NCCL id, barriers) goes through torch.distributed with the
gloo backend; no tensor data moves through torch.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import abi
from .abi import F32


class PeerLeft(RuntimeError):
    """A rank of the job has announced that it is leaving; the ranks that remain must not enter another collective."""

    def __init__(self, ranks):
        super().__init__(f"data-parallel rank(s) {sorted(ranks)} left the job: stopping before the next collective")
        self.ranks = sorted(ranks)


class DataParallel:
    def __init__(self, ctx, model, rank: int, world: int, dist=None, connect: bool = True):
        if world < 1 or not 0 <= rank < world:
            raise ValueError(f"rank {rank} is outside a world of {world}")
        if dist is not None and dist.is_initialized() and (dist.get_world_size() != world or dist.get_rank() != rank):
            # a launcher and a process group that disagree would leave some rank waiting in a collective for ever
            raise ValueError(f"rank {rank} of {world} does not match the process group (rank {dist.get_rank()} of {dist.get_world_size()})")
        self.ctx, self.model, self.rank, self.world, self.dist = ctx, model, rank, world, dist
        self.connected = False
        if connect and world > 1:
            self.connect()

    # ---- departures: a rank leaves only between steps and says so first; the others look before their next launch ----
    def _store(self):
        from torch.distributed import distributed_c10d
        return distributed_c10d._get_default_store()

    def announce_leave(self) -> None:
        """Called by a rank that is about to leave (between steps, nothing of its own in flight)."""
        self._store().set(f"gdb200/left/{self.rank}", "1")

    def departed(self) -> list[int]:
        store = self._store()
        return [r for r in range(self.world) if r != self.rank and store.check([f"gdb200/left/{r}"])]

    def check_peers(self) -> None:
        """Raises PeerLeft when a peer has announced its departure (one round trip to the rendezvous store: call it
        before a step whenever that cost is acceptable, not from inside the step)."""
        gone = self.departed()
        if gone:
            raise PeerLeft(gone)

    def exchange_unique_id(self) -> bytes:
        """Rank 0 creates the NCCL id; every rank returns the same 128 bytes."""
        import torch
        buf = torch.zeros(128, dtype=torch.uint8)
        if self.rank == 0:
            raw = (C.c_ubyte * 128)()
            self.ctx.check(self.ctx.lib.gdb200_dp_unique_id(raw), "dp_unique_id")
            buf = torch.tensor(list(raw), dtype=torch.uint8)
        self.dist.broadcast(buf, src=0)
        return bytes(buf.tolist())

    def connect(self) -> None:
        uid = self.exchange_unique_id()
        raw = (C.c_ubyte * 128).from_buffer_copy(uid)
        self.ctx.check(self.ctx.lib.gdb200_dp_init(self.ctx.backend, raw, self.rank, self.world), "dp_init")
        self.connected = True

    def shard(self, items: list) -> list:
        """Sequences rank, rank + world, ... of the global batch."""
        return items[self.rank::self.world]

    def shard_share(self, batch, pad_token_id: int) -> float:
        """Valid target rows of this rank's batch divided by those of the global batch (counts summed over the
        ranks on the host through the rendezvous group). Every rank must call it once per step."""
        import torch
        t = np.asarray(batch.targets)
        local = float(np.count_nonzero((t >= 0) & (t != pad_token_id)))
        total = torch.tensor([local], dtype=torch.float64)
        self.dist.all_reduce(total)
        return local / float(total[0]) if float(total[0]) > 0 else 1.0

    def reduce_gradients(self, optimizer, loss=None) -> None:
        """Python-host path: in-place sum all-reduce of every parameter gradient, in the optimizer's fixed
        parameter order on every rank (a parameter that received no gradient on this rank contributes zeros, so
        the ranks always issue the same collectives), and of the loss share. With the loss normalised by the
        global row count (shard_share) the sum IS the gradient of the global mean loss: no division by world."""
        ctx, lib = self.ctx, self.ctx.lib
        for slot in optimizer.slots:
            if slot.param.grad is None:
                slot.param.grad = ctx.zeros(ctx.scratch, slot.param.dtype, slot.param.shape, "zero_grad")
            g = slot.param.grad
            ctx.check(lib.gdb200_dp_all_reduce(ctx.backend, g.buffer, g.offset, g.count, g.dtype), "dp_all_reduce")
        if loss is not None:
            ctx.check(lib.gdb200_dp_all_reduce(ctx.backend, loss.buffer, loss.offset, 1, F32), "dp_all_reduce(loss)")
        ctx.check(lib.gdb200_dp_join(ctx.backend), "dp_join")


def split_global_batch(n_seqs: int, world: int) -> list[list[int]]:
    """Indices of the global batch owned by each rank (strided), used by tests and the launcher."""
    return [list(range(r, n_seqs, world)) for r in range(world)]


def balanced_shards(lengths, world: int) -> list[list[int]]:
    """Indices of the global batch per rank such that every rank gets the same number of sequences and nearly the
    same number of tokens: sequences are taken longest first and each goes to the lightest rank that still has room.
    A synchronous step runs at the pace of the heaviest rank, so a token-balanced shard is what keeps the ranks busy."""
    n = len(lengths)
    per = (n + world - 1) // world
    order = sorted(range(n), key=lambda i: (-int(lengths[i]), i))
    shards: list[list[int]] = [[] for _ in range(world)]
    load = [0] * world
    for i in order:
        r = min((r for r in range(world) if len(shards[r]) < per), key=lambda r: (load[r], r))
        shards[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(sh) for sh in shards]

