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


class DataParallel:
    def __init__(self, ctx, model, rank: int, world: int, dist=None, connect: bool = True):
        self.ctx, self.model, self.rank, self.world, self.dist = ctx, model, rank, world, dist
        self.connected = False
        if connect and world > 1:
            self.connect()

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

    def reduce_gradients(self, optimizer, scaler):
        """Python-host path: in-place sum all-reduce of every parameter gradient, then a device
        scalar inv_scale / world that the clip and AdamW kernels use as their gradient multiplier
        (mean over ranks with no extra pass over the gradients)."""
        ctx, lib = self.ctx, self.ctx.lib
        for slot in optimizer.slots:
            g = slot.param.grad
            if g is not None:
                ctx.check(lib.gdb200_dp_all_reduce(ctx.backend, g.buffer, g.offset, g.count, g.dtype), "dp_all_reduce")
        ctx.check(lib.gdb200_dp_join(ctx.backend), "dp_join")
        inv = ctx.scratch_empty(F32, (), "inv_scale_over_world")
        ctx.check(lib.gd_backend_scale(ctx.backend, inv.buffer, inv.offset, scaler.scale_state.buffer, scaler.scale_state.offset + 4,
                                       1, F32, 1.0 / self.world), "scale(inv_scale)")
        return inv


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

