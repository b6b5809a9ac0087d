"""One process per GPU (torchrun): the same step as group.PeerGroup, with the
mailboxes shared across processes through CUDA IPC handles that travel over
torch.distributed once, at set-up.  After that no collective runs on the data
path: q is pushed and partials are gathered with P2P stores of epoch-carrying
words by the library's own kernels.

Every rank calls `step(...)` once per decode step, in lockstep: rank `home`
publishes q, computes its own partial and merges; the others compute theirs and
push it.  Epochs count steps, so a rank that skips a step desynchronises the
group (the waits are bounded: a missing q or partial ends as a status bit, not a
hang).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from . import _lib, ops
from ._lib import PeerKVError, check
from .group import Exchange


class DistPeerGroup:
    def __init__(self, device, max_batch: int, n_q_heads: int, home: int = 0, group=None):
        if not dist.is_initialized():
            raise PeerKVError("torch.distributed must be initialised first")
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.home = home
        self.pg = group
        self.shard = ops.Shard(self.device, max_batch, n_q_heads)
        self.xchg = Exchange(self.device, self.rank, self.world, max_batch, n_q_heads)
        handles = [None] * self.world
        dist.all_gather_object(handles, self.xchg.export_handle(), group=group)
        for r, h in enumerate(handles):
            if r != self.rank:
                self.xchg.import_handle(r, h)
        dist.barrier(group=group)

    @property
    def is_home(self) -> bool:
        return self.rank == self.home

    def step(self, args: _lib.DecodeArgs, q: Optional[torch.Tensor] = None,
             out: Optional[torch.Tensor] = None):
        """args describes THIS rank's shard (q inside it is used on the home rank only)."""
        L = _lib.lib()
        st = ops._stream(self.device)
        if self.is_home:
            B = args.batch
            mask = ((1 << self.world) - 1) & ~(1 << self.rank)
            args.q = q.data_ptr()
            check(L.pkv_home_step(self.xchg._h, self.shard._h, C.byref(args), mask, out.data_ptr(),
                                  ops._DT[out.dtype], None, st))
            return out
        check(L.pkv_peer_step(self.xchg._h, self.shard._h, C.byref(args), self.home, 0, st))
        return None

    def status(self) -> int:
        return self.shard.status() | self.xchg.status()

    def barrier(self):
        dist.barrier(group=self.pg)

    # -- a sequence of steps as one CUDA graph per rank (every rank does the same) ------- #
    def capture_begin(self):
        self.xchg.capture_begin()

    def capture_end(self) -> int:
        return self.xchg.capture_end(ops._stream(self.device))

    def replayed(self):
        self.xchg.replayed()

    def resync(self):
        """After an error on any rank: all ranks agree on the largest epoch reached, so the
        next step's epoch words mean the same thing everywhere (a collective; call it on every rank)."""
        t = torch.tensor([self.xchg.epoch()], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.pg)
        self.xchg.resync(int(t.item()))

    def close(self):
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.pg)
        self.xchg.close()
        self.shard.close()
