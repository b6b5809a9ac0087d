"""Several GPUs driven by ONE process (the reference's model: its op takes tensors
on cuda:0 and cuda:1, PeerKV csrc/peer_fused_attn_ext.cu:37-137).

A PeerGroup owns, per GPU, a Shard (split-K scratch) and an Exchange (mailboxes)
created once and mapped into each other with peer access.  A step is:

    peers: one kernel each -- wait for q, partial over    pkv_peer_step
           their shard, push it into the home GPU's slot
           (P2P stores of words that carry the step's epoch)
    home:  one kernel -- push q to the peers the same     pkv_home_step
           way, partial over its own shard, wait for the
           peers' rows, merge

No stream, event or scratch is created per call and the host never blocks.
Calls on one group must come from one thread and, per GPU, one stream.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib, ops
from ._lib import PeerKVError, check


class Exchange:
    """One GPU's mailboxes (q inbox, one partial slot per rank; every word carries its epoch)."""

    def __init__(self, device, rank: int, world: int, max_batch: int, n_q_heads: int):
        self.device = torch.device(device)
        self.rank, self.world = rank, world
        self.max_batch, self.n_q_heads = max_batch, n_q_heads
        h = C.c_void_p()
        check(_lib.lib().pkv_exchange_create(C.byref(h), self.device.index, rank, world, max_batch,
                                             n_q_heads))
        self._h = h

    def export_handle(self) -> bytes:
        buf = C.create_string_buffer(64)
        check(_lib.lib().pkv_exchange_export(self._h, buf))
        return buf.raw

    def import_handle(self, peer_rank: int, handle: bytes):
        buf = C.create_string_buffer(handle, 64)
        check(_lib.lib().pkv_exchange_import(self._h, peer_rank, buf))

    def attach(self, peer: "Exchange"):
        check(_lib.lib().pkv_exchange_attach(self._h, peer.rank, peer._h))

    def status(self) -> int:
        v = C.c_uint32()
        check(_lib.lib().pkv_exchange_status(self._h, ops._stream(self.device), C.byref(v)))
        return int(v.value)

    def epoch(self) -> int:
        v = C.c_uint64()
        check(_lib.lib().pkv_exchange_epoch(self._h, C.byref(v)))
        return int(v.value)

    def capture_begin(self):
        """Before the stream capture of a sequence of steps starts."""
        check(_lib.lib().pkv_exchange_capture_begin(self._h))

    def capture_end(self, stream: int) -> int:
        """Inside the capture, after its last step: adds the node that advances the
        device-resident epoch base.  Returns the number of steps the graph holds."""
        n = C.c_uint64()
        check(_lib.lib().pkv_exchange_capture_end(self._h, stream, C.byref(n)))
        return int(n.value)

    def replayed(self):
        """After every launch of the captured graph: the host's epoch follows."""
        check(_lib.lib().pkv_exchange_replayed(self._h))

    def resync(self, epoch: int):
        """Sets the epoch (every rank passes the same value) after a failed or skipped step."""
        check(_lib.lib().pkv_exchange_resync(self._h, int(epoch)))

    def close(self):
        if getattr(self, "_h", None):
            _lib.lib().pkv_exchange_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class PeerGroup:
    """GPUs of one process; devices[0] is the home GPU (owns q, runs the merge)."""

    def __init__(self, devices: Sequence, max_batch: int, n_q_heads: int, max_pages: int = 0):
        self.devices = [torch.device(d) for d in devices]
        if len({d.index for d in self.devices}) != len(self.devices):
            raise PeerKVError("PeerGroup devices must be distinct GPUs")
        self.world = len(self.devices)
        self.max_batch, self.n_q_heads = max_batch, n_q_heads
        self.shards = [ops.Shard(d, max_batch, n_q_heads) for d in self.devices]
        self.xchg = [Exchange(d, r, self.world, max_batch, n_q_heads) for r, d in enumerate(self.devices)]
        for a in self.xchg:
            for b in self.xchg:
                if a is not b:
                    a.attach(b)
        self._lens = [torch.zeros(max_batch, dtype=torch.int32, device=d) for d in self.devices]
        self._tables = None
        self._max_pages = 0
        if max_pages:
            self._ensure_tables(max_pages)
        self._ev = torch.cuda.Event()

    def _ensure_tables(self, max_pages: int):
        if self._tables is None or self._max_pages < max_pages:
            for d in self.devices:
                torch.cuda.synchronize(d)
            self._max_pages = max_pages
            self._tables = [torch.zeros(self.max_batch, max_pages, dtype=torch.int32, device=d)
                            for d in self.devices]

    # -- one step over per-GPU argument blocks ---------------------------------- #
    def _step(self, q: torch.Tensor, args: List[_lib.DecodeArgs], out: torch.Tensor,
              after_event: Optional[torch.cuda.Event] = None):
        L = _lib.lib()
        home = self.devices[0]
        B = q.shape[0]
        hs = ops._stream(home)
        mask = 0
        for r in range(1, self.world):
            d = self.devices[r]
            with torch.cuda.device(d):
                st = torch.cuda.current_stream(d)
                if after_event is not None:
                    st.wait_event(after_event)
                check(L.pkv_peer_step(self.xchg[r]._h, self.shards[r]._h, C.byref(args[r]), 0, 0,
                                      st.cuda_stream))
            mask |= 1 << r
        check(L.pkv_home_step(self.xchg[0]._h, self.shards[0]._h, C.byref(args[0]), mask,
                              out.data_ptr(), ops._DT[out.dtype], None, hs))
        return out

    def decode_contiguous(self, q: torch.Tensor, shards: List[Tuple[torch.Tensor, torch.Tensor]],
                          scale: Optional[float] = None, out: Optional[torch.Tensor] = None):
        """q [B, Hq, D] on the home GPU; shards[r] = (K, V) [B, Hkv, T_r, D] on devices[r]."""
        q = ops._check_q(q)
        B, Hq, D = q.shape
        scale = 1.0 / math.sqrt(D) if scale is None else scale
        if len(shards) != self.world:
            raise PeerKVError("one (K, V) per GPU of the group is required")
        if q.device != self.devices[0]:
            raise PeerKVError(f"q lives on {q.device}, the group's home GPU is {self.devices[0]}")
        args = []
        for r, (K, V) in enumerate(shards):
            if K.device != self.devices[r]:
                raise PeerKVError(f"shard {r} lives on {K.device}, expected {self.devices[r]}")
            self._lens[r][:B].fill_(K.shape[2])
            args.append(ops.make_args(q, ops.contiguous_view(K, V), None, 1, self._lens[r], scale))
        out = torch.empty_like(q) if out is None else out
        return self._step(q, args, out)

    def decode_paged_local(self, q: torch.Tensor, pools: List[Tuple[torch.Tensor, torch.Tensor]],
                           tables: List[torch.Tensor], lens: List[torch.Tensor],
                           scale: Optional[float] = None, out: Optional[torch.Tensor] = None,
                           after_event: Optional[torch.cuda.Event] = None):
        """Per-GPU pools [n_pages_r, bs, Hkv, D] x2, LOCAL block tables and shard lengths
        that already live on each GPU (the steady state of a sharded KV cache)."""
        q = ops._check_q(q)
        B, Hq, D = q.shape
        scale = 1.0 / math.sqrt(D) if scale is None else scale
        args = []
        if q.device != self.devices[0]:
            raise PeerKVError(f"q lives on {q.device}, the group's home GPU is {self.devices[0]}")
        for r in range(self.world):
            kp, vp = pools[r]
            d = self.devices[r]
            ops._same_gpu(kp, d, f"pool {r}"); ops._same_gpu(vp, d, f"pool {r}")
            tab, ln = ops._meta(tables[r], d, "block table"), ops._meta(lens[r], d, "shard lengths")
            args.append(ops.make_args(q, ops.paged_view(kp, vp), tab, tab.stride(0), ln, scale))
            args[-1]._keep = (tab, ln)
        out = torch.empty_like(q) if out is None else out
        return self._step(q, args, out, after_event)

    def split_table(self, block_table: torch.Tensor, seq_lens: torch.Tensor, page_size: int,
                    bases: Optional[Sequence[int]] = None):
        """Device-side split of a GLOBAL block table (on the home GPU) into this group's
        per-GPU tables and shard lengths, written straight into each GPU's memory.
        bases=None means round robin (id mod N)."""
        B, W = block_table.shape
        self._ensure_tables(W)
        home = self.devices[0]
        bt, sl = ops._meta(block_table, home, "block_table"), ops._meta(seq_lens, home, "seq_lens")
        n = self.world
        tabs = (C.c_void_p * n)(*[t.data_ptr() for t in self._tables])
        lens = (C.c_void_p * n)(*[t.data_ptr() for t in self._lens])
        mode = 1 if bases is None else 0
        b = (C.c_int64 * n)(*([0] * n if bases is None else list(bases)))
        check(_lib.lib().pkv_split_block_table(home.index, bt.data_ptr(), bt.stride(0), sl.data_ptr(),
                                               B, page_size, n, mode, b, tabs, self._max_pages, lens,
                                               ops._stream(home)))
        self._ev.record(torch.cuda.current_stream(home))
        return self._tables, self._lens, self._ev

    def raise_on_status(self):
        for r, d in enumerate(self.devices):
            with torch.cuda.device(d):
                st = self.shards[r].status() | self.xchg[r].status()
            if st:
                raise PeerKVError(f"GPU {d}: device status 0x{st:x}")


_groups = {}


def group_for(devices: Sequence, batch: int, n_q_heads: int) -> PeerGroup:
    devs = tuple(torch.device(d).index for d in devices)
    key = (devs, n_q_heads)
    g = _groups.get(key)
    if g is None or g.max_batch < batch:
        cap = max(64, 1 << max(0, batch - 1).bit_length())
        g = PeerGroup([torch.device("cuda", i) for i in devs], cap, n_q_heads)
        _groups[key] = g
    return g
