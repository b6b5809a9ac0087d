"""Copy-back staging: the fallback corner of the policy (COPYBACK), for when the peers hold
KV blocks but must not be asked to compute (R1-busy).  Drop-in for the engine-independent
core of PeerKV umallm/vllm_integration/peerkv_staging.py:36-131 (`PeerKVLayout`,
`alloc_split_kv`, `PeerKVStager.stage`, `gather_kv`).

The home GPU's tensor has `c_local` real blocks followed by `c_scratch` scratch blocks.
`stage()` copies every peer block that the step's block table names into a scratch block
(over NVLink, by a kernel on the home GPU that reads the peers' pools directly) and returns
a block table that points at the scratch copies; a single-GPU decode over the home tensor
then gives the exact result.  Unlike the reference there is no host round trip (no
`unique`, no `.item()`): slots are ranked on the device, and running out of scratch is a
status bit.  Sharded compute (`paged_cfk_decode`) is the fast path; this one moves the KV
every step and exists so that a busy peer never has to lend its SMs.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .. import _lib, ops
from .._lib import PeerKVError, check
from .kv_alloc import _enable_peer_access


@dataclass
class StagingLayout:
    c_local: int
    c_scratch: int
    c_peers: List[int]
    block_size: int
    num_kv_heads: int
    head_size: int
    local_device: str = "cuda:0"
    peer_devices: List[str] = field(default_factory=lambda: ["cuda:1"])

    @property
    def peer_bases(self) -> List[int]:
        out, b = [], self.c_local
        for c in self.c_peers:
            out.append(b)
            b += c
        return out

    @property
    def peer_base(self) -> int:
        return self.c_local


def alloc_split_kv(layout: StagingLayout, dtype=torch.bfloat16):
    """(home tensor [2, c_local + c_scratch, bs, H, D], [peer tensors [2, c_peer, bs, H, D]])."""
    shape = (layout.block_size, layout.num_kv_heads, layout.head_size)
    local = torch.empty(2, layout.c_local + layout.c_scratch, *shape, dtype=dtype, device=layout.local_device)
    peers = [torch.empty(2, c, *shape, dtype=dtype, device=d) for c, d in zip(layout.c_peers, layout.peer_devices)]
    return local, peers


class PeerKVStager:
    """Stages the peer blocks of a step into the home tensor's scratch region."""

    def __init__(self, layout: StagingLayout, max_batch: int = 256, max_blocks_per_seq: int = 8192):
        self.L = layout
        dev = torch.device(layout.local_device)
        self._status = torch.zeros(1, dtype=torch.int32, device=dev)
        self._rows = torch.zeros(max_batch, dtype=torch.int32, device=dev)
        self._cap = (max_batch, max_blocks_per_seq)
        self._out = torch.zeros(max_batch * max_blocks_per_seq, dtype=torch.int32, device=dev)

    def stage(self, local_kv: torch.Tensor, peer_kvs: Sequence[torch.Tensor], block_table: torch.Tensor,
              seq_lens: torch.Tensor) -> torch.Tensor:
        """Returns the remapped block table [batch, width] (a view of a buffer this object
        owns, valid until the next call).  local_kv's scratch region is overwritten."""
        L = self.L
        dev = local_kv.device
        if isinstance(peer_kvs, torch.Tensor):
            peer_kvs = [peer_kvs]
        bt, sl = ops._meta(block_table, dev, "block_table"), ops._meta(seq_lens, dev, "seq_lens")
        B, W = bt.shape
        if bt.stride(0) != W:
            bt = bt.contiguous()           # the remapped table is written with the same row stride
        if B > self._cap[0] or B * W > self._out.numel():
            raise PeerKVError(f"batch {B} x {W} blocks exceeds this stager ({self._cap[0]} x {self._cap[1]})")
        if local_kv.shape[1] != L.c_local + L.c_scratch:
            raise PeerKVError("the home tensor must hold c_local + c_scratch blocks")
        _enable_peer_access(dev, [p.device for p in peer_kvs])
        n = 1 + len(peer_kvs)
        caches = [local_kv] + list(peer_kvs)
        for c in caches:
            if c.stride(4) != 1 or c[0, 0].numel() and not c[0, 0].is_contiguous():
                raise PeerKVError("blocks must be contiguous [bs, H, D]")
        arr64 = lambda xs: (C.c_int64 * n)(*[int(x) for x in xs])
        ptrs = lambda xs: (C.c_void_p * n)(*xs)
        out = self._out[:B * W].view(B, W)
        check(_lib.lib().pkv_stage_peer_blocks(
            dev.index, bt.data_ptr(), bt.stride(0), sl.data_ptr(), B, L.block_size, n,
            arr64([0] + L.peer_bases), arr64([L.c_local] + [p.shape[1] for p in peer_kvs]),
            ptrs([None] + [p[0].data_ptr() for p in peer_kvs]), ptrs([None] + [p[1].data_ptr() for p in peer_kvs]),
            arr64([0] + [p.stride(1) for p in peer_kvs]), local_kv[0].data_ptr(), local_kv[1].data_ptr(),
            local_kv.stride(1), L.c_local, L.c_scratch, local_kv[0, 0].numel(), local_kv.element_size(),
            out.data_ptr(), self._rows.data_ptr(),
            self._status.data_ptr(), ops._stream(dev)))
        return out

    def status(self) -> int:
        """Reads and clears the status word (synchronises): non-zero = scratch too small or a bad block id."""
        v = int(self._status.item())
        if v:
            self._status.zero_()
        return v


def copyback_decode(query, local_kv, peer_kvs, block_table, seq_lens, stager: PeerKVStager,
                    scale: Optional[float] = None):
    """The COPYBACK corner end to end: stage, then single-GPU decode over the home tensor."""
    bt = stager.stage(local_kv, peer_kvs, block_table, seq_lens)
    return ops.decode_paged(query, local_kv[0], local_kv[1], bt, seq_lens, scale)


@torch.no_grad()
def gather_kv(kv: torch.Tensor, block_table_row: torch.Tensor, n_blocks: int):
    """Test helper: the first n_blocks blocks named by a block-table row as (2, n_blocks*bs, H, D)."""
    ids = block_table_row[:n_blocks].to(kv.device).long()
    sel = kv.index_select(1, ids)
    return sel.reshape(2, -1, kv.shape[3], kv.shape[4])
