"""Drop-in for `umallm.peerkv.paged` (PeerKV umallm/peerkv/paged.py).

  paged_cfk_decode(query, local_cache, peer_cache, block_table, seq_lens, peer_base,
                   scale=None, splits=16) -> [num_seqs, H, D]                    :69-97
  gather_seq(local_cache, peer_cache, block_row, seq_len, peer_base)             :48-66

Block residency convention as in the reference: global id < peer_base lives in
local_cache[*, gid], id >= peer_base in peer_cache[*, gid - peer_base]; only a
sequence's final block may be partial.  Generalised: `peer_cache` may be a list of
caches (one per extra GPU) with `peer_base` a list of ascending thresholds.

Unlike the reference there is no per-sequence Python loop, no .item() and no KV
copy: the block table is split on the device and every GPU's kernel walks its own
pages.  `splits` is accepted and ignored.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..group import group_for


def gather_seq(local_cache, peer_cache, block_row, seq_len: int, peer_base: int):
    """Contiguous (K_local, V_local, K_peer, V_peer) [HKV, T, D] of one sequence, built
    with torch indexing.  Kept for callers that want the materialised shards; the
    decode path below never calls it."""
    bs = local_cache.size(2)
    n_blk = (seq_len + bs - 1) // bs
    row = block_row[:n_blk].to(torch.long)
    pos = torch.arange(n_blk, device=row.device)
    valid = torch.full((n_blk,), bs, device=row.device)
    if n_blk:
        valid[-1] = seq_len - (n_blk - 1) * bs
    is_peer = (row >= peer_base) if peer_cache is not None else torch.zeros_like(row, dtype=torch.bool)

    def cat(cache, ids, n_tok):
        H, D = cache.size(3), cache.size(4)
        if ids.numel() == 0:
            z = cache.new_empty((H, 0, D))
            return z, z
        ids = ids.to(cache.device)
        K = cache[0].index_select(0, ids).reshape(-1, H, D)[:n_tok].permute(1, 0, 2).contiguous()
        V = cache[1].index_select(0, ids).reshape(-1, H, D)[:n_tok].permute(1, 0, 2).contiguous()
        return K, V

    n_loc = int(valid[~is_peer].sum()) if n_blk else 0
    Kl, Vl = cat(local_cache, row[~is_peer], n_loc)
    if peer_cache is None or not bool(is_peer.any()):
        return Kl, Vl, None, None
    Kp, Vp = cat(peer_cache, row[is_peer] - peer_base, int(valid[is_peer].sum()))
    return Kl, Vl, Kp, Vp


def paged_cfk_decode(query: torch.Tensor,
                     local_cache: torch.Tensor,
                     peer_cache,
                     block_table: torch.Tensor,
                     seq_lens: torch.Tensor,
                     peer_base,
                     scale: Optional[float] = None,
                     splits: int = 16) -> torch.Tensor:
    """query [num_seqs, H, D] on the home GPU; local_cache [2, nb_l, bs, HKV, D] there;
    peer_cache [2, nb_p, bs, HKV, D] on the peer GPU (None for single-GPU), or a list
    of such; block_table [num_seqs, max_blk] global ids; seq_lens [num_seqs].
    Returns [num_seqs, H, D] on the home GPU in query.dtype."""
    num_seqs, H, D = query.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    bs = local_cache.size(2)
    peers = [] if peer_cache is None else (list(peer_cache) if isinstance(peer_cache, (list, tuple))
                                           else [peer_cache])
    if not peers:
        return ops.decode_paged(query, local_cache[0], local_cache[1], block_table, seq_lens, scale)
    bases = [0] + (list(peer_base) if isinstance(peer_base, (list, tuple)) else [int(peer_base)])
    caches = [local_cache] + peers
    devs = [c.device for c in caches]
    if len({d.index for d in devs}) != len(devs):
        # shards that share a GPU: split the table, run the partials back to back, merge
        return _same_device(query, caches, block_table, seq_lens, bases, bs, scale)
    grp = group_for(devs, num_seqs, H)
    tables, lens, ev = grp.split_table(block_table, seq_lens, bs, bases)
    pools = [(c[0], c[1]) for c in caches]
    return grp.decode_paged_local(query, pools, tables, lens, scale, after_event=ev)


def _same_device(query, caches, block_table, seq_lens, bases, bs, scale):
    import ctypes as C
    from .. import _lib
    n = len(caches)
    B, W = block_table.shape
    dev = query.device
    bt, sl = ops._meta(block_table, dev, "block_table"), ops._meta(seq_lens, dev, "seq_lens")
    tabs = [torch.zeros(B, W, dtype=torch.int32, device=dev) for _ in range(n)]
    lens = [torch.zeros(B, dtype=torch.int32, device=dev) for _ in range(n)]
    _lib.check(_lib.lib().pkv_split_block_table(
        dev.index, bt.data_ptr(), bt.stride(0), sl.data_ptr(), B, bs, n, 0,
        (C.c_int64 * n)(*bases), (C.c_void_p * n)(*[t.data_ptr() for t in tabs]), W,
        (C.c_void_p * n)(*[t.data_ptr() for t in lens]), ops._stream(dev)))
    H, D = query.shape[1], query.shape[2]
    o = torch.empty(n, B, H, D, dtype=torch.float32, device=dev)
    l = torch.empty(n, B, H, dtype=torch.float32, device=dev)
    for i, c in enumerate(caches):
        ops.partial_paged(query, c[0], c[1], tabs[i], lens[i], scale, o_part=o[i], lse_part=l[i])
    return ops.merge_partials(o, l, query.dtype)
