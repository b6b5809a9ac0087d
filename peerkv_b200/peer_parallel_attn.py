"""Drop-in for `umallm.peer_parallel_attn` (PeerKV umallm/peer_parallel_attn.py):
same names, shapes and conventions, computed by the sm_100a kernels.

  flash_partial(q, K, V, scale)            -> (O in q.dtype, lse fp32)      :46-71
  merge_partial(O0, lse0, O1, lse1)        -> (O fp32, lse)                 :74-80
  peer_parallel_attention(q, kv_shards, scale) -> O in q.dtype on q's device :143-173
  ring_prefill_attention(shards, scale)        -> [O_i] causal, sharded by position :112-140

q is (B, H, Lq, D); K, V are (B, Hkv, Tk, D) and may live on other GPUs: each
shard's partial is computed on the GPU that holds it and only (O, lse) moves.
Differences from the reference, by design: D must be 128 and tensors fp16/bf16 on
CUDA (there is no CPU or fp32-input path); partials stay fp32 until the final
cast, and the N partials are merged in one pass instead of a left fold.
"""
from __future__ import annotations

try:
    import torch  # noqa: F401
    HAS_TORCH = True
except Exception:  # pragma: no cover
    HAS_TORCH = False

from . import ops
from ._lib import PeerKVError


def _rows(q):
    """(B,H,Lq,D) -> ([B*Lq, H, D] contiguous, B, Lq)."""
    if q.dim() != 4:
        raise PeerKVError(f"q must be (B, H, Lq, D); got {tuple(q.shape)}")
    B, H, Lq, D = q.shape
    return q.permute(0, 2, 1, 3).reshape(B * Lq, H, D), B, Lq


def _decode_partial_rows(q_rows, K, V, row_page, row_len, scale):
    """The one call into the library that this module makes for a shard: every row of
    q_rows [R, H, D] is a "sequence" that attends to the first row_len[r] tokens of page
    row_page[r] of the contiguous K/V (B, Hkv, T, D) (one page per batch element).
    Returns fp32 (O [R, H, D], lse [R, H])."""
    import ctypes as C
    import torch
    from . import _lib
    R, H, D = q_rows.shape
    o = torch.empty(R, H, D, dtype=torch.float32, device=q_rows.device)
    lse = torch.empty(R, H, dtype=torch.float32, device=q_rows.device)
    view = ops.contiguous_view(K, V)
    step = 4096                                    # rows per launch (the shard scratch's batch limit)
    for r0 in range(0, R, step):
        r1 = min(R, r0 + step)
        qs = ops._check_q(q_rows[r0:r1])
        bt = row_page[r0:r1].to(torch.int32).contiguous().view(-1, 1)
        sl = row_len[r0:r1].to(torch.int32).contiguous()
        a = ops.make_args(qs, view, bt, 1, sl, scale)
        shard = ops.get_shard(q_rows.device, r1 - r0, H)
        _lib.check(_lib.lib().pkv_decode_partial(shard._h, C.byref(a), o[r0:r1].data_ptr(),
                                                 lse[r0:r1].data_ptr(), ops._stream(q_rows.device)))
    return o, lse


def _partial_f32(q, K, V, scale, causal_diagonal=False):
    """fp32 (O (B,H,Lq,D), lse (B,H,Lq)) of one shard on K's device.  With
    causal_diagonal, query position p of the shard sees keys 0..p of the same shard."""
    import torch
    if K.dim() != 4 or K.shape != V.shape:
        raise PeerKVError("K and V must both be (B, Hkv, Tk, D)")
    if K.dtype != q.dtype:
        raise PeerKVError(f"q ({q.dtype}) and K ({K.dtype}) must share a dtype")
    qr, B, Lq = _rows(q)
    H, D = qr.shape[1], qr.shape[2]
    Tk = K.shape[2]
    if Lq == 1 and not causal_diagonal:
        o, lse = ops.partial_contiguous(qr, K, V, scale)
    else:
        # every query position is its own "sequence" over its batch element's KV page
        row_page = torch.arange(B, device=q.device).repeat_interleave(Lq)
        if causal_diagonal:
            if Lq != Tk:
                raise PeerKVError("the causal diagonal needs as many queries as keys in the shard")
            row_len = torch.arange(1, Lq + 1, device=q.device).repeat(B)
        else:
            row_len = torch.full((B * Lq,), Tk, device=q.device)
        o, lse = _decode_partial_rows(qr, K, V, row_page, row_len, scale)
    o = o.view(B, Lq, H, D).permute(0, 2, 1, 3)
    lse = lse.view(B, Lq, H).permute(0, 2, 1)
    return o, lse


def flash_partial(q, K, V, scale=None):
    """Attention partial over one KV shard, on K's device -> (O, lse); O (B,H,Lq,D)
    in q.dtype, lse (B,H,Lq) fp32; pairs merge exactly with merge_partial."""
    if scale is None:
        scale = 1.0 / (q.shape[-1] ** 0.5)
    if q.device != K.device:
        q = q.to(K.device, non_blocking=True)
    o, lse = _partial_f32(q, K, V, scale)
    return o.to(q.dtype), lse


def merge_partial(O0, lse0, O1, lse1):
    """Exact merge of two (O, lse) partials -> (O fp32, lse)."""
    import torch
    o = torch.stack([O0.float(), O1.float()], 0)
    l = torch.stack([lse0.float(), lse1.float()], 0)
    out, lse = ops.merge_partials(o, l, torch.float32, return_lse=True)
    return out, lse


def peer_parallel_attention(q, kv_shards, scale=None):
    """Exact attention over KV shards resident on (possibly) different GPUs.  The KV
    never moves: q goes to each shard's GPU, fp32 (O, lse) comes back, one merge."""
    import torch
    if not kv_shards:
        raise ValueError("kv_shards must be non-empty")
    dev = q.device
    if scale is None:
        scale = 1.0 / (q.shape[-1] ** 0.5)
    B, H, Lq, D = q.shape
    N = len(kv_shards)
    o_all = torch.empty(N, B, H, Lq, D, dtype=torch.float32, device=dev)
    l_all = torch.empty(N, B, H, Lq, dtype=torch.float32, device=dev)
    remote = []
    for i, (K, V) in enumerate(kv_shards):
        if K.device == dev:
            o, lse = _partial_f32(q, K, V, scale)
            o_all[i].copy_(o)
            l_all[i].copy_(lse)
        else:
            with torch.cuda.device(K.device):
                qd = q.to(K.device, non_blocking=True)
                o, lse = _partial_f32(qd, K, V, scale)
                remote.append((i, o, lse))
    for i, o, lse in remote:                 # a few KB per shard cross the link
        o_all[i].copy_(o, non_blocking=True)
        l_all[i].copy_(lse, non_blocking=True)
    return ops.merge_partials(o_all, l_all, q.dtype)


def ring_prefill_attention(shards, scale=None):
    """Exact causal prefill over a sequence sharded by position (ring / context
    parallelism), the drop-in for umallm/peer_parallel_attn.py:112-140.

    shards: list of (Q, K, V) in sequence order, each (B, H, S_i, D) for a contiguous
    position range, resident on its own GPU.  Query shard i attends to all earlier key
    shards in full and to its own shard causally; as in the reference the earlier shards'
    KV is copied to the later GPU for that.  Returns the outputs O_i on each shard's GPU.

    Built from the decode kernel: a query row is a one-token "sequence" whose length is
    the number of keys it may see, so causality needs no mask.  This reads the shard's KV
    once per query row -- fine for checking a sharded prefill, not a prefill kernel.
    """
    import torch
    if scale is None:
        scale = 1.0 / (shards[0][0].shape[-1] ** 0.5)
    outs = []
    for i, (Qi, Ki, Vi) in enumerate(shards):
        dev = Qi.device
        parts = [_partial_f32(Qi, Ki, Vi, scale, causal_diagonal=True)]
        for j in range(i):
            _, Kj, Vj = shards[j]
            parts.append(_partial_f32(Qi, Kj.to(dev, non_blocking=True), Vj.to(dev, non_blocking=True), scale))
        o = torch.stack([p[0].contiguous() for p in parts])
        l = torch.stack([p[1].contiguous() for p in parts])
        outs.append(ops.merge_partials(o, l, Qi.dtype))
    return outs
