"""Drop-in for `umallm.peer_parallel_attn` (PeerKV umallm/peer_parallel_attn.py):
same names, shapes and conventions, computed by the sm_100a kernels.

  flash_partial(q, K, V, scale)            -> (O in q.dtype, lse fp32)      :46-71
  merge_partial(O0, lse0, O1, lse1)        -> (O fp32, lse)                 :74-80
  peer_parallel_attention(q, kv_shards, scale) -> O in q.dtype on q's device :143-173

q is (B, H, Lq, D); K, V are (B, Hkv, Tk, D) and may live on other GPUs: each
shard's partial is computed on the GPU that holds it and only (O, lse) moves.
Differences from the reference, by design: D must be 128 and tensors fp16/bf16 on
CUDA (there is no CPU or fp32-input path); partials stay fp32 until the final
cast, and the N partials are merged in one pass instead of a left fold.
"""
from __future__ import annotations

import math

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


def _partial_f32(q, K, V, scale):
    """fp32 (O (B,H,Lq,D), lse (B,H,Lq)) of one shard on K's device."""
    import torch
    if K.dim() != 4 or K.shape != V.shape:
        raise PeerKVError("K and V must both be (B, Hkv, Tk, D)")
    if K.dtype != q.dtype:
        raise PeerKVError(f"q ({q.dtype}) and K ({K.dtype}) must share a dtype")
    qr, B, Lq = _rows(q)
    H, D = qr.shape[1], qr.shape[2]
    if Lq == 1:
        o, lse = ops.partial_contiguous(qr, K, V, scale)
    else:
        # every query position is its own "sequence" over the same KV page
        view = ops.contiguous_view(K, V)
        bt = torch.arange(B, device=q.device, dtype=torch.int32).repeat_interleave(Lq).view(-1, 1)
        sl = torch.full((B * Lq,), K.shape[2], dtype=torch.int32, device=q.device)
        import ctypes as C
        from . import _lib
        a = ops.make_args(ops._check_q(qr), view, bt, 1, sl, scale)
        o = torch.empty(B * Lq, H, D, dtype=torch.float32, device=q.device)
        lse = torch.empty(B * Lq, H, dtype=torch.float32, device=q.device)
        shard = ops.get_shard(q.device, B * Lq, H)
        _lib.check(_lib.lib().pkv_decode_partial(shard._h, C.byref(a), o.data_ptr(), lse.data_ptr(),
                                                 ops._stream(q.device)))
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
