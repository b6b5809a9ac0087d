"""Drop-in for `umallm.peerkv.fused_attn` (PeerKV umallm/peerkv/fused_attn.py).

  peer_fused_attn(q, K_local, V_local, K_peer, V_peer, scale=None, splits=16) -> O   :62-80
  reference_attn(q, K_full, V_full, scale=None) -> O                                 :83-99
  load_fused_attn()                                                                  :32-46

Shapes as in the reference: q [H, D] on the local GPU, K/V_local [HKV, Tl, D] there,
K/V_peer [HKV, Tp, D] on the peer GPU (None / empty disables it), result [H, D] on
the local GPU.  fp16 or bf16 (the reference is fp16 only), D = 128.  `splits` is
accepted and ignored: the split-K factor is chosen by the persistent grid.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import _lib, ops
from ..group import group_for


def load_fused_attn(verbose: bool = False):
    """Returns the loaded C-ABI library (the reference JIT-compiles here; this one
    is built ahead of time by `python -m peerkv_b200.build`)."""
    return _lib.lib()


def peer_fused_attn(q: torch.Tensor,
                    K_local: torch.Tensor, V_local: torch.Tensor,
                    K_peer: Optional[torch.Tensor] = None,
                    V_peer: Optional[torch.Tensor] = None,
                    scale: Optional[float] = None,
                    splits: int = 16) -> torch.Tensor:
    """Multi-device compute-follows-KV attention; single-GPU when the peer is absent."""
    if q.dim() != 2:
        raise _lib.PeerKVError("q must be [H, D]")
    H, D = q.shape
    if D != 128:
        raise _lib.PeerKVError("this kernel requires head_dim D == 128")
    if K_local.dim() != 3 or V_local.dim() != 3:
        raise _lib.PeerKVError("K/V_local must be [HKV, Tl, D]")
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    q3 = q.unsqueeze(0)
    if K_peer is None or K_peer.numel() == 0:
        return ops.decode_contiguous(q3, K_local.unsqueeze(0), V_local.unsqueeze(0), scale)[0]
    if K_peer.device == q.device:
        o0, l0 = ops.partial_contiguous(q3, K_local.unsqueeze(0), V_local.unsqueeze(0), scale)
        o1, l1 = ops.partial_contiguous(q3, K_peer.unsqueeze(0), V_peer.unsqueeze(0), scale)
        return ops.merge_partials(torch.stack([o0, o1]), torch.stack([l0, l1]), q.dtype)[0]
    grp = group_for([q.device, K_peer.device], 1, H)
    return grp.decode_contiguous(q3, [(K_local.unsqueeze(0), V_local.unsqueeze(0)),
                                      (K_peer.unsqueeze(0), V_peer.unsqueeze(0))], scale)[0]


def reference_attn(q: torch.Tensor, K_full: torch.Tensor, V_full: torch.Tensor,
                   scale: Optional[float] = None) -> torch.Tensor:
    """Single-device GQA attention in fp32 torch math for numerics checks (not a
    product path).  q [H, D]; K/V_full [HKV, T, D] -> [H, D] in q.dtype."""
    H, D = q.shape
    HKV = K_full.shape[0]
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    g = H // HKV
    s = torch.einsum("hgd,htd->hgt", q.float().view(HKV, g, D), K_full.float()) * scale
    o = torch.einsum("hgt,htd->hgd", torch.softmax(s, dim=-1), V_full.float())
    return o.reshape(H, D).to(q.dtype)
