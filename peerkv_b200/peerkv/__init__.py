"""Drop-in for `umallm.peerkv` (PeerKV umallm/peerkv/__init__.py:13-15)."""
from __future__ import annotations

__all__ = ["load_fused_attn", "peer_fused_attn", "reference_attn"]

from .fused_attn import load_fused_attn, peer_fused_attn, reference_attn
