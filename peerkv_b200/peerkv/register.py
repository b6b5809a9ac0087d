"""Drop-in for `umallm.peerkv.register` (PeerKV umallm/peerkv/register.py:40-89): one
seam that routes vLLM's FlashAttention backend to the compute-follows-KV impl, and its
revert.  Import-safe without vLLM (both functions then return False).

Placing a share of each layer's KV pages on the peer GPUs is the other half: see
kv_alloc.patch_peer_kv_allocation (the reference leaves it open, register.py:21-27).
Until peer caches reach `PeerKVFusedAttentionImpl.set_peer_kv`, every layer falls back
to the stock kernel.
"""
from __future__ import annotations

import logging

logger = logging.getLogger("peerkv.attn")
_DONE = False


def _backend():
    from vllm.v1.attention.backends import flash_attn as v1fa
    return getattr(v1fa, "FlashAttentionBackend", None)


def install_cfk() -> bool:
    """Override FlashAttentionBackend.get_impl_cls once; idempotent."""
    global _DONE
    if _DONE:
        return True
    try:
        backend = _backend()
        from .vllm_backend import PeerKVFusedAttentionImpl, _HAVE_VLLM
    except Exception as e:  # noqa: BLE001
        logger.info("sharded decode not installed: vLLM cannot be imported (%s)", e)
        return False
    if not _HAVE_VLLM or backend is None or not hasattr(backend, "get_impl_cls"):
        logger.warning("sharded decode not installed: this vLLM has no FlashAttentionBackend.get_impl_cls")
        return False
    orig = backend.__dict__.get("get_impl_cls", None) or backend.get_impl_cls

    def _impl_cls():
        return PeerKVFusedAttentionImpl

    patched = staticmethod(_impl_cls)
    _impl_cls._peerkv_orig = orig  # type: ignore[attr-defined]
    backend.get_impl_cls = patched
    _DONE = True
    logger.info("sharded decode installed: FlashAttention layers now build PeerKVFusedAttentionImpl")
    return True


def uninstall_cfk() -> bool:
    """Restore vLLM's own get_impl_cls."""
    global _DONE
    try:
        backend = _backend()
        cur = backend.__dict__.get("get_impl_cls", None)
        fn = getattr(cur, "__func__", cur)
        orig = getattr(fn, "_peerkv_orig", None)
        if backend is not None and orig is not None:
            backend.get_impl_cls = orig
            _DONE = False
            return True
    except Exception:  # noqa: BLE001
        pass
    return False
