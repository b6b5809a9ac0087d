"""Drop-in for `umallm.peerkv.register` (PeerKV umallm/peerkv/register.py:40-89): one
seam that routes vLLM's FlashAttention backend to the compute-follows-KV impl, and its
revert.  Import-safe without vLLM (both functions then return False).

What this does NOT do (nor does the reference, register.py:21-27): make vLLM's block
manager place a share of each layer's KV pages on the peer GPUs.  Until an allocator
hands real peer caches to `PeerKVFusedAttentionImpl.set_peer_kv`, every layer falls
back to the stock kernel.
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
        logger.info("PeerKV-CFK: vLLM unavailable (%s); install_cfk() is a no-op.", e)
        return False
    if not _HAVE_VLLM or backend is None or not hasattr(backend, "get_impl_cls"):
        logger.warning("PeerKV-CFK: no FlashAttentionBackend.get_impl_cls seam found.")
        return False
    orig = backend.__dict__.get("get_impl_cls", None) or backend.get_impl_cls

    def _impl_cls():
        return PeerKVFusedAttentionImpl

    patched = staticmethod(_impl_cls)
    _impl_cls._peerkv_orig = orig  # type: ignore[attr-defined]
    backend.get_impl_cls = patched
    _DONE = True
    logger.info("PeerKV-CFK: FlashAttentionBackend.get_impl_cls -> PeerKVFusedAttentionImpl")
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
