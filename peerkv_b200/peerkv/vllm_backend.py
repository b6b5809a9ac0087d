"""Drop-in for `umallm.peerkv.vllm_backend` (PeerKV umallm/peerkv/vllm_backend.py:42-125):
a vLLM attention impl that keeps the peer KV pages ON the peer GPUs and runs the
compute-follows-KV decode there, merging on the home GPU.

Same names and contract as the reference: `PeerKVFusedAttentionImpl` with
`set_peer_kv(peer_cache, peer_base)`, `_try_fused` (returns None to fall back),
`forward`; `register_peerkv_fused()`.  Correct-or-fallback: decode-only batches with
head size 128 take the fused path, anything else -- prefill, chunked batches, a
missing peer cache, any exception -- defers to the parent FlashAttention impl.

Written against the vLLM that is installed here (0.22: `forward(layer, query, key,
value, kv_cache, attn_metadata, output, output_scale=None, output_block_scale=None)`,
KV-cache update done by the caller, metadata fields `num_actual_tokens`,
`max_query_len`, `seq_lens`, `block_table`); the reference targets 0.8.5's 7-argument
forward.  `peer_cache` / `peer_base` may be lists (one per extra GPU).
"""
from __future__ import annotations

import logging
import math
import os

import torch

from .. import metrics
from .paged import paged_cfk_decode

logger = logging.getLogger("peerkv.attn")

try:
    from vllm.v1.attention.backends.flash_attn import FlashAttentionImpl
    _HAVE_VLLM = True
except Exception:  # noqa: BLE001 - vLLM absent or not importable on this host
    FlashAttentionImpl = object  # type: ignore
    _HAVE_VLLM = False


class PeerKVFusedAttentionImpl(FlashAttentionImpl):
    """FlashAttention impl whose decode phase runs on the GPUs that hold the KV."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._init_peerkv()

    def _init_peerkv(self):
        self._peer_cache = None            # [2, nb_p, bs, HKV, D] on a peer GPU, or a list of them
        self._peer_base = 1 << 30          # global block id >= this -> peer (or a list of thresholds)
        self._splits = int(os.environ.get("PEERKV_SPLITS", 16))   # accepted for compatibility, unused
        self._scale_override = None
        self._point = "compute_follows_kv"  # operating point: the sharded path, or "copyback"
        self._c_local = self._c_scratch = 0
        self._stager = None
        self.fused_calls = 0
        self.copyback_calls = 0
        self.fallback_calls = 0

    def set_peer_kv(self, peer_cache, peer_base) -> None:
        """The allocator hands this layer its peer paged KV cache(s) and the global
        block-id threshold(s) at/above which blocks live on the peer(s)."""
        self._peer_cache = peer_cache
        self._peer_base = list(peer_base) if isinstance(peer_base, (list, tuple)) else int(peer_base)

    def set_scratch(self, c_local: int, c_scratch: int) -> None:
        """The allocator tells this layer that its local tensor ends in c_scratch staging blocks."""
        self._c_local, self._c_scratch = int(c_local), int(c_scratch)

    def set_operating_point(self, point) -> None:
        """What the policy decided for the running requests (elastic_policy.OperatingPoint or
        its value): compute-follows-KV on the peers, or copy-back when the peers are busy
        (umallm/elastic_policy.py:346-350).  Anything else takes the stock kernel."""
        self._point = getattr(point, "value", point)

    # --- the decode fast path ------------------------------------------------ #
    def _try_fused(self, query, kv_cache, attn_metadata):
        """O shaped [num_seqs, H, D] from the multi-GPU op, or None to signal fallback."""
        if self._peer_cache is None or attn_metadata is None:
            return None
        try:
            bt = getattr(attn_metadata, "block_table", None)
            seq_lens = getattr(attn_metadata, "seq_lens", None)
            if bt is None or seq_lens is None or kv_cache is None or kv_cache.dim() != 5:
                return None
            if getattr(attn_metadata, "use_cascade", False):
                return None
            q = query
            if q.dim() == 2:                               # a single [H, D] token
                q = q.unsqueeze(0)
            if q.dim() != 3:
                return None
            n_act = getattr(attn_metadata, "num_actual_tokens", q.shape[0])
            q = q[:n_act]
            num_tokens, H, D = q.shape
            bt2 = bt if bt.dim() == 2 else bt.unsqueeze(0)
            num_seqs = bt2.size(0)
            max_q = getattr(attn_metadata, "max_query_len", 1)
            if D != 128 or num_tokens != num_seqs or max_q != 1:
                return None                                # prefill / chunked batch: defer
            if q.dtype not in (torch.float16, torch.bfloat16) or kv_cache.dtype != q.dtype:
                return None                                # fp8 caches of vLLM use other scales
            scale = self._scale_override or getattr(self, "scale", None) or 1.0 / math.sqrt(D)
            if self._point == "copyback":
                return self._copyback(q, kv_cache, bt2, seq_lens[:num_seqs], float(scale))
            if self._point != "compute_follows_kv":
                return None
            return paged_cfk_decode(q, kv_cache, self._peer_cache, bt2, seq_lens[:num_seqs],
                                    self._peer_base, scale=float(scale), splits=self._splits)
        except Exception as e:  # noqa: BLE001 - any surprise -> safe fallback
            logger.warning("PeerKV fused decode declined: %s", e)
            return None

    def _copyback(self, q, kv_cache, bt, seq_lens, scale):
        """Peer blocks staged into the local tensor's scratch tail, then a one-GPU decode."""
        if self._c_scratch <= 0 or kv_cache.shape[1] != self._c_local + self._c_scratch:
            return None                                    # no staging area: defer
        from .staging import PeerKVStager, StagingLayout, copyback_decode
        peers = self._peer_cache if isinstance(self._peer_cache, (list, tuple)) else [self._peer_cache]
        if self._stager is None:
            lay = StagingLayout(self._c_local, self._c_scratch, [p.shape[1] for p in peers], kv_cache.shape[2],
                                kv_cache.shape[3], kv_cache.shape[4], str(kv_cache.device),
                                [str(p.device) for p in peers])
            self._stager = PeerKVStager(lay, max_batch=max(256, bt.shape[0]), max_blocks_per_seq=max(4096, bt.shape[1]))
        out = copyback_decode(q, kv_cache, peers, bt, seq_lens, self._stager, scale)
        self.copyback_calls += 1
        metrics.ATTN_CALLS.labels(path="copyback").inc()
        return out

    # --- vLLM hooks ----------------------------------------------------------- #
    def do_kv_cache_update(self, layer, key, value, kv_cache, slot_mapping):
        """vLLM calls this before `forward` to store the new tokens' K/V.  With peer caches
        set, a token whose block lives on a peer GPU must be written there: one library
        kernel routes every token to its owner (the stock op only knows the local tensor)."""
        if self._peer_cache is None or kv_cache is None or kv_cache.dim() != 5 \
                or kv_cache.dtype not in (torch.float16, torch.bfloat16) or key.dtype != kv_cache.dtype:
            return super().do_kv_cache_update(layer, key, value, kv_cache, slot_mapping)
        from .kv_alloc import sharded_kv_append
        peers = self._peer_cache if isinstance(self._peer_cache, (list, tuple)) else [self._peer_cache]
        bases = self._peer_base if isinstance(self._peer_base, (list, tuple)) else [self._peer_base]
        n = slot_mapping.shape[0]                     # key / value may be padded beyond it
        H, D = kv_cache.shape[3], kv_cache.shape[4]
        sharded_kv_append(key[:n].view(n, H, D), value[:n].view(n, H, D), slot_mapping, kv_cache, peers, bases)
        metrics.KV_APPEND_TOKENS.inc(n)

    def forward(self, layer, query, key, value, kv_cache, attn_metadata, output=None,
                output_scale=None, output_block_scale=None):
        O = None
        if output_scale is None and output_block_scale is None:
            O = self._try_fused(query, kv_cache, attn_metadata)
        if O is None:
            self.fallback_calls += 1
            metrics.ATTN_CALLS.labels(path="fallback").inc()
            return super().forward(layer, query, key, value, kv_cache, attn_metadata, output,
                                   output_scale, output_block_scale)
        if self._point == "compute_follows_kv":
            self.fused_calls += 1
            metrics.ATTN_CALLS.labels(path="sharded").inc()
        if output is not None:
            n = O.shape[0]                                  # rows past n are vLLM's padding
            flat = output if query.dim() != 2 else output.unsqueeze(0)
            flat[:n].view(n, -1).copy_(O.reshape(n, -1).to(output.dtype))
            return output
        O = O[0] if query.dim() == 2 else O
        return O.to(query.dtype)


def register_peerkv_fused() -> bool:
    """Route FlashAttentionBackend.get_impl_cls to PeerKVFusedAttentionImpl; True if patched."""
    from .register import install_cfk
    return install_cfk()
