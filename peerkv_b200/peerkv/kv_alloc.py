"""The allocator side of the sharded decode path inside vLLM: place a share of every
layer's KV blocks on peer GPUs, route the KV-cache writes to the GPU that owns the block,
and hand the peer caches to the attention impl.

This is the piece the reference names as missing for `vllm serve`
(PeerKV umallm/peerkv/register.py:21-27); its template is the reference's copy-back
allocator patch, umallm/vllm_integration/peer_kv_alloc.py:46-131 (wrap
`GPUModelRunner.initialize_kv_cache`, split each layer's tensor, publish the layout) and
umallm/vllm_integration/peerkv_staging.py:36-73 (`PeerKVLayout`, `alloc_split_kv`).
Differences: N peer GPUs instead of one, no scratch region (nothing is copied back: the
peers compute on their blocks in place), and the append is one kernel that writes a new
token straight into its owner's pool.

Block ids stay vLLM's: the block manager hands out 0 .. num_blocks-1 knowing nothing of
placement; ids below `c_local` live in the home GPU's tensor at the same index, ids in
[bases[d], bases[d+1]) in peer d's tensor at index id - bases[d].
"""
from __future__ import annotations

import ctypes as C
import functools
import logging
import os
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .. import _lib, ops
from .._lib import PeerKVError, check

logger = logging.getLogger("peerkv.alloc")
_DEFAULT_TARGET = "vllm.v1.worker.gpu_model_runner:GPUModelRunner.initialize_kv_cache"


@dataclass
class PeerKVLayout:
    """Where the blocks of one layer's KV cache live."""
    c_local: int                      # blocks on the home GPU (ids 0 .. c_local-1)
    c_peers: List[int]                # blocks on each peer GPU, in id order after the local ones
    block_size: int
    num_kv_heads: int
    head_size: int
    local_device: str = "cuda:0"
    peer_devices: List[str] = field(default_factory=lambda: ["cuda:1"])

    @property
    def peer_bases(self) -> List[int]:
        """First block id of each peer: the thresholds `set_peer_kv` and `paged_cfk_decode` take."""
        out, b = [], self.c_local
        for c in self.c_peers:
            out.append(b)
            b += c
        return out

    @property
    def peer_base(self) -> int:
        return self.c_local

    @property
    def num_blocks(self) -> int:
        return self.c_local + sum(self.c_peers)

    def owner(self, block_id: int):
        """(device index in [home, peers...], local block index) of a block id."""
        bases = [0] + self.peer_bases
        d = max(i for i, b in enumerate(bases) if block_id >= b)
        return d, block_id - bases[d]

    @classmethod
    def split(cls, num_blocks: int, block_size: int, num_kv_heads: int, head_size: int,
              peer_fraction: float, local_device: str, peer_devices: Sequence[str]) -> "PeerKVLayout":
        """`peer_fraction` of the blocks go to the peers, evenly (the remainder to the first ones)."""
        n = len(peer_devices)
        c_peer = int(num_blocks * peer_fraction)
        per = [c_peer // n + (1 if i < c_peer % n else 0) for i in range(n)]
        return cls(num_blocks - c_peer, per, block_size, num_kv_heads, head_size, str(local_device),
                   [str(d) for d in peer_devices])


def alloc_split_kv(layout: PeerKVLayout, dtype=torch.bfloat16):
    """(local [2, c_local, bs, H, D] on the home GPU, [peer [2, c_peer_d, bs, H, D] on each peer])."""
    shape = (layout.block_size, layout.num_kv_heads, layout.head_size)
    local = torch.empty(2, layout.c_local, *shape, dtype=dtype, device=layout.local_device)
    peers = [torch.empty(2, c, *shape, dtype=dtype, device=d) for c, d in zip(layout.c_peers, layout.peer_devices)]
    return local, peers


def sharded_kv_append(key: torch.Tensor, value: torch.Tensor, slot_mapping: torch.Tensor, local_cache: torch.Tensor,
                      peer_caches: Sequence[torch.Tensor], peer_bases: Sequence[int],
                      status_word: Optional[torch.Tensor] = None):
    """Writes the new tokens' K/V into the cache block that owns each slot, on whichever
    GPU it lives (one launch on key's GPU; peer pools are written through peer access).
    key / value [n_tokens, Hkv, D]; slot_mapping [n_tokens] int64 (negative = padding)."""
    dev = key.device
    if local_cache.device != dev or slot_mapping.device != dev or value.device != dev:
        raise PeerKVError("key, value, slot_mapping and the local cache must share a GPU")
    if key.dim() != 3 or key.shape != value.shape or key.stride(2) != 1 or key.stride(1) != key.shape[2] \
            or key.stride() != value.stride():
        raise PeerKVError("key / value must be [n_tokens, Hkv, D] with contiguous heads and equal strides")
    if slot_mapping.dtype != torch.int64:
        slot_mapping = slot_mapping.to(torch.int64)
    caches = [local_cache] + list(peer_caches)
    n = len(caches)
    _enable_peer_access(dev, [c.device for c in caches[1:]])
    arr64 = lambda xs: (C.c_int64 * n)(*[int(x) for x in xs])
    ptrs = lambda xs: (C.c_void_p * n)(*xs)
    check(_lib.lib().pkv_kv_append(
        dev.index, key.data_ptr(), value.data_ptr(), key.stride(0), slot_mapping.data_ptr(), slot_mapping.shape[0],
        key.shape[1], key.shape[2], local_cache.shape[2], n, arr64([0] + list(peer_bases)),
        arr64([c.shape[1] for c in caches]), ptrs([c[0].data_ptr() for c in caches]),
        ptrs([c[1].data_ptr() for c in caches]), arr64([c.stride(1) for c in caches]),
        arr64([c.stride(2) for c in caches]), arr64([c.stride(3) for c in caches]),
        status_word.data_ptr() if status_word is not None else None, ops._stream(dev)))


_peer_enabled = set()


def _enable_peer_access(dev: torch.device, others):
    """Kernels on `dev` may store into the others' memory (once per pair)."""
    for o in others:
        if o.index == dev.index or (dev.index, o.index) in _peer_enabled:
            continue
        check(_lib.lib().pkv_enable_peer_access(dev.index, o.index))
        _peer_enabled.add((dev.index, o.index))


def relayout_runner(runner, peer_fraction: float, peer_devices: Sequence[str],
                    scratch_blocks: int = 0) -> List[PeerKVLayout]:
    """Splits every layer's KV tensor of a vLLM model runner (`runner.kv_caches`, each
    [2, num_blocks, bs, H, D] on the home GPU) into a local part and per-peer parts, moves
    the peers' blocks over, replaces the engine's handles by the local part and hands the
    peer caches to every attention impl that has `set_peer_kv`.  With scratch_blocks > 0 the
    local part gets that many extra blocks at its tail: the staging area of the copy-back
    corner (staging.PeerKVStager), which the impl uses when the peers may not compute."""
    kv_caches = getattr(runner, "kv_caches", None)
    if not kv_caches:
        raise PeerKVError("runner.kv_caches not found")
    impls = attention_impls(runner)
    layouts = []
    for li, kv in enumerate(kv_caches):
        if kv.dim() != 5 or kv.shape[0] != 2:
            raise PeerKVError(f"layer {li}: expected a [2, num_blocks, bs, H, D] cache, got {tuple(kv.shape)}")
        _, nb, bs, H, D = kv.shape
        lay = PeerKVLayout.split(nb, bs, H, D, peer_fraction, kv.device, peer_devices)
        local, peers = alloc_split_kv(lay, kv.dtype)
        if scratch_blocks > 0:
            local = torch.empty(2, lay.c_local + scratch_blocks, bs, H, D, dtype=kv.dtype, device=kv.device)
        local[:, :lay.c_local].copy_(kv[:, :lay.c_local])
        for base, c, pk in zip(lay.peer_bases, lay.c_peers, peers):
            pk.copy_(kv[:, base:base + c])
        kv_caches[li] = local
        if li < len(impls):
            mod, impl = impls[li]
            impl.set_peer_kv(peers, lay.peer_bases)
            if scratch_blocks > 0 and hasattr(impl, "set_scratch"):
                impl.set_scratch(lay.c_local, scratch_blocks)
            bound = getattr(mod, "kv_cache", None)           # vLLM binds the tensor into the layer too
            if isinstance(bound, list):
                for i in range(len(bound)):
                    bound[i] = local
            elif isinstance(bound, torch.Tensor):
                mod.kv_cache = local
        layouts.append(lay)
        del kv
    if layouts:
        lay = layouts[0]
        os.environ["PEERKV_C_LOCAL"] = str(lay.c_local)
        os.environ["PEERKV_C_PEER"] = ",".join(str(c) for c in lay.c_peers)
        os.environ["PEERKV_BLOCK"] = str(lay.block_size)
        os.environ["PEERKV_LOCAL_DEV"] = lay.local_device
        os.environ["PEERKV_PEER_DEV"] = ",".join(lay.peer_devices)
    torch.cuda.empty_cache() if torch.cuda.is_available() else None
    logger.info("PeerKV: %d layers re-laid out; %.0f%% of the blocks on %s", len(layouts), peer_fraction * 100,
                ", ".join(str(d) for d in peer_devices))
    return layouts


def attention_impls(runner):
    """(module, impl) of every attention layer whose impl takes peer caches, in layer order."""
    out = []
    model = getattr(runner, "model", None)
    if model is None:
        return out
    for m in model.modules():
        impl = getattr(m, "impl", None)
        if impl is not None and hasattr(impl, "set_peer_kv"):
            out.append((m, impl))
    return out


def _resolve(spec: str):
    import importlib
    modpath, _, qual = spec.partition(":")
    owner = importlib.import_module(modpath)
    parts = qual.split(".")
    for p in parts[:-1]:
        owner = getattr(owner, p)
    return owner, parts[-1]


def patch_peer_kv_allocation(peer_fraction: float = 0.5, peer_devices: Sequence[str] = ("cuda:1",),
                             target: str = _DEFAULT_TARGET, scratch_blocks: int = 0) -> bool:
    """Wraps the runner's `initialize_kv_cache` so that, right after vLLM has allocated
    its KV cache, `peer_fraction` of each layer's blocks move to `peer_devices`.  Call it
    (together with `install_cfk`) before the engine builds its cache.  True if patched."""
    if not (0.0 < peer_fraction < 1.0) or not peer_devices:
        logger.info("PeerKV: peer_fraction=%.2f -> stock vLLM placement", peer_fraction)
        return False
    try:
        owner, name = _resolve(target)
        orig = getattr(owner, name)
    except Exception as e:  # noqa: BLE001
        logger.info("PeerKV: cannot patch %s (%s)", target, e)
        return False
    if getattr(orig, "_peerkv_wrapped", False):
        return True

    @functools.wraps(orig)
    def wrapper(self, *args, **kwargs):
        ret = orig(self, *args, **kwargs)
        try:
            relayout_runner(self, peer_fraction, peer_devices, scratch_blocks)
        except Exception as e:  # noqa: BLE001 - never break the engine
            logger.error("PeerKV: re-layout failed (%s); the KV cache stays on one GPU", e)
        return ret

    wrapper._peerkv_wrapped = True
    wrapper._peerkv_orig = orig
    setattr(owner, name, wrapper)
    return True


def unpatch_peer_kv_allocation(target: str = _DEFAULT_TARGET) -> bool:
    try:
        owner, name = _resolve(target)
        cur = getattr(owner, name)
    except Exception:  # noqa: BLE001
        return False
    orig = getattr(cur, "_peerkv_orig", None)
    if orig is None:
        return False
    setattr(owner, name, orig)
    return True
