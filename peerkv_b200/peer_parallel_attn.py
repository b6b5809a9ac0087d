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


def _prefill_partial(q, K, V, scale, causal, q_pos0=0, k_pos0=0):
    """The one call into the library for a shard with several query rows: q (B,H,Lq,D),
    K/V (B,Hkv,Tk,D) on the same GPU -> fp32 (O (B,H,Lq,D), lse (B,H,Lq)).  With `causal`
    query row i sees key j iff k_pos0 + j <= q_pos0 + i."""
    import ctypes as C
    import torch
    from . import _lib

    def strided(t):
        ok = t.numel() == 0 or (t.stride(3) == 1 and all(st % 8 == 0 for st in t.stride()[:3]) and t.data_ptr() % 16 == 0)
        return t if ok else t.contiguous()
    q, K, V = strided(q), strided(K), strided(V)
    if K.stride() != V.stride():
        K, V = K.contiguous(), V.contiguous()
    B, H, Lq, D = q.shape
    Hkv, Tk = K.shape[1], K.shape[2]
    o = torch.empty(B, H, Lq, D, dtype=torch.float32, device=q.device)
    lse = torch.empty(B, H, Lq, dtype=torch.float32, device=q.device)
    _lib.check(_lib.lib().pkv_prefill_partial(
        q.device.index, q.data_ptr(), q.stride(0), q.stride(1), q.stride(2),
        K.data_ptr() if Tk else None, V.data_ptr() if Tk else None, K.stride(0), K.stride(1), K.stride(2),
        B, H, Hkv, Lq, Tk, D, ops._DT[q.dtype], float(scale), 1 if causal else 0, int(q_pos0), int(k_pos0),
        o.data_ptr(), lse.data_ptr(), ops._stream(q.device)))
    return o, lse


def _partial_f32(q, K, V, scale, causal_diagonal=False):
    """fp32 (O (B,H,Lq,D), lse (B,H,Lq)) of one shard on K's device.  With
    causal_diagonal, query position p of the shard sees keys 0..p of the same shard.
    One query row per sequence is the decode kernel's case; more rows go to the prefill
    kernel, which reads the shard once per 64 rows instead of once per row."""
    if K.dim() != 4 or K.shape != V.shape:
        raise PeerKVError("K and V must both be (B, Hkv, Tk, D)")
    if K.dtype != q.dtype:
        raise PeerKVError(f"q ({q.dtype}) and K ({K.dtype}) must share a dtype")
    if q.dim() != 4:
        raise PeerKVError(f"q must be (B, H, Lq, D); got {tuple(q.shape)}")
    ops._require_cuda(q, "q")
    ops._same_gpu(K, q.device, "K"); ops._same_gpu(V, q.device, "V")
    B, H, Lq, D = q.shape
    if D != ops.HEAD_DIM or q.dtype not in (__import__("torch").float16, __import__("torch").bfloat16):
        raise PeerKVError(f"q must be fp16 or bf16 with D = {ops.HEAD_DIM}")
    Tk = K.shape[2]
    if causal_diagonal and Lq != Tk:
        raise PeerKVError("the causal diagonal needs as many queries as keys in the shard")
    if Lq == 1:                                   # causal or not, one row sees the whole shard
        qr, _, _ = _rows(q)
        o, lse = ops.partial_contiguous(qr, K, V, scale)
        return o.view(B, 1, H, D).permute(0, 2, 1, 3), lse.view(B, 1, H).permute(0, 2, 1)
    return _prefill_partial(q, K, V, scale, causal_diagonal)


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
    shard_devs = [K.device for K, _ in kv_shards]
    if Lq == 1 and q.is_cuda and any(d != dev for d in shard_devs) \
            and len({d.index for d in shard_devs}) == N and all(d.type == "cuda" for d in shard_devs):
        # Decode with one shard per GPU: the group's protocol -- q pushed into the peers'
        # inboxes by the home kernel, every peer's partial stored straight into the home
        # GPU's slot, merged in the home kernel's tail.  No copy_, no separate merge launch.
        from .group import group_for
        others = [d for d in shard_devs if d != dev]
        grp = group_for([dev] + others, B, H)
        by_dev = {d.index: kv for d, kv in zip(shard_devs, kv_shards)}
        K0 = kv_shards[0][0]
        ordered = []
        for d in grp.devices:
            if d.index in by_dev:
                ordered.append(by_dev[d.index])
            else:                                   # nothing of the KV lives with the query
                z = torch.empty(B, K0.shape[1], 0, D, dtype=q.dtype, device=d)
                ordered.append((z, z))
        out = grp.decode_contiguous(q[:, :, 0], ordered, scale)
        return out.view(B, H, 1, D)
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

    Every (query shard, key shard) pair is one launch of the prefill kernel
    (`pkv_prefill_partial`: 64 query rows per CTA stream the key shard once; the diagonal
    pair is causal), and one merge per query shard folds the partials.
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
