"""CPU oracle for peer-parallel split-K decode attention.  TEST INFRASTRUCTURE ONLY.

This file restates, in plain fp32 torch-on-CPU, the algorithm of the reference's
own torch implementation of the path.  It is the checker: only the tests, the
smoke entry and the bench's cpu_baseline / reference arm may import it.  The
product package never does.

Each function names the reference lines it follows (paths inside the PeerKV
project):

  flash_partial            umallm/peer_parallel_attn.py:46-71 (math branch :68-71,
                           GQA expansion :56-59)
  merge_partial            umallm/peer_parallel_attn.py:74-80
  peer_parallel_attention  umallm/peer_parallel_attn.py:143-173 (fold :162-173)
  reference_attn           umallm/peerkv/fused_attn.py:83-99
  cat_blocks / gather_seq / paged_cfk_decode
                           umallm/peerkv/paged.py:30-45, 48-66, 69-97
  partial_bytes / balanced_partition
                           umallm/multigpu.py:351-359, 362-377

Pinned against the reference itself: tests/golden/make_golden.py imports the real
`umallm` package, runs these same entry points on seeded inputs and stores
inputs + outputs; tests/test_oracle.py replays them through this file.

NOT in the reference, defined here once (parity unpinned for these):

  * quantize_kv / dequantize_kv : int8 and fp8-e4m3 KV codes with one fp16 scale
    per (token, kv-head) row.  For a row x (upcast to fp32): a = max|x|;
    s32 = a / QMAX (QMAX = 127 for int8, 448 for e4m3), s32 = 1 if a == 0;
    the STORED scale is s = fp16(s32) (round-to-nearest-even), bumped to the
    smallest positive fp16 subnormal if it rounded to zero; codes are computed
    against the stored scale with a true fp32 division:
        int8:  clamp(rint(x / float(s)), -127, 127)     (rint = ties-to-even)
        e4m3:  e4m3fn(clamp(x / float(s), -448, 448))   (RNE, saturating by the clamp)
    dequantised value = float(code) * float(s).
  * round_robin_shards / capacity_spill_shards : the page placements of the
    batched and ragged benchmark configurations (page p -> GPU p mod N at local
    index p div N; and a seeded per-GPU capacity with spill to the next GPU).
"""
from __future__ import annotations

import math
from typing import List, Sequence

import numpy as np
import torch

INT8_QMAX = 127.0
FP8_QMAX = 448.0


# --------------------------------------------------------------------------- #
# the reference's torch path, math branch
# --------------------------------------------------------------------------- #
def flash_partial(q, K, V, scale=None):
    """One shard's attention partial -> (O in q.dtype, lse fp32).

    q (B,Hq,Lq,D); K,V (B,Hkv,Tk,D).  Follows peer_parallel_attn.py:53-71: GQA by
    repeat_interleave on the head axis, then scores = (q.float()*scale) @ K.float()^T,
    lse = logsumexp, O = softmax @ V.float(), cast to q.dtype.
    """
    if scale is None:
        scale = 1.0 / (q.shape[-1] ** 0.5)
    if K.shape[1] != q.shape[1]:
        rep = q.shape[1] // K.shape[1]
        K = K.repeat_interleave(rep, dim=1)
        V = V.repeat_interleave(rep, dim=1)
    s = (q.float() * scale) @ K.float().transpose(-1, -2)
    lse = torch.logsumexp(s, dim=-1)
    O = (torch.softmax(s, dim=-1) @ V.float()).to(q.dtype)
    return O, lse


def merge_partial(O0, lse0, O1, lse1):
    """Exact two-way merge (peer_parallel_attn.py:74-80) -> (O fp32, lse)."""
    lse = torch.logaddexp(lse0, lse1)
    w0 = torch.exp(lse0 - lse).unsqueeze(-1)
    w1 = torch.exp(lse1 - lse).unsqueeze(-1)
    return O0.float() * w0 + O1.float() * w1, lse


def peer_parallel_attention(q, kv_shards, scale=None):
    """Left fold of flash_partial + merge_partial over the shards
    (peer_parallel_attn.py:158-173).  Result in q.dtype."""
    if not kv_shards:
        raise ValueError("kv_shards must be non-empty")
    if scale is None:
        scale = 1.0 / (q.shape[-1] ** 0.5)
    O_acc = lse_acc = None
    for K, V in kv_shards:
        O, lse = flash_partial(q, K, V, scale)
        if O_acc is None:
            O_acc, lse_acc = O.float(), lse
        else:
            O_acc, lse_acc = merge_partial(O_acc, lse_acc, O, lse)
    return O_acc.to(q.dtype)


def dense_attention_fp32(q, K, V, scale=None):
    """Unsplit fp32 attention with GQA expansion: softmax((q*scale) K^T) V.
    The comparator the single-layer configuration is checked against.  fp32 out."""
    if scale is None:
        scale = 1.0 / (q.shape[-1] ** 0.5)
    if K.shape[1] != q.shape[1]:
        rep = q.shape[1] // K.shape[1]
        K = K.repeat_interleave(rep, dim=1)
        V = V.repeat_interleave(rep, dim=1)
    s = (q.float() * scale) @ K.float().transpose(-1, -2)
    return torch.softmax(s, dim=-1) @ V.float()


def dense_attention_lse_fp32(q, K, V, scale=None):
    """(O fp32, lse fp32) of unsplit attention; q (B,Hq,Lq,D), K/V (B,Hkv,T,D).
    Empty T gives O = 0 and lse = -inf (the neutral element of the merge)."""
    if scale is None:
        scale = 1.0 / (q.shape[-1] ** 0.5)
    B, Hq, Lq, D = q.shape
    if K.shape[2] == 0:
        return (torch.zeros(B, Hq, Lq, D), torch.full((B, Hq, Lq), float("-inf")))
    if K.shape[1] != q.shape[1]:
        rep = q.shape[1] // K.shape[1]
        K = K.repeat_interleave(rep, dim=1)
        V = V.repeat_interleave(rep, dim=1)
    s = (q.float() * scale) @ K.float().transpose(-1, -2)
    return torch.softmax(s, dim=-1) @ V.float(), torch.logsumexp(s, dim=-1)


def reference_attn(q, K_full, V_full, scale=None):
    """Per-head fp32 softmax reference of the [H,D] / [HKV,T,D] form
    (peerkv/fused_attn.py:83-99).  Returns [H,D] fp32 (the reference casts to
    fp16 at the very end; callers cast as they need)."""
    H, D = q.shape
    HKV, T, _ = K_full.shape
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    groups = H // HKV
    qf = q.float()
    out = torch.empty((H, D), dtype=torch.float32)
    for h in range(H):
        kvh = h // groups
        s = (qf[h] @ K_full[kvh].float().T) * scale
        w = torch.softmax(s, dim=-1)
        out[h] = w @ V_full[kvh].float()
    return out


# --------------------------------------------------------------------------- #
# paged bridge (peerkv/paged.py)
# --------------------------------------------------------------------------- #
def cat_blocks(cache, block_idx: Sequence[int], total_valid: int):
    """cache [2, nb, bs, Hkv, D] -> (K, V) as [Hkv, T, D] with T = total_valid
    (paged.py:30-45; only the last listed block may be partial)."""
    Hkv, D = cache.size(3), cache.size(4)
    if len(block_idx) == 0:
        z = cache.new_empty((Hkv, 0, D))
        return z, z
    idx = torch.as_tensor(list(block_idx), dtype=torch.long)
    K = cache[0].index_select(0, idx)
    V = cache[1].index_select(0, idx)
    n, bs = K.size(0), K.size(1)
    K = K.reshape(n * bs, Hkv, D)[:total_valid].permute(1, 0, 2).contiguous()
    V = V.reshape(n * bs, Hkv, D)[:total_valid].permute(1, 0, 2).contiguous()
    return K, V


def split_block_row(block_row, seq_len: int, bs: int, bases: Sequence[int]):
    """Generalisation of gather_seq's id test (paged.py:52-61) to N devices.
    `bases` are ascending id thresholds: a global id g lives on the device d with
    bases[d] <= g < bases[d+1] at local index g - bases[d].
    Returns per device (local_ids, valid_tokens)."""
    n_blk = (seq_len + bs - 1) // bs
    n_dev = len(bases)
    ids: List[List[int]] = [[] for _ in range(n_dev)]
    val = [0] * n_dev
    for j in range(n_blk):
        gid = int(block_row[j])
        valid = bs if j < n_blk - 1 else (seq_len - (n_blk - 1) * bs)
        d = n_dev - 1
        while d > 0 and gid < bases[d]:
            d -= 1
        ids[d].append(gid - bases[d])
        val[d] += valid
    return ids, val


def paged_decode_oracle(query, caches, block_table, seq_lens, bases, scale=None):
    """Multi-sequence paged decode over N per-device caches -> [num_seqs, Hq, D] fp32.

    Follows paged_cfk_decode (paged.py:69-97): per sequence, gather each device's
    blocks into a contiguous shard, compute every shard's partial and fold them
    with merge_partial.  `caches[d]` is [2, nb_d, bs, Hkv, D] (None allowed for an
    absent device).  Partials are kept in fp32 (the fold's own precision)."""
    num_seqs, Hq, D = query.shape
    bs = next(c for c in caches if c is not None).size(2)
    out = torch.zeros((num_seqs, Hq, D), dtype=torch.float32)
    for i in range(num_seqs):
        L = int(seq_lens[i])
        ids, val = split_block_row(block_table[i].tolist(), L, bs, bases)
        O_acc = lse_acc = None
        qi = query[i].float().view(1, Hq, 1, D)
        for d, cache in enumerate(caches):
            if cache is None or val[d] == 0:
                continue
            K, V = cat_blocks(cache, ids[d], val[d])
            O, lse = dense_attention_lse_fp32(qi, K.unsqueeze(0), V.unsqueeze(0), scale)
            if O_acc is None:
                O_acc, lse_acc = O, lse
            else:
                O_acc, lse_acc = merge_partial(O_acc, lse_acc, O, lse)
        if O_acc is not None:
            out[i] = O_acc.view(Hq, D)
    return out


def paged_partial_oracle(query, cache, block_table, seq_lens, scale=None,
                         k_scale=None, v_scale=None):
    """One shard's (O fp32 [B,Hq,D], lse fp32 [B,Hq]) from its own paged cache.
    block_table holds LOCAL page ids, seq_lens the shard's token count per
    sequence (0 allowed).  With k_scale/v_scale ([nb, bs, Hkv] fp16 each) the
    cache holds codes that are dequantised first (code * scale)."""
    B, Hq, D = query.shape
    bs = cache.size(2)
    O = torch.zeros((B, Hq, D), dtype=torch.float32)
    lse = torch.full((B, Hq), float("-inf"), dtype=torch.float32)
    for i in range(B):
        L = int(seq_lens[i])
        if L == 0:
            continue
        n_blk = (L + bs - 1) // bs
        ids = [int(x) for x in block_table[i, :n_blk]]
        if k_scale is None:
            K, V = cat_blocks(cache, ids, L)
            K, V = K.float(), V.float()
        else:
            Kc, Vc = cat_blocks(cache, ids, L)
            idx = torch.as_tensor(ids, dtype=torch.long)
            ks = k_scale.index_select(0, idx).reshape(n_blk * bs, -1)[:L].t().float()
            vs = v_scale.index_select(0, idx).reshape(n_blk * bs, -1)[:L].t().float()
            K = code_to_float(Kc) * ks.unsqueeze(-1)
            V = code_to_float(Vc) * vs.unsqueeze(-1)
        o, l = dense_attention_lse_fp32(query[i].float().view(1, Hq, 1, D),
                                        K.unsqueeze(0), V.unsqueeze(0), scale)
        O[i] = o.view(Hq, D)
        lse[i] = l.view(Hq)
    return O, lse


def merge_n(O_parts, lse_parts):
    """Single-pass N-way merge of (O fp32 [..., D], lse [...]) partials; the
    closed form of folding merge_partial.  All-empty rows give O = 0, lse = -inf."""
    O = torch.stack([o.float() for o in O_parts], 0)
    l = torch.stack([x.float() for x in lse_parts], 0)
    L = torch.logsumexp(l, dim=0)
    w = torch.exp(l - torch.where(torch.isinf(L), torch.zeros_like(L), L))
    w = torch.where(torch.isinf(l) & (l < 0), torch.zeros_like(w), w)
    return (O * w.unsqueeze(-1)).sum(0), L


# --------------------------------------------------------------------------- #
# quantised KV (defined here; not in the reference)
# --------------------------------------------------------------------------- #
def code_to_float(codes):
    if codes.dtype == torch.int8:
        return codes.float()
    if codes.dtype == torch.float8_e4m3fn:
        return codes.float()
    if codes.dtype == torch.uint8:  # raw e4m3 bytes
        return codes.view(torch.float8_e4m3fn).float()
    raise TypeError(codes.dtype)


def quantize_kv(x, fmt: str):
    """x [..., D] (any float dtype) -> (codes [..., D], scales [...] fp16), one
    scale per row of D.  fmt 'int8' -> int8 codes; 'fp8' -> float8_e4m3fn codes."""
    qmax = INT8_QMAX if fmt == "int8" else FP8_QMAX
    xf = x.float()
    a = xf.abs().amax(dim=-1)
    s32 = a / qmax
    s32 = torch.where(a == 0, torch.ones_like(s32), s32)
    s16 = s32.to(torch.float16)
    tiny = torch.tensor(2.0 ** -24, dtype=torch.float16)
    s16 = torch.where(s16 == 0, tiny, s16)
    sf = s16.float().unsqueeze(-1)
    y = xf / sf
    if fmt == "int8":
        codes = torch.clamp(torch.round(y), -127, 127).to(torch.int8)
    elif fmt == "fp8":
        codes = torch.clamp(y, -FP8_QMAX, FP8_QMAX).to(torch.float8_e4m3fn)
    else:
        raise ValueError(fmt)
    return codes, s16


def dequantize_kv(codes, scales):
    return code_to_float(codes) * scales.float().unsqueeze(-1)


# --------------------------------------------------------------------------- #
# placements of the benchmark configurations (defined here; not in the reference)
# --------------------------------------------------------------------------- #
def round_robin_shards(block_table, seq_lens, bs: int, n_gpus: int):
    """Page p lives on GPU p mod N at local index p div N.  Returns per GPU
    (local_block_table [B, max_local] int32, local_seq_lens [B] int32).  Within a
    GPU the pages keep sequence order, so the only partial page is last."""
    B = len(seq_lens)
    tabs = [[[] for _ in range(B)] for _ in range(n_gpus)]
    lens = np.zeros((n_gpus, B), dtype=np.int64)
    for i in range(B):
        L = int(seq_lens[i])
        n_blk = (L + bs - 1) // bs
        for j in range(n_blk):
            p = int(block_table[i][j])
            valid = bs if j < n_blk - 1 else L - (n_blk - 1) * bs
            g = p % n_gpus
            tabs[g][i].append(p // n_gpus)
            lens[g, i] += valid
    return _pack_tables(tabs, lens)


def capacity_spill_shards(block_table, seq_lens, bs: int, caps: Sequence[float]):
    """Walk the GPUs in order; GPU g takes up to floor(caps[g] * total_pages / N)
    pages of the flattened (sequence-major) page list, the remainder spills to the
    next GPU and the last GPU takes what is left.  The returned tables hold the
    GLOBAL page ids (each GPU's pool is indexed by global id in the tests that use
    this); a caller that compacts pools remaps them."""
    n_gpus = len(caps)
    B = len(seq_lens)
    total = sum((int(L) + bs - 1) // bs for L in seq_lens)
    quota = [int(c * total / n_gpus) for c in caps]
    quota[-1] = total
    tabs = [[[] for _ in range(B)] for _ in range(n_gpus)]
    lens = np.zeros((n_gpus, B), dtype=np.int64)
    g, used = 0, 0
    for i in range(B):
        L = int(seq_lens[i])
        n_blk = (L + bs - 1) // bs
        for j in range(n_blk):
            while g < n_gpus - 1 and used >= quota[g]:
                g, used = g + 1, 0
            valid = bs if j < n_blk - 1 else L - (n_blk - 1) * bs
            tabs[g][i].append(int(block_table[i][j]))
            lens[g, i] += valid
            used += 1
    return _pack_tables(tabs, lens)


def _pack_tables(tabs, lens):
    out = []
    for g, per_seq in enumerate(tabs):
        width = max(1, max(len(r) for r in per_seq))
        t = np.zeros((len(per_seq), width), dtype=np.int32)
        for i, r in enumerate(per_seq):
            t[i, :len(r)] = r
        out.append((torch.from_numpy(t), torch.from_numpy(lens[g].astype(np.int32))))
    return out


# --------------------------------------------------------------------------- #
# cost helpers of the path (multigpu.py:351-377)
# --------------------------------------------------------------------------- #
def partial_bytes(heads: int, head_dim: int, lse_bytes: int = 4, o_bytes: int = 2) -> int:
    return heads * head_dim * o_bytes + heads * lse_bytes


def balanced_partition(n_blocks: int, hbm_bw_gbps_per_device) -> list:
    """Blocks per device in proportion to its HBM bandwidth, floors first, then the
    leftover handed out one block at a time starting from device 0."""
    w = np.asarray([float(b) for b in hbm_bw_gbps_per_device], dtype=np.float64)
    total_w = float(w.sum()) or 1.0
    share = [int(n_blocks * float(x) / total_w) for x in w]
    left = n_blocks - sum(share)
    for k in range(left):
        share[k % len(share)] += 1
    return share
