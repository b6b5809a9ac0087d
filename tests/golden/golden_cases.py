"""Seeded input generators shared by make_golden.py (which runs the reference on
them) and by the tests (which replay the stored outputs).  torch's CPU generator
is deterministic for a given torch version; every case carries a SHA-256 digest
of its inputs in the golden file so a drift would fail loudly instead of
comparing against the wrong vectors."""
from __future__ import annotations

import hashlib

import torch

# Shapes and seeds follow the reference's own unit tests of the sharded path
# (tests/test_peer_parallel.py:27-35, 38-50, 53-60, 98-111, 114-124) plus the
# single-layer GQA benchmark configuration at reduced and full context.
SEEDED_CASES = {
    "two_shards": dict(seed=0, B=1, Hq=4, Hkv=4, Lq=1, T=500, D=64, dtype="float32",
                       shards=[300, 200], store_inputs=True),
    "four_ragged": dict(seed=1, B=1, Hq=8, Hkv=8, Lq=1, T=1000, D=128, dtype="float32",
                        shards=[128, 256, 384, 232]),
    "single_shard": dict(seed=2, B=1, Hq=2, Hkv=2, Lq=1, T=137, D=32, dtype="float32",
                         shards=[137], store_inputs=True),
    "fp16_16x512": dict(seed=7, B=1, Hq=8, Hkv=8, Lq=1, T=8192, D=128, dtype="float16",
                        shards=[512] * 16),
    "partial_merge": dict(seed=4, B=1, Hq=2, Hkv=2, Lq=1, T=64, D=48, dtype="float32",
                          shards=[40, 24], store_inputs=True),
    "gqa_c1_small": dict(seed=11, B=1, Hq=32, Hkv=8, Lq=1, T=2048, D=128, dtype="float16",
                         shards=[1024, 1024]),
    "gqa_c1_full": dict(seed=12, B=1, Hq=32, Hkv=8, Lq=1, T=16384, D=128, dtype="float16",
                        shards=[8192, 8192]),
    "gqa_bf16_batch": dict(seed=13, B=3, Hq=32, Hkv=8, Lq=1, T=1500, D=128, dtype="bfloat16",
                           shards=[700, 33, 767]),
    "gqa8_bf16": dict(seed=14, B=2, Hq=64, Hkv=8, Lq=1, T=1024, D=128, dtype="bfloat16",
                      shards=[512, 512]),
}


def gen_seeded_case(spec):
    torch.manual_seed(spec["seed"])
    dt = getattr(torch, spec["dtype"])
    q = torch.randn(spec["B"], spec["Hq"], spec["Lq"], spec["D"]).to(dt)
    K = torch.randn(spec["B"], spec["Hkv"], spec["T"], spec["D"]).to(dt)
    V = torch.randn(spec["B"], spec["Hkv"], spec["T"], spec["D"]).to(dt)
    return q, K, V


def digest(*tensors) -> str:
    h = hashlib.sha256()
    for t in tensors:
        t = t.contiguous()
        if t.dtype == torch.bfloat16:
            t = t.view(torch.int16)
        h.update(t.numpy().tobytes())
    return h.hexdigest()


def gen_paged_case(dtype=torch.float16):
    """Paged two-device case with the sequence lengths, block size and tail-40%-on-
    the-peer split of the reference's paged check (experiments/test_paged_cfk.py:21-81),
    built on CPU.  Global ids >= peer_base live in the peer cache at id - peer_base."""
    torch.manual_seed(0)
    H, HKV, D, bs = 32, 8, 128, 16
    seq_lens = [777, 1024, 1600, 33, 4096]
    per_seq = [(L + bs - 1) // bs for L in seq_lens]
    total = sum(per_seq)
    peer_base = total
    max_blk = max(per_seq)
    q = (torch.randn(len(seq_lens), H, D) * 0.1).to(dtype)
    local_cache = torch.zeros(2, total, bs, HKV, D, dtype=dtype)
    peer_cache = torch.zeros(2, total, bs, HKV, D, dtype=dtype)
    block_table = torch.zeros(len(seq_lens), max_blk, dtype=torch.long)
    nl = npeer = 0
    full = []
    for i, L in enumerate(seq_lens):
        nblk = per_seq[i]
        Kf = (torch.randn(HKV, L, D) * 0.1).to(dtype)
        Vf = (torch.randn(HKV, L, D) * 0.1).to(dtype)
        full.append((Kf, Vf))
        n_peer = int(nblk * 0.4)
        n_local = nblk - n_peer
        for j in range(nblk):
            valid = bs if j < nblk - 1 else L - (nblk - 1) * bs
            t0 = j * bs
            kb = torch.zeros(bs, HKV, D, dtype=dtype)
            vb = torch.zeros(bs, HKV, D, dtype=dtype)
            kb[:valid] = Kf[:, t0:t0 + valid].permute(1, 0, 2)
            vb[:valid] = Vf[:, t0:t0 + valid].permute(1, 0, 2)
            if j < n_local:
                gid = nl
                nl += 1
                local_cache[0, gid], local_cache[1, gid] = kb, vb
            else:
                gid = peer_base + npeer
                npeer += 1
                peer_cache[0, gid - peer_base], peer_cache[1, gid - peer_base] = kb, vb
            block_table[i, j] = gid
    return dict(q=q, local_cache=local_cache, peer_cache=peer_cache,
                block_table=block_table, seq_lens=seq_lens, peer_base=peer_base,
                full=full, H=H, HKV=HKV, D=D, bs=bs)
