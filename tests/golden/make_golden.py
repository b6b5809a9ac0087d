"""Generate golden vectors by running the REAL reference package.

Run once, in a container that has the reference checked out, as

    PEERKV_REFERENCE=/path/to/PeerKV python tests/golden/make_golden.py

It imports `umallm` from that checkout, calls the reference's own entry points
for the path (peer_parallel_attention, flash_partial, merge_partial,
reference_attn, gather_seq, partial_bytes, balanced_partition) on seeded inputs
and writes `tests/golden/peerkv_golden.npz`.  Small cases store inputs and
outputs; large ones store the seed, a checksum of the regenerated inputs and
the outputs.  The tests never import the reference: they replay these vectors.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE0 = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("PEERKV_REFERENCE",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE0))), "reference"))
sys.path.insert(0, REF)

from umallm.peer_parallel_attn import (flash_partial, merge_partial,  # noqa: E402
                                       peer_parallel_attention)
from umallm.peerkv.fused_attn import reference_attn  # noqa: E402
from umallm.peerkv.paged import gather_seq  # noqa: E402
from umallm.multigpu import balanced_partition, partial_bytes  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from golden_cases import (SEEDED_CASES, digest, gen_paged_case,  # noqa: E402
                          gen_seeded_case)


def main():
    out = {}
    # ---- seeded sharded-attention cases (shapes of the reference's unit tests) -- #
    for name, spec in SEEDED_CASES.items():
        q, K, V = gen_seeded_case(spec)
        shards = list(zip(K.split(spec["shards"], dim=2), V.split(spec["shards"], dim=2)))
        o = peer_parallel_attention(q, shards)
        out[f"{name}/out"] = o.float().numpy()
        out[f"{name}/digest"] = np.frombuffer(bytes.fromhex(digest(q, K, V)), dtype=np.uint8)
        # per-shard partials of the first two shards + their merge
        O0, l0 = flash_partial(q, *shards[0])
        out[f"{name}/p0_o"] = O0.float().numpy()
        out[f"{name}/p0_lse"] = l0.float().numpy()
        if len(shards) > 1:
            O1, l1 = flash_partial(q, *shards[1])
            Om, lm = merge_partial(O0, l0, O1, l1)
            out[f"{name}/m01_o"] = Om.float().numpy()
            out[f"{name}/m01_lse"] = lm.float().numpy()
        if spec.get("store_inputs"):
            out[f"{name}/q"] = q.float().numpy()
            out[f"{name}/K"] = K.float().numpy()
            out[f"{name}/V"] = V.float().numpy()

    # ---- [H,D] / [HKV,T,D] form: reference_attn ------------------------------- #
    torch.manual_seed(0)
    H, HKV, D, T = 32, 8, 128, 1024
    q = (torch.randn(H, D) * 0.1).half()
    Kf = (torch.randn(HKV, T, D) * 0.1).half()
    Vf = (torch.randn(HKV, T, D) * 0.1).half()
    out["refattn/out"] = reference_attn(q, Kf, Vf).float().numpy()
    out["refattn/digest"] = np.frombuffer(bytes.fromhex(digest(q, Kf, Vf)), dtype=np.uint8)

    # ---- paged bridge: gather_seq + fold (seq lens of the reference's paged check) #
    case = gen_paged_case()
    outs = []
    for i, L in enumerate(case["seq_lens"]):
        Kl, Vl, Kp, Vp = gather_seq(case["local_cache"], case["peer_cache"],
                                    case["block_table"][i], L, case["peer_base"])
        qi = case["q"][i].view(1, H, 1, D)
        shards = [(Kl.unsqueeze(0), Vl.unsqueeze(0))]
        if Kp is not None:
            shards.append((Kp.unsqueeze(0), Vp.unsqueeze(0)))
        outs.append(peer_parallel_attention(qi, shards).view(H, D).float().numpy())
        out[f"paged/n_local_tok_{i}"] = np.int64(Kl.shape[1])
    out["paged/out"] = np.stack(outs)
    out["paged/digest"] = np.frombuffer(bytes.fromhex(
        digest(case["q"], case["local_cache"], case["peer_cache"],
               case["block_table"].to(torch.int32))), dtype=np.uint8)

    # ---- cost helpers ---------------------------------------------------------- #
    out["cost/partial_bytes_8_128"] = np.int64(partial_bytes(8, 128))
    out["cost/partial_bytes_32_128"] = np.int64(partial_bytes(32, 128))
    out["cost/bp_1000_773_773"] = np.asarray(balanced_partition(1000, [773, 773]))
    out["cost/bp_1001_3eq"] = np.asarray(balanced_partition(1001, [1, 1, 1]))
    out["cost/bp_8192_8"] = np.asarray(balanced_partition(8192, [6549.4] * 8))
    out["cost/bp_777_uneven"] = np.asarray(balanced_partition(777, [2000, 773, 773, 1555]))

    path = os.path.join(HERE, "peerkv_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
