"""The oracle against the reference's own outputs (golden vectors produced by
tests/golden/make_golden.py, which runs the real reference package) and against
the assertions of the reference's unit tests for the path."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from golden_cases import SEEDED_CASES, digest, gen_paged_case, gen_seeded_case
from oracle import peerkv_oracle as orc


def _check_digest(golden, name, *tensors):
    want = bytes(golden[f"{name}/digest"]).hex()
    assert digest(*tensors) == want, f"seeded inputs of {name} drifted from the golden file"


@pytest.mark.parametrize("name", list(SEEDED_CASES))
def test_fold_matches_reference_output(golden, name):
    spec = SEEDED_CASES[name]
    q, K, V = gen_seeded_case(spec)
    _check_digest(golden, name, q, K, V)
    shards = list(zip(K.split(spec["shards"], dim=2), V.split(spec["shards"], dim=2)))
    out = orc.peer_parallel_attention(q, shards).float().numpy()
    assert np.array_equal(out, golden[f"{name}/out"])          # same ops, same order: bit-exact
    O0, l0 = orc.flash_partial(q, *shards[0])
    assert np.array_equal(O0.float().numpy(), golden[f"{name}/p0_o"])
    assert np.array_equal(l0.numpy(), golden[f"{name}/p0_lse"])
    if len(shards) > 1:
        O1, l1 = orc.flash_partial(q, *shards[1])
        Om, lm = orc.merge_partial(O0, l0, O1, l1)
        assert np.array_equal(Om.numpy(), golden[f"{name}/m01_o"])
        assert np.array_equal(lm.numpy(), golden[f"{name}/m01_lse"])


@pytest.mark.parametrize("name", [n for n, s in SEEDED_CASES.items() if s.get("store_inputs")])
def test_stored_inputs_agree_with_generator(golden, name):
    q, K, V = gen_seeded_case(SEEDED_CASES[name])
    assert np.array_equal(q.float().numpy(), golden[f"{name}/q"])
    assert np.array_equal(K.float().numpy(), golden[f"{name}/K"])


@pytest.mark.parametrize("name", list(SEEDED_CASES))
def test_fold_matches_dense_and_merge_n(golden, name):
    """The reference's own acceptance: sharded == dense (test_peer_parallel.py:27-35)."""
    spec = SEEDED_CASES[name]
    q, K, V = gen_seeded_case(spec)
    dense = orc.dense_attention_fp32(q, K, V)
    sdpa = F.scaled_dot_product_attention(q.float(), K.float().repeat_interleave(spec["Hq"] // spec["Hkv"], 1),
                                          V.float().repeat_interleave(spec["Hq"] // spec["Hkv"], 1))
    assert torch.allclose(dense, sdpa, atol=1e-5, rtol=1e-5)
    tol = 1e-4 if spec["dtype"] == "float32" else 5e-3
    assert torch.allclose(torch.from_numpy(golden[f"{name}/out"]), dense, atol=tol, rtol=tol)
    parts = [orc.dense_attention_lse_fp32(q, k, v) for k, v in
             zip(K.split(spec["shards"], dim=2), V.split(spec["shards"], dim=2))]
    O, lse = orc.merge_n([p[0] for p in parts], [p[1] for p in parts])
    assert torch.allclose(O, dense, atol=1e-5, rtol=1e-4)


def test_order_invariance():
    """test_peer_parallel.py:46-50."""
    torch.manual_seed(1)
    q = torch.randn(1, 8, 1, 128); K = torch.randn(1, 8, 1000, 128); V = torch.randn(1, 8, 1000, 128)
    shards = list(zip(K.split([500, 500], 2), V.split([500, 500], 2)))
    o1 = orc.peer_parallel_attention(q, shards)
    o2 = orc.peer_parallel_attention(q, list(reversed(shards)))
    assert torch.allclose(o1, o2, atol=1e-5, rtol=1e-5)


def test_reference_attn_golden(golden):
    torch.manual_seed(0)
    H, HKV, D, T = 32, 8, 128, 1024
    q = (torch.randn(H, D) * 0.1).half()
    Kf = (torch.randn(HKV, T, D) * 0.1).half()
    Vf = (torch.randn(HKV, T, D) * 0.1).half()
    _check_digest(golden, "refattn", q, Kf, Vf)
    out = orc.reference_attn(q, Kf, Vf).half().float().numpy()
    assert np.array_equal(out, golden["refattn/out"])


def test_paged_bridge_golden(golden):
    c = gen_paged_case()
    _check_digest(golden, "paged", c["q"], c["local_cache"], c["peer_cache"],
                  c["block_table"].to(torch.int32))
    out = orc.paged_decode_oracle(c["q"], [c["local_cache"], c["peer_cache"]], c["block_table"],
                                  c["seq_lens"], [0, c["peer_base"]])
    ref = torch.from_numpy(golden["paged/out"])            # fp16-rounded fold of the reference
    assert torch.allclose(out, ref, atol=2e-4, rtol=1e-2)
    for i, L in enumerate(c["seq_lens"]):
        ids, val = orc.split_block_row(c["block_table"][i].tolist(), L, c["bs"], [0, c["peer_base"]])
        assert val[0] == int(golden[f"paged/n_local_tok_{i}"])
        assert val[0] + val[1] == L
        Kf, Vf = c["full"][i]
        dense = orc.reference_attn(c["q"][i], Kf, Vf)
        assert torch.allclose(out[i], dense, atol=1e-5, rtol=1e-3)


def test_paged_partial_matches_fold():
    c = gen_paged_case()
    bt_local = c["block_table"].clone()
    # device 0's view: only its own blocks, in order
    B = len(c["seq_lens"])
    tabs, lens = [[], []], [[], []]
    for i, L in enumerate(c["seq_lens"]):
        ids, val = orc.split_block_row(c["block_table"][i].tolist(), L, c["bs"], [0, c["peer_base"]])
        for d in range(2):
            tabs[d].append(ids[d]); lens[d].append(val[d])
    parts = []
    for d, cache in enumerate([c["local_cache"], c["peer_cache"]]):
        w = max(len(r) for r in tabs[d])
        t = torch.zeros(B, w, dtype=torch.int32)
        for i, r in enumerate(tabs[d]):
            t[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
        parts.append(orc.paged_partial_oracle(c["q"], cache, t, torch.tensor(lens[d])))
    O, _ = orc.merge_n([p[0] for p in parts], [p[1] for p in parts])
    ref = orc.paged_decode_oracle(c["q"], [c["local_cache"], c["peer_cache"]], c["block_table"],
                                  c["seq_lens"], [0, c["peer_base"]])
    assert torch.allclose(O, ref, atol=1e-6, rtol=1e-4)


def test_cost_helpers_golden(golden):
    assert orc.partial_bytes(8, 128) == int(golden["cost/partial_bytes_8_128"]) == 2080
    assert orc.partial_bytes(32, 128) == int(golden["cost/partial_bytes_32_128"])
    assert orc.balanced_partition(1000, [773, 773]) == golden["cost/bp_1000_773_773"].tolist()
    assert orc.balanced_partition(1001, [1, 1, 1]) == golden["cost/bp_1001_3eq"].tolist()
    assert orc.balanced_partition(8192, [6549.4] * 8) == golden["cost/bp_8192_8"].tolist()
    assert orc.balanced_partition(777, [2000, 773, 773, 1555]) == golden["cost/bp_777_uneven"].tolist()


@pytest.mark.parametrize("fmt", ["int8", "fp8"])
def test_quantiser_definition(fmt):
    torch.manual_seed(3)
    x = torch.randn(64, 8, 128).bfloat16()
    x[0, 0] = 0                         # zero row -> scale 1, codes 0
    x[1, 1] = 1e-30                     # underflowing scale -> smallest subnormal
    codes, s = orc.quantize_kv(x, fmt)
    assert s.dtype == torch.float16 and s.shape == (64, 8)
    assert float(s[0, 0]) == 1.0 and orc.code_to_float(codes[0, 0]).abs().max() == 0
    assert float(s[1, 1]) > 0
    xh = orc.dequantize_kv(codes, s)
    err = (xh - x.float()).abs().amax(-1)
    step = s.float() * (0.5 if fmt == "int8" else 16.0)   # e4m3 half-ulp at 448 is 16
    assert bool((err <= step * 1.01 + 1e-6).all())
    # idempotence: re-quantising the dequantised values with the same scale gives the same codes
    y = xh / s.float().unsqueeze(-1)
    if fmt == "int8":
        assert torch.equal(torch.round(y).to(torch.int8), codes)
    else:
        assert torch.equal(y.to(torch.float8_e4m3fn).view(torch.uint8), codes.view(torch.uint8))


def test_placements_cover_every_token_once():
    rng = np.random.default_rng(5)
    bs, B = 16, 6
    lens = rng.integers(1, 700, size=B)
    n_pages = [(int(L) + bs - 1) // bs for L in lens]
    perm = rng.permutation(sum(n_pages))
    bt = np.zeros((B, max(n_pages)), dtype=np.int64)
    k = 0
    for i, n in enumerate(n_pages):
        bt[i, :n] = perm[k:k + n]; k += n
    for N in (1, 2, 4, 8):
        sh = orc.round_robin_shards(bt, lens, bs, N)
        assert sum(int(s[1].sum()) for s in sh) == int(lens.sum())
        for i in range(B):
            pages = sorted(int(p) * N + g for g, s in enumerate(sh)
                           for p in s[0][i, :(int(s[1][i]) + bs - 1) // bs])
            assert pages == sorted(bt[i, :n_pages[i]].tolist())
    caps = [0.6, 1.0, 0.5, 0.9]
    sh = orc.capacity_spill_shards(bt, lens, bs, caps)
    assert sum(int(s[1].sum()) for s in sh) == int(lens.sum())
    total = sum(n_pages)
    for g in range(3):
        used = sum((int(x) + bs - 1) // bs for x in sh[g][1])
        assert used <= int(caps[g] * total / 4) + B    # a sequence's partial page may round up
