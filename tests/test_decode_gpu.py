"""GPU parity tests, through the C-ABI library, against the CPU oracle and the
golden vectors.  Tolerance (16-bit KV, fp32 accumulate): |out - ref| <= 2e-3 or
relative <= 1e-2, i.e. allclose(atol=2e-3, rtol=1e-2); quantiser codes and scales
and all index work are bit-exact."""
import numpy as np
import pytest
import torch

from golden_cases import SEEDED_CASES, gen_paged_case, gen_seeded_case
from oracle import peerkv_oracle as orc

pytestmark = pytest.mark.gpu

ATOL, RTOL = 2e-3, 1e-2


def close(a, b, atol=ATOL, rtol=RTOL):
    a, b = a.float().cpu(), b.float().cpu()
    ok = torch.allclose(a, b, atol=atol, rtol=rtol)
    if not ok:
        d = (a - b).abs()
        print("max abs", float(d.max()), "at", int(d.argmax()), "ref", float(b.flatten()[d.argmax()]))
    return ok


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


def make_paged(B, lens, Hkv, D, bs, dtype, dev, seed, extra_pages=3, poison=True):
    """Random pool + permuted block table; the unused tail of partial pages and unused
    pages are filled with NaN so any read of them shows."""
    g = torch.Generator().manual_seed(seed)
    n_pages = [(int(L) + bs - 1) // bs for L in lens]
    total = sum(n_pages) + extra_pages
    pool = torch.randn(2, total, bs, Hkv, D, generator=g).to(dtype)
    perm = torch.randperm(total, generator=g)
    W = max(1, max(n_pages))
    bt = torch.zeros(B, W, dtype=torch.int32)
    k = 0
    used = torch.zeros(total, dtype=torch.bool)
    for i, n in enumerate(n_pages):
        bt[i, :n] = perm[k:k + n].to(torch.int32)
        used[perm[k:k + n]] = True
        if n and poison and lens[i] % bs:
            pool[:, perm[k + n - 1], lens[i] % bs:] = float("nan")
        k += n
    if poison:
        pool[:, ~used] = float("nan")
    return pool, bt, torch.tensor(lens, dtype=torch.int32)


@pytest.mark.parametrize("name", ["gqa_c1_small", "gqa_c1_full", "gqa_bf16_batch", "gqa8_bf16", "fp16_16x512"])
def test_sharded_contiguous_matches_reference_golden(golden, dev, name):
    from peerkv_b200.peer_parallel_attn import peer_parallel_attention
    spec = SEEDED_CASES[name]
    q, K, V = gen_seeded_case(spec)
    qd, Kd, Vd = q.to(dev), K.to(dev), V.to(dev)
    shards = list(zip(Kd.split(spec["shards"], dim=2), Vd.split(spec["shards"], dim=2)))
    out = peer_parallel_attention(qd, shards)
    assert out.dtype == q.dtype and out.shape == q.shape
    ref = torch.from_numpy(golden[f"{name}/out"])              # the reference's own output
    assert close(out, ref)
    assert close(out, orc.dense_attention_fp32(q, K, V))       # unsplit fp32 attention
    # order invariance (reference tests/test_peer_parallel.py:46-50)
    out2 = peer_parallel_attention(qd, list(reversed(shards)))
    assert close(out2, out, atol=1e-3, rtol=1e-2)


@pytest.mark.parametrize("name", ["gqa_c1_small", "gqa_bf16_batch"])
def test_flash_partial_and_merge(golden, dev, name):
    from peerkv_b200.peer_parallel_attn import flash_partial, merge_partial
    spec = SEEDED_CASES[name]
    q, K, V = gen_seeded_case(spec)
    Ks, Vs = K.split(spec["shards"], 2), V.split(spec["shards"], 2)
    O0, l0 = flash_partial(q.to(dev), Ks[0].to(dev), Vs[0].to(dev))
    O1, l1 = flash_partial(q.to(dev), Ks[1].to(dev), Vs[1].to(dev))
    assert O0.dtype == q.dtype and l0.dtype == torch.float32 and l0.shape == q.shape[:3]
    assert close(O0, torch.from_numpy(golden[f"{name}/p0_o"]))
    assert close(l0, torch.from_numpy(golden[f"{name}/p0_lse"]), atol=2e-3, rtol=1e-4)
    Om, lm = merge_partial(O0, l0, O1, l1)
    assert Om.dtype == torch.float32
    assert close(Om, torch.from_numpy(golden[f"{name}/m01_o"]))
    assert close(lm, torch.from_numpy(golden[f"{name}/m01_lse"]), atol=2e-3, rtol=1e-4)


@pytest.mark.parametrize("T", [1, 2, 15, 16, 17, 31, 32, 33, 47, 100, 255, 256, 257, 1000])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_contiguous_edge_lengths(dev, T, dtype):
    from peerkv_b200 import ops
    torch.manual_seed(T)
    B, Hq, Hkv, D = 2, 32, 8, 128
    q = torch.randn(B, Hq, D).to(dtype)
    K = torch.randn(B, Hkv, T, D).to(dtype)
    V = torch.randn(B, Hkv, T, D).to(dtype)
    out = ops.decode_contiguous(q.to(dev), K.to(dev), V.to(dev))
    ref = orc.dense_attention_fp32(q.unsqueeze(2), K, V).squeeze(2)
    assert close(out, ref)
    o, lse = ops.partial_contiguous(q.to(dev), K.to(dev), V.to(dev))
    ro, rl = orc.dense_attention_lse_fp32(q.unsqueeze(2), K, V)
    assert close(o, ro.squeeze(2)) and close(lse, rl.squeeze(2), atol=2e-3, rtol=1e-4)


@pytest.mark.parametrize("Hq,Hkv", [(32, 8), (64, 8), (8, 8), (32, 32), (16, 4), (4, 1), (48, 12), (24, 24)])
def test_head_geometries(dev, Hq, Hkv):
    from peerkv_b200 import ops
    torch.manual_seed(Hq * 100 + Hkv)
    B, D, T = 3, 128, 333
    q = torch.randn(B, Hq, D).bfloat16()
    K = torch.randn(B, Hkv, T, D).bfloat16()
    V = torch.randn(B, Hkv, T, D).bfloat16()
    out = ops.decode_contiguous(q.to(dev), K.to(dev), V.to(dev))
    assert close(out, orc.dense_attention_fp32(q.unsqueeze(2), K, V).squeeze(2))


def test_unsupported_shapes_raise(dev):
    from peerkv_b200 import ops, PeerKVError
    q = torch.randn(1, 32, 64, device=dev).half()
    with pytest.raises(PeerKVError):
        ops.decode_contiguous(q, torch.randn(1, 8, 10, 64, device=dev).half(),
                              torch.randn(1, 8, 10, 64, device=dev).half())
    q = torch.randn(1, 32, 128, device=dev).half()
    with pytest.raises(PeerKVError):      # group of 16 query heads per kv head
        ops.decode_contiguous(q, torch.randn(1, 2, 10, 128, device=dev).half(),
                              torch.randn(1, 2, 10, 128, device=dev).half())
    with pytest.raises(PeerKVError):      # CPU tensors: no fallback
        ops.decode_contiguous(q.cpu(), torch.randn(1, 8, 10, 128).half(), torch.randn(1, 8, 10, 128).half())
    with pytest.raises(PeerKVError):      # dtype mismatch
        ops.decode_contiguous(q, torch.randn(1, 8, 10, 128, device=dev).bfloat16(),
                              torch.randn(1, 8, 10, 128, device=dev).bfloat16())


@pytest.mark.parametrize("bs", [16, 32, 64])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_paged_ragged_with_poisoned_padding(dev, bs, dtype):
    from peerkv_b200 import ops
    lens = [777, 1024, 1600, 33, 4096, 0, 1, 16, 17, 5000]
    B, Hq, Hkv, D = len(lens), 32, 8, 128
    pool, bt, sl = make_paged(B, lens, Hkv, D, bs, dtype, dev, seed=bs)
    torch.manual_seed(1)
    q = torch.randn(B, Hq, D).to(dtype)
    shard = ops.Shard(dev, B, Hq)
    pd = pool.to(dev)
    out, lse = ops.decode_paged(q.to(dev), pd[0], pd[1], bt.to(dev), sl.to(dev), return_lse=True, shard=shard)
    assert shard.status() == 0
    clean = torch.nan_to_num(pool.float(), nan=0.0).to(dtype)
    ro, rl = orc.paged_partial_oracle(q, clean, bt, sl)
    assert not torch.isnan(out).any()
    assert close(out, ro)
    assert close(lse[torch.tensor(lens) > 0], rl[torch.tensor(lens) > 0], atol=2e-3, rtol=1e-4)
    assert torch.isinf(lse[5]).all() and (out[5] == 0).all()      # empty sequence
    o, l2 = ops.partial_paged(q.to(dev), pd[0], pd[1], bt.to(dev), sl.to(dev), shard=shard)
    assert close(o, ro)


def test_paged_two_device_layout_on_one_gpu_matches_golden(golden, dev):
    """The reference's paged check (experiments/test_paged_cfk.py): 5 sequences, tail
    40 % of each one's blocks in a second cache with its own id space."""
    from peerkv_b200.peerkv.paged import paged_cfk_decode, gather_seq
    c = gen_paged_case()
    out = paged_cfk_decode(c["q"].to(dev), c["local_cache"].to(dev), c["peer_cache"].to(dev),
                           c["block_table"].to(dev), torch.tensor(c["seq_lens"], device=dev),
                           c["peer_base"])
    assert out.shape == c["q"].shape and out.dtype == c["q"].dtype
    assert close(out, torch.from_numpy(golden["paged/out"]), atol=2e-3, rtol=1e-2)
    for i, (Kf, Vf) in enumerate(c["full"]):
        assert close(out[i], orc.reference_attn(c["q"][i], Kf, Vf))
    # single-cache form
    Kl, Vl, Kp, Vp = gather_seq(c["local_cache"].to(dev), c["peer_cache"].to(dev),
                                c["block_table"][0].to(dev), c["seq_lens"][0], c["peer_base"])
    assert Kl.shape[1] == int(golden["paged/n_local_tok_0"])
    assert Kl.shape[1] + Kp.shape[1] == c["seq_lens"][0]


def test_peer_fused_attn_surface(golden, dev):
    """experiments/test_fused_attn_op.py: H=32, HKV=8, D=128, randn*0.1 fp16, KV split in half."""
    from peerkv_b200.peerkv import peer_fused_attn, reference_attn, load_fused_attn
    assert load_fused_attn() is not None
    torch.manual_seed(0)
    H, HKV, D = 32, 8, 128
    for T in (1024, 4096, 16384):
        q = (torch.randn(H, D) * 0.1).half()
        Kf = (torch.randn(HKV, T, D) * 0.1).half()
        Vf = (torch.randn(HKV, T, D) * 0.1).half()
        ref = orc.reference_attn(q, Kf, Vf)
        qd, Kd, Vd = q.to(dev), Kf.to(dev), Vf.to(dev)
        O = peer_fused_attn(qd, Kd[:, :T // 2].contiguous(), Vd[:, :T // 2].contiguous(),
                            Kd[:, T // 2:].contiguous(), Vd[:, T // 2:].contiguous())
        O1 = peer_fused_attn(qd, Kd, Vd, None, None)
        assert O.shape == (H, D) and O.dtype == torch.float16
        assert close(O, ref) and close(O1, ref)
        assert close(reference_attn(qd, Kd, Vd), ref)
        cos = torch.nn.functional.cosine_similarity(O.float().flatten().cpu(), ref.flatten(), dim=0)
        assert cos > 0.999


def test_merge_kernel_matches_oracle(dev):
    from peerkv_b200 import ops
    torch.manual_seed(5)
    N, B, H, D = 8, 7, 32, 128
    o = torch.randn(N, B, H, D)
    l = torch.randn(N, B, H) * 3
    l[2] = float("-inf")                 # an empty shard
    l[:, 3, 5] = float("-inf")           # a row empty everywhere
    ref_o, ref_l = orc.merge_n(list(o), list(l))
    out, lse = ops.merge_partials(o.to(dev), l.to(dev), torch.float32, return_lse=True)
    assert close(out, ref_o, atol=1e-5, rtol=1e-4)
    fin = ~torch.isinf(ref_l)
    assert close(lse.cpu()[fin], ref_l[fin], atol=1e-5, rtol=1e-5)
    assert torch.isinf(lse[3, 5]) and (out[3, 5] == 0).all()
    for dt in (torch.float16, torch.bfloat16):
        assert close(ops.merge_partials(o.to(dev), l.to(dev), dt), ref_o.to(dt))


@pytest.mark.parametrize("fmt", ["int8", "fp8"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_quantiser_bit_exact(dev, fmt, dtype):
    from peerkv_b200 import ops
    torch.manual_seed(9)
    x = (torch.randn(4096, 8, 128) * torch.rand(4096, 8, 1) * 4).to(dtype)
    x[0, 0] = 0
    x[1, 1] = 1e-7 if dtype == torch.float16 else 1e-30
    x[2, 2, 0] = 60000.0 if dtype == torch.float16 else 3e38
    codes, scales = ops.quantize_kv(x.to(dev), fmt)
    rc, rs = orc.quantize_kv(x, fmt)
    assert torch.equal(scales.cpu().view(torch.int16), rs.view(torch.int16))
    assert torch.equal(codes.cpu().view(torch.uint8), rc.view(torch.uint8))


@pytest.mark.parametrize("n_dev", [2, 4, 8])
def test_split_block_table_bit_exact(dev, n_dev):
    import ctypes as C
    from peerkv_b200 import _lib
    rng = np.random.default_rng(n_dev)
    bs, B = 16, 9
    lens = rng.integers(0, 3000, size=B); lens[3] = 0; lens[4] = 16; lens[5] = 17
    n_pages = [(int(L) + bs - 1) // bs for L in lens]
    total = sum(n_pages)
    perm = rng.permutation(total)
    W = max(n_pages)
    bt = np.zeros((B, W), dtype=np.int32)
    k = 0
    for i, n in enumerate(n_pages):
        bt[i, :n] = perm[k:k + n]; k += n
    btd = torch.from_numpy(bt).to(dev); sld = torch.from_numpy(lens.astype(np.int32)).to(dev)
    for mode in (1, 0):
        tabs = [torch.full((B, W), -1, dtype=torch.int32, device=dev) for _ in range(n_dev)]
        outl = [torch.full((B,), -1, dtype=torch.int32, device=dev) for _ in range(n_dev)]
        bases = [d * (total // n_dev) for d in range(n_dev)]
        _lib.check(_lib.lib().pkv_split_block_table(
            0, btd.data_ptr(), W, sld.data_ptr(), B, bs, n_dev, mode, (C.c_int64 * n_dev)(*bases),
            (C.c_void_p * n_dev)(*[t.data_ptr() for t in tabs]), W,
            (C.c_void_p * n_dev)(*[t.data_ptr() for t in outl]), None))
        torch.cuda.synchronize()
        if mode == 1:
            ref = orc.round_robin_shards(bt, lens, bs, n_dev)
            for d in range(n_dev):
                assert torch.equal(outl[d].cpu(), ref[d][1])
                for i in range(B):
                    n = (int(ref[d][1][i]) + bs - 1) // bs
                    assert torch.equal(tabs[d][i, :n].cpu(), ref[d][0][i, :n])
        else:
            for i in range(B):
                ids, val = orc.split_block_row(bt[i].tolist(), int(lens[i]), bs, bases)
                for d in range(n_dev):
                    assert int(outl[d][i]) == val[d]
                    assert tabs[d][i, :len(ids[d])].cpu().tolist() == ids[d]


def test_bad_page_id_sets_status_not_a_fault(dev):
    from peerkv_b200 import ops, _lib
    B, Hq, Hkv, D, bs = 2, 32, 8, 128, 16
    pool, bt, sl = make_paged(B, [100, 200], Hkv, D, bs, torch.bfloat16, dev, seed=3, poison=False)
    bt[1, 2] = 10 ** 6
    q = torch.randn(B, Hq, D).bfloat16()
    shard = ops.Shard(dev, B, Hq)
    pd = pool.to(dev)
    ops.decode_paged(q.to(dev), pd[0], pd[1], bt.to(dev), sl.to(dev), shard=shard)
    assert shard.status() & _lib.ST_BAD_PAGE
    assert shard.status() == 0            # reading clears it


def test_large_shard_split_consistency(dev):
    """Size-independent property at a pool well above L2 (1 GiB): attention over the
    whole pool equals the merge of attention over any partition of its pages, and a
    permuted block table with permuted pages gives the same result."""
    from peerkv_b200 import ops
    torch.manual_seed(0)
    B, Hq, Hkv, D, bs = 4, 32, 8, 128, 16
    T = 32768
    n_pages = B * T // bs
    pool = torch.randn(2, n_pages, bs, Hkv, D, device=dev, dtype=torch.bfloat16)
    q = torch.randn(B, Hq, D, device=dev, dtype=torch.bfloat16)
    bt = torch.randperm(n_pages, device=dev).to(torch.int32).view(B, -1)
    sl = torch.full((B,), T, dtype=torch.int32, device=dev)
    whole = ops.decode_paged(q, pool[0], pool[1], bt, sl)
    W = bt.shape[1]
    cut = [0, W // 3, W // 3 + 1, W]
    parts = []
    for a, b in zip(cut[:-1], cut[1:]):
        sub = bt[:, a:b].contiguous()
        parts.append(ops.partial_paged(q, pool[0], pool[1], sub, torch.full((B,), (b - a) * bs,
                                       dtype=torch.int32, device=dev)))
    merged = ops.merge_partials(torch.stack([p[0] for p in parts]), torch.stack([p[1] for p in parts]),
                                torch.bfloat16)
    assert close(merged, whole, atol=1e-3, rtol=1e-2)
    # a slice small enough for the oracle pins the absolute values
    sub = bt[:1, :64].cpu()
    ro, _ = orc.paged_partial_oracle(q[:1].cpu(), pool.cpu() if False else
                                     torch.stack([pool[0].cpu(), pool[1].cpu()]), sub,
                                     torch.tensor([64 * bs], dtype=torch.int32))
    po, _ = ops.partial_paged(q[:1], pool[0], pool[1], sub.to(dev), torch.tensor([64 * bs], dtype=torch.int32, device=dev))
    assert close(po, ro)


@pytest.mark.parametrize("fmt", ["int8", "fp8"])
@pytest.mark.parametrize("qdtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Hq,Hkv", [(64, 8), (32, 8), (16, 16), (8, 2)])
def test_quantised_kv_decode(dev, fmt, qdtype, Hq, Hkv):
    """int8 / e4m3 codes with per-(token, kv-head) fp16 scales, dequantised inside the
    kernel's load path: codes and scales come from the library's own quantiser (bit-exact
    to the oracle's, see test_quantiser_bit_exact) and the attention is compared with the
    oracle run over the dequantised values.  Scales of unused rows are NaN."""
    from peerkv_b200 import ops
    bs, D = 16, 128
    lens = [700, 1024, 33, 0, 16, 2500, 1]
    B = len(lens)
    pool, bt, sl = make_paged(B, lens, Hkv, D, bs, torch.bfloat16, dev, seed=Hq + Hkv, poison=False)
    torch.manual_seed(2)
    q = torch.randn(B, Hq, D).to(qdtype)
    codes, scales = ops.quantize_kv(pool.to(dev), fmt)                  # [2, nb, bs, Hkv, D], [2, nb, bs, Hkv]
    rc, rs = orc.quantize_kv(pool, fmt)
    assert torch.equal(codes.cpu().view(torch.uint8), rc.view(torch.uint8))
    assert torch.equal(scales.cpu().view(torch.int16), rs.view(torch.int16))
    # poison the scales of every row that no sequence owns
    owned = torch.zeros(pool.shape[1], bs, dtype=torch.bool)
    for i, L in enumerate(lens):
        n = (L + bs - 1) // bs
        for j in range(n):
            owned[bt[i, j], :min(bs, L - j * bs)] = True
    sc_p = scales.clone()
    sc_p[:, ~owned.to(dev)] = float("nan")
    shard = ops.Shard(dev, B, Hq)
    out, lse = ops.decode_paged(q.to(dev), codes[0], codes[1], bt.to(dev), sl.to(dev), return_lse=True,
                                k_scale=sc_p[0], v_scale=sc_p[1], shard=shard)
    assert shard.status() == 0
    assert not torch.isnan(out).any()
    ro, rl = orc.paged_partial_oracle(q, rc, bt, sl, k_scale=rs[0], v_scale=rs[1])
    assert close(out, ro)
    has = torch.tensor(lens) > 0
    assert close(lse[has], rl[has], atol=2e-3, rtol=1e-4)
    assert torch.isinf(lse[3]).all() and (out[3] == 0).all()
    # and against the un-quantised pool: the quantisation error itself stays small
    rf, _ = orc.paged_partial_oracle(q, pool, bt, sl)
    tol = 4e-2 if fmt == "int8" else 0.3           # a 1-token sequence returns V itself: up to 2^-4 relative in e4m3
    assert (out.float().cpu() - rf)[has].abs().max() < tol
