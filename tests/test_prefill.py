"""ring_prefill_attention and multi-query partials (reference
umallm/peer_parallel_attn.py:112-140 and tests/test_peer_parallel.py:63-95).

CPU: the host-side construction (which shard pairs are computed, which one is causal,
what is merged) is checked against dense causal attention with the CPU oracle standing in
for the per-shard library call.  GPU: the same entry points on the real kernels, and the
prefill kernel itself against fp32 attention over edge shapes."""
import pytest
import torch
import torch.nn.functional as F

from oracle import peerkv_oracle as orc


@pytest.fixture
def oracle_backed(monkeypatch):
    from peerkv_b200 import ops, peer_parallel_attn as ppa

    def fake_partial(q, K, V, scale, causal_diagonal=False):
        """What the library computes for a shard, from the oracle: every key, or keys <= the row."""
        B, H, Lq, D = q.shape
        if not causal_diagonal:
            return orc.dense_attention_lse_fp32(q, K, V, scale)
        o = torch.zeros(B, H, Lq, D)
        l = torch.full((B, H, Lq), float("-inf"))
        for r in range(Lq):
            oo, ll = orc.dense_attention_lse_fp32(q[:, :, r:r + 1], K[:, :, :r + 1], V[:, :, :r + 1], scale)
            o[:, :, r], l[:, :, r] = oo[:, :, 0], ll[:, :, 0]
        return o, l

    def fake_merge(o_parts, lse_parts, out_dtype=torch.float32, return_lse=False):
        O, L = orc.merge_n(list(o_parts), list(lse_parts))
        return (O.to(out_dtype), L) if return_lse else O.to(out_dtype)

    monkeypatch.setattr(ppa, "_partial_f32", fake_partial)
    monkeypatch.setattr(ops, "merge_partials", fake_merge)
    return ppa


def test_ring_prefill_host_logic_matches_dense_causal(oracle_backed):
    """Shapes of the reference's test_ring_prefill_causal_exact_vs_dense (3 x 200, H 4, D 64)."""
    torch.manual_seed(5)
    B, H, S, D = 1, 4, 600, 64
    Q, K, V = torch.randn(B, H, S, D), torch.randn(B, H, S, D), torch.randn(B, H, S, D)
    ref = F.scaled_dot_product_attention(Q, K, V, is_causal=True)
    cuts = [200, 200, 200]
    shards = list(zip(Q.split(cuts, 2), K.split(cuts, 2), V.split(cuts, 2)))
    out = torch.cat(oracle_backed.ring_prefill_attention(shards), dim=2)
    assert torch.allclose(ref, out, atol=1e-4, rtol=1e-4)
    one = oracle_backed.ring_prefill_attention([(Q[:, :, :130], K[:, :, :130], V[:, :, :130])])[0]
    assert torch.allclose(F.scaled_dot_product_attention(Q[:, :, :130], K[:, :, :130], V[:, :, :130], is_causal=True),
                          one, atol=1e-4, rtol=1e-4)


def test_multi_query_host_logic(oracle_backed):
    torch.manual_seed(3)
    q, K, V = torch.randn(2, 4, 5, 64), torch.randn(2, 4, 200, 64), torch.randn(2, 4, 200, 64)
    o, lse = oracle_backed._partial_f32(q, K, V, 1.0 / 8)
    assert torch.allclose(o, F.scaled_dot_product_attention(q, K, V), atol=1e-5, rtol=1e-4)
    assert lse.shape == (2, 4, 5)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("Sq,Sk,causal,qp,kp", [
    (1, 1, True, 0, 0), (64, 64, True, 0, 0), (65, 65, True, 0, 0), (200, 200, True, 0, 0),
    (130, 1000, False, 0, 0), (63, 7, False, 0, 0), (300, 300, True, 300, 300),
    (128, 256, True, 256, 64),          # a later query shard against an earlier, overlapping key range
    (100, 50, True, 0, 80),             # keys that start after some rows: those rows see nothing
    (17, 0, False, 0, 0),               # an empty shard
])
def test_prefill_partial_kernel(dt, Sq, Sk, causal, qp, kp):
    """pkv_prefill_partial against fp32 attention with the same visibility rule."""
    from peerkv_b200 import peer_parallel_attn as ppa
    dev = torch.device("cuda", 0)
    torch.manual_seed(Sq * 1000 + Sk)
    B, H, Hkv, D = 2, 8, 2, 128
    q = torch.randn(B, H, Sq, D).to(dt)
    K = torch.randn(B, Hkv, Sk, D).to(dt)
    V = torch.randn(B, Hkv, Sk, D).to(dt)
    o, lse = ppa._prefill_partial(q.to(dev), K.to(dev), V.to(dev), 1.0 / D ** 0.5, causal, qp, kp)
    Ke, Ve = K.float().repeat_interleave(H // Hkv, 1), V.float().repeat_interleave(H // Hkv, 1)
    s = (q.float() / D ** 0.5) @ Ke.transpose(-1, -2)
    if causal:
        vis = (kp + torch.arange(Sk))[None, :] <= (qp + torch.arange(Sq))[:, None]
        s = s.masked_fill(~vis, float("-inf"))
    ref_lse = torch.logsumexp(s, dim=-1) if Sk else torch.full((B, H, Sq), float("-inf"))
    seen = torch.isfinite(ref_lse)
    w = torch.softmax(s, dim=-1) if Sk else s
    w = torch.where(seen[..., None], w, torch.zeros_like(w))
    ref = w @ Ve
    assert torch.allclose(o.cpu(), ref, atol=2e-3, rtol=1e-2)
    assert torch.equal(torch.isfinite(lse.cpu()), seen)
    assert torch.allclose(lse.cpu()[seen], ref_lse[seen], atol=2e-3, rtol=1e-3)
    assert (o.cpu()[~seen] == 0).all()


@pytest.mark.gpu
def test_ring_prefill_on_gpu():
    from peerkv_b200.peer_parallel_attn import ring_prefill_attention
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    B, H, Hkv, S, D = 1, 8, 2, 300, 128
    Q = torch.randn(B, H, S, D).half()
    K = torch.randn(B, Hkv, S, D).half()
    V = torch.randn(B, Hkv, S, D).half()
    ref = F.scaled_dot_product_attention(Q.float(), K.float().repeat_interleave(4, 1), V.float().repeat_interleave(4, 1),
                                         is_causal=True)
    cuts = [100, 70, 130]
    shards = [(q.contiguous().to(dev), k.contiguous().to(dev), v.contiguous().to(dev))
              for q, k, v in zip(Q.split(cuts, 2), K.split(cuts, 2), V.split(cuts, 2))]
    out = torch.cat([o.cpu() for o in ring_prefill_attention(shards)], dim=2)
    assert torch.allclose(out.float(), ref, atol=2e-3, rtol=1e-2)


@pytest.mark.gpu
def test_multi_query_partial_on_gpu():
    from peerkv_b200.peer_parallel_attn import flash_partial, peer_parallel_attention
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    q = torch.randn(2, 8, 5, 128).bfloat16()
    K = torch.randn(2, 2, 200, 128).bfloat16()
    V = torch.randn(2, 2, 200, 128).bfloat16()
    ref = orc.dense_attention_fp32(q, K, V)
    out = peer_parallel_attention(q.to(dev), [(K[:, :, :50].to(dev), V[:, :, :50].to(dev)),
                                              (K[:, :, 50:].to(dev), V[:, :, 50:].to(dev))])
    assert torch.allclose(out.float().cpu(), ref, atol=2e-3, rtol=1e-2)
    O, lse = flash_partial(q.to(dev), K.to(dev), V.to(dev))
    assert O.shape == q.shape and lse.shape == q.shape[:3]
