"""ring_prefill_attention and multi-query partials (reference
umallm/peer_parallel_attn.py:112-140 and tests/test_peer_parallel.py:63-95).

CPU: the host-side construction (one "sequence" per query row, causality by length) is
checked against dense causal attention with the CPU oracle standing in for the one
library call.  GPU: the same entry points on the real kernels."""
import pytest
import torch
import torch.nn.functional as F

from oracle import peerkv_oracle as orc


@pytest.fixture
def oracle_backed(monkeypatch):
    from peerkv_b200 import ops, peer_parallel_attn as ppa

    def fake_rows(q_rows, K, V, row_page, row_len, scale):
        R, H, D = q_rows.shape
        o = torch.zeros(R, H, D)
        l = torch.full((R, H), float("-inf"))
        for r in range(R):
            b, n = int(row_page[r]), int(row_len[r])
            oo, ll = orc.dense_attention_lse_fp32(q_rows[r].view(1, H, 1, D), K[b:b + 1, :, :n], V[b:b + 1, :, :n], scale)
            o[r], l[r] = oo.view(H, D), ll.view(H)
        return o, l

    def fake_merge(o_parts, lse_parts, out_dtype=torch.float32, return_lse=False):
        O, L = orc.merge_n(list(o_parts), list(lse_parts))
        return (O.to(out_dtype), L) if return_lse else O.to(out_dtype)

    monkeypatch.setattr(ppa, "_decode_partial_rows", fake_rows)
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
