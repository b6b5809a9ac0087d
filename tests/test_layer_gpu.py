"""The decoder-layer kernels around the attention call (RMSNorm with the residual add,
RoPE with the KV append, SwiGLU) against plain torch fp32 references of the same ops, and
the whole decode step -- eager and as ONE captured CUDA graph -- against a torch
restatement of the layer with its attention computed by the CPU oracle."""
import math

import pytest
import torch
import torch.nn.functional as F

from oracle import peerkv_oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,hidden", [(1, 4096), (4, 4096), (3, 1024), (7, 8192), (2, 136)])
def test_add_rmsnorm(dev, dt, rows, hidden):
    from peerkv_b200.decoder import add_rmsnorm
    torch.manual_seed(rows * hidden)
    x = torch.randn(rows, hidden, device=dev).to(dt)
    d = torch.randn(rows, hidden, device=dev).to(dt)
    w = (1 + 0.1 * torch.randn(hidden, device=dev)).to(dt)
    out = torch.empty_like(x)
    # without a residual: x untouched
    x0 = x.clone()
    add_rmsnorm(x, None, w, out, 1e-5)
    ref = (x0.float() * torch.rsqrt(x0.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float())
    assert torch.equal(x, x0)
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=1e-2)
    # with the residual add: x is updated exactly as a separate add would
    add_rmsnorm(x, d, w, out, 1e-5)
    xs = (x0.float() + d.float()).to(dt)
    assert torch.equal(x, xs)
    ref = (xs.float() * torch.rsqrt(xs.float().pow(2).mean(-1, keepdim=True) + 1e-5) * w.float())
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=1e-2)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
def test_rope_append(dev, dt):
    from peerkv_b200.decoder import rope, rope_append, rope_inv_freq, rope_tables
    torch.manual_seed(1)
    B, Hq, Hkv, D, bs, n_pages = 5, 32, 8, 128, 16, 12
    qkv = torch.randn(B, (Hq + 2 * Hkv) * D, device=dev).to(dt)
    pos = torch.tensor([0, 1, 77, 131071, 1048575], device=dev)
    inv = rope_inv_freq(D, 500000.0, dev)
    pool = torch.zeros(2, n_pages, bs, Hkv, D, dtype=dt, device=dev)
    pages = torch.tensor([3, 0, 11, 7, 5], device=dev)
    slots = torch.tensor([0, 15, 4, 9, 1], device=dev)
    q = torch.empty(B, Hq, D, dtype=dt, device=dev)
    rope_append(qkv, pos, inv, q, Hq, Hkv, pool, pages, slots)
    cos, sin = rope_tables(pos, D, 500000.0)
    heads = qkv.view(B, Hq + 2 * Hkv, D)
    ref = rope(heads[:, :Hq + Hkv], cos, sin)
    assert torch.allclose(q.float(), ref[:, :Hq].float(), atol=2e-2, rtol=1e-2)
    assert torch.allclose(pool[0, pages, slots].float(), ref[:, Hq:].float(), atol=2e-2, rtol=1e-2)
    assert torch.equal(pool[1, pages, slots], heads[:, Hq + Hkv:])
    untouched = torch.ones(n_pages, bs, dtype=torch.bool, device=dev)
    untouched[pages, slots] = False
    assert (pool[:, untouched] == 0).all()
    # no pools: q only
    q2 = torch.empty_like(q)
    rope_append(qkv, pos, inv, q2, Hq, Hkv)
    assert torch.equal(q, q2)


@pytest.mark.parametrize("dt", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,ffn", [(4, 14336), (1, 2048), (3, 8)])
def test_swiglu(dev, dt, rows, ffn):
    from peerkv_b200.decoder import swiglu
    torch.manual_seed(ffn)
    gu = torch.randn(rows, 2 * ffn, device=dev).to(dt)
    out = torch.empty(rows, ffn, dtype=dt, device=dev)
    swiglu(gu, out)
    ref = F.silu(gu[:, :ffn].float()) * gu[:, ffn:].float()
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)


def _torch_step(g, w, layers, tokens, pos, append):
    """The decode step in plain torch ops, attention by the CPU oracle on the gathered KV."""
    from peerkv_b200.decoder import rope, rope_tables
    x = w.embed[tokens].clone()
    B = x.shape[0]
    nq, nkv = g.n_q_heads * g.head_dim, g.n_kv_heads * g.head_dim
    cos, sin = rope_tables(pos, g.head_dim, g.rope_theta)
    for li, lw in enumerate(w.layers):
        h = F.rms_norm(x, (g.hidden,), lw.norm1, g.rms_eps)
        qkv = h @ lw.wqkv
        qk = rope(qkv[:, :nq + nkv].view(B, g.n_q_heads + g.n_kv_heads, g.head_dim), cos, sin)
        pages, slots = append
        pool = layers[li].pool
        pool[0, pages, slots] = qk[:, g.n_q_heads:]
        pool[1, pages, slots] = qkv[:, nq + nkv:].view(B, g.n_kv_heads, g.head_dim)
        l = layers[li]
        o, _ = orc.paged_partial_oracle(qk[:, :g.n_q_heads].contiguous().cpu(), l.pool.cpu(), l.table.cpu(), l.lens.cpu())
        ao = o.to(x.dtype).to(x.device)
        x = x + ao.view(B, nq) @ lw.wo
        h = F.rms_norm(x, (g.hidden,), lw.norm2, g.rms_eps)
        gu = h @ lw.w_gate_up
        x = x + (F.silu(gu[:, :g.ffn]) * gu[:, g.ffn:]) @ lw.w_down
    h = F.rms_norm(x, (g.hidden,), w.final_norm, g.rms_eps)
    return h @ w.lm_head


def test_decode_step_eager_and_as_one_graph(dev):
    from peerkv_b200.decoder import DecodeStep, LlamaGeometry, ModelWeights, ShardedKVLayer
    torch.manual_seed(0)
    g = LlamaGeometry(n_layers=2, hidden=1024, n_q_heads=8, n_kv_heads=2, head_dim=128, ffn=2048, vocab=512)
    B, bs = 3, 16
    lens = [48, 160, 16]                                   # whole pages; the new token opens a new page
    n_pages = [L // bs for L in lens]
    total = sum(n_pages)
    W = max(n_pages) + 1
    layers = []
    for li in range(g.n_layers):
        pool = torch.zeros(2, total + B, bs, g.n_kv_heads, g.head_dim, dtype=torch.bfloat16, device=dev)
        pool[:, :total].normal_()
        tab = torch.zeros(B, W, dtype=torch.int32, device=dev)
        k = 0
        for i, n in enumerate(n_pages):
            tab[i, :n] = torch.arange(k, k + n, dtype=torch.int32)
            tab[i, n] = total + i
            k += n
        ln = torch.tensor([L + 1 for L in lens], dtype=torch.int32, device=dev)
        layers.append(ShardedKVLayer(pool, tab, ln))
    w = ModelWeights(g, dev)
    append = (torch.arange(total, total + B, device=dev), torch.zeros(B, dtype=torch.int64, device=dev))
    tokens = torch.tensor([5, 17, 400], device=dev)
    pos = torch.tensor(lens, device=dev)
    pools0 = [l.pool.clone() for l in layers]

    def restore():
        for l, p0 in zip(layers, pools0):
            l.pool.copy_(p0)

    ref_logits = _torch_step(g, w, layers, tokens, pos, append).float()
    k_ref = layers[0].pool[0, total:total + B, 0].clone()
    restore()
    ds = DecodeStep(g, w, layers, B, dev, append_slots=append)
    nxt = ds.step(tokens, pos).clone()
    torch.cuda.synchronize()
    assert ds.shard.status() == 0
    assert torch.allclose(ds.logits.float(), ref_logits, atol=3e-2, rtol=3e-2)
    assert torch.allclose(layers[0].pool[0, total:total + B, 0].float(), k_ref.float(), atol=2e-2, rtol=1e-2)
    assert k_ref.abs().sum() > 0
    top2 = ref_logits.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 0.1                 # where the winner is not a rounding toss-up
    assert torch.equal(nxt[clear], ref_logits.argmax(-1)[clear])
    eager_logits = ds.logits.clone()
    # the same step as ONE graph: identical launches, so identical bits, replay after replay
    restore()
    ds.capture()
    for rep in range(3):
        restore()
        out = ds.step(tokens, pos)
        torch.cuda.synchronize()
        assert torch.equal(ds.logits, eager_logits), f"replay {rep}"
        assert torch.equal(out, nxt)
    assert ds.shard.status() == 0
