"""A Llama-architecture decode step whose attention runs on the sharded-KV path.

The counterpart of PeerKV's full-layer bench (csrc/peer_fused_decoder.cu:188-239,
`peer_decoder_layer`: rmsnorm -> q/k/v projections -> attention over a local and a
peer KV shard -> output projection -> residual -> rmsnorm -> gate/up -> swiglu -> down
-> residual), extended to what the Llama-3 configuration needs (RoPE, appending the
new token's K/V to the paged cache, batch > 1, N GPUs).

Everything except attention runs on the home GPU with plain torch ops (the
projections are weight-bandwidth-bound library GEMMs, as in the reference, which
calls cuBLAS); attention is one `pkv_home_step` per layer on the home GPU and one
`pkv_peer_step` per layer on every peer.  New tokens are appended to pages that the
home GPU owns ("newest page local"), so the append is a local write.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import _lib, ops


@dataclass
class LlamaGeometry:
    n_layers: int = 32
    hidden: int = 4096
    n_q_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0


class LayerWeights:
    def __init__(self, g: LlamaGeometry, device, dtype=torch.bfloat16, std: float = 0.02):
        def w(*shape):
            return torch.empty(*shape, dtype=dtype, device=device).normal_(0.0, std)
        kv = g.n_kv_heads * g.head_dim
        self.wqkv = w(g.hidden, g.n_q_heads * g.head_dim + 2 * kv)   # fused q|k|v projection
        self.wo = w(g.n_q_heads * g.head_dim, g.hidden)
        self.w_gate_up = w(g.hidden, 2 * g.ffn)
        self.w_down = w(g.ffn, g.hidden)
        self.norm1 = torch.ones(g.hidden, dtype=dtype, device=device)
        self.norm2 = torch.ones(g.hidden, dtype=dtype, device=device)


class ModelWeights:
    """Random-init weights of the whole model on the home GPU."""

    def __init__(self, g: LlamaGeometry, device, dtype=torch.bfloat16):
        self.g = g
        self.embed = torch.empty(g.vocab, g.hidden, dtype=dtype, device=device).normal_(0.0, 0.02)
        self.layers = [LayerWeights(g, device, dtype) for _ in range(g.n_layers)]
        self.final_norm = torch.ones(g.hidden, dtype=dtype, device=device)
        self.lm_head = torch.empty(g.hidden, g.vocab, dtype=dtype, device=device).normal_(0.0, 0.02)

    def bytes(self) -> int:
        n = self.embed.numel() + self.lm_head.numel() + self.final_norm.numel()
        for l in self.layers:
            n += sum(t.numel() for t in (l.wqkv, l.wo, l.w_gate_up, l.w_down, l.norm1, l.norm2))
        return n * self.embed.element_size()


def rope_tables(pos: torch.Tensor, head_dim: int, theta: float):
    """cos / sin [B, 1, D/2] (fp32) for integer positions pos [B]."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=pos.device, dtype=torch.float32) / head_dim))
    ang = pos.to(torch.float32)[:, None] * inv[None, :]
    return ang.cos()[:, None, :], ang.sin()[:, None, :]


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, H, D]; rotate-half convention."""
    D = x.shape[-1]
    x1, x2 = x[..., : D // 2].float(), x[..., D // 2:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class ShardedKVLayer:
    """One layer's share of the paged KV on this GPU: pool [2, n_pages, page, Hkv, D], the
    local block table and the per-sequence token counts of this shard."""

    def __init__(self, pool, table, lens):
        self.pool, self.table, self.lens = pool, table, lens
        self.view = ops.paged_view(pool[0], pool[1])


class DecodeStep:
    """Runs decode steps of the model.  `attend(layer, q, out)` is supplied by the caller:
    one GPU -> pkv_decode; several -> the group's home step.  Peers run `peer_layers`."""

    def __init__(self, g: LlamaGeometry, weights: Optional[ModelWeights], kv: List[ShardedKVLayer],
                 attend, append_slots=None):
        self.g, self.w, self.kv, self.attend = g, weights, kv, attend
        self.append_slots = append_slots          # (page ids [B], slot in page [B]) on the home GPU, or None
        self.scale = 1.0 / math.sqrt(g.head_dim)

    # -- the per-layer pieces around the attention call ------------------------------ #
    def _pre(self, li, x, cos, sin, q_out):
        g, lw, F = self.g, self.w.layers[li], torch.nn.functional
        B = x.shape[0]
        nq, nkv = g.n_q_heads * g.head_dim, g.n_kv_heads * g.head_dim
        h = F.rms_norm(x, (g.hidden,), lw.norm1, g.rms_eps)
        qkv = h @ lw.wqkv
        qk = rope(qkv[:, :nq + nkv].view(B, g.n_q_heads + g.n_kv_heads, g.head_dim), cos, sin)
        q_out.copy_(qk[:, :g.n_q_heads])
        if self.append_slots is not None:         # the new token's K/V into home-owned pages
            pages, slots = self.append_slots
            pool = self.kv[li].pool
            pool[0, pages, slots] = qk[:, g.n_q_heads:]
            pool[1, pages, slots] = qkv[:, nq + nkv:].view(B, g.n_kv_heads, g.head_dim)

    def _post(self, li, x, attn_out):
        g, lw, F = self.g, self.w.layers[li], torch.nn.functional
        B = x.shape[0]
        x.add_(attn_out.view(B, g.n_q_heads * g.head_dim) @ lw.wo)
        h = F.rms_norm(x, (g.hidden,), lw.norm2, g.rms_eps)
        gu = h @ lw.w_gate_up
        x.add_((F.silu(gu[:, :g.ffn]) * gu[:, g.ffn:]) @ lw.w_down)

    def capture(self, batch: int):
        """Records the non-attention pieces as CUDA graphs over static buffers (one graph
        before and one after each layer's attention call, as the reference's bench captures
        its layer, csrc/peer_fused_decoder.cu:433-455).  The attention call itself stays a
        plain launch between them: its epoch changes every step."""
        g, dev = self.g, self.w.embed.device
        dt = self.w.embed.dtype
        self._tok = torch.zeros(batch, dtype=torch.int64, device=dev)
        self._pos = torch.zeros(batch, dtype=torch.int64, device=dev)
        self._x = torch.zeros(batch, g.hidden, dtype=dt, device=dev)
        self._q = torch.zeros(batch, g.n_q_heads, g.head_dim, dtype=dt, device=dev)
        self._ao = torch.zeros(batch, g.n_q_heads, g.head_dim, dtype=dt, device=dev)
        self._next = torch.zeros(batch, dtype=torch.int64, device=dev)

        self._cos = torch.zeros(batch, 1, g.head_dim // 2, dtype=torch.float32, device=dev)
        self._sin = torch.zeros_like(self._cos)

        def head():
            self._x.copy_(self.w.embed[self._tok])
            c, s_ = rope_tables(self._pos, g.head_dim, g.rope_theta)
            self._cos.copy_(c)
            self._sin.copy_(s_)

        def tail():
            F = torch.nn.functional
            h = F.rms_norm(self._x, (g.hidden,), self.w.final_norm, g.rms_eps)
            self._next.copy_((h @ self.w.lm_head).argmax(dim=-1))

        pieces = [head]
        for li in range(g.n_layers):
            pieces.append(lambda li=li: self._pre(li, self._x, self._cos, self._sin, self._q))
            pieces.append(lambda li=li: self._post(li, self._x, self._ao))
        pieces.append(tail)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(2):
                for f in pieces:
                    f()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self._graphs = []
        pool = None
        for f in pieces:
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr, pool=pool):
                f()
            pool = gr.pool()
            self._graphs.append(gr)

    def home_step(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """tokens [B] int64, positions [B] (index of the new token) -> next tokens [B]."""
        g = self.g
        if getattr(self, "_graphs", None):
            self._tok.copy_(tokens)
            self._pos.copy_(positions)
            self._graphs[0].replay()
            for li in range(g.n_layers):
                self._graphs[1 + 2 * li].replay()
                self.attend(li, self._q, self._ao)
                self._graphs[2 + 2 * li].replay()
            self._graphs[-1].replay()
            return self._next
        F = torch.nn.functional
        x = self.w.embed[tokens].clone()
        B = x.shape[0]
        q = torch.empty(B, g.n_q_heads, g.head_dim, dtype=x.dtype, device=x.device)
        attn_out = torch.empty_like(q)
        cos, sin = rope_tables(positions, g.head_dim, g.rope_theta)
        for li in range(g.n_layers):
            self._pre(li, x, cos, sin, q)
            self.attend(li, q, attn_out)
            self._post(li, x, attn_out)
        x = F.rms_norm(x, (g.hidden,), self.w.final_norm, g.rms_eps)
        return (x @ self.w.lm_head).argmax(dim=-1)


def make_args(q_like: torch.Tensor, layer: ShardedKVLayer, scale: float) -> _lib.DecodeArgs:
    return ops.make_args(q_like, layer.view, layer.table, layer.table.stride(0), layer.lens, scale)
