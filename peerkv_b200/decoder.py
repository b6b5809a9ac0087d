"""A Llama-architecture decode step whose attention runs on the sharded-KV path.

The counterpart of PeerKV's full-layer bench (csrc/peer_fused_decoder.cu:188-239,
`peer_decoder_layer`: rmsnorm -> q/k/v projections -> attention over a local and a
peer KV shard -> output projection -> residual -> rmsnorm -> gate/up -> swiglu -> down
-> residual), extended to what the Llama-3 configuration needs (RoPE, appending the
new token's K/V to the paged cache, batch > 1, N GPUs).

Per layer, on the home GPU (everything but attention lives there, as in the reference):

    pkv_add_rmsnorm   x += previous MLP output; h = rmsnorm(x) * w1        (library kernel)
    h @ Wqkv                                                                (cuBLAS, weight-bandwidth bound)
    pkv_rope_append   RoPE on q and k; k, v into the page slot of the pool  (library kernel)
    pkv_home_step     q out to the peers, own shard, peers' partials merged (library kernel)
    attn @ Wo                                                               (cuBLAS)
    pkv_add_rmsnorm   x += attention output; h = rmsnorm(x) * w2
    h @ Wgate_up ; pkv_swiglu ; act @ Wdown                                 (cuBLAS, library kernel, cuBLAS)

and one `pkv_peer_step` per layer on every peer.  New tokens are appended to pages that
the home GPU owns ("newest page local"), so the append is a local write.

`capture()` records the WHOLE step of a rank -- all layers, attention launches included --
as one CUDA graph per GPU (the reference captures its two-device step the same way,
csrc/peer_rt_bench.cu:134-154, csrc/peer_fused_decoder.cu:433-455).  The attention kernels
take their epoch relative to a device-resident base that the graph's last node advances,
so a replay is a valid next step.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import List, Optional

import torch

from . import _lib, ops
from ._lib import check


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


def rope_inv_freq(head_dim: int, theta: float, device) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device, dtype=torch.float32) / head_dim))


def rope_tables(pos: torch.Tensor, head_dim: int, theta: float):
    """cos / sin [B, 1, D/2] (fp32) for integer positions pos [B] (torch reference of the kernel)."""
    ang = pos.to(torch.float32)[:, None] * rope_inv_freq(head_dim, theta, pos.device)[None, :]
    return ang.cos()[:, None, :], ang.sin()[:, None, :]


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, H, D]; rotate-half convention (torch reference of the kernel)."""
    D = x.shape[-1]
    x1, x2 = x[..., : D // 2].float(), x[..., D // 2:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


# ---- the library's layer kernels on torch tensors ------------------------------------- #
def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, out: torch.Tensor,
                eps: float):
    """x [rows, hidden] (updated in place when delta is given) -> out = rmsnorm(x) * weight."""
    check(_lib.lib().pkv_add_rmsnorm(x.device.index, x.data_ptr(), delta.data_ptr() if delta is not None else None,
                                     weight.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], float(eps),
                                     ops._DT[x.dtype], ops._stream(x.device)))
    return out


def rope_append(qkv: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, q_out: torch.Tensor,
                n_q_heads: int, n_kv_heads: int, pool: Optional[torch.Tensor] = None,
                pages: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None):
    """qkv [B, (Hq + 2 Hkv) D]; q_out [B, Hq, D]; pool [2, n_pages, page, Hkv, D] or None."""
    D = q_out.shape[-1]
    if pool is not None:
        k, v = pool[0], pool[1]
        args = (k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1), k.stride(2), pages.data_ptr(), slots.data_ptr())
    else:
        args = (None, None, 0, 0, 0, None, None)
    check(_lib.lib().pkv_rope_append(qkv.device.index, qkv.data_ptr(), positions.data_ptr(), inv_freq.data_ptr(),
                                     qkv.shape[0], n_q_heads, n_kv_heads, D, q_out.data_ptr(), *args,
                                     ops._DT[qkv.dtype], ops._stream(qkv.device)))
    return q_out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor):
    check(_lib.lib().pkv_swiglu(gate_up.device.index, gate_up.data_ptr(), out.data_ptr(), gate_up.shape[0],
                                out.shape[1], ops._DT[gate_up.dtype], ops._stream(gate_up.device)))
    return out


class ShardedKVLayer:
    """One layer's share of the paged KV on this GPU: pool [2, n_pages, page, Hkv, D], the
    local block table and the per-sequence token counts of this shard."""

    def __init__(self, pool, table, lens):
        self.pool, self.table, self.lens = pool, table, lens
        self.view = ops.paged_view(pool[0], pool[1])


def make_args(q_like: torch.Tensor, layer: ShardedKVLayer, scale: float) -> _lib.DecodeArgs:
    return ops.make_args(q_like, layer.view, layer.table, layer.table.stride(0), layer.lens, scale)


class DecodeStep:
    """Decode steps of the model on one rank.

    Home rank (weights given): the whole model, attention through `group` (a
    distributed.DistPeerGroup) or, with no group, through a one-GPU shard.  Peer rank
    (weights None): one peer step per layer.  `append_slots` = (page ids [B], token slots
    [B]) int64 on the home GPU: where each sequence's new token goes in every layer's pool.
    """

    def __init__(self, g: LlamaGeometry, weights: Optional[ModelWeights], kv: List[ShardedKVLayer], batch: int,
                 device, group=None, append_slots=None):
        self.g, self.w, self.kv, self.group = g, weights, kv, group
        self.dev = torch.device(device)
        self.B = batch
        self.append_slots = append_slots
        self.scale = 1.0 / math.sqrt(g.head_dim)
        self._graph = None
        dev, dt = self.dev, torch.bfloat16 if weights is None else weights.embed.dtype
        self.q = torch.zeros(batch, g.n_q_heads, g.head_dim, dtype=dt, device=dev)
        self.args = [make_args(self.q, l, self.scale) for l in kv]
        self.shard = group.shard if group is not None else ops.Shard(dev, batch, g.n_q_heads)
        if weights is not None:
            nq, nkv = g.n_q_heads * g.head_dim, g.n_kv_heads * g.head_dim
            z = lambda *s, d=dt: torch.zeros(*s, dtype=d, device=dev)
            self.tok, self.pos = z(batch, d=torch.int64), z(batch, d=torch.int64)
            self.x, self.h = z(batch, g.hidden), z(batch, g.hidden)
            self.qkv = z(batch, nq + 2 * nkv)
            self.ao = z(batch, g.n_q_heads, g.head_dim)
            self.proj, self.mlp = z(batch, g.hidden), z(batch, g.hidden)
            self.gu, self.act = z(batch, 2 * g.ffn), z(batch, g.ffn)
            self.logits = z(batch, g.vocab)
            self.next = z(batch, d=torch.int64)
            self.inv_freq = rope_inv_freq(g.head_dim, g.rope_theta, dev)

    # -- attention of one layer ---------------------------------------------------------- #
    def _attend(self, li: int):
        L, st = _lib.lib(), ops._stream(self.dev)
        if self.group is None:
            check(L.pkv_decode(self.shard._h, C.byref(self.args[li]), self.ao.data_ptr(), ops._DT[self.ao.dtype],
                               None, st))
        else:
            self.group.step(self.args[li], q=self.q, out=self.ao)

    # -- the step as a sequence of launches (what the graph records) ---------------------- #
    def _body(self):
        g = self.g
        if self.w is None:                                   # a peer: its shard's partial, layer by layer
            for li in range(g.n_layers):
                self.group.step(self.args[li])
            return
        torch.index_select(self.w.embed, 0, self.tok, out=self.x)
        delta = None
        for li, lw in enumerate(self.w.layers):
            add_rmsnorm(self.x, delta, lw.norm1, self.h, g.rms_eps)
            torch.matmul(self.h, lw.wqkv, out=self.qkv)
            pool = self.kv[li].pool if self.append_slots is not None else None
            pages, slots = self.append_slots if self.append_slots is not None else (None, None)
            rope_append(self.qkv, self.pos, self.inv_freq, self.q, g.n_q_heads, g.n_kv_heads, pool, pages, slots)
            self._attend(li)
            torch.matmul(self.ao.view(self.B, -1), lw.wo, out=self.proj)
            add_rmsnorm(self.x, self.proj, lw.norm2, self.h, g.rms_eps)
            torch.matmul(self.h, lw.w_gate_up, out=self.gu)
            swiglu(self.gu, self.act)
            torch.matmul(self.act, lw.w_down, out=self.mlp)
            delta = self.mlp
        add_rmsnorm(self.x, delta, self.w.final_norm, self.h, g.rms_eps)
        torch.matmul(self.h, self.w.lm_head, out=self.logits)
        torch.argmax(self.logits, dim=-1, out=self.next)

    def capture(self, warmup: int = 2):
        """Records the whole step of this rank as ONE CUDA graph.  Every rank of the group
        calls this together (the warm-up steps are real steps)."""
        dev = self.dev
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._body()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        if self.group is not None:
            self.group.barrier()
        gr = torch.cuda.CUDAGraph()
        if self.group is not None:
            self.group.capture_begin()
        with torch.cuda.graph(gr):
            self._body()
            if self.group is not None:
                self.group.capture_end()          # last node: advances the device-resident epoch base
        self._graph = gr

    def step(self, tokens: Optional[torch.Tensor] = None, positions: Optional[torch.Tensor] = None):
        """One decode step: tokens [B] int64, positions [B] (index of the new token) ->
        next tokens [B] on the home rank; peers pass nothing and get None."""
        if self.w is not None:
            self.tok.copy_(tokens)
            self.pos.copy_(positions)
        if self._graph is not None:
            self._graph.replay()
            if self.group is not None:
                self.group.replayed()
        else:
            self._body()
        return self.next if self.w is not None else None

    # kept for callers of the earlier interface
    def home_step(self, tokens, positions):
        return self.step(tokens, positions)

    def attention_only(self):
        """The attention launches of one step and nothing else (timing aid)."""
        for li in range(self.g.n_layers):
            if self.w is None:
                self.group.step(self.args[li])
            else:
                self._attend(li)
