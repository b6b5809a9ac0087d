"""Tensor-level entry points over the C-ABI library: one GPU's shard context, the
paged / contiguous decode calls, the N-way merge and the KV quantiser.

torch is used for device memory and the current stream only; all device work is
done by libpeerkv.so.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import DecodeArgs, KvView, PeerKVError, check

_DT = {torch.float16: _lib.PKV_F16, torch.bfloat16: _lib.PKV_BF16, torch.float32: _lib.PKV_F32,
       torch.int8: _lib.PKV_INT8, torch.float8_e4m3fn: _lib.PKV_FP8_E4M3}
HEAD_DIM = 128


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str):
    if not t.is_cuda:
        raise PeerKVError(f"{name} must be a CUDA tensor (this package has no CPU path)")


class Shard:
    """One GPU's attention context: persistent split-K scratch and status word
    (replaces the per-call scratch of PeerKV csrc/peer_fused_attn_ext.cu:56-63)."""

    def __init__(self, device, max_batch: int, n_q_heads: int):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise PeerKVError("Shard needs a CUDA device")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.max_batch, self.n_q_heads = int(max_batch), int(n_q_heads)
        h = C.c_void_p()
        check(_lib.lib().pkv_shard_create(C.byref(h), self.device.index, self.max_batch, self.n_q_heads))
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            _lib.lib().pkv_shard_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def status(self) -> int:
        """Reads and clears the device status word (synchronises the current stream)."""
        v = C.c_uint32()
        check(_lib.lib().pkv_shard_status(self._h, _stream(self.device), C.byref(v)))
        return int(v.value)

    def stats(self, element_size: int = 2) -> dict:
        """Cumulative launches and KV bytes read by this shard's kernels (synchronises);
        also adds what is new since the last call to the package's counters."""
        from . import metrics
        a, b = C.c_uint64(), C.c_uint64()
        check(_lib.lib().pkv_shard_stats(self._h, _stream(self.device), C.byref(a), C.byref(b)))
        kv_bytes = int(b.value) * 16 * HEAD_DIM * 2 * element_size
        new = kv_bytes - getattr(self, "_bytes_seen", 0)
        self._bytes_seen = kv_bytes
        metrics.KV_BYTES_READ.labels(gpu=self.device.index).inc(new)
        return {"launches": int(a.value), "kv_bytes_read": kv_bytes}

    def raise_on_status(self):
        st = self.status()
        if st:
            names = [n for b, n in ((1, "pipeline wait timed out"), (2, "block-table id outside the pool"),
                                    (4, "query never arrived"), (8, "a peer partial never arrived")) if st & b]
            raise PeerKVError("device status 0x%x: %s" % (st, "; ".join(names)))


_shards = {}
_retired = []          # (shard, event): outgrown contexts whose scratch queued kernels may still use


def get_shard(device: torch.device, batch: int, n_q_heads: int) -> Shard:
    """Cached per (device, n_q_heads); regrown when a larger batch shows up.  The outgrown
    context is not freed under kernels that may still be queued on it, and the host does
    not wait for them either: it is retired with an event and freed once that has passed."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    key = (device.index, n_q_heads)
    for item in list(_retired):
        if item[1].query():
            item[0].close()
            _retired.remove(item)
    s = _shards.get(key)
    if s is None or s.max_batch < batch:
        if s is not None:
            ev = torch.cuda.Event()
            with torch.cuda.device(device):
                ev.record(torch.cuda.current_stream(device))
            _retired.append((s, ev))
        cap = min(4096, max(64, 1 << max(0, batch - 1).bit_length()))   # next power of two, 64..4096
        s = Shard(device, max(cap, batch), n_q_heads)                    # > 4096: let the library refuse it
        _shards[key] = s
    return s


def make_args(q: torch.Tensor, kv_view: KvView, block_table: Optional[torch.Tensor],
              bt_stride: int, seq_lens: torch.Tensor, scale: float) -> DecodeArgs:
    a = DecodeArgs()
    a.q = q.data_ptr()
    a.q_dtype = _DT[q.dtype]
    a.batch, a.n_q_heads = q.shape[0], q.shape[1]
    a.kv = kv_view
    a.block_table = block_table.data_ptr() if block_table is not None else None
    a.block_table_stride = bt_stride
    a.seq_lens = seq_lens.data_ptr()
    a.scale = float(scale)
    return a


def paged_view(k_pool: torch.Tensor, v_pool: torch.Tensor,
               k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None) -> KvView:
    """k_pool / v_pool: [n_pages, page_size, Hkv, D] (any strides with a unit last
    stride), e.g. cache[0] and cache[1] of vLLM's [2, nb, bs, Hkv, D]."""
    if k_pool.dim() != 4 or k_pool.shape != v_pool.shape or k_pool.stride() != v_pool.stride():
        raise PeerKVError("k_pool and v_pool must be [n_pages, page_size, Hkv, D] with equal strides")
    if k_pool.stride(3) != 1 and k_pool.numel() > 0:
        raise PeerKVError("the head dimension must be contiguous")
    if k_pool.dtype not in _DT or k_pool.dtype == torch.float32:
        raise PeerKVError(f"unsupported KV dtype {k_pool.dtype}")
    v = KvView()
    v.k, v.v = k_pool.data_ptr(), v_pool.data_ptr()
    v.k_scale = k_scale.data_ptr() if k_scale is not None else None
    v.v_scale = v_scale.data_ptr() if v_scale is not None else None
    v.dtype = _DT[k_pool.dtype]
    v.n_pages, v.page_size, v.n_kv_heads, v.head_dim = k_pool.shape
    v.page_stride, v.token_stride, v.head_stride = k_pool.stride(0), k_pool.stride(1), k_pool.stride(2)
    return v


def contiguous_view(K: torch.Tensor, V: torch.Tensor) -> KvView:
    """K / V: [B, Hkv, T, D] (the reference's shard layout, any batch/head/token
    strides with a unit last stride; slices along T are fine).  Each sequence is
    one page of T tokens."""
    if K.dim() != 4 or K.shape != V.shape:
        raise PeerKVError("K and V must both be [B, Hkv, T, D]")
    if K.stride() != V.stride() and K.numel() > 0:
        V = V.contiguous(); K = K.contiguous()
    if K.numel() > 0 and K.stride(3) != 1:
        K = K.contiguous(); V = V.contiguous()
    v = KvView()
    v.k, v.v = K.data_ptr(), V.data_ptr()
    v.dtype = _DT[K.dtype]
    B, Hkv, T, D = K.shape
    v.n_pages, v.n_kv_heads, v.page_size, v.head_dim = (B if T > 0 else 0), Hkv, max(T, 1), D
    v.page_stride, v.head_stride, v.token_stride = K.stride(0), K.stride(1), K.stride(2)
    v._keep = (K, V)
    return v


def _meta(t: torch.Tensor, device: torch.device, name: str) -> torch.Tensor:
    """Block tables and lengths as the kernels need them: int32, on `device`, rows
    contiguous.  The reference accepts host-side metadata (it calls .item() on it), so a
    CPU tensor or one on another GPU is moved here rather than refused; a pointer that is
    not valid on `device` must never reach a kernel."""
    if not isinstance(t, torch.Tensor):
        t = torch.as_tensor(t)
    if t.dtype != torch.int32:
        t = t.to(torch.int32)
    if t.device != device:
        t = t.to(device, non_blocking=True)
    if t.dim() > 0 and t.stride(-1) != 1:
        t = t.contiguous()
    return t


def _same_gpu(t: torch.Tensor, device: torch.device, name: str):
    if t is not None and t.device != device:
        raise PeerKVError(f"{name} lives on {t.device}, expected {device}")


def _check_q(q: torch.Tensor):
    _require_cuda(q, "q")
    if q.dim() != 3 or q.shape[2] != HEAD_DIM:
        raise PeerKVError(f"q must be [batch, n_q_heads, {HEAD_DIM}]; got {tuple(q.shape)}")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise PeerKVError(f"q must be fp16 or bf16; got {q.dtype}")
    return q if q.is_contiguous() else q.contiguous()


def decode_paged(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                 block_table: torch.Tensor, seq_lens: torch.Tensor, scale: Optional[float] = None,
                 out: Optional[torch.Tensor] = None, return_lse: bool = False,
                 k_scale=None, v_scale=None, shard: Optional[Shard] = None):
    """Whole decode attention of one GPU over its paged pool -> out [B, Hq, D] in q.dtype."""
    q = _check_q(q)
    B, Hq, D = q.shape
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    shard = shard or get_shard(q.device, B, Hq)
    bt, sl = _meta(block_table, q.device, "block_table"), _meta(seq_lens, q.device, "seq_lens")
    for t, n in ((k_pool, "k_pool"), (v_pool, "v_pool"), (k_scale, "k_scale"), (v_scale, "v_scale")):
        _same_gpu(t, q.device, n)
    if shard.device != q.device:
        raise PeerKVError(f"the shard context is on {shard.device}, q on {q.device}")
    view = paged_view(k_pool, v_pool, k_scale, v_scale)
    a = make_args(q, view, bt, bt.stride(0), sl, scale)
    if out is None:
        out = torch.empty_like(q)
    lse = torch.empty(B, Hq, dtype=torch.float32, device=q.device) if return_lse else None
    check(_lib.lib().pkv_decode(shard._h, C.byref(a), out.data_ptr(), _DT[out.dtype],
                                lse.data_ptr() if lse is not None else None, _stream(q.device)))
    return (out, lse) if return_lse else out


def partial_paged(q, k_pool, v_pool, block_table, seq_lens, scale=None, k_scale=None, v_scale=None,
                  shard: Optional[Shard] = None, o_part=None, lse_part=None):
    """One shard's (O fp32 [B,Hq,D] normalised, lse fp32 [B,Hq]) from a paged pool."""
    q = _check_q(q)
    B, Hq, D = q.shape
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    shard = shard or get_shard(q.device, B, Hq)
    bt, sl = _meta(block_table, q.device, "block_table"), _meta(seq_lens, q.device, "seq_lens")
    for t, n in ((k_pool, "k_pool"), (v_pool, "v_pool"), (k_scale, "k_scale"), (v_scale, "v_scale")):
        _same_gpu(t, q.device, n)
    if shard.device != q.device:
        raise PeerKVError(f"the shard context is on {shard.device}, q on {q.device}")
    view = paged_view(k_pool, v_pool, k_scale, v_scale)
    a = make_args(q, view, bt, bt.stride(0), sl, scale)
    if o_part is None:
        o_part = torch.empty(B, Hq, D, dtype=torch.float32, device=q.device)
        lse_part = torch.empty(B, Hq, dtype=torch.float32, device=q.device)
    check(_lib.lib().pkv_decode_partial(shard._h, C.byref(a), o_part.data_ptr(), lse_part.data_ptr(),
                                        _stream(q.device)))
    return o_part, lse_part


def partial_contiguous(q, K, V, scale=None, shard: Optional[Shard] = None, o_part=None, lse_part=None):
    """One shard's partial from contiguous K/V [B, Hkv, T, D]; q [B, Hq, D]."""
    q = _check_q(q)
    _require_cuda(K, "K")
    _same_gpu(K, q.device, "K"); _same_gpu(V, q.device, "V")
    B, Hq, D = q.shape
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    shard = shard or get_shard(q.device, B, Hq)
    view = contiguous_view(K, V)
    T = K.shape[2]
    sl = torch.full((B,), T, dtype=torch.int32, device=q.device)
    a = make_args(q, view, None, 1, sl, scale)
    if o_part is None:
        o_part = torch.empty(B, Hq, D, dtype=torch.float32, device=q.device)
        lse_part = torch.empty(B, Hq, dtype=torch.float32, device=q.device)
    check(_lib.lib().pkv_decode_partial(shard._h, C.byref(a), o_part.data_ptr(), lse_part.data_ptr(),
                                        _stream(q.device)))
    return o_part, lse_part


def decode_contiguous(q, K, V, scale=None, out=None, shard: Optional[Shard] = None):
    """Whole attention over contiguous K/V [B, Hkv, T, D] on one GPU -> [B, Hq, D]."""
    q = _check_q(q)
    _require_cuda(K, "K")
    _same_gpu(K, q.device, "K"); _same_gpu(V, q.device, "V")
    B, Hq, D = q.shape
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    shard = shard or get_shard(q.device, B, Hq)
    view = contiguous_view(K, V)
    sl = torch.full((B,), K.shape[2], dtype=torch.int32, device=q.device)
    a = make_args(q, view, None, 1, sl, scale)
    if out is None:
        out = torch.empty_like(q)
    check(_lib.lib().pkv_decode(shard._h, C.byref(a), out.data_ptr(), _DT[out.dtype], None,
                                _stream(q.device)))
    return out


def merge_partials(o_parts: torch.Tensor, lse_parts: torch.Tensor, out_dtype=torch.float32,
                   return_lse: bool = False):
    """Single-pass N-way LSE merge.  o_parts [N, ..., D] fp32, lse_parts [N, ...] fp32
    (contiguous, same device) -> out [..., D] in out_dtype (and lse [...])."""
    _require_cuda(o_parts, "o_parts")
    if o_parts.dtype != torch.float32 or lse_parts.dtype != torch.float32:
        raise PeerKVError("partials must be fp32")
    o_parts, lse_parts = o_parts.contiguous(), lse_parts.contiguous()
    N, D = o_parts.shape[0], o_parts.shape[-1]
    rows = lse_parts[0].numel()
    out = torch.empty(o_parts.shape[1:], dtype=out_dtype, device=o_parts.device)
    lse = torch.empty(lse_parts.shape[1:], dtype=torch.float32, device=o_parts.device) if return_lse else None
    check(_lib.lib().pkv_merge_partials(o_parts.device.index, o_parts.data_ptr(), rows * D,
                                        lse_parts.data_ptr(), rows, N, rows, D, out.data_ptr(),
                                        _DT[out_dtype], lse.data_ptr() if lse is not None else None,
                                        _stream(o_parts.device)))
    return (out, lse) if return_lse else out


def quantize_kv(x: torch.Tensor, fmt: str) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-(token, kv-head) absmax quantiser: x [..., 128] fp16/bf16 ->
    (codes [..., 128] int8 or float8_e4m3fn, scales [...] fp16)."""
    _require_cuda(x, "x")
    if x.shape[-1] != HEAD_DIM or x.dtype not in (torch.float16, torch.bfloat16):
        raise PeerKVError("x must be [..., 128] fp16 or bf16")
    x = x.contiguous()
    rows = x.numel() // HEAD_DIM
    code_dt = torch.int8 if fmt == "int8" else torch.float8_e4m3fn
    if fmt not in ("int8", "fp8"):
        raise PeerKVError("fmt must be 'int8' or 'fp8'")
    codes = torch.empty(x.shape, dtype=code_dt, device=x.device)
    scales = torch.empty(x.shape[:-1], dtype=torch.float16, device=x.device)
    check(_lib.lib().pkv_quantize_kv(x.device.index, x.data_ptr(), _DT[x.dtype], rows, codes.data_ptr(),
                                     scales.data_ptr(), _DT[code_dt], _stream(x.device)))
    return codes, scales
