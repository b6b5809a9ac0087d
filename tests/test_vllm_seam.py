"""The vLLM seam: names, decode-only gate and correct-or-fallback behaviour
(reference umallm/peerkv/vllm_backend.py:65-106, register.py:40-89).  The host-side
logic runs on CPU with a stand-in metadata object; the fused path itself is a GPU test."""
from types import SimpleNamespace

import pytest
import torch

from golden_cases import gen_paged_case


def _impl():
    from peerkv_b200.peerkv.vllm_backend import PeerKVFusedAttentionImpl
    impl = PeerKVFusedAttentionImpl.__new__(PeerKVFusedAttentionImpl)   # no vLLM config needed
    impl._init_peerkv()
    impl.scale = 1.0 / 128 ** 0.5
    return impl


def test_names_and_gate_on_cpu():
    from peerkv_b200.peerkv import vllm_backend, register
    assert hasattr(vllm_backend, "PeerKVFusedAttentionImpl") and hasattr(vllm_backend, "register_peerkv_fused")
    assert hasattr(register, "install_cfk") and hasattr(register, "uninstall_cfk")
    impl = _impl()
    q = torch.zeros(4, 32, 128, dtype=torch.float16)
    kv = torch.zeros(2, 8, 16, 8, 128, dtype=torch.float16)
    md = SimpleNamespace(block_table=torch.zeros(4, 2, dtype=torch.int32), seq_lens=torch.ones(4, dtype=torch.int32),
                         num_actual_tokens=4, max_query_len=1, use_cascade=False)
    assert impl._try_fused(q, kv, md) is None                       # no peer cache yet -> fallback
    impl.set_peer_kv(kv.clone(), 100)
    assert impl._peer_base == 100
    md_prefill = SimpleNamespace(block_table=md.block_table[:2], seq_lens=md.seq_lens[:2],
                                 num_actual_tokens=4, max_query_len=2, use_cascade=False)
    assert impl._try_fused(q, kv, md_prefill) is None               # prefill / chunked -> fallback
    assert impl._try_fused(q[:, :, :64], kv[..., :64], md) is None  # head size != 128 -> fallback
    assert impl._try_fused(q, kv, md) is None                       # CPU tensors: the op raises -> fallback


def test_install_uninstall_roundtrip():
    from peerkv_b200.peerkv import register
    try:
        from vllm.v1.attention.backends import flash_attn as v1fa
    except Exception:
        assert register.install_cfk() is False
        return
    from peerkv_b200.peerkv.vllm_backend import PeerKVFusedAttentionImpl
    orig_cls = v1fa.FlashAttentionBackend.get_impl_cls()
    assert register.install_cfk() is True
    assert v1fa.FlashAttentionBackend.get_impl_cls() is PeerKVFusedAttentionImpl
    assert register.install_cfk() is True                           # idempotent
    assert register.uninstall_cfk() is True
    assert v1fa.FlashAttentionBackend.get_impl_cls() is orig_cls


@pytest.mark.gpu
def test_fused_decode_through_the_impl(golden):
    """Decode batch through `_try_fused` / `forward` with vLLM-shaped inputs: kv_cache
    [2, nb, 16, HKV, D], block_table of global ids, tail blocks in a second cache."""
    dev = torch.device("cuda", 0)
    n = torch.cuda.device_count()
    peer_dev = torch.device("cuda", 1 if n > 1 else 0)
    c = gen_paged_case()
    impl = _impl()
    impl.set_peer_kv(c["peer_cache"].to(peer_dev), c["peer_base"])
    B, H, D = c["q"].shape
    md = SimpleNamespace(block_table=c["block_table"].to(torch.int32).to(dev),
                         seq_lens=torch.tensor(c["seq_lens"], dtype=torch.int32, device=dev),
                         num_actual_tokens=B, max_query_len=1, use_cascade=False)
    out = torch.zeros(B + 3, H * D, dtype=torch.float16, device=dev)     # padded like vLLM's buffer
    q_pad = torch.zeros(B + 3, H, D, dtype=torch.float16, device=dev)
    q_pad[:B] = c["q"].to(dev)
    res = impl.forward(None, q_pad, None, None, c["local_cache"].to(dev), md, out)
    assert res is out and impl.fused_calls == 1 and impl.fallback_calls == 0
    ref = torch.from_numpy(golden["paged/out"])
    assert torch.allclose(out[:B].view(B, H, D).float().cpu(), ref, atol=2e-3, rtol=1e-2)
    assert (out[B:] == 0).all()
