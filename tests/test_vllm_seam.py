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


# ---- the allocator side: placement, hand-over, append -------------------------------------- #
def test_layout_arithmetic():
    from peerkv_b200.peerkv.kv_alloc import PeerKVLayout
    lay = PeerKVLayout.split(1000, 16, 8, 128, 0.7, "cuda:0", ["cuda:1", "cuda:2", "cuda:3"])
    assert lay.c_local == 300 and lay.c_peers == [234, 233, 233] and lay.num_blocks == 1000
    assert lay.peer_bases == [300, 534, 767] and lay.peer_base == 300
    assert lay.owner(0) == (0, 0) and lay.owner(299) == (0, 299) and lay.owner(300) == (1, 0)
    assert lay.owner(533) == (1, 233) and lay.owner(534) == (2, 0) and lay.owner(999) == (3, 232)


class _StandInRunner:
    """What relayout_runner touches of a vLLM GPUModelRunner: kv_caches and the model's
    attention modules (.impl, .kv_cache)."""

    def __init__(self, n_layers, nb, device, dtype):
        import torch.nn as nn
        self.kv_caches = [torch.randn(2, nb, 16, 2, 128, device=device).to(dtype) for _ in range(n_layers)]

        class Attn(nn.Module):
            pass
        self.model = nn.Sequential()
        for li in range(n_layers):
            a = Attn()
            a.impl = _impl()
            a.kv_cache = [self.kv_caches[li]]
            self.model.add_module(f"attn{li}", a)

    def initialize_kv_cache(self, cfg=None):
        return "done"


def test_relayout_on_cpu_tensors():
    """Host logic of the re-layout with every 'GPU' being the CPU: block values land where
    the layout says, the engine's handles are replaced, the impls get their peer caches."""
    from peerkv_b200.peerkv import kv_alloc
    r = _StandInRunner(3, 40, "cpu", torch.float16)
    before = [k.clone() for k in r.kv_caches]
    lays = kv_alloc.relayout_runner(r, 0.5, ["cpu", "cpu"])
    assert len(lays) == 3 and lays[0].c_local == 20 and lays[0].c_peers == [10, 10]
    for li, (mod, impl) in enumerate(kv_alloc.attention_impls(r)):
        assert r.kv_caches[li].shape[1] == 20 and mod.kv_cache[0] is r.kv_caches[li]
        assert torch.equal(r.kv_caches[li], before[li][:, :20])
        assert torch.equal(impl._peer_cache[0], before[li][:, 20:30])
        assert torch.equal(impl._peer_cache[1], before[li][:, 30:40])
        assert impl._peer_base == [20, 30]


def test_patch_wraps_and_survives_a_failing_relayout(monkeypatch):
    import sys
    import types
    from peerkv_b200.peerkv import kv_alloc
    mod = types.ModuleType("fake_runner_mod")
    mod.Runner = _StandInRunner
    sys.modules["fake_runner_mod"] = mod
    target = "fake_runner_mod:Runner.initialize_kv_cache"
    try:
        assert kv_alloc.patch_peer_kv_allocation(0.0, ["cpu"], target) is False        # no tiering asked
        assert kv_alloc.patch_peer_kv_allocation(0.25, ["cpu"], target) is True
        assert kv_alloc.patch_peer_kv_allocation(0.25, ["cpu"], target) is True        # idempotent
        r = _StandInRunner(2, 16, "cpu", torch.float16)
        assert r.initialize_kv_cache() == "done"
        assert r.kv_caches[0].shape[1] == 12
        broken = _StandInRunner(1, 16, "cpu", torch.float16)
        broken.kv_caches = None
        assert broken.initialize_kv_cache() == "done"                                  # the engine is not broken
        assert kv_alloc.unpatch_peer_kv_allocation(target) is True
        assert not getattr(_StandInRunner.initialize_kv_cache, "_peerkv_wrapped", False)
    finally:
        sys.modules.pop("fake_runner_mod", None)


@pytest.mark.gpu
def test_append_then_decode_through_the_seam():
    """The whole allocator path on real GPUs: split a runner's caches over the GPUs of the
    box, append one token per sequence through the impl's do_kv_cache_update (some land on
    peers), decode through forward, and compare with the oracle on the unsplit cache."""
    from oracle import peerkv_oracle as orc
    from peerkv_b200.peerkv import kv_alloc
    dev = torch.device("cuda", 0)
    n = torch.cuda.device_count()
    peers = [f"cuda:{i}" for i in range(1, n)] or ["cuda:0"]
    nb, bs, Hkv, D, Hq = 64, 16, 2, 128, 8
    r = _StandInRunner(2, nb, dev, torch.bfloat16)
    full = [k.clone() for k in r.kv_caches]                      # the unsplit truth, kept up to date below
    lays = kv_alloc.relayout_runner(r, 0.6, peers)
    lens = [100, 16, 333]                                        # before the append
    B = len(lens)
    g = torch.Generator().manual_seed(3)
    perm = torch.randperm(nb, generator=g)
    W = 24
    bt = torch.zeros(B, W, dtype=torch.int32)
    k = 0
    for i, L in enumerate(lens):
        m = L // bs + 1                                          # room for the new token
        bt[i, :m] = perm[k:k + m].to(torch.int32)
        k += m
    slot = torch.tensor([int(bt[i, L // bs]) * bs + L % bs for i, L in enumerate(lens)], dtype=torch.int64)
    assert any(lays[0].owner(int(s) // bs)[0] > 0 for s in slot) or n == 1
    for li, (mod, impl) in enumerate(kv_alloc.attention_impls(r)):
        key = torch.randn(B + 2, Hkv * D, generator=g).bfloat16()       # padded like vLLM's buffers
        val = torch.randn(B + 2, Hkv * D, generator=g).bfloat16()
        impl.do_kv_cache_update(mod, key.to(dev), val.to(dev), r.kv_caches[li], slot.to(dev))
        for i in range(B):
            blk, off = int(slot[i]) // bs, int(slot[i]) % bs
            full[li][0, blk, off] = key[i].view(Hkv, D).to(dev)
            full[li][1, blk, off] = val[i].view(Hkv, D).to(dev)
        q = torch.randn(B, Hq, D, generator=g).bfloat16()
        new_lens = torch.tensor([L + 1 for L in lens], dtype=torch.int32)
        md = SimpleNamespace(block_table=bt.to(dev), seq_lens=new_lens.to(dev), num_actual_tokens=B,
                             max_query_len=1, use_cascade=False)
        out = torch.zeros(B, Hq * D, dtype=torch.bfloat16, device=dev)
        res = impl.forward(mod, q.to(dev), None, None, r.kv_caches[li], md, out)
        assert res is out and impl.fused_calls == 1, "the sharded path was not taken"
        ref, _ = orc.paged_partial_oracle(q, full[li].cpu(), bt, new_lens)
        assert torch.allclose(out.view(B, Hq, D).float().cpu(), ref, atol=2e-3, rtol=1e-2)
