"""The copy-back corner (reference umallm/vllm_integration/peerkv_staging.py:82-131, checked
there by experiments/serve/m3_staging_test.py): staging is value preserving, the decode
over the staged tensor is exact, and running out of scratch is a status bit."""
from types import SimpleNamespace

import pytest
import torch

from oracle import peerkv_oracle as orc

pytestmark = pytest.mark.gpu


def _setup(n_peer_devs, c_scratch, seed=0):
    from peerkv_b200.peerkv.staging import StagingLayout, alloc_split_kv
    n = torch.cuda.device_count()
    peers = [f"cuda:{1 + i % max(1, n - 1)}" if n > 1 else "cuda:0" for i in range(n_peer_devs)]
    lay = StagingLayout(c_local=24, c_scratch=c_scratch, c_peers=[20] * n_peer_devs, block_size=16,
                        num_kv_heads=2, head_size=128, local_device="cuda:0", peer_devices=peers)
    g = torch.Generator().manual_seed(seed)
    total = lay.c_local + sum(lay.c_peers)
    full = torch.randn(2, total, 16, 2, 128, generator=g).bfloat16()       # the unsplit truth, by global id
    local, peer_kvs = alloc_split_kv(lay)
    local.zero_()
    local[:, :lay.c_local] = full[:, :lay.c_local].to(local.device)
    for base, c, pk in zip(lay.peer_bases, lay.c_peers, peer_kvs):
        pk.copy_(full[:, base:base + c])
    lens = [100, 16, 333, 1]
    bt = torch.zeros(len(lens), 24, dtype=torch.int32)
    perm = torch.randperm(total, generator=g)
    k = 0
    for i, L in enumerate(lens):
        m = (L + 15) // 16
        bt[i, :m] = perm[k:k + m].to(torch.int32)
        k += m
    return lay, full, local, peer_kvs, bt, torch.tensor(lens, dtype=torch.int32)


@pytest.mark.parametrize("n_peer_devs", [1, 2])
def test_staging_preserves_values_and_decode_is_exact(n_peer_devs):
    from peerkv_b200.peerkv.staging import PeerKVStager, copyback_decode, gather_kv
    lay, full, local, peer_kvs, bt, sl = _setup(n_peer_devs, c_scratch=40)
    dev = torch.device("cuda", 0)
    st = PeerKVStager(lay)
    out_bt = st.stage(local, peer_kvs, bt.to(dev), sl.to(dev))
    torch.cuda.synchronize()
    assert st.status() == 0
    for i, L in enumerate(sl.tolist()):
        m = (L + 15) // 16
        got = gather_kv(local, out_bt[i], m).cpu()
        want = gather_kv(full, bt[i], m)
        assert torch.equal(got, want), f"sequence {i}: staged blocks differ"
        assert ((out_bt[i, :m].cpu() < lay.c_local) == (bt[i, :m] < lay.c_local)).all()      # local ids pass through
    q = torch.randn(len(sl), 8, 128).bfloat16()
    out = copyback_decode(q.to(dev), local, peer_kvs, bt.to(dev), sl.to(dev), st)
    ref, _ = orc.paged_partial_oracle(q, full, bt, sl)
    assert torch.allclose(out.float().cpu(), ref, atol=2e-3, rtol=1e-2)


def test_scratch_too_small_is_a_status_bit():
    from peerkv_b200 import _lib
    from peerkv_b200.peerkv.staging import PeerKVStager
    lay, full, local, peer_kvs, bt, sl = _setup(1, c_scratch=3)
    dev = torch.device("cuda", 0)
    st = PeerKVStager(lay)
    out_bt = st.stage(local, peer_kvs, bt.to(dev), sl.to(dev))
    torch.cuda.synchronize()
    assert st.status() == _lib.ST_BAD_PAGE
    assert int(out_bt.max()) < lay.c_local + lay.c_scratch            # nothing points outside the tensor
    assert st.status() == 0


def test_impl_takes_the_copyback_corner_when_told():
    """The vLLM impl under the policy's COPYBACK decision: stage + one-GPU decode, same answer."""
    from peerkv_b200 import elastic_policy as ep
    from peerkv_b200.peerkv.vllm_backend import PeerKVFusedAttentionImpl
    lay, full, local, peer_kvs, bt, sl = _setup(1, c_scratch=40, seed=5)
    dev = torch.device("cuda", 0)
    impl = PeerKVFusedAttentionImpl.__new__(PeerKVFusedAttentionImpl)
    impl._init_peerkv()
    impl.scale = 1.0 / 128 ** 0.5
    impl.set_peer_kv(peer_kvs, lay.peer_bases)
    impl.set_scratch(lay.c_local, lay.c_scratch)
    impl.set_operating_point(ep.OperatingPoint.COPYBACK)
    B = len(sl)
    q = torch.randn(B, 8, 128).bfloat16()
    md = SimpleNamespace(block_table=bt.to(dev), seq_lens=sl.to(dev), num_actual_tokens=B, max_query_len=1,
                         use_cascade=False)
    out = torch.zeros(B, 8 * 128, dtype=torch.bfloat16, device=dev)
    res = impl.forward(None, q.to(dev), None, None, local, md, out)
    assert res is out and impl.copyback_calls == 1 and impl.fallback_calls == 0
    ref, _ = orc.paged_partial_oracle(q, full, bt, sl)
    assert torch.allclose(out.view(B, 8, 128).float().cpu(), ref, atol=2e-3, rtol=1e-2)
