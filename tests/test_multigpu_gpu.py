"""Two or more GPUs: the single-process group (the reference's calling model, tensors
on cuda:0 and cuda:1) and the one-process-per-GPU group, both through the C ABI,
against the CPU oracle.  Also the bounded-wait behaviour: a peer whose query never
arrives ends with a status bit, not a hang."""
import os
import subprocess
import sys

import pytest
import torch

from golden_cases import SEEDED_CASES, gen_paged_case, gen_seeded_case
from oracle import peerkv_oracle as orc

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def close(a, b, atol=2e-3, rtol=1e-2):
    return torch.allclose(a.float().cpu(), b.float().cpu(), atol=atol, rtol=rtol)


def test_peer_fused_attn_two_devices(golden):
    """experiments/test_fused_attn_op.py on real peers: local half on cuda:0, peer half on cuda:1."""
    from peerkv_b200.peerkv import peer_fused_attn
    torch.manual_seed(0)
    H, HKV, D = 32, 8, 128
    for T in (1024, 4096, 16384, 1000):
        q = (torch.randn(H, D) * 0.1).half()
        Kf = (torch.randn(HKV, T, D) * 0.1).half()
        Vf = (torch.randn(HKV, T, D) * 0.1).half()
        Tl = T // 2
        O = peer_fused_attn(q.to("cuda:0"), Kf[:, :Tl].contiguous().to("cuda:0"), Vf[:, :Tl].contiguous().to("cuda:0"),
                            Kf[:, Tl:].contiguous().to("cuda:1"), Vf[:, Tl:].contiguous().to("cuda:1"))
        assert O.device == torch.device("cuda:0") and O.shape == (H, D)
        assert close(O, orc.reference_attn(q, Kf, Vf))
    from peerkv_b200.group import _groups
    for g in _groups.values():
        g.raise_on_status()


@pytest.mark.parametrize("name", ["gqa_c1_full", "gqa_bf16_batch"])
def test_peer_parallel_attention_across_devices(golden, name):
    from peerkv_b200.peer_parallel_attn import peer_parallel_attention
    spec = SEEDED_CASES[name]
    q, K, V = gen_seeded_case(spec)
    n = torch.cuda.device_count()
    shards = []
    for i, (k, v) in enumerate(zip(K.split(spec["shards"], 2), V.split(spec["shards"], 2))):
        d = torch.device("cuda", i % n)
        shards.append((k.to(d), v.to(d)))
    out = peer_parallel_attention(q.to("cuda:0"), shards)
    assert out.device == torch.device("cuda:0")
    assert close(out, torch.from_numpy(golden[f"{name}/out"]))


def test_paged_cfk_decode_two_devices(golden):
    """experiments/test_paged_cfk.py: tail 40 % of each sequence's blocks on the peer."""
    from peerkv_b200.peerkv.paged import paged_cfk_decode
    c = gen_paged_case()
    for rep in range(3):      # repeated steps: epochs advance, mailboxes are reused
        out = paged_cfk_decode(c["q"].to("cuda:0"), c["local_cache"].to("cuda:0"), c["peer_cache"].to("cuda:1"),
                               c["block_table"].to("cuda:0"), torch.tensor(c["seq_lens"], device="cuda:0"),
                               c["peer_base"])
        assert close(out, torch.from_numpy(golden["paged/out"]))
    for i, (Kf, Vf) in enumerate(c["full"]):
        assert close(out[i], orc.reference_attn(c["q"][i], Kf, Vf))


def test_group_round_robin_all_devices():
    """Round-robin page placement over every GPU of the box, ragged lengths."""
    from peerkv_b200.group import PeerGroup
    n = torch.cuda.device_count()
    bs, Hq, Hkv, D = 16, 32, 8, 128
    lens = [3000, 17, 0, 4096, 1, 777]
    B = len(lens)
    g = torch.Generator().manual_seed(4)
    n_pages = [(L + bs - 1) // bs for L in lens]
    total = sum(n_pages)
    total_pad = (total + n - 1) // n * n
    pool = torch.randn(2, total_pad, bs, Hkv, D, generator=g).bfloat16()
    perm = torch.randperm(total, generator=g)
    bt = torch.zeros(B, max(n_pages), dtype=torch.int32)
    k = 0
    for i, m in enumerate(n_pages):
        bt[i, :m] = perm[k:k + m].to(torch.int32); k += m
    sl = torch.tensor(lens, dtype=torch.int32)
    q = torch.randn(B, Hq, D, generator=g).bfloat16()
    ref, _ = orc.paged_partial_oracle(q, pool, bt, sl)
    devs = [torch.device("cuda", i) for i in range(n)]
    grp = PeerGroup(devs, B, Hq)
    pools = []
    for r, d in enumerate(devs):
        local = pool[:, r::n].contiguous().to(d)           # page p -> GPU p mod n at index p div n
        pools.append((local[0], local[1]))
    tables, lens_d, ev = grp.split_table(bt.to(devs[0]), sl.to(devs[0]), bs, None)
    for rep in range(2):
        out = grp.decode_paged_local(q.to(devs[0]), pools, tables, lens_d, after_event=ev)
        assert close(out, ref)
    grp.raise_on_status()


def test_query_that_never_arrives_is_a_status_bit_not_a_hang():
    """A peer step with no publish: the bounded device-side wait runs out, the kernel
    returns, the status word says why and the context stays usable."""
    import ctypes as C
    from peerkv_b200 import _lib, ops
    from peerkv_b200.group import Exchange
    dev0, dev1 = torch.device("cuda:0"), torch.device("cuda:1")
    # long enough that every CTA has more tiles than ring slots: the producers fill their
    # rings and then block on the consumers, which are waiting for the query
    B, Hq, Hkv, D, T = 1, 32, 8, 128, 16 * 8 * 160
    x0, x1 = Exchange(dev0, 0, 2, B, Hq), Exchange(dev1, 1, 2, B, Hq)
    x0.attach(x1); x1.attach(x0)
    shard = ops.Shard(dev1, B, Hq)
    K = torch.randn(B, Hkv, T, D, device=dev1).half()
    V = torch.randn(B, Hkv, T, D, device=dev1).half()
    q = torch.randn(B, Hq, D, device=dev1).half()
    sl = torch.full((B,), T, dtype=torch.int32, device=dev1)
    a = ops.make_args(q, ops.contiguous_view(K, V), None, 1, sl, 0.1)
    with torch.cuda.device(dev1):
        _lib.check(_lib.lib().pkv_peer_step(x1._h, shard._h, C.byref(a), 0, 0, ops._stream(dev1)))
        torch.cuda.synchronize(dev1)
        assert shard.status() == _lib.ST_Q_TIMEOUT      # that bit and no other (no pipeline time-out)
        # the GPU still works: an ordinary decode on the same shard object
        out = ops.decode_contiguous(q, K, V, shard=shard)
        ref = orc.dense_attention_fp32(q.cpu().unsqueeze(2), K.cpu(), V.cpu()).squeeze(2)
        assert close(out, ref)
    # and a merge that waits for a partial nobody sends
    out0 = torch.empty(B, Hq, D, device=dev0, dtype=torch.float16)
    with torch.cuda.device(dev0):
        _lib.check(_lib.lib().pkv_home_publish_q(x0._h, q.to(dev0).data_ptr(), B, ops._stream(dev0)))
        _lib.check(_lib.lib().pkv_home_merge(x0._h, B, 0b10, out0.data_ptr(), _lib.PKV_F16, None,
                                             ops._stream(dev0)))
        torch.cuda.synchronize(dev0)
        assert x0.status() & _lib.ST_PARTIAL_TIMEOUT
    x0.close(); x1.close(); shard.close()


def test_back_to_back_steps_with_a_sequence_that_leaves_the_peer():
    """Two steps enqueued with no synchronisation in between.  In the first, sequence 1
    has tokens on the peer GPU; in the second it has none there (its rows from the peer
    become the neutral ones).  The peer's second kernel starts while the home GPU may
    still be merging the first step: nothing of the second step may land in the home
    GPU's slot before the home GPU has finished reading the first."""
    from peerkv_b200.group import PeerGroup
    devs = [torch.device("cuda:0"), torch.device("cuda:1")]
    bs, Hq, Hkv, D = 16, 32, 8, 128
    g = torch.Generator().manual_seed(9)
    n_pages = 4096
    pools_cpu = [torch.randn(2, n_pages, bs, Hkv, D, generator=g).bfloat16() for _ in devs]
    B = 3
    q = torch.randn(B, Hq, D, generator=g).bfloat16()
    # per GPU: local block tables; GPU 0 holds a long shard so that its merge comes late
    tab = [torch.arange(B * 1024, dtype=torch.int32).view(B, 1024) for _ in devs]
    lens1 = [torch.tensor([16000, 16000, 16000], dtype=torch.int32), torch.tensor([800, 4000, 16], dtype=torch.int32)]
    lens2 = [torch.tensor([16000, 16000, 16000], dtype=torch.int32), torch.tensor([800, 0, 16], dtype=torch.int32)]
    grp = PeerGroup(devs, B, Hq)
    pools = [(p[0].to(d), p[1].to(d)) for p, d in zip(pools_cpu, devs)]
    tabs = [t.to(d) for t, d in zip(tab, devs)]
    l1 = [t.to(d) for t, d in zip(lens1, devs)]
    l2 = [t.to(d) for t, d in zip(lens2, devs)]
    qd = q.to(devs[0])
    out1, out2 = torch.empty_like(qd), torch.empty_like(qd)
    for d in devs:
        torch.cuda.synchronize(d)
    for rep in range(20):                         # the window is narrow: many tries
        grp.decode_paged_local(qd, pools, tabs, l1, out=out1)
        grp.decode_paged_local(qd, pools, tabs, l2, out=out2)
    for d in devs:
        torch.cuda.synchronize(d)

    def want(lens):
        parts = [orc.paged_partial_oracle(q, pools_cpu[r], tab[r], lens[r]) for r in range(2)]
        return orc.merge_n([p[0] for p in parts], [p[1] for p in parts])[0]
    assert close(out1, want(lens1))
    assert close(out2, want(lens2))
    grp.raise_on_status()


def test_a_rejected_step_leaves_the_epoch_where_it_was():
    import ctypes as C
    from peerkv_b200 import _lib, ops
    from peerkv_b200.group import Exchange
    dev0, dev1 = torch.device("cuda:0"), torch.device("cuda:1")
    B, Hq, Hkv, D, T = 2, 32, 8, 128, 64
    x0, x1 = Exchange(dev0, 0, 2, B, Hq), Exchange(dev1, 1, 2, B, Hq)
    x0.attach(x1); x1.attach(x0)
    shard = ops.Shard(dev1, B, Hq)
    K = torch.randn(B, Hkv, T, D, device=dev1).half()
    q = torch.randn(B, Hq, D, device=dev1).half()
    sl = torch.full((B,), T, dtype=torch.int32, device=dev1)
    a = ops.make_args(q, ops.contiguous_view(K, K), None, 1, sl, 0.1)
    a.kv.head_dim = 64                                   # refused by the argument check
    with torch.cuda.device(dev1):
        rc = _lib.lib().pkv_peer_step(x1._h, shard._h, C.byref(a), 0, 0, ops._stream(dev1))
    assert rc == -3 and x1.epoch() == 0
    x1.resync(5)
    assert x1.epoch() == 5
    with pytest.raises(_lib.PeerKVError):
        x1.resync(4)
    x0.close(); x1.close(); shard.close()


def _two_exchanges(B, Hq):
    from peerkv_b200.group import Exchange
    dev0, dev1 = torch.device("cuda:0"), torch.device("cuda:1")
    x0, x1 = Exchange(dev0, 0, 2, B, Hq), Exchange(dev1, 1, 2, B, Hq)
    x0.attach(x1); x1.attach(x0)
    return dev0, dev1, x0, x1


def _three_call_step(x0, x1, sh0, sh1, q0, a0, a1, out0):
    """publish, the two shard partials, merge: the long form of pkv_home_step."""
    import ctypes as C
    from peerkv_b200 import _lib, ops
    L = _lib.lib()
    dev0, dev1 = x0.device, x1.device
    with torch.cuda.device(dev0):
        _lib.check(L.pkv_home_publish_q(x0._h, q0.data_ptr(), q0.shape[0], ops._stream(dev0)))
    with torch.cuda.device(dev1):
        _lib.check(L.pkv_peer_step(x1._h, sh1._h, C.byref(a1), 0, 0, ops._stream(dev1)))
    with torch.cuda.device(dev0):
        _lib.check(L.pkv_home_partial(x0._h, sh0._h, C.byref(a0), ops._stream(dev0)))
        _lib.check(L.pkv_home_merge(x0._h, q0.shape[0], 0b10, out0.data_ptr(), _lib.PKV_F16, None,
                                    ops._stream(dev0)))


def test_three_call_form_against_the_oracle_two_steps_in_a_row():
    """pkv_home_publish_q + pkv_peer_step + pkv_home_partial + pkv_home_merge, twice with no
    synchronisation in between and a new query the second time: both results must be the
    unsplit attention over the two shards."""
    from peerkv_b200 import ops
    B, Hq, Hkv, D, T0, T1 = 3, 32, 8, 128, 400, 272
    dev0, dev1, x0, x1 = _two_exchanges(B, Hq)
    g = torch.Generator().manual_seed(21)
    K = torch.randn(B, Hkv, T0 + T1, D, generator=g).half()
    V = torch.randn(B, Hkv, T0 + T1, D, generator=g).half()
    qs = [torch.randn(B, Hq, D, generator=g).half() for _ in range(2)]
    K0, V0 = K[:, :, :T0].contiguous().to(dev0), V[:, :, :T0].contiguous().to(dev0)
    K1, V1 = K[:, :, T0:].contiguous().to(dev1), V[:, :, T0:].contiguous().to(dev1)
    sh0, sh1 = ops.Shard(dev0, B, Hq), ops.Shard(dev1, B, Hq)
    sl0 = torch.full((B,), T0, dtype=torch.int32, device=dev0)
    sl1 = torch.full((B,), T1, dtype=torch.int32, device=dev1)
    q0s = [q.to(dev0) for q in qs]
    q_unused = torch.zeros(B, Hq, D, dtype=torch.float16, device=dev1)
    outs = [torch.empty(B, Hq, D, device=dev0, dtype=torch.float16) for _ in range(2)]
    scale = 1.0 / D ** 0.5
    for q0, out0 in zip(q0s, outs):
        a0 = ops.make_args(q0, ops.contiguous_view(K0, V0), None, 1, sl0, scale)
        a1 = ops.make_args(q_unused, ops.contiguous_view(K1, V1), None, 1, sl1, scale)
        _three_call_step(x0, x1, sh0, sh1, q0, a0, a1, out0)
    torch.cuda.synchronize(dev0); torch.cuda.synchronize(dev1)
    assert x0.status() == 0 and x1.status() == 0 and sh0.status() == 0 and sh1.status() == 0
    assert x0.epoch() == 2 and x1.epoch() == 2
    for q, out0 in zip(qs, outs):
        ref = orc.dense_attention_fp32(q.unsqueeze(2), K, V).squeeze(2)
        assert close(out0, ref)
    x0.close(); x1.close(); sh0.close(); sh1.close()


def test_hop_probe_both_forms_and_steps_after_it():
    """The latency probe bounces a flag, a fenced payload and a payload of self-validating
    words between two GPUs; none of its waits may run out, and what it leaves in the query
    inbox must not pass for a query afterwards."""
    from peerkv_b200 import _lib, ops
    from peerkv_b200.group import PeerGroup
    devs = [torch.device("cuda:0"), torch.device("cuda:1")]
    B, Hq, Hkv, D, T = 2, 32, 8, 128, 256
    grp = PeerGroup(devs, B, Hq)
    L = _lib.lib()
    x0, x1 = grp.xchg[0], grp.xchg[1]
    res = [torch.zeros(2, dtype=torch.int64, device=d) for d in devs]
    for form, payload in ((0, 0), (0, 1024), (2, 1024)):
        for x, d in ((x0, devs[0]), (x1, devs[1])):
            with torch.cuda.device(d):
                _lib.check(L.pkv_exchange_hop_probe_reset(x._h, ops._stream(d)))
            torch.cuda.synchronize(d)
        with torch.cuda.device(devs[1]):      # the answering side first
            _lib.check(L.pkv_exchange_hop_probe(x1._h, 0, 1 | form, 64, payload, res[1].data_ptr(),
                                                ops._stream(devs[1])))
        with torch.cuda.device(devs[0]):
            _lib.check(L.pkv_exchange_hop_probe(x0._h, 1, 0 | form, 64, payload, res[0].data_ptr(),
                                                ops._stream(devs[0])))
        for d in devs:
            torch.cuda.synchronize(d)
        for r in res:
            assert int(r[1]) == 0 and int(r[0]) > 0          # no wait ran out
        one_way_us = int(res[0][0]) / (2 * 64) / 1e3
        assert 0.1 < one_way_us < 1000.0
    with pytest.raises(_lib.PeerKVError):                      # the word form needs a payload
        _lib.check(L.pkv_exchange_hop_probe(x0._h, 1, 2, 4, 0, res[0].data_ptr(), ops._stream(devs[0])))
    g = torch.Generator().manual_seed(5)
    K = torch.randn(B, Hkv, 2 * T, D, generator=g).half()
    V = torch.randn(B, Hkv, 2 * T, D, generator=g).half()
    q = torch.randn(B, Hq, D, generator=g).half()
    shards = [(K[:, :, r * T:(r + 1) * T].contiguous().to(devs[r]), V[:, :, r * T:(r + 1) * T].contiguous().to(devs[r]))
              for r in range(2)]
    out = grp.decode_contiguous(q.to(devs[0]), shards)
    for d in devs:
        torch.cuda.synchronize(d)
    grp.raise_on_status()
    assert close(out, orc.dense_attention_fp32(q.unsqueeze(2), K, V).squeeze(2))


@pytest.mark.parametrize("nproc", [2])
def test_one_process_per_gpu(nproc):
    """torchrun-style launch of tests/dist_worker.py: mailboxes shared through IPC handles."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", "29517",
           os.path.join(ROOT, "tests", "dist_worker.py"), "--backend", "nccl"]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "DIST_OK" in res.stdout
