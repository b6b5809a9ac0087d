"""pkv_decode_static: the decode entry point for callers that are not allowed to
allocate GPU memory (a plugin inside a runtime whose memory pool is fully handed out,
a server that fixes all device memory at start-up).  Its split-K scratch is static
device memory inside the library, so it must give the same result as pkv_decode, which
uses a shard object's cudaMalloc'ed scratch, and as the CPU oracle -- on a first call,
and again on a second call that finds the scratch as the first one left it, without the
free device memory changing.  Its device status is read with pkv_static_status.
Collected last on purpose: a run that stops at the first failure has then already run
every other test."""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(dev, seed):
    g = torch.Generator().manual_seed(seed)
    bs, Hq, Hkv, D = 16, 32, 8, 128
    lens = [1500, 16, 0, 4096, 33, 7]
    B = len(lens)
    n_pages = [(L + bs - 1) // bs for L in lens]
    total = sum(n_pages) + 2
    pool = torch.randn(2, total, bs, Hkv, D, generator=g).bfloat16().to(dev)
    perm = torch.randperm(total, generator=g)
    bt = torch.zeros(B, max(n_pages), dtype=torch.int32)
    k = 0
    for i, n in enumerate(n_pages):
        bt[i, :n] = perm[k:k + n].to(torch.int32)
        k += n
    q = torch.randn(B, Hq, D, generator=g).bfloat16().to(dev)
    return q, pool, bt.to(dev), torch.tensor(lens, dtype=torch.int32, device=dev)


def _static_status(L, dev, st):
    v = C.c_uint32(0xffffffff)
    from peerkv_b200 import _lib
    _lib.check(L.pkv_static_status(dev.index, st, C.byref(v)))
    return int(v.value)


def test_static_scratch_decode_matches_shard_decode_twice():
    from oracle import peerkv_oracle as orc
    from peerkv_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    st = ops._stream(dev)
    free_before = None
    for call, seed in enumerate((21, 22)):          # two calls in a row, different inputs
        q, pool, bt, sl = _case(dev, seed)
        B, Hq, D = q.shape
        a = ops.make_args(q, ops.paged_view(pool[0], pool[1]), bt, bt.stride(0), sl, 1.0 / math.sqrt(D))
        ref, ref_lse = ops.decode_paged(q, pool[0], pool[1], bt, sl, return_lse=True)
        want, want_lse = orc.paged_partial_oracle(q.cpu(), pool.cpu(), bt.cpu(), sl.cpu())
        out = torch.full_like(q, float("nan"))
        lse = torch.full((B, Hq), float("nan"), dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        if call == 1:                                # the first call did the per-device set-up
            free_before = torch.cuda.mem_get_info(dev)[0]
        _lib.check(L.pkv_decode_static(dev.index, C.byref(a), out.data_ptr(), _lib.PKV_BF16,
                                       lse.data_ptr(), st))
        torch.cuda.synchronize()
        if call == 1:
            assert torch.cuda.mem_get_info(dev)[0] == free_before, "the call changed the free device memory"
        assert torch.allclose(out.float(), ref.float(), atol=2e-3, rtol=1e-2), f"call {call} differs from pkv_decode"
        assert torch.allclose(out.float().cpu(), want, atol=2e-3, rtol=1e-2), f"call {call} differs from the oracle"
        has = sl > 0
        assert torch.allclose(lse[has], ref_lse[has], atol=2e-3, rtol=1e-4)
        assert torch.allclose(lse[has].cpu(), want_lse[has.cpu()], atol=2e-3, rtol=1e-4)
        assert torch.isinf(lse[~has]).all() and (out[~has] == 0).all()
        assert _static_status(L, dev, st) == 0


def test_static_scratch_reports_a_bad_page_and_stays_usable():
    """A block-table id outside the pool is skipped (no fault) and shows up as a status bit
    that stays until it is read; the next call is clean again."""
    from peerkv_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    st = ops._stream(dev)
    q, pool, bt, sl = _case(dev, 24)
    D = q.shape[2]
    bad = bt.clone()
    bad[0, 1] = pool.shape[1] + 5
    out = torch.empty_like(q)
    a = ops.make_args(q, ops.paged_view(pool[0], pool[1]), bad, bad.stride(0), sl, 1.0 / math.sqrt(D))
    _lib.check(L.pkv_decode_static(dev.index, C.byref(a), out.data_ptr(), _lib.PKV_BF16, None, st))
    a = ops.make_args(q, ops.paged_view(pool[0], pool[1]), bt, bt.stride(0), sl, 1.0 / math.sqrt(D))
    _lib.check(L.pkv_decode_static(dev.index, C.byref(a), out.data_ptr(), _lib.PKV_BF16, None, st))
    assert _static_status(L, dev, st) == _lib.ST_BAD_PAGE        # from the first call, still there
    assert _static_status(L, dev, st) == 0                       # read once, cleared
    ref = ops.decode_paged(q, pool[0], pool[1], bt, sl)
    assert torch.allclose(out.float(), ref.float(), atol=2e-3, rtol=1e-2)


def test_static_scratch_rejects_sizes_beyond_its_maximum():
    from peerkv_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    q, pool, bt, sl = _case(dev, 23)
    D = q.shape[2]
    big_q = torch.zeros(33, 32, D, dtype=torch.bfloat16, device=dev)          # 33 sequences > 32
    big_sl = torch.zeros(33, dtype=torch.int32, device=dev)
    big_bt = torch.zeros(33, bt.shape[1], dtype=torch.int32, device=dev)
    a = ops.make_args(big_q, ops.paged_view(pool[0], pool[1]), big_bt, big_bt.stride(0), big_sl, 0.1)
    out = torch.empty_like(big_q)
    rc = L.pkv_decode_static(dev.index, C.byref(a), out.data_ptr(), _lib.PKV_BF16, None, ops._stream(dev))
    assert rc == -1 and b"at most 32 sequences" in L.pkv_last_error()
    wide_q = torch.zeros(2, 128, D, dtype=torch.bfloat16, device=dev)        # 128 query heads > 64
    a = ops.make_args(wide_q, ops.paged_view(pool[0], pool[1]), bt[:2], bt.stride(0), sl[:2], 0.1)
    out = torch.empty_like(wide_q)
    rc = L.pkv_decode_static(dev.index, C.byref(a), out.data_ptr(), _lib.PKV_BF16, None, ops._stream(dev))
    assert rc == -1 and b"at most 64 query heads" in L.pkv_last_error()
