"""pkv_decode_static: the decode entry point for callers that are not allowed to
allocate GPU memory (a plugin inside a runtime whose memory pool is fully handed out,
a server that fixes all device memory at start-up).  Its split-K scratch is static
device memory inside the library, so it must give the same result as pkv_decode, which
uses a shard object's cudaMalloc'ed scratch -- on a first call, and again on a second
call that finds the scratch as the first one left it.  Collected last on purpose: a
run that stops at the first failure has then already run every other test."""
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


def test_static_scratch_decode_matches_shard_decode_twice():
    from peerkv_b200 import _lib, ops
    dev = torch.device("cuda", 0)
    L = _lib.lib()
    st = ops._stream(dev)
    for call, seed in enumerate((21, 22)):          # two calls in a row, different inputs
        q, pool, bt, sl = _case(dev, seed)
        B, Hq, D = q.shape
        a = ops.make_args(q, ops.paged_view(pool[0], pool[1]), bt, bt.stride(0), sl, 1.0 / math.sqrt(D))
        ref, ref_lse = ops.decode_paged(q, pool[0], pool[1], bt, sl, return_lse=True)
        out = torch.full_like(q, float("nan"))
        lse = torch.full((B, Hq), float("nan"), dtype=torch.float32, device=dev)
        _lib.check(L.pkv_decode_static(dev.index, C.byref(a), out.data_ptr(), _lib.PKV_BF16,
                                       lse.data_ptr(), st))
        torch.cuda.synchronize()
        assert torch.allclose(out.float(), ref.float(), atol=2e-3, rtol=1e-2), f"call {call} differs"
        has = sl > 0
        assert torch.allclose(lse[has], ref_lse[has], atol=2e-3, rtol=1e-4)
        assert torch.isinf(lse[~has]).all() and (out[~has] == 0).all()


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
