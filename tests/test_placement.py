"""Cost helpers, selector and do-no-harm rules of the compute-follows-KV path: the
assertions of the reference's tests/test_peer_parallel_cost.py and the CFK-relevant
rules of tests/test_no_harm.py, on the B200-calibrated model."""
import pytest

from peerkv_b200 import placement as pl

BLK = 256 * 1024


def test_partial_bytes_independent_of_kv_size(golden):
    pb = pl.partial_bytes(heads=8, head_dim=128)
    assert pb == 8 * 128 * 2 + 8 * 4 == int(golden["cost/partial_bytes_8_128"])
    assert pl.partial_bytes(32, 128) == int(golden["cost/partial_bytes_32_128"])
    assert pl.partial_bytes(32, 128, o_bytes=4) == 32 * 128 * 4 + 32 * 4


def test_balanced_partition_matches_reference(golden):
    assert pl.balanced_partition(1000, [773, 773]) == golden["cost/bp_1000_773_773"].tolist()
    assert pl.balanced_partition(1001, [1, 1, 1]) == golden["cost/bp_1001_3eq"].tolist()
    assert pl.balanced_partition(8192, [6549.4] * 8) == golden["cost/bp_8192_8"].tolist()
    assert pl.balanced_partition(777, [2000, 773, 773, 1555]) == golden["cost/bp_777_uneven"].tolist()
    a = pl.balanced_partition(900, [600.0, 300.0])
    assert sum(a) == 900 and a[0] > a[1]


def test_parallel_step_uses_max_not_sum():
    m = pl.PeerKVCostModel()
    big = 40000                                  # 10 GB of 256 KiB blocks
    t_par = m.decode_step_parallel_us([big // 2, big // 2], BLK, heads=8, head_dim=128)
    t_one = m.decode_step_parallel_us([big], BLK, heads=8, head_dim=128)
    assert t_par < t_one and t_one / t_par > 1.5
    assert m.decode_step_parallel_us([], BLK, compute_us=3.0) == 3.0


def test_parallel_capacity_scales_with_devices():
    m = pl.PeerKVCostModel()
    common = dict(deadline_us=5000.0, block_bytes=BLK, compute_us=1500.0, attn_us=200.0)
    one = m.max_context_for_slo_parallel(n_devices=1, **common)
    two = m.max_context_for_slo_parallel(n_devices=2, **common)
    eight = m.max_context_for_slo_parallel(n_devices=8, **common)
    assert one["feasible"] and two["feasible"]
    assert two["max_blocks"] > 1.8 * one["max_blocks"]
    assert eight["max_blocks"] > 7.5 * one["max_blocks"]
    assert not m.max_context_for_slo_parallel(deadline_us=10.0, block_bytes=BLK, compute_us=20.0)["feasible"]


def test_calibrate_recovers_constants():
    true = pl.PeerKVCostModel(hbm_gbps=6900.0, kernel_fixed_us=9.0, exchange_us=21.0)
    single = {b: true.kernel_fixed_us + b / (true.hbm_gbps * 1e3) for b in (1 << 30, 8 << 30)}
    multi = (8 << 30, true.kernel_fixed_us + (1 << 30) / (true.hbm_gbps * 1e3) + true.exchange_us)
    fit = pl.PeerKVCostModel.calibrate(single, multi, n_devices=8)
    assert abs(fit.hbm_gbps - 6900.0) < 1.0 and abs(fit.kernel_fixed_us - 9.0) < 0.1
    assert abs(fit.exchange_us - 21.0) < 0.1
    with pytest.raises(ValueError):
        pl.PeerKVCostModel.calibrate({1: 5.0}, multi, 8)
    with pytest.raises(ValueError):
        pl.PeerKVCostModel.calibrate({1 << 30: 50.0, 2 << 30: 40.0}, multi, 8)   # time falls with size


def test_capacity_spill_split_matches_the_oracle():
    import numpy as np
    from oracle import peerkv_oracle as orc
    rng = np.random.default_rng(0)
    for _ in range(25):
        B, N, bs = int(rng.integers(1, 9)), int(rng.integers(1, 6)), 16
        lens = rng.integers(1, 3000, size=B)
        pages = (lens + bs - 1) // bs
        caps = rng.uniform(0.5, 1.0, size=N)
        start = np.concatenate([[0], np.cumsum(pages)[:-1]])
        bt = [list(range(int(s0), int(s0 + p))) for s0, p in zip(start, pages)]
        tab, tok, used = pl.capacity_spill_split(pages, lens, bs, caps)
        ref = orc.capacity_spill_shards(bt, lens, bs, list(caps))
        assert int(used.sum()) == int(pages.sum())
        for g, (t, l) in enumerate(ref):
            assert (l.numpy() == tok[g]).all()
            flat = [int(x) for i in range(B) for x in t[i, :-(-int(tok[g, i]) // bs)]]
            mine = [int(x) for i in range(B) for x in tab[g, i, :-(-int(tok[g, i]) // bs)]]
            assert mine == [f - flat[0] for f in flat]          # compact pools: arrival order


def test_page_placer_policies():
    rr = pl.PagePlacer(4, "round_robin")
    got = [rr.place() for _ in range(9)]
    assert got[:5] == [(0, 0), (1, 0), (2, 0), (3, 0), (0, 1)]
    sp = pl.PagePlacer(3, "capacity_spill", capacity_pages=[2, 1, 5])
    assert [sp.place()[0] for _ in range(6)] == [0, 0, 1, 2, 2, 2]
    bal = pl.PagePlacer(2, "balanced", bandwidth_gbps=[2.0, 1.0])
    for _ in range(300):
        bal.place()
    assert bal.used == pl.balanced_partition(300, [2.0, 1.0])
    full = pl.PagePlacer(2, "round_robin", capacity_pages=[1, 1])
    full.place(); full.place()
    with pytest.raises(MemoryError):
        full.place()
