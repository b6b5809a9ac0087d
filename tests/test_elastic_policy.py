"""The policy (peerkv_b200.elastic_policy) against the reference's own answers.

tests/golden/policy_golden.json.gz was written by tests/golden/make_policy_golden.py, which
runs the real `umallm.elastic_policy` / `umallm.runtime.selector` over ~1000 scenarios.
Under the reference's hardware constants (A100_NV12, two devices) this package must give
the same calibrated constants, predictions, admissible sets, decisions and gate verdicts.
The assertions of the reference's tests/test_elastic_policy.py and tests/test_no_harm.py
are restated below as well, and the N-device / B200 extensions are checked on their own."""
import gzip
import json
import math
import os

import pytest

from peerkv_b200 import elastic_policy as ep
from peerkv_b200 import metrics

HERE = os.path.dirname(os.path.abspath(__file__))
HW = ep.A100_NV12


@pytest.fixture(scope="module")
def gold():
    with gzip.open(os.path.join(HERE, "golden", "policy_golden.json.gz")) as f:
        return json.loads(f.read().decode())


def _geom(name):
    return ep.Geometry.llama2_7b_mha() if name == "mha" else ep.Geometry.gqa_8kv()


def _model(c):
    return ep.DecodeStepModel.calibrate(
        _geom(c["geom"]), {int(k): v for k, v in c["single_pts"].items()}, tuple(c["cfk_pt"]),
        tuple(c["copyback_pt"]), n_devices=2, hw=HW)


def test_hardware_record_matches_the_reference_constants(gold):
    h = gold["hardware"]
    assert (HW.hbm_gbps, HW.nvlink_gbps, HW.pcie_gbps) == (h["hbm"], h["nvlink"], h["pcie"])
    assert (HW.c_nvlink_us, HW.c_pcie_us, HW.c_hbm_us) == (h["c_nvlink_us"], h["c_pcie_us"], h["c_hbm_us"])


def test_calibration_reproduces_the_reference(gold):
    for name, c in gold["calibrations"].items():
        m = _model(c)
        assert m.A_ms == pytest.approx(c["A_ms"], rel=1e-12)
        assert m.beta_eff_gbps == pytest.approx(c["beta_eff_gbps"], rel=1e-12)
        assert m.roundtrip_ms_per_layer == pytest.approx(c["roundtrip_ms_per_layer"], rel=1e-9, abs=1e-12)
        assert m.copyback_eff == pytest.approx(c["copyback_eff"], rel=1e-9)
        assert m.predict_tp_bound_ms(143360) == pytest.approx(c["tp_bound_143360"], rel=1e-9)


def test_every_golden_scenario(gold):
    models = {n: _model(c) for n, c in gold["calibrations"].items()}
    n = 0
    for s in gold["scenarios"]:
        m = models[s["calibration"]]
        geom = m.geom
        peer = ep.PeerState(n_peers=1, **s["peer"])
        dep = ep.Deployment(**s["deploy"])
        link = ep.LinkState.from_peer(peer, HW)
        adm = ep.admissible_points(s["ctx"], geom, peer, dep, HW)
        assert sorted(p.value for p in adm) == s["admissible"], s
        for pv, want in s["predict_ms"].items():
            got = m.predict_ms(ep.OperatingPoint(pv), s["ctx"], peer, dep)
            if want is None:
                assert math.isinf(got), (s, pv)
            else:
                assert got == pytest.approx(want, rel=1e-9), (s, pv)
        d = ep.select_point(s["ctx"], geom, peer, dep, m)
        assert d.point.value == s["select"]["point"], s
        assert d.reason == s["select"]["reason"], s
        assert ep.select_point(s["ctx"], geom, peer, dep, m, 1.0).meets_deadline == s["select_deadline_1ms_meets"]
        on = ep.online_select(s["ctx"], geom, dep, m, peer=peer, link=link, strict=False)
        assert on.point.value == s["online"], s
        for pv, want in s["gate"].items():
            try:
                ep.enforce_do_no_harm(ep.OperatingPoint(pv), s["ctx"], geom, peer, link, deploy=dep)
                got = "ok"
            except ep.DoNoHarmViolation as e:
                got = str(e).split(":", 1)[0]
            assert got == want, (s, pv)
        n += 1
    assert n > 500


# ---- the reference's own assertions, restated (tests/test_elastic_policy.py) ------------ #
def _mha():
    g = ep.Geometry.llama2_7b_mha()
    return g, ep.DecodeStepModel.calibrate(g, {16384: 17.257, 32768: 22.151}, (16384, 20.336),
                                           (16384, 38.402), hw=HW)


def _peer(**kw):
    kw.setdefault("nvlink_bw_gbps", HW.nvlink_gbps)
    return ep.PeerState(**kw)


def test_reference_selector_assertions():
    g, m = _mha()
    dep = ep.Deployment()
    assert ep.OperatingPoint.SINGLE in ep.admissible_points(16384, g, _peer(), dep, HW)
    assert ep.OperatingPoint.SINGLE not in ep.admissible_points(143360, g, _peer(), dep, HW)
    busy = ep.admissible_points(143360, g, _peer(compute_idle=False), dep, HW)
    assert ep.OperatingPoint.CFK not in busy and ep.OperatingPoint.COPYBACK in busy
    slow = ep.admissible_points(143360, g, _peer(nvlink_bw_gbps=HW.pcie_gbps / 2), dep, HW)
    assert not ({ep.OperatingPoint.CFK, ep.OperatingPoint.COPYBACK} & slow) and ep.OperatingPoint.HOST in slow
    assert ep.select_point(16384, g, _peer(), dep, m).point is ep.OperatingPoint.SINGLE
    assert ep.select_point(143360, g, _peer(), dep, m).point is ep.OperatingPoint.CFK
    assert ep.select_point(143360, g, _peer(compute_idle=False), dep, m).point is ep.OperatingPoint.COPYBACK
    assert m.predict_ms(ep.OperatingPoint.SINGLE, 16384, _peer(), dep) < \
        m.predict_ms(ep.OperatingPoint.CFK, 16384, _peer(), dep)
    assert ep._single_capacity_tokens(ep.Geometry.gqa_8kv(), dep) > ep._single_capacity_tokens(g, dep)


def test_reference_no_harm_assertions():
    g = ep.Geometry.llama2_7b_mha()
    m = ep.DecodeStepModel.calibrate(g, {16384: 17.3, 32768: 22.2}, (32768, 25.1), (32768, 65.5), hw=HW)
    dep = ep.Deployment()
    cap = ep._single_capacity_tokens(g, dep)
    healthy = ep.LinkState(HW.nvlink_gbps, HW.pcie_gbps)
    idle, busy = _peer(), _peer(compute_idle=False)
    for ctx in (1, 1024, cap - 1, cap):
        d = ep.online_select(ctx, g, dep, m, peer=busy, link=healthy, strict=True)
        assert d.point is ep.OperatingPoint.SINGLE
    with pytest.raises(ep.DoNoHarmViolation, match="R1-fit"):
        ep.enforce_do_no_harm(ep.OperatingPoint.CFK, 1024, g, idle, healthy, deploy=dep)

    class Evil(ep.DecodeStepModel):          # pretends CFK is always fastest
        def predict_ms(self, point, ctx_tokens, peer, deploy):
            return 0.0 if point is ep.OperatingPoint.CFK else 100.0
    evil = Evil(g, m.A_ms, m.beta_eff_gbps, m.roundtrip_ms_per_layer, hw=HW)
    assert ep.online_select(1024, g, dep, evil, peer=idle, link=healthy).point is ep.OperatingPoint.SINGLE

    ctx = cap + 50_000
    assert ep.OperatingPoint.CFK not in ep.admissible_points(ctx, g, busy, dep, HW)
    assert ep.select_point(ctx, g, busy, dep, m).point in {ep.OperatingPoint.COPYBACK, ep.OperatingPoint.HOST}
    with pytest.raises(ep.DoNoHarmViolation, match="R1-busy"):
        ep.enforce_do_no_harm(ep.OperatingPoint.CFK, ctx, g, busy, healthy, deploy=dep)
    deg_peer, deg_link = _peer(nvlink_bw_gbps=20.0), ep.LinkState(20.0, 24.0)
    assert ep.online_select(ctx, g, dep, m, peer=deg_peer, link=deg_link, strict=True).point is ep.OperatingPoint.HOST
    for bad in (ep.OperatingPoint.CFK, ep.OperatingPoint.COPYBACK):
        with pytest.raises(ep.DoNoHarmViolation, match="R1-route"):
            ep.enforce_do_no_harm(bad, ctx, g, deg_peer, deg_link, deploy=dep)
    assert ep.enforce_do_no_harm(ep.OperatingPoint.COPYBACK, ctx, g, idle,
                                 ep.LinkState(HW.nvlink_gbps, HW.pcie_gbps, "pull"), deploy=dep) \
        is ep.OperatingPoint.COPYBACK
    tp = ep.Deployment(tp_enabled=True)
    assert math.isinf(m.predict_ms(ep.OperatingPoint.TP, ctx, idle, tp))
    assert ep.select_point(ctx, g, idle, tp, m).point is not ep.OperatingPoint.TP
    with pytest.raises(ep.DoNoHarmViolation, match="R1-tp-oracle"):
        ep.enforce_do_no_harm(ep.OperatingPoint.TP, ctx, g, idle, healthy, deploy=tp)
    meas = ep.Deployment(tp_enabled=True, tp_tpot_ms_per_token=20.6)
    assert m.predict_ms(ep.OperatingPoint.TP, ctx, idle, meas) == 20.6
    assert ep.enforce_do_no_harm(ep.OperatingPoint.TP, ctx, g, idle, healthy, deploy=meas) is ep.OperatingPoint.TP


# ---- what this package adds --------------------------------------------------------------- #
def test_n_device_model_and_relaxed_fit_rule():
    """Eight B200s: the KV read divides by eight, the per-peer memory test uses the per-peer
    share, and with allow_faster_cfk a fitting request may shard when predicted not slower."""
    g = ep.Geometry.llama3_8b()
    hw = ep.B200_NVSWITCH
    # anchors in the shape this library measures: ~2.3 ms weights, 7 TB/s KV reads, 25 us per layer exchanged
    kv = lambda t: t * g.kv_bytes_per_token / 7.0e12 * 1e3
    m = ep.DecodeStepModel.calibrate(g, {131072: 2.3 + kv(131072), 524288: 2.3 + kv(524288)},
                                     (1048576, 2.3 + kv(1048576 / 8) + 32 * 0.025), n_devices=8, hw=hw)
    assert m.beta_eff_gbps == pytest.approx(7000, rel=1e-6) and m.roundtrip_ms_per_layer == pytest.approx(0.025, rel=1e-6)
    peer = ep.PeerState(hbm_free_bytes=150 * 1024 ** 3, n_peers=7, nvlink_bw_gbps=hw.nvlink_gbps)
    dep = ep.Deployment(single_capacity_tokens=1_100_000, capacity_kv_bytes_per_token=g.kv_bytes_per_token)
    ctx = 1_000_000
    s = m.predict_ms(ep.OperatingPoint.SINGLE, ctx, peer, dep)
    c = m.predict_ms(ep.OperatingPoint.CFK, ctx, peer, dep)
    assert c < s / 3                                         # eight HBMs add up
    # the reference's rule: fits one GPU -> SINGLE
    assert ep.online_select(ctx, g, dep, m, peer=peer, strict=True).point is ep.OperatingPoint.SINGLE
    relaxed = ep.Deployment(single_capacity_tokens=1_100_000, capacity_kv_bytes_per_token=g.kv_bytes_per_token,
                            allow_faster_cfk=True)
    assert ep.online_select(ctx, g, relaxed, m, peer=peer, strict=True).point is ep.OperatingPoint.CFK
    # a short context is not worth the exchange even when relaxed
    assert ep.online_select(2048, g, relaxed, m, peer=peer, strict=True).point is ep.OperatingPoint.SINGLE
    # busy peers: never CFK, relaxed or not
    busy = ep.PeerState(hbm_free_bytes=150 * 1024 ** 3, n_peers=7, compute_idle=False, nvlink_bw_gbps=hw.nvlink_gbps)
    assert ep.online_select(ctx, g, relaxed, m, peer=busy, strict=True).point is ep.OperatingPoint.SINGLE
    # per-peer share: 8M tokens over 8 GPUs is 1M tokens = 128 GiB per peer
    big = 8_000_000
    assert ep.OperatingPoint.CFK in ep.admissible_points(big, g, peer, dep, hw)
    small = ep.PeerState(hbm_free_bytes=100 * 1024 ** 3, n_peers=7, nvlink_bw_gbps=hw.nvlink_gbps)
    assert ep.OperatingPoint.CFK not in ep.admissible_points(big, g, small, dep, hw)


def test_selector_counters():
    metrics.reset()
    g, m = _mha()
    ep.online_select(16384, g, ep.Deployment(), m, peer=_peer(), link=ep.LinkState(HW.nvlink_gbps, HW.pcie_gbps))
    snap = metrics.snapshot()
    assert snap["peerkv_selected_point_total{point=single}"] == 1
    assert snap["peerkv_admissible_points"] >= 1


def test_calibration_fit_from_injected_measurements():
    """The fit of calibration.py, with the GPU measurement replaced by numbers of the shape
    this library produces (7 TB/s reads, 9 us fixed, 20 us exchange on 8 GPUs)."""
    from peerkv_b200 import calibration as cal

    def fake(sizes, devices):
        us = lambda b: 9.0 + b / 7.0e6
        return {"device": "fake B200", "single_us": {s: us(s) for s in sizes},
                "multi_us": 9.0 + (4 << 30) / 8 / 7.0e6 + 20.0, "multi_bytes": 4 << 30,
                "nvlink_gbps": 760.0, "pcie_gbps": 52.0, "c_nvlink_us": 7.0, "c_pcie_us": 9.0}
    res = cal.calibrate_box(devices=[f"cuda:{i}" for i in range(8)], measure=fake)
    cm = cal.cost_model(res)
    assert cm.hbm_gbps == pytest.approx(7000, rel=1e-6) and cm.kernel_fixed_us == pytest.approx(9.0, abs=1e-6)
    assert cm.exchange_us == pytest.approx(20.0, abs=1e-6) and cm.nvlink_gbps == 760.0
    hw = cal.hardware(res)
    assert hw.pcie_gbps == 52.0 and hw.hbm_gbps == pytest.approx(7000, rel=1e-6)
    g = ep.Geometry.llama3_8b()
    m = cal.step_model(res, g, rest_of_step_ms=2.3)
    peer = ep.PeerState(hbm_free_bytes=150 * 1024 ** 3, n_peers=7, nvlink_bw_gbps=hw.nvlink_gbps)
    dep = ep.Deployment(single_capacity_tokens=1_100_000, capacity_kv_bytes_per_token=g.kv_bytes_per_token,
                        allow_faster_cfk=True)
    assert m.predict_ms(ep.OperatingPoint.CFK, 1_000_000, peer, dep) < m.predict_ms(ep.OperatingPoint.SINGLE, 1_000_000, peer, dep)
    one = cal.calibrate_box(devices=["cuda:0"], measure=lambda s, d: dict(fake(s, d), multi_us=None, multi_bytes=0))
    assert cal.cost_model(one).hbm_gbps == pytest.approx(7000, rel=1e-6)


@pytest.mark.gpu
def test_calibrate_box_on_the_gpu():
    """The constants come from this library's own kernels on this box and land in a plausible range."""
    import torch
    from peerkv_b200 import calibration as cal
    res = cal.calibrate_box(sizes=(1 << 29, 2 << 30))
    cm = cal.cost_model(res)
    assert 3000 < cm.hbm_gbps < 9000, res.to_dict()
    assert 0 <= cm.kernel_fixed_us < 100
    assert res.pcie_gbps > 5
    if torch.cuda.device_count() > 1:
        assert res.nvlink_gbps > 100 and 0 <= cm.exchange_us < 200
