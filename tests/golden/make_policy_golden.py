"""Golden decisions of the policy, made by running the REAL reference package.

    PEERKV_REFERENCE=/path/to/PeerKV python tests/golden/make_policy_golden.py

Imports `umallm.elastic_policy` and `umallm.runtime.selector` from that checkout and
records, for a grid of scenarios (the calibration anchors, contexts, peer and link states
of the reference's tests/test_elastic_policy.py and tests/test_no_harm.py plus a seeded
sweep), what the reference answers: the calibrated constants, predict_ms of every corner,
the admissible set, select_point's decision, online_select's decision, and which rule
enforce_do_no_harm trips for every (scenario, forced corner).  Written to
tests/golden/policy_golden.json.gz; tests/test_elastic_policy.py replays it under the
reference's hardware constants.
"""
from __future__ import annotations

import json
import math
import os
import random
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("PEERKV_REFERENCE",
                     os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference"))
sys.path.insert(0, REF)

from umallm import elastic_policy as ep  # noqa: E402
from umallm.runtime.selector import online_select  # noqa: E402

CALIBRATIONS = {
    # name: (geometry, single anchors, cfk point, copyback point)
    "mha_e27": ("mha", {16384: 17.257, 32768: 22.151}, (16384, 20.336), (16384, 38.402)),
    "mha_noharm": ("mha", {16384: 17.3, 32768: 22.2}, (32768, 25.1), (32768, 65.5)),
    "gqa_synth": ("gqa", {32768: 15.1, 131072: 21.4}, (131072, 19.9), (131072, 47.0)),
}


def fin(x):
    return None if (isinstance(x, float) and math.isinf(x)) else x


def main():
    geoms = {"mha": ep.Geometry.llama2_7b_mha(), "gqa": ep.Geometry.gqa_8kv()}
    out = {"hardware": {"hbm": ep.BETA_HBM_GBPS, "nvlink": ep.BETA_NVLINK_GBPS, "pcie": ep.BETA_PCIE_GBPS,
                        "c_nvlink_us": ep.C_NVLINK_US, "c_pcie_us": ep.C_PCIE_US, "c_hbm_us": ep.C_HBM_US},
           "calibrations": {}, "scenarios": []}
    rng = random.Random(7)
    for cname, (gname, singles, cfk, cb) in CALIBRATIONS.items():
        geom = geoms[gname]
        model = ep.DecodeStepModel.calibrate(geom, single_pts=singles, cfk_pt=cfk, copyback_pt=cb)
        out["calibrations"][cname] = {
            "geom": gname, "single_pts": {str(k): v for k, v in singles.items()}, "cfk_pt": list(cfk),
            "copyback_pt": list(cb), "A_ms": model.A_ms, "beta_eff_gbps": model.beta_eff_gbps,
            "roundtrip_ms_per_layer": model.roundtrip_ms_per_layer, "copyback_eff": model.copyback_eff,
            "tp_bound_143360": model.predict_tp_bound_ms(143360)}
        cap = ep._single_capacity_tokens(geom, ep.Deployment())
        ctxs = [1, 1024, 16384, 32768, cap - 1, cap, cap + 1, 143360, cap + 50000, 253536, 400000]
        peers = [dict(hbm_free_bytes=70 * 1024 ** 3, compute_idle=True, nvlink_bw_gbps=ep.BETA_NVLINK_GBPS),
                 dict(hbm_free_bytes=70 * 1024 ** 3, compute_idle=False, nvlink_bw_gbps=ep.BETA_NVLINK_GBPS),
                 dict(hbm_free_bytes=70 * 1024 ** 3, compute_idle=True, nvlink_bw_gbps=ep.BETA_PCIE_GBPS / 2),
                 dict(hbm_free_bytes=70 * 1024 ** 3, compute_idle=True, nvlink_bw_gbps=20.0),
                 dict(hbm_free_bytes=0, compute_idle=True, nvlink_bw_gbps=ep.BETA_NVLINK_GBPS)]
        for _ in range(6):
            peers.append(dict(hbm_free_bytes=rng.choice([0, 8, 35, 70]) * 1024 ** 3,
                              compute_idle=rng.random() < 0.5,
                              nvlink_bw_gbps=rng.choice([ep.BETA_NVLINK_GBPS, 100.0, 10.0])))
        deploys = [dict(), dict(tp_enabled=True), dict(tp_enabled=True, tp_tpot_ms_per_token=20.6)]
        for ctx in ctxs:
            for pk in peers:
                for dk in deploys:
                    peer, dep = ep.PeerState(**pk), ep.Deployment(**dk)
                    link = ep.LinkState.from_peer(peer)
                    adm = ep.admissible_points(ctx, geom, peer, dep)
                    dec = ep.select_point(ctx, geom, peer, dep, model)
                    on = online_select(ctx, geom, dep, model, peer=peer, link=link, strict=False)
                    gate = {}
                    for p in ep.OperatingPoint:
                        if p is ep.OperatingPoint.INFEASIBLE:
                            continue
                        try:
                            ep.enforce_do_no_harm(p, ctx, geom, peer, link, deploy=dep)
                            gate[p.value] = "ok"
                        except ep.DoNoHarmViolation as e:
                            gate[p.value] = str(e).split(":", 1)[0]
                    out["scenarios"].append({
                        "calibration": cname, "ctx": ctx, "peer": pk, "deploy": dk,
                        "admissible": sorted(p.value for p in adm),
                        "predict_ms": {p.value: fin(model.predict_ms(p, ctx, peer, dep))
                                       for p in ep.OperatingPoint if p is not ep.OperatingPoint.INFEASIBLE},
                        "select": {"point": dec.point.value, "predicted_ms": fin(dec.predicted_ms),
                                   "reason": dec.reason},
                        "select_deadline_1ms_meets": ep.select_point(ctx, geom, peer, dep, model, 1.0).meets_deadline,
                        "online": on.point.value, "gate": gate})
    import gzip
    path = os.path.join(HERE, "policy_golden.json.gz")
    with gzip.GzipFile(path, "wb", mtime=0) as f:
        f.write(json.dumps(out, separators=(",", ":")).encode())
    print("wrote", path, os.path.getsize(path), "bytes,", len(out["scenarios"]), "scenarios")


if __name__ == "__main__":
    main()
