"""Drop-in for `umallm.elastic_policy` (PeerKV umallm/elastic_policy.py): the policy that
decides, per request, whether decode attention runs on one GPU or follows the KV.

Same names, arguments and decisions as the reference:

  OperatingPoint, Geometry, PeerState, Deployment, LinkState, Decision      :56-62, 65-101, 288-304
  DecodeStepModel.predict_ms / predict_tp_bound_ms / calibrate               :103-219
  admissible_points, select_point, link_degraded                             :222-241, 261-288
  DoNoHarmViolation, enforce_do_no_harm  (R1-fit, R1-busy, R1-route, R1-tp-oracle)  :307-365
  online_select (single exit: candidate set that obeys R1 by construction, the
  gate as tripwire, repair when not strict)        umallm/runtime/selector.py:112-190

What is different, on purpose:

  * The hardware numbers are not module constants baked into the formulas but a
    `Hardware` record.  `A100_NV12` holds the reference's dual-A100 measurements (its
    tests and golden decisions replay under it); `B200_NVSWITCH` holds what this library
    measures on B200 and is the default.  The reference's constant names (BETA_*, C_*)
    are exported and mean the default record's values.
  * N devices, not two: a context splits evenly over `n_devices` GPUs
    (`DecodeStepModel.n_devices`, `PeerState.n_peers`), and the peers' free memory is per
    peer.  With n_devices = 2 every formula reduces to the reference's.
  * On B200 the sharded path can beat one GPU even when the context fits (the HBM
    bandwidths add and the exchange costs microseconds), so R1-fit has an opt-in relaxed
    form (`Deployment.allow_faster_cfk`): a fitting request may take CFK when the
    calibrated model predicts it is not slower.  Off by default: the reference's rule.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field, replace
from typing import Dict, Optional, Set, Tuple


@dataclass(frozen=True)
class Hardware:
    """Measured constants of one box: bandwidths in GB/s, per-transfer set-up costs in us."""
    name: str
    hbm_gbps: float               # effective KV read bandwidth of the decode kernel
    nvlink_gbps: float            # one way, peer to peer
    pcie_gbps: float              # pinned host memory to GPU
    c_nvlink_us: float
    c_pcie_us: float
    c_hbm_us: float
    hbm_bytes: int
    lender_flops_retained: float = 0.6676    # a GPU that lends attention compute keeps ~2/3 of its FLOPs
    borrower_bw_retained: float = 0.9974


A100_NV12 = Hardware("dual A100-SXM4-80GB, NV12", 773.0, 273.0, 24.0, 23.6, 12.6, 12.3, 80 * 1024 ** 3)
B200_NVSWITCH = Hardware("B200, NVLink 5 / NVSwitch", 7000.0, 770.0, 55.0, 8.0, 10.0, 10.0, 180 * 1024 ** 3)
DEFAULT_HW = B200_NVSWITCH

BETA_HBM_GBPS = DEFAULT_HW.hbm_gbps
BETA_NVLINK_GBPS = DEFAULT_HW.nvlink_gbps
BETA_PCIE_GBPS = DEFAULT_HW.pcie_gbps
C_NVLINK_US = DEFAULT_HW.c_nvlink_us
C_PCIE_US = DEFAULT_HW.c_pcie_us
C_HBM_US = DEFAULT_HW.c_hbm_us
PARTIAL_BYTES_DEFAULT = 2080
BORROWER_BW_RETAINED = DEFAULT_HW.borrower_bw_retained
LENDER_FLOPS_RETAINED = DEFAULT_HW.lender_flops_retained


class OperatingPoint(enum.Enum):
    SINGLE = "single"                 # the whole context on the query's GPU
    COPYBACK = "copyback"             # KV on peers, streamed back over NVLink every step
    CFK = "compute_follows_kv"        # KV on peers, partials computed there, (O, lse) exchanged
    TP = "tp"                         # tensor parallelism, a deploy-time choice
    HOST = "host"                     # KV in host memory over PCIe
    INFEASIBLE = "infeasible"


_PEER_PATHS = (OperatingPoint.CFK, OperatingPoint.COPYBACK)


@dataclass(frozen=True)
class Geometry:
    name: str
    layers: int
    kv_bytes_per_token: int          # K + V over all layers
    weight_bytes: int

    @staticmethod
    def llama2_7b_mha() -> "Geometry":
        return Geometry("MHA", 32, 32 * 2 * 32 * 128 * 2, int(12.0625 * 1024 ** 3))

    @staticmethod
    def gqa_8kv() -> "Geometry":
        return Geometry("GQA", 32, 32 * 2 * 8 * 128 * 2, int(13.0 * 1024 ** 3))

    @staticmethod
    def llama3_8b() -> "Geometry":
        return Geometry("Llama-3-8B", 32, 32 * 2 * 8 * 128 * 2, int(14.96 * 1024 ** 3))


@dataclass
class PeerState:
    """What the peers can lend right now (per peer)."""
    hbm_free_bytes: int = 70 * 1024 ** 3
    compute_idle: bool = True
    nvlink_bw_gbps: float = BETA_NVLINK_GBPS
    n_peers: int = 1


@dataclass
class Deployment:
    tp_enabled: bool = False
    single_capacity_tokens: int = 116016       # measured ceiling for the MHA geometry on one GPU
    tp_capacity_tokens: int = 253536
    tp_tpot_ms_per_token: Optional[float] = None
    capacity_kv_bytes_per_token: int = 524288  # the geometry single_capacity_tokens was measured with
    allow_faster_cfk: bool = False             # relaxed R1-fit (see the module text)


@dataclass(frozen=True)
class LinkState:
    """Interconnect state when the decision is taken.  transfer_dir is recorded only."""
    nvlink_eff_gbps: float = BETA_NVLINK_GBPS
    pcie_eff_gbps: float = BETA_PCIE_GBPS
    transfer_dir: str = "push"

    @classmethod
    def from_peer(cls, peer: PeerState, hw: Hardware = DEFAULT_HW) -> "LinkState":
        return cls(nvlink_eff_gbps=peer.nvlink_bw_gbps, pcie_eff_gbps=hw.pcie_gbps)


@dataclass
class Decision:
    point: OperatingPoint
    predicted_ms: float
    admissible: Set[OperatingPoint] = field(default_factory=set)
    meets_deadline: bool = True
    reason: str = ""


class DoNoHarmViolation(RuntimeError):
    """A chosen operating point would break a do-no-harm rule."""


def _single_capacity_tokens(geom: Geometry, deploy: Deployment) -> int:
    """One GPU's token capacity for `geom`, scaled from the measured ceiling by KV bytes per token."""
    return int(deploy.single_capacity_tokens * deploy.capacity_kv_bytes_per_token / geom.kv_bytes_per_token)


@dataclass
class DecodeStepModel:
    """Calibrated decode-step latency (ms per token) of each corner:

        SINGLE    A + kv(ctx)
        CFK       A + kv(ctx / n) + layers * roundtrip
        COPYBACK  A + kv(ctx / n) + eff * (remote bytes / nvlink + layers * c_nvlink)
        HOST      A + kv(ctx / n) + remote bytes / pcie + layers * c_pcie
        TP        the measured TPOT when there is one, else inf (admissibility only)

    kv(t) = t * kv_bytes_per_token / beta_eff; A is the weights + compute intercept."""
    geom: Geometry
    A_ms: float
    beta_eff_gbps: float
    roundtrip_ms_per_layer: float
    copyback_eff: float = 1.0
    n_devices: int = 2
    hw: Hardware = DEFAULT_HW

    def _kv_read_ms(self, n_tokens: float) -> float:
        return (n_tokens * self.geom.kv_bytes_per_token) / (self.beta_eff_gbps * 1e9) * 1e3

    def _stream_ms(self, tokens: float, gbps: float, setup_us: float) -> float:
        if gbps <= 0:
            return math.inf
        return tokens * self.geom.kv_bytes_per_token / (gbps * 1e9) * 1e3 + self.geom.layers * setup_us / 1e3

    def _copyback_ms(self, peer_tokens: float, nvlink_bw_gbps: float) -> float:
        return self.copyback_eff * self._stream_ms(peer_tokens, nvlink_bw_gbps, self.hw.c_nvlink_us)

    def predict_ms(self, point: OperatingPoint, ctx_tokens: int, peer: PeerState,
                   deploy: Deployment) -> float:
        local = ctx_tokens / self.n_devices
        remote = ctx_tokens - local
        if point is OperatingPoint.SINGLE:
            return self.A_ms + self._kv_read_ms(ctx_tokens)
        if point is OperatingPoint.TP:
            return math.inf if deploy.tp_tpot_ms_per_token is None else deploy.tp_tpot_ms_per_token
        if point is OperatingPoint.CFK:
            extra = self.geom.layers * self.roundtrip_ms_per_layer
        elif point is OperatingPoint.COPYBACK:
            extra = self._copyback_ms(remote, peer.nvlink_bw_gbps)
        elif point is OperatingPoint.HOST:
            extra = self._stream_ms(remote, self.hw.pcie_gbps, self.hw.c_pcie_us)
        else:
            return math.inf
        return self.A_ms + self._kv_read_ms(local) + extra

    def predict_tp_bound_ms(self, ctx_tokens: int, allreduce_us_per_layer: Optional[float] = None,
                            weight_stream_gbps: Optional[float] = None) -> float:
        """Optimistic analytic bound for TP over n_devices (a diagnostic; never used to choose):
        the weight-read share of A and the KV read divide by n, one exchange per layer is added."""
        ar = self.hw.c_nvlink_us if allreduce_us_per_layer is None else allreduce_us_per_layer
        gbps = weight_stream_gbps or self.beta_eff_gbps
        weight_ms = min(self.geom.weight_bytes / (gbps * 1e9) * 1e3, self.A_ms)
        return ((self.A_ms - weight_ms) + weight_ms / self.n_devices
                + self._kv_read_ms(ctx_tokens / self.n_devices) + self.geom.layers * ar / 1e3)

    @classmethod
    def calibrate(cls, geom: Geometry, single_pts: Dict[int, float], cfk_pt: Tuple[int, float],
                  copyback_pt: Optional[Tuple[int, float]] = None, n_devices: int = 2,
                  hw: Hardware = DEFAULT_HW) -> "DecodeStepModel":
        """A and beta_eff from the two smallest SINGLE anchors {ctx: ms}, the round trip from
        one CFK point (ctx, ms), the copy-back efficiency from one COPYBACK point (optional
        here: this library has no copy-back data path of its own to measure)."""
        if len(single_pts) < 2:
            raise ValueError("calibrate needs >=2 SINGLE anchors")
        (c1, m1), (c2, m2) = sorted(single_pts.items())[:2]
        if c1 == c2:
            raise ValueError(f"degenerate SINGLE anchors: equal ctx {c1}")
        slope = (m2 - m1) / (c2 - c1)                       # ms per token
        if slope <= 0:
            raise ValueError(f"non-physical anchors: latency not increasing with context "
                             f"(slope {slope:.3e} ms/token from {single_pts}); remeasure")
        m = cls(geom, m1 - slope * c1, geom.kv_bytes_per_token / (slope * 1e-3) / 1e9, 0.0,
                n_devices=n_devices, hw=hw)
        cctx, cms = cfk_pt
        m.roundtrip_ms_per_layer = max(0.0, (cms - m.A_ms - m._kv_read_ms(cctx / n_devices)) / geom.layers)
        if copyback_pt is not None:
            pctx, pms = copyback_pt
            plocal = pctx / n_devices
            ideal = m._kv_read_ms(plocal) + m._stream_ms(pctx - plocal, hw.nvlink_gbps, hw.c_nvlink_us)
            m.copyback_eff = max(1.0, (pms - m.A_ms) / ideal) if ideal > 0 else 1.0
        return m


def link_degraded(peer: PeerState, hw: Hardware = DEFAULT_HW) -> bool:
    return peer.nvlink_bw_gbps < hw.pcie_gbps


def admissible_points(ctx_tokens: int, geom: Geometry, peer: PeerState, deploy: Deployment,
                      hw: Hardware = DEFAULT_HW) -> Set[OperatingPoint]:
    """Corners that are available to this request right now."""
    pts = {OperatingPoint.HOST}                              # slow, but always there
    if ctx_tokens <= _single_capacity_tokens(geom, deploy):
        pts.add(OperatingPoint.SINGLE)
    n = max(1, peer.n_peers) + 1
    per_peer_tokens = (ctx_tokens - ctx_tokens // n + (n - 2)) // (n - 1)      # ceil of the remote share per peer
    fits_peers = per_peer_tokens * geom.kv_bytes_per_token <= peer.hbm_free_bytes
    if fits_peers and peer.n_peers > 0 and not link_degraded(peer, hw):
        pts.add(OperatingPoint.COPYBACK)                     # needs the peers' memory and the link
        if peer.compute_idle:
            pts.add(OperatingPoint.CFK)                      # and their compute
    if deploy.tp_enabled and ctx_tokens <= deploy.tp_capacity_tokens:
        pts.add(OperatingPoint.TP)
    return pts


def select_point(ctx_tokens: int, geom: Geometry, peer: PeerState, deploy: Deployment,
                 model: DecodeStepModel, deadline_ms: Optional[float] = None) -> Decision:
    """The admissible corner with the lowest predicted step latency; an SLO miss is flagged,
    not refused."""
    adm = admissible_points(ctx_tokens, geom, peer, deploy, model.hw)
    if not adm:
        return Decision(OperatingPoint.INFEASIBLE, math.inf, adm, False, "no admissible point")
    preds = {p: model.predict_ms(p, ctx_tokens, peer, deploy) for p in adm}
    best = min(preds, key=preds.get)
    notes = []
    if OperatingPoint.SINGLE not in adm:
        notes.append("ctx OOMs single GPU")
    if OperatingPoint.COPYBACK in adm and OperatingPoint.CFK not in adm:
        notes.append("peer compute busy -> CFK inadmissible, copy-back only")
    if link_degraded(peer, model.hw):
        notes.append("NVLink degraded -> route to host")
    return Decision(best, preds[best], adm, deadline_ms is None or preds[best] <= deadline_ms,
                    "; ".join(notes) or "fastest admissible")


def enforce_do_no_harm(point: OperatingPoint, ctx_tokens: int, geom: Geometry, peer: PeerState,
                       link: Optional[LinkState] = None, deploy: Optional[Deployment] = None,
                       single_capacity_tokens: Optional[int] = None,
                       model: Optional[DecodeStepModel] = None) -> OperatingPoint:
    """The one place the R1 rules live.  Returns `point` when legal, raises otherwise."""
    link = link or LinkState.from_peer(peer, model.hw if model else DEFAULT_HW)
    cap = single_capacity_tokens
    if cap is None and deploy is not None:
        cap = _single_capacity_tokens(geom, deploy)
    if cap is not None and ctx_tokens <= cap and point is not OperatingPoint.SINGLE:
        relaxed = (deploy is not None and deploy.allow_faster_cfk and point is OperatingPoint.CFK
                   and model is not None
                   and model.predict_ms(point, ctx_tokens, peer, deploy)
                   <= model.predict_ms(OperatingPoint.SINGLE, ctx_tokens, peer, deploy))
        if not relaxed:
            raise DoNoHarmViolation(f"R1-fit: fits single ({ctx_tokens} <= {cap} tokens) but chose {point.value}")
    if point is OperatingPoint.CFK and not peer.compute_idle:
        raise DoNoHarmViolation("R1-busy: peer compute-busy, CFK forbidden "
                                f"(lender retains only {LENDER_FLOPS_RETAINED:.2%} FLOPs)")
    if point in _PEER_PATHS and link.nvlink_eff_gbps < link.pcie_eff_gbps:
        raise DoNoHarmViolation(f"R1-route: nvlink {link.nvlink_eff_gbps:.1f} < pcie "
                                f"{link.pcie_eff_gbps:.1f} GB/s, route host")
    if point is OperatingPoint.TP and deploy is not None and deploy.tp_tpot_ms_per_token is None:
        raise DoNoHarmViolation("R1-tp-oracle: TP chosen without a measured TPOT (admissibility-only corner)")
    return point


# --------------------------------------------------------------------------- #
# the selector's single exit (umallm/runtime/selector.py)
# --------------------------------------------------------------------------- #
def _r1_candidates(ctx_tokens, geom, peer, link, deploy, model) -> Set[OperatingPoint]:
    """The admissible set cut down so that the rules hold by construction."""
    adm = admissible_points(ctx_tokens, geom, peer, deploy, model.hw)
    if ctx_tokens <= _single_capacity_tokens(geom, deploy) and OperatingPoint.SINGLE in adm:
        keep = {OperatingPoint.SINGLE}
        if deploy.allow_faster_cfk and OperatingPoint.CFK in adm and peer.compute_idle \
                and link.nvlink_eff_gbps >= link.pcie_eff_gbps \
                and model.predict_ms(OperatingPoint.CFK, ctx_tokens, peer, deploy) \
                <= model.predict_ms(OperatingPoint.SINGLE, ctx_tokens, peer, deploy):
            keep.add(OperatingPoint.CFK)
        return keep
    if link.nvlink_eff_gbps < link.pcie_eff_gbps:
        adm -= set(_PEER_PATHS)
    if not peer.compute_idle:
        adm.discard(OperatingPoint.CFK)
    return adm


def online_select(ctx_tokens: int, geom: Geometry, deploy: Deployment, model: DecodeStepModel,
                  deadline_ms: Optional[float] = None, peer: Optional[PeerState] = None,
                  link: Optional[LinkState] = None, strict: bool = False) -> Decision:
    """Live state -> candidates that obey R1 -> fastest of them -> the gate as a tripwire ->
    counters.  With strict a violation raises; otherwise the decision is repaired to the
    safest legal corner and the violation is counted."""
    from . import metrics as _m
    peer = peer or PeerState()
    link = link or LinkState.from_peer(peer, model.hw)
    cands = _r1_candidates(ctx_tokens, geom, peer, link, deploy, model)
    d = select_point(ctx_tokens, geom, peer, deploy, model, deadline_ms)
    if cands and d.point not in cands:
        preds = {p: model.predict_ms(p, ctx_tokens, peer, deploy) for p in cands}
        best = min(preds, key=preds.get)
        d = replace(d, point=best, predicted_ms=preds[best], admissible=cands,
                    meets_deadline=deadline_ms is None or preds[best] <= deadline_ms,
                    reason=d.reason + "; R1-restricted")
    try:
        enforce_do_no_harm(d.point, ctx_tokens, geom, peer, link, deploy=deploy, model=model)
    except DoNoHarmViolation as e:
        rule = str(e).split(":", 1)[0]
        _m.DO_NO_HARM_VIOL.labels(rule=rule).inc()
        if strict:
            raise
        legal = _r1_candidates(ctx_tokens, geom, peer, link, deploy, model) - {d.point}
        point = (min(legal, key=lambda p: model.predict_ms(p, ctx_tokens, peer, deploy))
                 if legal else OperatingPoint.HOST)
        enforce_do_no_harm(point, ctx_tokens, geom, peer, link, deploy=deploy, model=model)
        pred = model.predict_ms(point, ctx_tokens, peer, deploy)
        d = replace(d, point=point, predicted_ms=pred,
                    meets_deadline=deadline_ms is None or pred <= deadline_ms,
                    reason=f"{d.reason}; repaired({rule})->{point.value}")
    _m.SELECTED_POINT.labels(point=d.point.value).inc()
    _m.ADMISSIBLE_POINTS.set(len(d.admissible))
    _m.PEER_BUSY.labels(peer="all").set(0 if peer.compute_idle else 1)
    _m.LINK_EFF_GBPS.labels(fabric="nvlink").set(link.nvlink_eff_gbps)
    return d
