"""Measures this box's cost-model constants with the library's own kernels and turns them
into the models the policy uses (the recipe of PeerKV umallm/runtime/calibration.py:76-148,
which times a decode-attention kernel over resident KV and divides the KV bytes by the
kernel time, plus one-way peer and host copies).

  calibrate_box()            -> CalibrationResult      (needs a GPU; ~2 s)
  cost_model(result)         -> placement.PeerKVCostModel   (per-layer attention model)
  hardware(result)           -> elastic_policy.Hardware
  step_model(result, ...)    -> elastic_policy.DecodeStepModel for a whole decode step

The measuring functions can be replaced (`measure=`) so the fitting is testable without a GPU.
"""
from __future__ import annotations

import math
import statistics
import time
from dataclasses import asdict, dataclass
from typing import Callable, Dict, Optional, Sequence

from . import elastic_policy as ep
from .placement import PeerKVCostModel

PAGE, HKV, HQ, D = 16, 8, 32, 128
BYTES_PER_TOKEN = 2 * HKV * D * 2


@dataclass
class CalibrationResult:
    device: str
    n_gpu: int
    single_us: Dict[int, float]          # KV bytes -> us of one single-GPU decode over them
    multi_us: Optional[float]            # us of one sharded decode over multi_bytes on n_gpu GPUs
    multi_bytes: int
    nvlink_gbps: float
    pcie_gbps: float
    c_nvlink_us: float
    c_pcie_us: float
    measured_at: float

    def to_dict(self):
        return asdict(self)


def _median_us(fn: Callable[[], None], dev, warmup: int = 3, reps: int = 9) -> float:
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(dev)
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(torch.cuda.current_stream(dev))
        fn()
        e1.record(torch.cuda.current_stream(dev))
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3)
    return statistics.median(ts)


def _gpu_measure(sizes: Sequence[int], devices) -> dict:
    """The real measurement: decode over `sizes` bytes of bf16 KV on devices[0], the same
    total sharded over all devices, and the copy engines."""
    import torch
    from . import ops
    from .group import PeerGroup
    devs = [torch.device(d) for d in devices]
    d0 = devs[0]
    B = 8
    out: dict = {"single_us": {}, "multi_us": None, "multi_bytes": 0}
    with torch.cuda.device(d0):
        big = max(sizes)
        n_pages = big // (BYTES_PER_TOKEN * PAGE)
        pool = torch.empty(2, n_pages, PAGE, HKV, D, dtype=torch.bfloat16, device=d0).normal_()
        q = torch.randn(B, HQ, D, device=d0).bfloat16()
        shard = ops.Shard(d0, B, HQ)
        for size in sizes:
            pages = size // (BYTES_PER_TOKEN * PAGE) // B * B
            bt = torch.arange(pages, dtype=torch.int32, device=d0).view(B, -1)
            sl = torch.full((B,), pages // B * PAGE, dtype=torch.int32, device=d0)
            o = torch.empty_like(q)
            out["single_us"][pages * PAGE * BYTES_PER_TOKEN] = _median_us(
                lambda: ops.decode_paged(q, pool[0], pool[1], bt, sl, out=o, shard=shard), d0)
        shard.close()
        # copies: large for bandwidth, 4 KiB for the set-up cost
        host = torch.empty(64 << 20, dtype=torch.uint8).pin_memory()
        dst = torch.empty(64 << 20, dtype=torch.uint8, device=d0)
        us = _median_us(lambda: dst.copy_(host, non_blocking=True), d0)
        out["pcie_gbps"] = host.numel() / us / 1e3
        out["c_pcie_us"] = _median_us(lambda: dst[:4096].copy_(host[:4096], non_blocking=True), d0)
        out["nvlink_gbps"], out["c_nvlink_us"] = 0.0, math.inf
        if len(devs) > 1:
            src = torch.empty(256 << 20, dtype=torch.uint8, device=devs[1])
            dstp = torch.empty(256 << 20, dtype=torch.uint8, device=d0)
            us = _median_us(lambda: dstp.copy_(src, non_blocking=True), d0)
            out["nvlink_gbps"] = src.numel() / us / 1e3
            out["c_nvlink_us"] = _median_us(lambda: dstp[:4096].copy_(src[:4096], non_blocking=True), d0)
    if len(devs) > 1:
        n = len(devs)
        total = max(sizes)
        per = total // n // (BYTES_PER_TOKEN * PAGE) // B * B        # pages per GPU
        grp = PeerGroup(devs, B, HQ)
        pools, tabs, lens = [], [], []
        for d in devs:
            p = pool[:, :per] if d == d0 else torch.empty(2, per, PAGE, HKV, D, dtype=torch.bfloat16, device=d).normal_()
            pools.append((p[0], p[1]))
            tabs.append(torch.arange(per, dtype=torch.int32, device=d).view(B, -1))
            lens.append(torch.full((B,), per // B * PAGE, dtype=torch.int32, device=d))
        o = torch.empty_like(q)
        with torch.cuda.device(d0):
            out["multi_us"] = _median_us(lambda: grp.decode_paged_local(q, pools, tabs, lens, out=o), d0)
        out["multi_bytes"] = per * n * PAGE * BYTES_PER_TOKEN
        grp.raise_on_status()
    out["device"] = torch.cuda.get_device_name(d0)
    return out


def calibrate_box(devices=None, sizes: Sequence[int] = (1 << 30, 4 << 30),
                  measure: Optional[Callable] = None) -> CalibrationResult:
    """Times the decode kernel over two KV sizes on one GPU, the same step sharded over
    all `devices`, and the copy paths.  `measure(sizes, devices) -> dict` replaces the GPU
    measurement (tests)."""
    if devices is None:
        import torch
        devices = [f"cuda:{i}" for i in range(torch.cuda.device_count())]
    m = (measure or _gpu_measure)(list(sizes), list(devices))
    return CalibrationResult(device=m.get("device", "?"), n_gpu=len(devices), single_us=dict(m["single_us"]),
                             multi_us=m.get("multi_us"), multi_bytes=int(m.get("multi_bytes", 0)),
                             nvlink_gbps=float(m.get("nvlink_gbps", 0.0)), pcie_gbps=float(m.get("pcie_gbps", 0.0)),
                             c_nvlink_us=float(m.get("c_nvlink_us", math.inf)),
                             c_pcie_us=float(m.get("c_pcie_us", math.inf)), measured_at=time.time())


def cost_model(res: CalibrationResult) -> PeerKVCostModel:
    """Per-layer attention model: KV read bandwidth and the kernel's fixed cost from the
    single-GPU points, the exchange cost from the sharded point (the defaults' exchange cost
    when the box has one GPU)."""
    if res.multi_us is not None and res.n_gpu > 1:
        m = PeerKVCostModel.calibrate(res.single_us, (res.multi_bytes, res.multi_us), res.n_gpu)
    else:
        big = max(res.single_us)
        m = PeerKVCostModel.calibrate(res.single_us, (big, res.single_us[big]), 1)
        m.exchange_us = PeerKVCostModel().exchange_us
    if res.nvlink_gbps > 0:
        m.nvlink_gbps = res.nvlink_gbps
    return m


def hardware(res: CalibrationResult, base: ep.Hardware = ep.B200_NVSWITCH) -> ep.Hardware:
    cm = cost_model(res)
    return ep.Hardware(name=res.device, hbm_gbps=cm.hbm_gbps,
                       nvlink_gbps=res.nvlink_gbps or base.nvlink_gbps, pcie_gbps=res.pcie_gbps or base.pcie_gbps,
                       c_nvlink_us=res.c_nvlink_us if math.isfinite(res.c_nvlink_us) else base.c_nvlink_us,
                       c_pcie_us=res.c_pcie_us if math.isfinite(res.c_pcie_us) else base.c_pcie_us,
                       c_hbm_us=cm.kernel_fixed_us, hbm_bytes=base.hbm_bytes)


def step_model(res: CalibrationResult, geom: ep.Geometry, rest_of_step_ms: float,
               n_devices: Optional[int] = None) -> ep.DecodeStepModel:
    """Whole-step model for `geom`: the attention part from the measured per-layer model
    (scaled by the layer count), everything else (`rest_of_step_ms`: weights + compute of
    one token) as the intercept."""
    cm = cost_model(res)
    n = n_devices or max(res.n_gpu, 1)
    A = rest_of_step_ms + geom.layers * cm.kernel_fixed_us / 1e3
    return ep.DecodeStepModel(geom, A, cm.hbm_gbps, cm.exchange_us / 1e3, n_devices=max(n, 2) if n > 1 else 2,
                              hw=hardware(res))
