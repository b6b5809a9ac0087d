"""Placement and operating-point logic of the compute-follows-KV path, re-expressed
for N uniform B200 peers behind an NVSwitch.

Mirrors, for this path only, PeerKV's host-side cost helpers and selector:

  partial_bytes, balanced_partition            umallm/multigpu.py:351-359, 362-377
  PeerKVCostModel.decode_step_parallel_us      umallm/multigpu.py:191-215
  PeerKVCostModel.max_context_for_slo_parallel umallm/multigpu.py:217-239
(the operating-point selector and the do-no-harm rules are in elastic_policy.py)

The reference's constants are dual-A100 measurements (773 / 273 GB/s, 12-24 us set-up).
The defaults here are what this library measures on B200 (effective KV read bandwidth
of the decode kernel, cost of one exchange); `PeerKVCostModel.calibrate` refits them
from two timed single-GPU points and one N-GPU point, and calibration.calibrate_box
measures those points with the library's own kernels (the recipe of
umallm/runtime/calibration.py:76-148).

The page -> GPU maps themselves are made on the device (`pkv_split_block_table`,
group.PeerGroup.split_table); `PagePlacer` is the allocation-time counterpart that
decides where a NEW page goes.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

# measured with this library on B200 (bf16, Hkv 8, D 128, 16-token pages)
B200_KV_READ_GBPS = 7000.0       # decode kernel, >= 4 GiB per GPU
B200_NVLINK_GBPS = 770.0         # per direction per GPU, measured peer copy
B200_KERNEL_FIXED_US = 10.0      # launch + pipeline fill + split-K tail of one shard kernel
B200_EXCHANGE_US = 18.0          # q publish + flag hops + final merge, all peers together
B200_HBM_BYTES = 180 * 1024 ** 3


def partial_bytes(heads: int, head_dim: int, lse_bytes: int = 4, o_bytes: int = 2) -> int:
    """Bytes of one decode-step partial (O + lse) exchanged per remote shard; independent
    of the KV size.  Defaults as in the reference (fp16 O); this library sends fp32 O
    (`o_bytes=4`)."""
    return heads * head_dim * o_bytes + heads * lse_bytes


def balanced_partition(n_blocks: int, hbm_bw_gbps_per_device: Sequence[float]) -> List[int]:
    """Blocks per device in proportion to its HBM bandwidth (equal GPUs: an even split,
    the optimum); floors first, the remainder handed out one block at a time from
    device 0."""
    w = [float(b) for b in hbm_bw_gbps_per_device]
    tot = sum(w) or 1.0
    share = [int(n_blocks * x / tot) for x in w]
    for k in range(n_blocks - sum(share)):
        share[k % len(share)] += 1
    return share


@dataclass
class PeerKVCostModel:
    """step = compute + max_d(c_kernel + bytes_d / beta_hbm) + exchange(n_remote)."""
    hbm_gbps: float = B200_KV_READ_GBPS
    nvlink_gbps: float = B200_NVLINK_GBPS
    kernel_fixed_us: float = B200_KERNEL_FIXED_US
    exchange_us: float = B200_EXCHANGE_US

    def decode_step_parallel_us(self, blocks_per_device: Sequence[int], block_bytes: int,
                                compute_us: float = 0.0, part_bytes: Optional[int] = None,
                                heads: int = 0, head_dim: int = 0) -> float:
        bpd = [int(n) for n in blocks_per_device if int(n) > 0]
        if not bpd:
            return compute_us
        reads = [self.kernel_fixed_us + n * block_bytes / (self.hbm_gbps * 1e3) for n in bpd]
        if part_bytes is None:
            part_bytes = partial_bytes(heads, head_dim) if (heads and head_dim) else 2080
        n_remote = max(0, len(bpd) - 1)
        # one latency-bound exchange for all peers (NVSwitch: peers do not share a link),
        # plus the bytes that land on the home GPU's ingress
        transfer = (self.exchange_us + n_remote * part_bytes / (self.nvlink_gbps * 1e3)) if n_remote else 0.0
        return compute_us + max(reads) + transfer

    def max_context_for_slo_parallel(self, deadline_us: float, block_bytes: int, n_devices: int = 2,
                                     compute_us: float = 0.0, attn_us: float = 0.0,
                                     part_bytes: int = 2080) -> dict:
        transfer = (self.exchange_us + (n_devices - 1) * part_bytes / (self.nvlink_gbps * 1e3)) \
            if n_devices > 1 else 0.0
        budget = deadline_us - compute_us - attn_us - transfer - self.kernel_fixed_us
        if budget <= 0:
            return {"feasible": False, "max_blocks": 0, "max_blocks_per_device": 0, "n_devices": n_devices}
        per_dev = budget * self.hbm_gbps * 1e3 / block_bytes
        return {"feasible": True, "max_blocks": int(n_devices * per_dev),
                "max_blocks_per_device": int(per_dev), "n_devices": n_devices,
                "speedup_vs_single": float(n_devices)}

    @classmethod
    def calibrate(cls, single_pts: dict, multi_pt, n_devices: int) -> "PeerKVCostModel":
        """single_pts = {bytes: us} (>= 2 single-GPU timings), multi_pt = (total_bytes, us)
        on n_devices with an even split.  Fits beta_hbm and the kernel's fixed cost from
        the single-GPU line and the exchange cost from the multi-GPU point."""
        if len(single_pts) < 2:
            raise ValueError("calibrate needs >= 2 single-GPU anchors")
        (b1, t1), (b2, t2) = sorted(single_pts.items())[:2]
        if b1 == b2:
            raise ValueError("degenerate anchors: equal sizes")
        slope = (t2 - t1) / (b2 - b1)
        if slope <= 0:
            raise ValueError("non-physical anchors: time does not grow with bytes; remeasure")
        m = cls(hbm_gbps=1e-3 / slope, kernel_fixed_us=max(0.0, t1 - slope * b1))
        tb, tt = multi_pt
        m.exchange_us = max(0.0, tt - m.kernel_fixed_us - (tb / n_devices) * slope)
        return m


def capacity_spill_split(pages_per_seq: Sequence[int], seq_lens: Sequence[int], page_size: int,
                         caps: Sequence[float]):
    """Capacity-limited placement of a batch's pages (the ragged benchmark configuration).

    The pages of all sequences form one list, sequence after sequence.  GPU g takes up to
    floor(caps[g] * total / N) of them in order; what is left spills to the next GPU and
    the last GPU takes the rest.  Pools are compact: a page's local id is its arrival order
    on its GPU.  Returns (tables [N, B, W] int32 local ids, tokens [N, B] int64, pages used
    per GPU [N]); only a sequence's last page can be partial and it stays last in its
    owner's list."""
    import numpy as np
    n = len(caps)
    pages = np.asarray(pages_per_seq, dtype=np.int64)
    lens = np.asarray(seq_lens, dtype=np.int64)
    B, total = len(pages), int(pages.sum())
    quota = [int(c * total / n) for c in caps]
    quota[-1] = total
    hi = np.minimum(np.cumsum(quota), total)          # GPU g owns flat pages [lo[g], hi[g])
    hi[-1] = total
    lo = np.concatenate([[0], hi[:-1]])
    W = int(pages.max()) if B else 1
    tab = np.zeros((n, B, max(W, 1)), dtype=np.int32)
    tok = np.zeros((n, B), dtype=np.int64)
    start = np.concatenate([[0], np.cumsum(pages)])
    for i in range(B):
        p0, p1 = int(start[i]), int(start[i + 1])
        for g in range(n):
            a, b = max(p0, int(lo[g])), min(p1, int(hi[g]))
            if a >= b:
                continue
            tab[g, i, :b - a] = np.arange(a - lo[g], b - lo[g], dtype=np.int32)
            tok[g, i] = (b - a) * page_size - ((p1 * page_size - (start[i] * page_size + lens[i])) if b == p1 else 0)
    used = (hi - lo).astype(np.int64)
    return tab, tok, used


class PagePlacer:
    """Allocation-time page -> (gpu, local id) decisions for a sharded KV pool.

    policy 'round_robin': page p -> GPU p mod N (the batched benchmark configuration);
    policy 'balanced': keep every GPU's page count proportional to its bandwidth
    (`balanced_partition`), new pages going to the most under-filled GPU;
    policy 'capacity_spill': fill GPUs in order up to their capacity, then spill on.
    """

    def __init__(self, n_gpus: int, policy: str = "round_robin",
                 capacity_pages: Optional[Sequence[int]] = None,
                 bandwidth_gbps: Optional[Sequence[float]] = None):
        if policy not in ("round_robin", "balanced", "capacity_spill"):
            raise ValueError(policy)
        self.n, self.policy = n_gpus, policy
        self.capacity = list(capacity_pages) if capacity_pages is not None else [1 << 62] * n_gpus
        self.bw = list(bandwidth_gbps) if bandwidth_gbps is not None else [1.0] * n_gpus
        self.used = [0] * n_gpus
        self._next = 0

    def place(self) -> tuple:
        """Returns (gpu, local page id) for one new page."""
        if self.policy == "round_robin":
            for _ in range(self.n):
                g = self._next % self.n
                self._next += 1
                if self.used[g] < self.capacity[g]:
                    break
            else:
                raise MemoryError("every GPU is at capacity")
        elif self.policy == "capacity_spill":
            g = next((i for i in range(self.n) if self.used[i] < self.capacity[i]), None)
            if g is None:
                raise MemoryError("every GPU is at capacity")
        else:
            tot = sum(self.used) + 1
            want = balanced_partition(tot, self.bw)
            cands = [i for i in range(self.n) if self.used[i] < self.capacity[i]]
            if not cands:
                raise MemoryError("every GPU is at capacity")
            g = max(cands, key=lambda i: (want[i] - self.used[i], -i))
        local = self.used[g]
        self.used[g] += 1
        return g, local
