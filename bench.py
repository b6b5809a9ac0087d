"""Benchmark of peer-parallel split-K decode attention on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline workload `paged-bf16` (batched paged decode attention): batch 16, 32 query / 8
kv heads, head_dim 128, 131072-token context per sequence, bf16 KV in 16-token pages,
block table = seeded random permutation of the page pool; for N > 1 page p lives on GPU
p mod N (strong scaling: the same 8 GiB of KV is split), q is resident on GPU 0 and the
partials are merged on GPU 0.  A step is one decode-attention layer.  Synthetic N(0,1)
data stands in for everything (the path has no dataset).

Prints ONE JSON line: effective KV GB/s (algorithmic KV bytes / step time) with the
per-layer latency, the roofline of the dominant kernel, an end-to-end number with host
buffers, a parity check of the timed output against the CPU oracle at full context
(every rank checks its own shard, partials are gathered and merged on rank 0; the run
exits non-zero when it fails), the same for the other attention shapes (`workloads`,
a few steps each), and the CPU baseline: the reference's torch path timed on this box's
host cores on a bounded sample.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

D, PAGE = 128, 16
PEAK_FALLBACK_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of decode_partial_kernel per launch and
# algorithmic byte, from ncu captures on 1 GiB pools (traffic grows in proportion to the
# tokens read)
NCU_TRAFFIC_PER_ALGO_BYTE = {"bf16": (1.07455e9 + 4.46e6) / 1073741824, "int8": 1.002, "fp8": 1.002}
METRIC = "decode_attn_effective_kv_bandwidth"

WORKLOADS = {
    # name: batch, Hq, Hkv, tokens per sequence (None = ragged), kv format, placement
    "paged-bf16": dict(B=16, HQ=32, HKV=8, ctx=131072, fmt="bf16", place="round_robin"),
    "ragged-bf16": dict(B=64, HQ=32, HKV=8, ctx=None, fmt="bf16", place="capacity_spill"),
    "quant-int8": dict(B=8, HQ=64, HKV=8, ctx=524288, fmt="int8", place="round_robin"),
    "quant-fp8": dict(B=8, HQ=64, HKV=8, ctx=524288, fmt="fp8", place="round_robin"),
    "long-bf16": dict(B=4, HQ=32, HKV=8, ctx=1048576, fmt="bf16", place="round_robin"),
}
EXTRA_WORKLOADS = ["long-bf16", "ragged-bf16", "quant-int8", "quant-fp8"]


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return PEAK_FALLBACK_GBS, "fallback"


def bytes_per_token(w):
    return 2 * w["HKV"] * D * 2 if w["fmt"] == "bf16" else 2 * w["HKV"] * D + 2 * w["HKV"] * 2


def workload_lengths(name, context):
    import numpy as np
    w = WORKLOADS[name]
    rng = np.random.default_rng(1234)
    if w["ctx"] is None:
        lens = rng.integers(4096, 262144 + 1, size=w["B"]).astype(np.int64)
        if context:
            lens = np.maximum(1, lens * context // 262144)
    else:
        lens = np.full(w["B"], context or w["ctx"], dtype=np.int64)
    return lens, rng


def workload_config(name, n, context=0):
    """The one description of a workload that both arms print."""
    w = WORKLOADS[name]
    lens, _ = workload_lengths(name, context)
    ctx_desc = "ragged U[4096, 262144]" if w["ctx"] is None else str(int(lens[0]))
    if w["ctx"] is None and context:
        ctx_desc += f" scaled by {context}/262144"
    return {"workload": f"{name}: batch {w['B']}, Hq {w['HQ']}, Hkv {w['HKV']}, head_dim {D}, context "
                        f"{ctx_desc}/seq, {w['fmt']} KV, {PAGE}-token pages, random-permutation block table",
            "batch": w["B"], "context": ctx_desc, "page_size": PAGE,
            "kv_bytes_per_layer": int(lens.sum()) * bytes_per_token(w),
            "sharding": f"{w['place']} pages over {n} GPU(s), q and merge on GPU 0",
            "l2_policy": "inputs larger than L2 (KV per GPU >= 1 GiB, read once per step)"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML (read only)."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            import torch
            uuid = str(torch.cuda.get_device_properties(index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.nv = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception as e:  # pragma: no cover
            self.nv = None
            self.err = repr(e)

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonGpuIdle", 0x1): "gpu_idle",
            getattr(nv, "nvmlClocksEventReasonApplicationsClocksSetting", 0x2): "applications_clocks_setting",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonSyncBoost", 0x10): "sync_boost",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake_slowdown",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, n in names.items():
                    if r & bit and n != "gpu_idle":
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.02)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self):
        self._stop.set()
        if self._thr is not None:
            self._thr.join()
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


# --------------------------------------------------------------------------- #
# reference arm / cpu baseline: the reference's own torch path on host cores
# --------------------------------------------------------------------------- #
def load_reference():
    """The reference's Python implementation of the path, when `make -C oracle` placed it
    under oracle/_ref (kind "reference"); else the oracle's restatement (kind "port").
    Returns (gather_seq, peer_parallel_attention, kind)."""
    ref_root = os.path.join(ROOT, "oracle", "_ref", "ref_py")
    if os.path.exists(os.path.join(ref_root, "umallm", "peer_parallel_attn.py")):
        if ref_root not in sys.path:
            sys.path.insert(0, ref_root)
        try:
            from umallm.peer_parallel_attn import peer_parallel_attention
            from umallm.peerkv.paged import gather_seq
            return gather_seq, peer_parallel_attention, "reference"
        except Exception:      # an incomplete copy: fall through to the port
            pass
    from oracle import peerkv_oracle as orc

    def gather_seq(local_cache, peer_cache, block_row, seq_len, peer_base):
        n_blk = (seq_len + PAGE - 1) // PAGE
        ids, val = orc.split_block_row(block_row[:n_blk].tolist(), seq_len, PAGE,
                                       [0] if peer_cache is None else [0, peer_base])
        Kl, Vl = orc.cat_blocks(local_cache, ids[0], val[0])
        if peer_cache is None or val[1] == 0:
            return Kl, Vl, None, None
        Kp, Vp = orc.cat_blocks(peer_cache, ids[1], val[1])
        return Kl, Vl, Kp, Vp
    return gather_seq, orc.peer_parallel_attention, "port"


def cpu_sample_inputs(name, tokens: int, n_shards: int, seed: int = 0):
    """One sequence of the workload at `tokens` tokens: paged pool(s) and a permuted block
    table.  With two or more shards the pages are split in the reference's own form: ids
    below peer_base in a local cache, the rest in a peer cache."""
    import torch
    w = WORKLOADS[name]
    g = torch.Generator().manual_seed(seed)
    n_pages = tokens // PAGE
    pool = torch.randn(2, n_pages, PAGE, w["HKV"], D, generator=g).bfloat16()
    bt = torch.randperm(n_pages, generator=g).to(torch.int32)
    q = torch.randn(1, w["HQ"], 1, D, generator=g).bfloat16()
    if n_shards > 1:
        base = n_pages // 2
        return q, pool[:, :base].contiguous(), pool[:, base:].contiguous(), bt, tokens, base
    return q, pool, None, bt, tokens, 1 << 62


def cpu_reference_step(fns, inputs):
    """The reference's path on CPU for one sequence: paged gather into contiguous shards
    (umallm/peerkv/paged.py gather_seq), one partial per shard with GQA expansion and
    fp32 math, then the merge fold (umallm/peer_parallel_attn.py peer_parallel_attention)."""
    gather_seq, ppa, _ = fns
    q, local, peer, bt, tokens, base = inputs
    Kl, Vl, Kp, Vp = gather_seq(local, peer, bt, tokens, base)
    shards = [(Kl.unsqueeze(0), Vl.unsqueeze(0))]
    if Kp is not None:
        shards.append((Kp.unsqueeze(0), Vp.unsqueeze(0)))
    return ppa(q, shards)


def run_reference(args):
    import torch
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    name = args.workload if args.workload in WORKLOADS else "paged-bf16"
    w = WORKLOADS[name]
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    fns = load_reference()
    tokens = 32768
    n_shards = 1 if args.gpus == 1 else 2
    inputs = cpu_sample_inputs(name, tokens, n_shards)
    for _ in range(args.warmup):
        cpu_reference_step(fns, inputs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_reference_step(fns, inputs)
    dt = (time.perf_counter() - t0) / args.steps
    gbs = tokens * 2 * w["HKV"] * D * 2 / dt / 1e9
    sample = (f"1 sequence x {tokens} tokens of the workload per step (bf16 pool), {n_shards} shard(s) in the "
              f"reference's local/peer form, paged gather + GQA expansion + fp32 math + merge; the rate is "
              f"extrapolated to the whole workload linearly in tokens")
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "extrapolated": True,
        "config": workload_config(name, args.gpus, args.context),
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": fns[2], "sample": sample,
                         "sample_tokens": tokens, "extrapolated": True},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- #
# workloads (synthetic stand-ins with the shapes, sizes and value distributions of the
# benchmark configurations; N(0,1) KV, seeded)
# --------------------------------------------------------------------------- #
def build_workload(name, context, N, rank, dev):
    """This rank's pool, local block table and shard lengths.  The global block table
    is the same seeded permutation on every rank; placement decides which pages are
    this rank's (round robin: page p -> GPU p mod N at index p div N, split on the device
    by the library; capacity spill: GPUs are filled in order up to a seeded fraction in
    [0.5, 1.0] of an equal share, the rest spills to the next GPU)."""
    import numpy as np
    import torch
    from peerkv_b200 import _lib, ops, placement
    w = WORKLOADS[name]
    B, HQ, HKV = w["B"], w["HQ"], w["HKV"]
    lens, rng = workload_lengths(name, context)
    n_pages = (lens + PAGE - 1) // PAGE
    total_pages = int(n_pages.sum())
    W = int(n_pages.max())
    perm = rng.permutation(total_pages).astype(np.int32)
    bt = np.zeros((B, W), dtype=np.int32)
    k = 0
    for i in range(B):
        bt[i, :n_pages[i]] = perm[k:k + n_pages[i]]
        k += int(n_pages[i])
    sl = lens.astype(np.int32)
    caps = None

    if w["place"] == "round_robin":
        btd, sld = torch.from_numpy(bt).to(dev), torch.from_numpy(sl).to(dev)
        tabs = [torch.zeros(B, W, dtype=torch.int32, device=dev) for _ in range(N)]
        lns = [torch.zeros(B, dtype=torch.int32, device=dev) for _ in range(N)]
        _lib.check(_lib.lib().pkv_split_block_table(
            dev.index, btd.data_ptr(), W, sld.data_ptr(), B, PAGE, N, 1, None,
            (C.c_void_p * N)(*[t.data_ptr() for t in tabs]), W,
            (C.c_void_p * N)(*[t.data_ptr() for t in lns]), ops._stream(dev)))
        torch.cuda.synchronize()
        my_tab, my_len = tabs[rank], lns[rank]
        n_local = (total_pages + N - 1) // N
        all_tokens = torch.stack(lns).cpu().numpy().astype(np.int64)          # [N, B]
    else:
        caps = np.random.default_rng(99).uniform(0.5, 1.0, size=N)
        tab, tok, used = placement.capacity_spill_split(n_pages, lens, PAGE, caps)
        my_tab = torch.from_numpy(tab[rank]).to(dev)
        my_len = torch.from_numpy(tok[rank].astype(np.int32)).to(dev)
        n_local = max(1, int(used[rank]))
        all_tokens = tok

    torch.manual_seed(100 + rank)
    fmt = w["fmt"]
    scales = None
    if fmt == "bf16":
        pool = torch.empty(2, n_local, PAGE, HKV, D, dtype=torch.bfloat16, device=dev)
        chunk = max(1, n_local // 8)
        for i in range(0, n_local, chunk):
            pool[:, i:i + chunk].normal_()
    else:
        code_dt = torch.int8 if fmt == "int8" else torch.float8_e4m3fn
        pool = torch.empty(2, n_local, PAGE, HKV, D, dtype=code_dt, device=dev)
        sc = torch.empty(2, n_local, PAGE, HKV, dtype=torch.float16, device=dev)
        chunk = max(1, n_local // 32)
        for i in range(0, n_local, chunk):                    # quantise N(0,1) bf16 with the library's quantiser
            x = torch.randn(2, min(chunk, n_local - i), PAGE, HKV, D, device=dev).bfloat16()
            c, s_ = ops.quantize_kv(x, fmt)
            pool[:, i:i + chunk] = c
            sc[:, i:i + chunk] = s_
        scales = (sc[0], sc[1])
    return dict(name=name, B=B, HQ=HQ, HKV=HKV, fmt=fmt, pool=pool, scales=scales, tab=my_tab, len=my_len,
                bytes_per_token=bytes_per_token(w), total_tokens=int(lens.sum()),
                rank_tokens=[int(x) for x in all_tokens.sum(1)], all_tokens=all_tokens,
                lens=lens, n_pages=n_pages, global_bt=bt, caps=caps,
                q_dtype=torch.bfloat16, dtype="bf16" if fmt == "bf16" else "f16",
                config=workload_config(name, N, context))


# --------------------------------------------------------------------------- #
# parity of the timed output against the CPU oracle, at the workload's full context
# --------------------------------------------------------------------------- #
def oracle_shard_partial(wl, q_cpu, seq, chunk_tokens):
    """CPU oracle partial (O fp32 [Hq, D], lse fp32 [Hq]) of this rank's shard for one
    sequence.  The shard's pages of the sequence are fetched from the GPU in chunks; each
    chunk is one call of the oracle's paged partial, and the chunks are merged with the
    oracle's N-way merge (exactly what the path itself does across shards)."""
    import torch
    from oracle import peerkv_oracle as orc
    L = int(wl["len"][seq])
    Hq = wl["HQ"]
    if L == 0:
        return torch.zeros(Hq, D), torch.full((Hq,), float("-inf"))
    n_blk = (L + PAGE - 1) // PAGE
    ids = wl["tab"][seq, :n_blk].long()
    pool, scales = wl["pool"], wl["scales"]
    Os, Ls = [], []
    per = max(1, chunk_tokens // PAGE)
    for c0 in range(0, n_blk, per):
        c1 = min(n_blk, c0 + per)
        idc = ids[c0:c1]
        toks = min(L, c1 * PAGE) - c0 * PAGE
        raw = pool.view(torch.uint8) if pool.dtype == torch.float8_e4m3fn else pool
        cache = raw.index_select(1, idc).cpu()
        ks = vs = None
        if scales is not None:
            ks, vs = scales[0].index_select(0, idc).cpu(), scales[1].index_select(0, idc).cpu()
        bt = torch.arange(c1 - c0, dtype=torch.int32).view(1, -1)
        o, l = orc.paged_partial_oracle(q_cpu[seq:seq + 1], cache, bt, torch.tensor([toks]), None, ks, vs)
        Os.append(o[0]); Ls.append(l[0])
    if len(Os) == 1:
        return Os[0], Ls[0]
    return orc.merge_n(Os, Ls)


def check_placement(wl, N, seqs):
    """The placement this run used against the oracle's definition of it."""
    import numpy as np
    from oracle import peerkv_oracle as orc
    if wl["caps"] is None:
        rows = [wl["global_bt"][s] for s in seqs]
        ref = orc.round_robin_shards(rows, [int(wl["lens"][s]) for s in seqs], PAGE, N)
        return all(np.array_equal(ref[g][1].numpy().astype(np.int64), wl["all_tokens"][g][seqs]) for g in range(N))
    # capacity spill over the whole batch (the oracle walks every page once)
    bt = [wl["global_bt"][i, :int(wl["n_pages"][i])] for i in range(wl["B"])]
    ref = orc.capacity_spill_shards(bt, [int(x) for x in wl["lens"]], PAGE, list(wl["caps"]))
    return all(np.array_equal(ref[g][1].numpy().astype(np.int64), wl["all_tokens"][g]) for g in range(N))


def parity_check(wl, q, out, N, rank, dev, n_seqs=2):
    """Every rank: oracle partial of its own shard for the sampled sequences; rank 0 merges
    the gathered partials with the oracle's merge and compares with the timed output at
    |diff| <= 2e-3 + 1e-2 |ref|."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from oracle import peerkv_oracle as orc
    lens = wl["lens"]
    seqs = sorted({int(np.argmax(lens)), int(np.argmin(lens))} if wl["caps"] is not None else {0, wl["B"] - 1})
    seqs = seqs[:n_seqs]
    cores = os.cpu_count() or 1
    torch.set_num_threads(max(1, cores // N))
    t0 = time.perf_counter()
    q_cpu = q.cpu()
    chunk = 65536 if wl["HQ"] <= 32 else 32768
    parts = [oracle_shard_partial(wl, q_cpu, s, chunk) for s in seqs]
    O = torch.stack([p[0] for p in parts]).to(dev)
    Lse = torch.stack([p[1] for p in parts]).to(dev)
    if N > 1:
        Og = [torch.empty_like(O) for _ in range(N)]
        Lg = [torch.empty_like(Lse) for _ in range(N)]
        dist.all_gather(Og, O)
        dist.all_gather(Lg, Lse)
    else:
        Og, Lg = [O], [Lse]
    res = None
    if rank == 0:
        ref, _ = orc.merge_n([o.cpu() for o in Og], [l.cpu() for l in Lg])
        got = out[seqs].float().cpu()
        diff = (got - ref).abs()
        ok = bool(torch.allclose(got, ref, atol=2e-3, rtol=1e-2))
        res = {"checked": True, "against": "CPU oracle, per-rank shard partials at full context merged on rank 0",
               "seqs": seqs, "seq_tokens": [int(lens[s]) for s in seqs], "tolerance": "abs 2e-3 + rel 1e-2",
               "max_abs_err": float(diff.max()), "max_abs_ref": float(ref.abs().max()),
               "placement_matches_oracle": bool(check_placement(wl, N, seqs)),
               "oracle_seconds": round(time.perf_counter() - t0, 2), "ok": ok}
        res["ok"] = bool(res["ok"] and res["placement_matches_oracle"])
    return res


# --------------------------------------------------------------------------- #
# full decode step (BASELINE configuration 5): random-init Llama-3-8B architecture,
# attention over the sharded KV, everything else on GPU 0
# --------------------------------------------------------------------------- #
def run_llama_step(args):
    import torch
    import torch.distributed as dist
    from peerkv_b200.decoder import DecodeStep, LlamaGeometry, ModelWeights, ShardedKVLayer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    N = args.gpus
    if world != N:
        raise SystemExit(f"--gpus {N} but WORLD_SIZE={world}")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if N > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    t_setup = time.perf_counter()

    def note(msg):
        if rank == 0:
            print(f"[llama-step +{time.perf_counter() - t_setup:6.1f}s] {msg}", file=sys.stderr, flush=True)

    HKV = WORKLOADS["long-bf16"]["HKV"]
    g = LlamaGeometry(n_layers=args.layers)
    ctx = args.context or 1048576
    wl = build_workload("long-bf16", ctx, N, rank, dev)
    note("placement and layer 0's KV built")
    B, HQ = wl["B"], wl["HQ"]
    base, tab, lens = wl["pool"], wl["tab"], wl["len"]
    append = None
    if rank == 0:
        # the new token of every sequence goes to one more page that GPU 0 owns
        n0 = base.shape[1]
        base = torch.cat([base, torch.zeros(2, B, PAGE, HKV, D, dtype=base.dtype, device=dev)], dim=1)
        used = (lens.to(torch.int64) + PAGE - 1) // PAGE
        tab = torch.cat([tab, torch.zeros(B, 1, dtype=torch.int32, device=dev)], dim=1)
        tab[torch.arange(B, device=dev), used] = torch.arange(n0, n0 + B, device=dev, dtype=torch.int32)
        full = (lens % PAGE) == 0
        assert bool(full.all()), "the bench context puts whole pages on every GPU"
        lens = lens + 1
        append = (torch.arange(n0, n0 + B, device=dev), torch.zeros(B, dtype=torch.int64, device=dev))
    wl["pool"] = None
    # every layer has its own KV of the same shape; the values of layers 1.. are copies of
    # layer 0's N(0,1) pool (the step's time does not depend on them)
    layers = []
    for li in range(g.n_layers):
        pool = base if li == 0 else torch.empty_like(base).copy_(base)
        layers.append(ShardedKVLayer(pool, tab, lens))
    note(f"{g.n_layers} layers of KV resident ({base.numel() * 2 * g.n_layers / 2**30:.1f} GiB on this GPU)")
    grp = None
    if N > 1:
        from peerkv_b200.distributed import DistPeerGroup
        grp = DistPeerGroup(dev, B, HQ, home=0)
    weights = ModelWeights(g, dev) if rank == 0 else None
    note("weights built")
    step = DecodeStep(g, weights, layers, B, dev, group=grp, append_slots=append)
    tokens = torch.randint(0, g.vocab, (B,), device=dev)
    positions = torch.full((B,), ctx, device=dev, dtype=torch.int64)

    def one_token():
        step.step(tokens, positions)

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if N > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if N > 1:
            dist.barrier()
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms / n

    warm = max(args.warmup, 3)
    for _ in range(2):
        one_token()
    eager_logits = step.logits.float().clone() if rank == 0 else None
    eager = timed(one_token, max(2, args.steps // 4))
    note(f"eager step {eager:.3f} ms")
    if not args.no_graphs:
        step.capture()
        note("whole step captured as one graph per GPU")
    for _ in range(warm):
        one_token()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    tpot = timed(one_token, args.steps)
    attn = timed(step.attention_only, args.steps)
    clocks = sampler.stop() if sampler else None
    status = step.shard.status() | (grp.xchg.status() if grp else 0)
    if rank == 0:
        logit_diff = float((step.logits.float() - eager_logits).abs().max())
        peak, kind = measured_peak()
        kv_bytes = wl["total_tokens"] * wl["bytes_per_token"] * g.n_layers
        w_bytes = weights.bytes() - weights.embed.numel() * 2          # the embedding is gathered, not read
        floor_ms = (kv_bytes / N + w_bytes) / (peak * 1e9) * 1e3
        rest = tpot - attn
        print(json.dumps({
            "metric": "tpot_ms", "value": tpot, "unit": "ms", "n_gpus": N, "steps": args.steps,
            "warmup": warm, "ms_per_step": tpot, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"llama-step: random-init Llama-3-8B architecture ({g.n_layers} layers, hidden "
                                   f"{g.hidden}, {g.n_q_heads}/{g.n_kv_heads} heads, FFN {g.ffn}, vocab {g.vocab}), "
                                   f"batch {B}, {ctx}-token KV per sequence, pages round-robin over {N} GPU(s), "
                                   "attention on the sharded path, the rest on GPU 0 (library GEMMs + this library's "
                                   "rmsnorm / rope+append / swiglu kernels)"
                                   + ("" if args.no_graphs else ", the whole step one CUDA graph per GPU"),
                       "kv_bytes_per_token_step": kv_bytes, "weight_bytes": weights.bytes()},
            "attention_ms_per_token": attn, "attention_us_per_layer": attn / g.n_layers * 1e3,
            "rest_ms_per_token": rest, "rest_floor_ms": w_bytes / (peak * 1e9) * 1e3,
            "rest_over_floor": rest / (w_bytes / (peak * 1e9) * 1e3),
            "eager_ms_per_token": eager,
            "hbm_floor_ms": floor_ms, "tpot_over_floor": tpot / floor_ms, "peak_kind": kind,
            "graph_vs_eager_max_abs_logit_diff": logit_diff,
            "gpu_launches": args.steps * g.n_layers * (N + 3),
            "clocks": clocks, "device_status": status}), flush=True)
    if grp:
        grp.close()
        dist.destroy_process_group()


# --------------------------------------------------------------------------- #
# single-layer configuration (BASELINE configuration 1): the one shape the reference's
# own CUDA prototype supports, so its kernels (built for sm_100a into oracle/_ref) are
# timed beside ours
# --------------------------------------------------------------------------- #
def run_single_layer(args):
    import torch
    import torch.distributed as dist
    from peerkv_b200 import _lib, ops
    from oracle import peerkv_oracle as orc

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    N = args.gpus
    if world != N:
        raise SystemExit(f"--gpus {N} but WORLD_SIZE={world}")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if N > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    Bq, H, HK, T = 1, 32, 8, args.context or 16384
    BYTES_PER_TOKEN = 2 * HK * D * 2
    n_sh = max(2, N)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(Bq, H, 1, D, generator=g).half()
    K = torch.randn(Bq, HK, T, D, generator=g).half()
    V = torch.randn(Bq, HK, T, D, generator=g).half()
    cuts = [T // n_sh] * n_sh
    cuts[-1] += T - sum(cuts)
    Ks, Vs = K.split(cuts, 2), V.split(cuts, 2)
    scale = 1.0 / math.sqrt(D)
    L = _lib.lib()
    st = ops._stream(dev)
    qd = q.view(Bq, H, D).to(dev)
    out = torch.empty(Bq, H, D, dtype=torch.float16, device=dev)
    if N == 1:
        shard = ops.Shard(dev, Bq, H)
        Kd = [k.contiguous().to(dev) for k in Ks]
        Vd = [v.contiguous().to(dev) for v in Vs]
        lens = [torch.full((Bq,), k.shape[2], dtype=torch.int32, device=dev) for k in Kd]
        views = [ops.contiguous_view(k, v) for k, v in zip(Kd, Vd)]
        a = [ops.make_args(qd, vw, None, 1, ln, scale) for vw, ln in zip(views, lens)]
        po = torch.empty(n_sh, Bq, H, D, dtype=torch.float32, device=dev)
        pl = torch.empty(n_sh, Bq, H, dtype=torch.float32, device=dev)

        def step():
            for i in range(n_sh):
                _lib.check(L.pkv_decode_partial(shard._h, C.byref(a[i]), po[i].data_ptr(), pl[i].data_ptr(), st))
            _lib.check(L.pkv_merge_partials(dev.index, po.data_ptr(), Bq * H * D, pl.data_ptr(), Bq * H, n_sh,
                                            Bq * H, D, out.data_ptr(), _lib.PKV_F16, None, st))
        launches = n_sh + 1
        grp = None
    else:
        from peerkv_b200.distributed import DistPeerGroup
        grp = DistPeerGroup(dev, Bq, H, home=0)
        shard = grp.shard
        Kd, Vd = Ks[rank].contiguous().to(dev), Vs[rank].contiguous().to(dev)
        ln = torch.full((Bq,), Kd.shape[2], dtype=torch.int32, device=dev)
        a1 = ops.make_args(qd, ops.contiguous_view(Kd, Vd), None, 1, ln, scale)

        def step():
            grp.step(a1, q=qd, out=out)
        launches = N + 1

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if N > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if N > 1:
            dist.barrier()
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t)
        return ms / n

    # the 64 MiB of this configuration fit the 126 MB L2: flush it between timed steps
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def step_flushed():
        flush.zero_()
        step()

    for _ in range(max(args.warmup, 3)):
        step()
    ms_hot = timed(step, args.steps)
    ms_flush_only = timed(flush.zero_, args.steps)
    ms_cold = timed(step_flushed, args.steps) - ms_flush_only
    status = shard.status() | (grp.xchg.status() if grp else 0)
    if rank == 0:
        dense = orc.dense_attention_fp32(q, K, V).view(Bq, H, D)
        err = float((out.float().cpu() - dense).abs().max())
        ref_fold = orc.peer_parallel_attention(q, list(zip(Ks, Vs))).view(Bq, H, D).float()
        line = {"metric": "decode_attn_effective_kv_bandwidth", "unit": "GB/s", "n_gpus": N,
                "steps": args.steps, "warmup": max(args.warmup, 3), "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                "config": {"workload": f"single-fp16: batch 1, Hq 32, Hkv 8, head_dim 128, context {T}, fp16, "
                                       f"contiguous KV in {n_sh} equal shards, partial per shard + LSE merge",
                           "kv_bytes_per_layer": T * BYTES_PER_TOKEN,
                           "l2_policy": "64 MiB of KV fit L2: reported cold (192 MB written between steps, its "
                                        "time subtracted) and hot"},
                "value": T * BYTES_PER_TOKEN / (ms_cold * 1e-3) / 1e9, "ms_per_step": ms_cold,
                "us_per_layer": ms_cold * 1e3, "us_per_layer_l2_hot": ms_hot * 1e3,
                "max_abs_err_vs_unsplit_fp32": err,
                "max_abs_err_vs_reference_fold": float((out.float().cpu() - ref_fold).abs().max()),
                "gpu_launches": launches * args.steps, "device_status": status}
        ref_so = os.path.join(ROOT, "oracle", "_ref", "libref_attn.so")
        if N == 1 and os.path.exists(ref_so):
            R = C.CDLL(ref_so)
            R.ref_attn_two_shards.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p,
                                              C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p,
                                              C.c_void_p]
            half = T // 2
            K0 = K[0, :, :half].contiguous().to(dev); V0 = V[0, :, :half].contiguous().to(dev)
            K1 = K[0, :, half:].contiguous().to(dev); V1 = V[0, :, half:].contiguous().to(dev)
            q2 = q.view(H, D).to(dev)
            ro = torch.empty(H, D, dtype=torch.float16, device=dev)

            def ref_step():
                rc = R.ref_attn_two_shards(q2.data_ptr(), K0.data_ptr(), V0.data_ptr(), half, K1.data_ptr(),
                                           V1.data_ptr(), T - half, H, HK, D, 16, scale, ro.data_ptr(), st)
                assert rc == 0

            def ref_flushed():
                flush.zero_()
                ref_step()
            for _ in range(3):
                ref_step()
            r_hot = timed(ref_step, args.steps)
            r_cold = timed(ref_flushed, args.steps) - ms_flush_only
            line["reference_cuda_kernels"] = {
                "what": "the reference's attn_split_gqa / attn_combine / merge2_h (S = 16), built for sm_100a "
                        "from its own source, same inputs, both shards on this GPU",
                "us_per_layer": r_cold * 1e3, "us_per_layer_l2_hot": r_hot * 1e3,
                "max_abs_err_vs_unsplit_fp32": float((ro.float().cpu() - dense.view(H, D)).abs().max()),
                "speedup_ours": r_cold / ms_cold}
        print(json.dumps(line), flush=True)
    if grp:
        grp.close()
        dist.destroy_process_group()


# --------------------------------------------------------------------------- #
# our arm
# --------------------------------------------------------------------------- #
def measure_workload(name, args, N, rank, local_rank, dev, steps, headline):
    """Builds one workload on this rank, times `steps` steps (CUDA events between barriers,
    max over ranks), times the shard kernel alone on every rank, checks the timed output
    against the CPU oracle and, for the headline, measures the end-to-end step with host
    buffers.  Returns the result dict on rank 0 (None elsewhere)."""
    import torch
    import torch.distributed as dist
    from peerkv_b200 import _lib, ops

    wl = build_workload(name, args.context, N, rank, dev)
    B, HQ = wl["B"], wl["HQ"]
    pool, my_tab, my_len = wl["pool"], wl["tab"], wl["len"]
    local_tokens = int(my_len.sum())
    bpt = wl["bytes_per_token"]
    qdt = wl["q_dtype"]

    torch.manual_seed(7)
    # One pinned staging buffer per rank holds everything a decode step can change -- the
    # query (home rank), every sequence's shard length and one page id per sequence -- and
    # one device buffer mirrors it: q, the lengths and the new page ids are views of it, so
    # the end-to-end step is ONE host-to-device copy per rank.
    q_bytes = B * HQ * D * 2
    stage_host = torch.zeros(q_bytes + 8 * B, dtype=torch.uint8).pin_memory()
    stage_dev = torch.zeros(q_bytes + 8 * B, dtype=torch.uint8, device=dev)
    q_host = stage_host[:q_bytes].view(qdt).view(B, HQ, D)
    q_host.copy_(torch.randn(B, HQ, D).to(qdt))
    q = stage_dev[:q_bytes].view(qdt).view(B, HQ, D)
    len_dev = stage_dev[q_bytes:q_bytes + 4 * B].view(torch.int32)
    new_page_dev = stage_dev[q_bytes + 4 * B:].view(torch.int32)
    stage_host[q_bytes:q_bytes + 4 * B].view(torch.int32).copy_(my_len.cpu())
    # the page a decode step may have to add per sequence: the last one of each row
    used = ((my_len.to(torch.int64) + PAGE - 1) // PAGE - 1).clamp_(min=0)
    stage_host[q_bytes + 4 * B:].view(torch.int32).copy_(my_tab.gather(1, used.view(-1, 1)).view(-1).cpu())
    stage_dev.copy_(stage_host)
    my_len = len_dev                       # the kernels read the lengths where the copy lands
    out = torch.zeros(B, HQ, D, dtype=qdt, device=dev)
    out_host = torch.empty(B, HQ, D, dtype=qdt).pin_memory()
    rows = torch.arange(B, device=dev)
    scale = 1.0 / math.sqrt(D)
    view = ops.paged_view(pool[0], pool[1], *(wl["scales"] or (None, None)))
    out_code = ops._DT[qdt]
    L = _lib.lib()
    st = ops._stream(dev)
    a = ops.make_args(q, view, my_tab, my_tab.stride(0), my_len, scale)

    if N == 1:
        shard = ops.Shard(dev, B, HQ)
        grp = None

        def step():
            _lib.check(L.pkv_decode(shard._h, C.byref(a), out.data_ptr(), out_code, None, st))
    else:
        from peerkv_b200.distributed import DistPeerGroup
        grp = DistPeerGroup(dev, B, HQ, home=0)
        shard = grp.shard
        _GROUP["grp"] = grp

        def step():
            grp.step(a, q=q, out=out)
    launches_per_step = N          # one kernel per GPU per step (the home kernel also publishes q and merges)

    def barrier():
        if N > 1:
            dist.barrier()
        torch.cuda.synchronize()

    rank_ms = []

    def timed(fn, n):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        barrier()
        ms = e0.elapsed_time(e1)
        if N > 1:
            t = torch.tensor([ms], device=dev)
            allt = [torch.zeros_like(t) for _ in range(N)]
            dist.all_gather(allt, t)
            rank_ms[:] = [float(x) / n for x in allt]
            ms = max(float(x) for x in allt)
        return ms

    warm = max(args.warmup, 3)
    sampler = ClockSampler(local_rank) if (rank == 0 and headline) else None
    for _ in range(warm):
        step()
    barrier()
    if sampler:
        sampler.start()
    total_ms = timed(step, steps)
    ms_per_step = total_ms / steps
    step_rank_ms = list(rank_ms)
    # keep the GPU under the same load long enough for the clock sampler to see it
    soak_steps = 0
    if headline and total_ms < 1500.0 and not args.lean:
        soak_steps = int(min(20000, (1500.0 - total_ms) / max(ms_per_step, 1e-3))) + 1
        timed(step, soak_steps)
    clocks = sampler.stop() if sampler else None
    status = shard.status() | (grp.xchg.status() if grp else 0)

    algo_bytes = wl["total_tokens"] * bpt
    value = algo_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- optional: where the microseconds of a step go (device time stamps) ----------- #
    timeline = None
    if args.timeline:
        timeline = step_timeline(L, shard, step, barrier, dev, N, rank)

    # ---- parity: the output of the last timed step against the CPU oracle ------------ #
    parity = None
    if not args.lean:
        parity = parity_check(wl, q, out, N, rank, dev)

    # ---- end to end: host buffers in, host result out, every step ------------------- #
    e2e = None
    if headline:
        def e2e_step():
            # what a decode step changes: the query, every sequence's length on the GPU that
            # took the new token, and at most one new page id per sequence
            if rank == 0:
                stage_dev.copy_(stage_host, non_blocking=True)
            else:
                stage_dev[q_bytes:].copy_(stage_host[q_bytes:], non_blocking=True)
            my_tab[rows, used] = new_page_dev
            step()
            if rank == 0:
                out_host.copy_(out, non_blocking=True)
                torch.cuda.current_stream().synchronize()
        for _ in range(3):
            e2e_step()
        e2e_n = 3 if args.lean else max(5, min(steps, 100))
        e2e_ms = timed(e2e_step, e2e_n) / e2e_n
        h2d = q_bytes + N * 8 * B
        e2e = {"value": algo_bytes / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": out_host.numel() * 2,
               "note": "per step, one copy per GPU from pinned host memory: q (GPU 0 only), the shard lengths "
                       "and one page id per sequence (what a decode step can change; the block tables stay "
                       "resident and take the page ids by a scatter); the result is copied back to the host "
                       "and GPU 0's stream synchronised"}

    # ---- the shard kernel alone on every rank, CUDA events around each launch -------- #
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
           for _ in range(2 if args.lean else 20)]
    for _ in range(3):
        _lib.check(L.pkv_decode_splits_only(shard._h, C.byref(a), st))
    for e0, e1 in evs:
        e0.record()
        _lib.check(L.pkv_decode_splits_only(shard._h, C.byref(a), st))
        e1.record()
    torch.cuda.synchronize()
    kern_ms = sum(e0.elapsed_time(e1) for e0, e1 in evs) / len(evs)
    kern_all = [kern_ms]
    if N > 1:
        t = torch.tensor([kern_ms], device=dev)
        allt = [torch.zeros_like(t) for _ in range(N)]
        dist.all_gather(allt, t)
        kern_all = [float(x) for x in allt]
    barrier()
    if grp:
        grp.close()
    shard.close() if N == 1 else None
    del pool, view, a
    wl["pool"] = wl["scales"] = None
    torch.cuda.empty_cache()

    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    kern_bytes = local_tokens * bpt
    achieved = kern_bytes / (kern_ms * 1e-3) / 1e9
    slowest = max(range(N), key=lambda r: kern_all[r])
    res = {
        "value": value, "unit": "GB/s", "steps": steps, "warmup": warm, "ms_per_step": ms_per_step,
        "us_per_layer": ms_per_step * 1e3, "dtype": wl["dtype"],
        "config": dict(wl["config"], max_rank_kv_bytes=max(wl["rank_tokens"]) * bpt),
        "frac_of_aggregate_hbm": value / (peak * N), "frac_of_8tbs_nominal": value / (8000.0 * N),
        "roofline": {"kernel": "decode_partial_kernel", "bound": "hbm", "achieved": achieved, "peak": peak,
                     "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                     "bytes_per_launch": kern_bytes, "us_per_launch": kern_ms * 1e3,
                     "traffic": NCU_TRAFFIC_PER_ALGO_BYTE[wl["fmt"]] * kern_bytes},
        "exchange": {"slowest_shard_kernel_us": kern_all[slowest] * 1e3, "slowest_rank": slowest,
                     "step_minus_kernel_us": (ms_per_step - kern_all[slowest]) * 1e3,
                     "frac_of_step": (ms_per_step - kern_all[slowest]) / ms_per_step,
                     "what": "step time minus the slowest rank's shard kernel timed alone: split-K combine, "
                             "q publish, partial return, final merge and the launch gap"},
        "parity": parity,
        "gpu_launches": launches_per_step * steps,
        "device_status": status,
        "rank_ms_per_step": step_rank_ms, "rank_kv_bytes": [t * bpt for t in wl["rank_tokens"]],
    }
    if e2e:
        res["e2e"] = e2e
    if timeline:
        res["timeline"] = timeline
    if clocks is not None:
        res["clocks"] = dict(clocks, note=f"sampled over the timed steps plus {soak_steps} more identical steps")
    return res


_GROUP = {}


def hop_latency(L, shard, dev, N, rank, iters=2000):
    """One-way latency between GPU 0 and GPU 1 of a bare flag, of a payload + system fence +
    flag (what a partial return is) and of a payload of {payload, epoch} words with nothing
    behind it (what the query publish is), measured by the library's probe kernels."""
    import torch
    import torch.distributed as dist
    from peerkv_b200 import _lib, ops
    xchg = _GROUP["grp"].xchg
    out = torch.zeros(2, dtype=torch.int64, device=dev)
    res = {}
    for name, payload, ll in (("flag_only", 0, 0), ("payload_4096B_fence_flag", 4096, 0),
                              ("payload_4096B_self_validating_words", 4096, 2)):
        if rank < 2:
            _lib.check(L.pkv_exchange_hop_probe_reset(xchg._h, ops._stream(dev)))
        torch.cuda.synchronize()
        dist.barrier()
        if rank < 2:
            _lib.check(L.pkv_exchange_hop_probe(xchg._h, 1 - rank, rank | ll, iters, payload, out.data_ptr(),
                                                ops._stream(dev)))
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            ns, bad = int(out[0]), int(out[1])
            res[name] = None if bad else ns / (2.0 * iters) / 1e3
    return res if rank == 0 else None


def step_timeline(L, shard, step, barrier, dev, N, rank, reps=5):
    """%globaltimer stamps of one step in steady state (three untraced steps are queued in
    front of the traced one, no host synchronisation in between), per rank, in microseconds
    after that rank's first CTA started.  Median over `reps` traced steps."""
    import torch
    import torch.distributed as dist
    from peerkv_b200 import _lib
    tr = torch.zeros(1024 * 8, dtype=torch.int64, device=dev)
    names = ["cta_start_spread", "q_published_or_first_q_seen", "last_tile_consumed", "last_local_combine",
             "last_peer_tag_seen", "last_row_written"]
    rows = []
    for _ in range(reps):
        barrier()
        for _ in range(3):
            step()
        _lib.check(L.pkv_shard_trace(shard._h, tr.data_ptr()))
        tr.zero_()
        step()
        torch.cuda.synchronize()
        _lib.check(L.pkv_shard_trace(shard._h, None))
        t = tr.view(-1, 8).cpu()
        t = t[t[:, 0] > 0]
        t0 = int(t[:, 0].min())
        row = [float(int(t[:, 0].max()) - t0) / 1e3]
        for w in range(1, 6):
            col = t[:, w][t[:, w] > 0]
            row.append(float(int(col.max()) - t0) / 1e3 if col.numel() else None)
        rows.append(row + [t0])
    med = []
    for w in range(6):
        vals = sorted(r[w] for r in rows if r[w] is not None)
        med.append(vals[len(vals) // 2] if vals else None)
    mine = dict(zip(names, med), rank=rank, first_cta_start_ns=rows[-1][6])
    if N > 1:
        allr = [None] * N
        dist.all_gather_object(allr, mine)
    else:
        allr = [mine]
    hops = hop_latency(L, shard, dev, N, rank) if N > 1 else None
    if rank != 0:
        return None
    base = allr[0]["first_cta_start_ns"]
    for r in allr:      # the GPUs' timers are separate clocks: only a rough cross-rank offset
        r["first_cta_start_vs_rank0_us"] = (r.pop("first_cta_start_ns") - base) / 1e3
    return {"unit": "us after the rank's first CTA start; rank 0 is the home GPU", "ranks": allr,
            "fabric_one_way_us": hops}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--workload", default="paged-bf16",
                    choices=list(WORKLOADS) + ["llama-step", "single-fp16"],
                    help="paged-bf16 is the headline configuration; the others are the remaining "
                         "benchmark configurations' attention shapes")
    ap.add_argument("--context", type=int, default=0, help="tokens per sequence, 0 = the workload's own")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the `workloads` block (the other shapes)")
    ap.add_argument("--timeline", action="store_true",
                    help="add per-rank device time stamps of one steady-state step to the line")
    ap.add_argument("--lean", action="store_true", help="timed steps only (for runs under a profiler)")
    ap.add_argument("--layers", type=int, default=32, help="llama-step only")
    ap.add_argument("--no-graphs", action="store_true", help="llama-step only: eager launches instead of one graph")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.workload == "llama-step":
        return run_llama_step(args)
    if args.workload == "single-fp16":
        return run_single_layer(args)

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    N = args.gpus
    if world != N:
        raise SystemExit(f"--gpus {N} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {N}")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if N > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)

    head = measure_workload(args.workload, args, N, rank, local_rank, dev, args.steps, headline=True)
    extras = {}
    if args.workload == "paged-bf16" and not args.no_extra and not args.lean and not args.context:
        for name in EXTRA_WORKLOADS:
            r = measure_workload(name, args, N, rank, local_rank, dev, min(args.steps, 20), headline=False)
            if r is not None:
                extras[name] = {k: r[k] for k in ("us_per_layer", "value", "unit", "steps", "dtype",
                                                  "frac_of_aggregate_hbm", "frac_of_8tbs_nominal", "exchange",
                                                  "parity", "device_status")}
                extras[name]["kernel_frac_of_peak"] = r["roofline"]["frac"]
                extras[name]["kv_bytes_per_layer"] = r["config"]["kv_bytes_per_layer"]
                extras[name]["max_rank_kv_bytes"] = r["config"]["max_rank_kv_bytes"]

    ok = True
    if rank == 0:
        line = {"metric": METRIC, "value": head["value"], "unit": "GB/s", "n_gpus": N, "steps": args.steps,
                "warmup": head["warmup"], "ms_per_step": head["ms_per_step"], "us_per_layer": head["us_per_layer"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": head["dtype"],
                "data": "synthetic", "config": workload_config(args.workload, N, args.context)}
        for k in ("frac_of_aggregate_hbm", "frac_of_8tbs_nominal", "roofline", "e2e", "exchange", "parity", "timeline",
                  "gpu_launches", "clocks", "device_status", "rank_ms_per_step", "rank_kv_bytes"):
            if k in head:
                line[k] = head[k]
        line["max_rank_kv_bytes"] = head["config"]["max_rank_kv_bytes"]
        if extras:
            line["workloads"] = extras
        checks = [head["parity"]] + [e["parity"] for e in extras.values()]
        ok = all(c is None or c["ok"] for c in checks) and not head["device_status"] and \
            not any(e["device_status"] for e in extras.values())
        if N == 1 and not args.no_cpu_baseline and not args.lean and args.workload == "paged-bf16":
            cores = os.cpu_count() or 1
            torch.set_num_threads(cores)
            fns = load_reference()
            tokens = 131072
            inputs = cpu_sample_inputs("paged-bf16", tokens, 1)
            cpu_reference_step(fns, inputs)
            ts = []
            for _ in range(5):
                t0 = time.perf_counter()
                cpu_reference_step(fns, inputs)
                ts.append(time.perf_counter() - t0)
            med = sorted(ts)[len(ts) // 2]
            w = WORKLOADS["paged-bf16"]
            line["cpu_baseline"] = {
                "value": tokens * bytes_per_token(w) / med / 1e9, "unit": "GB/s", "cores": cores, "kind": fns[2],
                "sample": f"1 of the 16 sequences ({tokens} tokens, 512 MiB of KV): the reference's paged gather + "
                          f"GQA expansion + fp32 attention, median of 5 after 1 warm-up; a rate, extrapolated "
                          f"to the workload linearly in tokens",
                "sample_tokens": tokens, "extrapolated": True}
        print(json.dumps(line), flush=True)
    if N > 1:
        flag = torch.tensor([1 if ok else 0], device=dev)
        dist.broadcast(flag, 0)
        ok = bool(flag.item())
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("parity or device status failed: see the JSON line")


if __name__ == "__main__":
    main()
