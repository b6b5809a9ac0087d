"""Worker of the multi-process tests (launched with torch.distributed.run).

--backend nccl : every rank owns one GPU; rank 0 is the home rank.  Runs a few decode
                 steps through DistPeerGroup (C-ABI kernels, P2P mailboxes) and rank 0
                 checks the result against the CPU oracle.
--backend gloo : no GPU.  Every rank computes its shard's partial with the CPU oracle,
                 the partials are gathered to rank 0 and merged there: the same
                 placement, protocol and merge semantics as the GPU path, host side only.
"""
import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch
import torch.distributed as dist

from oracle import peerkv_oracle as orc


def make_case(world):
    bs, Hq, Hkv, D = 16, 32, 8, 128
    lens = [2000, 33, 0, 1024, 517]
    B = len(lens)
    g = torch.Generator().manual_seed(11)
    n_pages = [(L + bs - 1) // bs for L in lens]
    total = sum(n_pages)
    total_pad = (total + world - 1) // world * world
    pool = torch.randn(2, total_pad, bs, Hkv, D, generator=g).bfloat16()
    perm = torch.randperm(total, generator=g)
    bt = torch.zeros(B, max(n_pages), dtype=torch.int32)
    k = 0
    for i, m in enumerate(n_pages):
        bt[i, :m] = perm[k:k + m].to(torch.int32)
        k += m
    sl = torch.tensor(lens, dtype=torch.int32)
    q = torch.randn(B, Hq, D, generator=g).bfloat16()
    return dict(bs=bs, Hq=Hq, Hkv=Hkv, D=D, B=B, pool=pool, bt=bt, sl=sl, q=q)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="gloo")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    c = make_case(world)
    shards = orc.round_robin_shards(c["bt"].numpy(), c["sl"].numpy(), c["bs"], world)
    my_tab, my_len = shards[rank]
    my_pool = c["pool"][:, rank::world].contiguous()
    ref, _ = orc.paged_partial_oracle(c["q"], c["pool"], c["bt"], c["sl"])

    if args.backend == "gloo":
        dist.init_process_group("gloo")
        o, lse = orc.paged_partial_oracle(c["q"], my_pool, my_tab, my_len)
        os_, ls_ = [torch.empty_like(o) for _ in range(world)], [torch.empty_like(lse) for _ in range(world)]
        dist.gather(o, os_ if rank == 0 else None, dst=0)
        dist.gather(lse, ls_ if rank == 0 else None, dst=0)
        if rank == 0:
            out, _ = orc.merge_n(os_, ls_)
            assert torch.allclose(out, ref, atol=1e-5, rtol=1e-4)
            print("DIST_OK gloo world", world, flush=True)
        dist.barrier()
        dist.destroy_process_group()
        return

    import math
    local_rank = int(os.environ.get("LOCAL_RANK", rank))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    from peerkv_b200 import ops
    from peerkv_b200.distributed import DistPeerGroup
    grp = DistPeerGroup(dev, c["B"], c["Hq"], home=0)
    pool_d = my_pool.to(dev)
    tab_d, len_d = my_tab.to(dev), my_len.to(dev)
    q_d = c["q"].to(dev)
    out = torch.zeros(c["B"], c["Hq"], c["D"], dtype=torch.bfloat16, device=dev)
    a = ops.make_args(q_d, ops.paged_view(pool_d[0], pool_d[1]), tab_d, tab_d.stride(0), len_d,
                      1.0 / math.sqrt(c["D"]))
    for step in range(4):
        if rank == 0:
            q_d.copy_((c["q"].float() * (1 + step)).bfloat16())     # a new q every step
        grp.step(a, q=q_d, out=out)
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            qs = (c["q"].float() * (1 + step)).bfloat16()
            want, _ = orc.paged_partial_oracle(qs, c["pool"], c["bt"], c["sl"])
            assert torch.allclose(out.float().cpu(), want, atol=2e-3, rtol=1e-2), f"step {step} differs"
    st = grp.status()
    assert st == 0, f"device status {st:#x}"
    grp.close()
    if rank == 0:
        print("DIST_OK nccl world", world, flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
