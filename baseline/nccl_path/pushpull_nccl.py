#!/usr/bin/env python
"""Baseline (b): full-table push + pull done with library collectives only - NCCL reduce_scatter of the
workers' updates, an elementwise momentum-SGD apply on the owned shard (torch ops), NCCL all_gather of
the new rows.  Run under torchrun; prints GB/s per GPU (table bytes / clock time, max over ranks)."""
import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=float, nargs="+", default=[1, 16, 64, 256, 1024])
    ap.add_argument("--clocks", type=int, default=10)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    for mb in a.mb:
        n = int(mb * 1024 * 1024 / 4) // (128 * world) * (128 * world)
        upd = torch.randn(n, device=dev) * 0.01
        table = torch.zeros(n, device=dev)
        shard = torch.zeros(n // world, device=dev)
        master = torch.zeros(n // world, device=dev)
        mom = torch.zeros(n // world, device=dev)

        def clock():
            dist.reduce_scatter_tensor(shard, upd)
            mom.mul_(0.9).add_(shard, alpha=0.01)
            master.sub_(mom)
            dist.all_gather_into_tensor(table, master)

        for _ in range(3):
            clock()
        torch.cuda.synchronize(); dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.clocks):
            clock()
        e1.record(); e1.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.clocks], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            print(json.dumps({"baseline": "nccl_reduce_scatter_apply_all_gather", "world": world, "table_mb": n * 4 / 2**20,
                              "ms_per_clock": t.item(), "gb_s_per_gpu": n * 4 / t.item() / 1e6}), flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
