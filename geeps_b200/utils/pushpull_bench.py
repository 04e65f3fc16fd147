"""Parameter-server push/pull sweep: python -m geeps_b200.utils.pushpull_bench (under torchrun for N > 1)

One table of rows of 128 floats, total size swept from 1 MB to 1 GB, row ids partitioned round-robin over
the shards, update values ~N(0, 0.01).  Every clock each worker pushes a full-table update and pulls the
full table (Read all rows, PreUpdate / Update all rows, Clock) at SSP slack 0 / 1 / 4.  Reports GB/s per
GPU = table bytes / time per clock (device-timed, max over ranks) and, for N > 1, the fraction of the
NVLink roofline: (N-1)/N of the table crosses the link once per direction in each of push and pull,
at 770 GB/s measured per direction (900 nominal)."""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..parallel.ps import GeePs
from ..utils.config import (DEVICE_CUDA, PARTITION_ROUND_ROBIN, TABLE_SGD_MOMENTUM, TRANSPORT_NVLINK, TRANSPORT_TCP,
                            GeePsConfig)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mb", type=float, nargs="+", default=[1, 16, 64, 256, 1024])
    ap.add_argument("--slack", type=int, nargs="+", default=[0, 1, 4])
    ap.add_argument("--clocks", type=int, default=10)
    ap.add_argument("--transport", default="nvlink")
    ap.add_argument("--multicast", type=int, default=0,
                    help="1: reduce and publish through the NVSwitch multicast view (multimem) instead of peer loads / stores")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    port = 10000 + (int(os.environ.get("MASTER_PORT", "29500")) % 10) * 2000   # below the ephemeral range
    run = 0
    for mb in a.mb:
        for slack in a.slack:
            run += 1
            rows = max(world, int(mb * 1024 * 1024 / 512))
            cfg = GeePsConfig(host_list=["127.0.0.1"] * world,
                              port_list=[port + (run % 19) * 100 + 10 * r for r in range(world)],
                              device=DEVICE_CUDA, cuda_device=local,
                              transport=TRANSPORT_NVLINK if a.transport == "nvlink" else TRANSPORT_TCP,
                              partitioner=PARTITION_ROUND_ROBIN, table_mode=TABLE_SGD_MOMENTUM, grad_scale=1.0 / world,
                              use_multicast=a.multicast)
            with torch.cuda.stream(torch.cuda.Stream(device=dev)):
                g = GeePs(rank, cfg)
                ids = range(rows)
                r = g.virtual_read(0, ids, slack); u = g.virtual_pre_update(0, ids)
                pr = g.virtual_post_read(r); up = g.virtual_update(u); g.virtual_clock()
                g.finish_virtual_iteration()
                g.pre_update(u).zero_(); g.update(up); g.clock(); g.start_iterations()
                upd = torch.randn(rows, 128, device=dev, generator=torch.Generator(device=dev).manual_seed(rank)) * 0.01
                sink = torch.zeros(1, device=dev)

                def clock():
                    x = g.read(r)
                    sink.add_(x[0, 0])                      # the pulled rows are consumed
                    b = g.pre_update(u)
                    g.post_read(pr)
                    b.copy_(upd)                            # the worker produces its update in place
                    g.update(up)
                    g.clock()

                for _ in range(3):
                    clock()
                torch.cuda.synchronize()
                if dist: dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(a.clocks):
                    clock()
                torch.cuda.synchronize()
                e1.record(); e1.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / a.clocks], device=dev, dtype=torch.float64)
                if dist: dist.all_reduce(t, op=dist.ReduceOp.MAX)
                err = g.last_error()
                multicast = bool(g.get_stats().get("multicast", False))
                g.shutdown(); g.close()
            if rank == 0:
                nbytes = rows * 512
                out = {"bench": "ps_pushpull", "transport": a.transport, "world": world, "table_mb": nbytes / 2**20,
                       "slack": slack, "ms_per_clock": t.item(), "gb_s_per_gpu": nbytes / t.item() / 1e6, "error": err,
                       "multicast": multicast}
                if world > 1:
                    link_ms = 2 * (world - 1) / world * nbytes / 770e9 * 1e3
                    out["nvlink_roofline_ms"] = link_ms
                    out["frac_of_nvlink_roofline"] = link_ms / t.item()
                print(json.dumps(out), flush=True)
    if dist: dist.destroy_process_group()


if __name__ == "__main__":
    main()
