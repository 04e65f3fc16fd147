#!/usr/bin/env python
"""Headline benchmark: AlexNet training throughput (images/s) through the parameter server.

  python bench.py --gpus N --steps K --warmup W            (N=1: this process; N>1: under torchrun)
  python bench.py --impl reference ...                      (the unmodified reference, if it could be built)

Config (the AlexNet entry of the benchmark spec): 5 conv + 3 FC with LRN, ~61 M parameters,
synthetic 3x227x227 fp32 input ~N(0,1), labels uniform over 1000 classes, batch 256 per GPU
(weak scaling), fp32 parameter tables with momentum SGD applied by the owning server shard,
bf16 tensor-core compute, SSP slack 0.  One step = one parameter-server clock: Read every table,
forward, backward (gradients written into the PreUpdate buffers), Update, Clock.

Prints ONE JSON line on rank 0.  `value` is device-timed (CUDA events, max over ranks) with inputs
resident on the device (158 MB per step, larger than L2); `e2e` runs the same public API call with a
host->device copy of the step's batch from pinned memory and a device->host read of the loss in
every step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

MODEL = "alexnet"
BATCH_PER_GPU = 256
IMAGE = (3, 227, 227)
CLASSES = 1000


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None
        self.t_begin = self.t_end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        inside = [s for t, s in self.samples if self.t_begin is not None and self.t_begin <= t <= (self.t_end or t)]
        if not inside:   # region shorter than the sampling period: take the samples taken under load just before it
            inside = [s for _, s in self.samples[-3:]]
        for s in inside:
            f = [x.strip() for x in s.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> None:
    """The reference is a C++ library (SCons + ZeroMQ/boost/tbb/glog/gflags/cblas) with no Python
    package, and its Caffe application (the only program in it that trains AlexNet) is an empty submodule: the
    offline pip install answers "neither setup.py nor pyproject.toml found".  The last line of the install
    attempt's record, when present, is reported as the reason."""
    marker = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", "INSTALL_RESULT.txt")
    why = "reference cannot be installed offline: no setup.py/pyproject, needs zmq.hpp, boost, tbb, glog, gflags, cblas, scons; its Caffe app (the only AlexNet trainer) is an empty submodule"
    if os.path.exists(marker):
        with open(marker) as f:
            txt = f.read().strip().splitlines()
        if txt:
            why = txt[-1][:300]
    print(json.dumps({"impl": "reference", "unavailable": why}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default=MODEL)
    ap.add_argument("--batch", type=int, default=BATCH_PER_GPU)
    ap.add_argument("--transport", default="nvlink", choices=["nvlink", "tcp"])
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--cache-frac", type=float, default=None,
                    help="manage activations through the PS memory plan and cap the GPU budget at this fraction of the working set")
    ap.add_argument("--slack", type=int, default=0)
    ap.add_argument("--input-dtype", default="bf16", choices=["fp32", "bf16"],
                    help="dtype of the synthetic input batches on the host and on the device; the input layer rounds "
                         "either to bf16 NHWC, so the results are identical and bf16 halves the host-to-device bytes")
    ap.add_argument("--fp32-weight-cache", action="store_true",
                    help="also refresh the workers' fp32 copies of the weights every clock (the layers read bf16 only)")
    ap.add_argument("--no-tape", action="store_true",
                    help="re-run the Python layer code every step instead of replaying the recorded native calls")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from geeps_b200.models.alexnet import alexnet
    from geeps_b200.models.inception_bn import inception_bn_22k, inception_bn_small
    from geeps_b200.ops import _lib as L
    from geeps_b200.parallel.ps_module import PSModule
    from geeps_b200.utils.feeder import HostFeeder, LossMailbox
    from geeps_b200.utils.config import (DEVICE_CUDA, TABLE_SGD_MOMENTUM, TRANSPORT_NVLINK, TRANSPORT_TCP, GeePsConfig)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    # before any pinned allocation: keep this rank's host buffers and threads on the socket next to its GPU
    from geeps_b200.utils.affinity import bind_to_gpu_cores
    cores = bind_to_gpu_cores(local_rank)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    model_name = args.model
    if model_name == "alexnet":
        net, image, classes = alexnet(), IMAGE, CLASSES
    elif model_name == "inception_bn_small":
        net, image, classes = inception_bn_small(), (3, 32, 32), 10
    else:
        net, image, classes = inception_bn_22k(), (3, 224, 224), 21841
    B = args.batch
    # below the kernel's ephemeral port range (32768+), or an outgoing connection may already own the port
    base_port = 10000 + (int(os.environ.get("MASTER_PORT", "29500")) % 500) * 40
    cfg = GeePsConfig(host_list=["127.0.0.1"] * world, port_list=[base_port + 10 * r for r in range(world)],
                      device=DEVICE_CUDA, cuda_device=local_rank,
                      transport=TRANSPORT_NVLINK if args.transport == "nvlink" else TRANSPORT_TCP,
                      table_mode=TABLE_SGD_MOMENTUM, learning_rate=0.01, momentum=0.9, weight_decay=5e-4,
                      grad_scale=1.0 / world, bf16_compute_cache=1)
    stream = torch.cuda.Stream(device=dev, priority=-1)     # ahead of the runtime's comm stream
    with torch.cuda.stream(stream):
        mod = PSModule(net, (B,) + image, cfg, rank=rank, world=world, device=dev, slack=args.slack, seed=1,
                       manage_activations=args.cache_frac is not None, cache_fraction=args.cache_frac,
                       use_tape=not args.no_tape, bf16_weights_only=not args.fp32_weight_cache)
        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        in_dtype = torch.bfloat16 if args.input_dtype == "bf16" else torch.float32
        x_dev = torch.randn((B,) + image, device=dev, generator=gen).to(in_dtype)
        y_dev = torch.randint(0, classes, (B,), device=dev, generator=gen)
        x_host = torch.randn((B,) + image).to(in_dtype).pin_memory()
        y_host = torch.randint(0, classes, (B,)).pin_memory()

        def barrier():
            torch.cuda.synchronize(dev)
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(dev)

        def timed(step_fn, steps):
            sampler = ClockSampler(local_rank)
            sampler.start()
            for _ in range(3):       # keeps the GPU under load while nvidia-smi starts sampling (untimed)
                step_fn()
            barrier()
            sampler.mark_begin()
            launches0 = L.launch_count()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            loss = None
            for _ in range(steps):
                loss = step_fn()
            torch.cuda.synchronize(dev)      # the runtime's comm stream (push / apply kernels) included
            e1.record(stream)
            e1.synchronize()
            ms = e0.elapsed_time(e1)
            sampler.mark_end()
            clocks = sampler.stop()
            barrier()
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item(), clocks, L.launch_count() - launches0, float(loss.item()) if loss is not None else None

        def step_device():
            return mod.step(x_dev, y_dev)

        feeder = HostFeeder((B,) + image, (B,), dev, x_dtype=in_dtype)
        mailbox = LossMailbox(dev)
        feeder.submit(x_host, y_host)

        def step_e2e():
            # every step: this step's batch comes from pinned host memory (its copy was started one step
            # earlier on the copy stream), the next batch's copy starts now, and the loss goes back to the
            # host; the host reads each step's loss one step later, so the launch queue never drains
            xb, yb, slot = feeder.next(stream)
            feeder.submit(x_host, y_host)
            loss = mod.step(xb, yb)
            feeder.release(slot, stream)
            mailbox.post(loss, stream)
            mailbox.collect(lag=1)
            return loss

        for _ in range(max(args.warmup, 3)):
            step_device()
        ms, clocks, launches, last_loss = timed(step_device, args.steps)
        e2e = None
        if not args.no_e2e:
            for _ in range(2):
                step_e2e()
            ms_e, _, _, _ = timed(step_e2e, args.steps)
            e2e = {"value": B * world * args.steps / (ms_e / 1e3), "unit": "images/s",
                   "h2d_bytes_per_step": feeder.bytes_per_batch, "d2h_bytes_per_step": mailbox.bytes_per_step,
                   "ms_per_step": ms_e / args.steps}
        stats = mod.ps.get_stats()
        # kernels launched inside the runtime (flag signal + flag wait + push/apply per table per clock,
        # one data-age wait per table per clock) are not seen by the Python-side counter
        runtime_launches = stats["bgthread"]["nr_push"] * 3 // max(1, mod.steps) * args.steps + len(mod.tables) * args.steps
        if rank == 0:
            out = {
                "metric": "images/sec (device-timed, max over ranks)", "value": B * world * args.steps / (ms / 1e3),
                "unit": "images/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic", "impl": "ours",
                "config": {"model": model_name, "global_batch": B * world, "batch_per_gpu": B, "image": list(image),
                           "parallelism": f"dp{world}+ps{world}", "transport": args.transport, "slack": args.slack, "input_dtype": args.input_dtype, "cpu_cores_bound": len(cores) if cores else 0,
                           "weight_publish": "bf16+fp32" if args.fp32_weight_cache else "bf16 (biases / BN fp32)",
                           "host_replay_tapes": len(mod._tapes),
                           "tables": "fp32 master rows, momentum SGD on the owning shard",
                           "l2": "inputs (158 MB/step) and activations exceed the 126 MB L2; no explicit flush"},
                "memory_plan": ({"cache_fraction_of_activations": args.cache_frac, "budget_rows": mod.budget_rows,
                                 "working_set_rows": mod.working_set_rows, "managed_activation_rows": mod.managed_rows,
                                 "param_rows": mod.param_rows,
                                 "swap_h2d_gb_per_s": stats["client"]["swap_h2d_bytes"] / max(1, mod.steps) / (ms / args.steps) / 1e6,
                                 "swap_d2h_gb_per_s": stats["client"]["swap_d2h_bytes"] / max(1, mod.steps) / (ms / args.steps) / 1e6,
                                 "cpu_local_rows": stats["client"]["cpu_local_rows"], "gpu_local_rows": stats["client"]["gpu_local_rows"]}
                                if args.cache_frac is not None else None),
                "clocks": clocks, "e2e": e2e, "gpu_launches": launches + runtime_launches, "final_loss": last_loss,
            }
            print(json.dumps(out))
        mod.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
