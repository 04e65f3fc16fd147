"""Pin a worker process to the CPU cores next to its GPU.

One process per GPU copies its input batches from pinned host memory every step.  Pinned pages are placed on the
NUMA node of the thread that first touches them, so a process that happens to run on the far socket reads every
batch across the inter-socket link, and eight such processes share that link.  Binding the process to the GPU's
ideal cores (as NVML reports them) before anything is allocated keeps buffers, feeder threads and the launch
thread local.  Reading NVML does not change any device setting.
"""
from __future__ import annotations

import os


def split_shared_mask(cores: list[int], sharers: int, position: int) -> list[int]:
    """The slice of a core list that the `position`-th of `sharers` processes takes when they all got the same
    list: contiguous, disjoint, sizes differing by at most one; the whole list when there are fewer cores than
    processes."""
    if sharers <= 1 or len(cores) < sharers:
        return list(cores)
    lo = position * len(cores) // sharers
    hi = (position + 1) * len(cores) // sharers
    return list(cores[lo:hi])


def bind_to_gpu_cores(device_index: int, local_world: int = 1, nvml=None) -> list[int] | None:
    """Set this process's CPU affinity to the cores NVML lists for GPU `device_index`.  When the GPUs of the
    `local_world` processes on this host report the same core list (a virtual machine with one NUMA node, for
    instance), the list is cut into disjoint slices, one per process, so that the launch thread of one rank never
    competes with the threads of another.  Returns the core list, or None when NVML / the affinity call is
    unavailable (nothing is changed then).  `nvml` lets a test pass a stand-in for the pynvml module."""
    try:
        pynvml = nvml
        if pynvml is None:
            import pynvml
        pynvml.nvmlInit()
        try:
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            ids = [v.strip() for v in visible.split(",") if v.strip()] if visible else []

            def physical(i: int) -> int:
                return int(ids[i]) if i < len(ids) and ids[i].isdigit() else i

            ncpu = os.cpu_count() or 1
            masks = []
            for i in range(max(local_world, device_index + 1)):
                try:
                    words = pynvml.nvmlDeviceGetCpuAffinity(pynvml.nvmlDeviceGetHandleByIndex(physical(i)), (ncpu + 63) // 64)
                    masks.append([64 * w + b for w, mask in enumerate(words) for b in range(64) if (mask >> b) & 1])
                except Exception:
                    masks.append(None)
        finally:
            pynvml.nvmlShutdown()
        allowed = os.sched_getaffinity(0)
        cores = [c for c in (masks[device_index] or []) if c in allowed]
        if not cores:
            return None
        sharers = [i for i in range(local_world) if masks[i] == masks[device_index]]
        if len(sharers) > 1 and device_index in sharers:
            cores = split_shared_mask(cores, len(sharers), sharers.index(device_index))
        os.sched_setaffinity(0, cores)
        return cores
    except Exception:
        return None
