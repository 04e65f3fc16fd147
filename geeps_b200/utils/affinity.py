"""Pin a worker process to the CPU cores next to its GPU.

One process per GPU copies its input batches from pinned host memory every step.  Pinned pages are placed on the
NUMA node of the thread that first touches them, so a process that happens to run on the far socket reads every
batch across the inter-socket link, and eight such processes share that link.  Binding the process to the GPU's
ideal cores (as NVML reports them) before anything is allocated keeps buffers, feeder threads and the launch
thread local.  Reading NVML does not change any device setting.
"""
from __future__ import annotations

import os


def bind_to_gpu_cores(device_index: int) -> list[int] | None:
    """Set this process's CPU affinity to the cores NVML lists for GPU `device_index`.  Returns the core list, or
    None when NVML / the affinity call is unavailable (nothing is changed then)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = device_index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if device_index < len(ids) and ids[device_index].isdigit():
                    index = int(ids[device_index])
            handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            ncpu = os.cpu_count() or 1
            words = pynvml.nvmlDeviceGetCpuAffinity(handle, (ncpu + 63) // 64)
        finally:
            pynvml.nvmlShutdown()
        cores = [64 * w + b for w, mask in enumerate(words) for b in range(64) if (mask >> b) & 1]
        allowed = os.sched_getaffinity(0)
        cores = [c for c in cores if c in allowed]
        if not cores:
            return None
        os.sched_setaffinity(0, cores)
        return cores
    except Exception:
        return None
