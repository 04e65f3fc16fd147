"""Bounded device-side waits: a flag that nothing sets makes the wait kernel run out of its budget,
the kernel records TIMEOUT in the status block and returns, the runtime turns it into an error code,
and the CUDA context stays usable.  Nothing here faults, traps or hangs the GPU."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

from geeps_b200.ops import _lib as L
from geeps_b200.ops._lib import lib, ptr, stream_ptr
from geeps_b200.parallel.ps import GeePs, GeePsError
from geeps_b200.utils.config import DEVICE_CUDA, TRANSPORT_NVLINK, GeePsConfig
import ctypes as C


def test_flag_wait_kernel_times_out_and_reports():
    dev = torch.device("cuda:0")
    flags = torch.zeros(8, dtype=torch.int32, device=dev)
    status = L.new_status(dev)
    t0 = time.time()
    rc = lib().geeps_flag_wait(ptr(flags), 4, 7, C.c_ulonglong(200_000_000), ptr(status), stream_ptr())   # 0.2 s budget
    assert rc == 0
    torch.cuda.synchronize()
    assert time.time() - t0 < 5
    s = L.read_status(status)
    assert s["name"] == "timeout" and s["kernel"] == 13 and s["seen"] == 0
    # the context is alive: ordinary work still runs
    assert float((torch.ones(10, device=dev) * 2).sum()) == 20.0
    # and a satisfied wait does not report
    flags.fill_(9)
    status.zero_()
    lib().geeps_flag_wait(ptr(flags), 4, 7, C.c_ulonglong(200_000_000), ptr(status), stream_ptr())
    torch.cuda.synchronize()
    assert L.read_status(status)["code"] == 0


def test_withheld_push_signal_surfaces_as_device_timeout():
    dev = torch.device("cuda:0")
    cfg = GeePsConfig(device=DEVICE_CUDA, cuda_device=0, transport=TRANSPORT_NVLINK, tcp_base_port=28111,
                      device_wait_budget_us=300_000)
    with torch.cuda.stream(torch.cuda.Stream(device=dev)):
        g = GeePs(0, cfg)
        rows = list(range(32))
        r = g.virtual_read(0, rows, 0); u = g.virtual_pre_update(0, rows)
        pr = g.virtual_post_read(r); up = g.virtual_update(u); g.virtual_clock()
        g.finish_virtual_iteration()
        g.pre_update(u).zero_(); g.update(up); g.clock(); g.start_iterations()
        x = g.read(r); b = g.pre_update(u); g.post_read(pr); b.fill_(1.0)
        g.inject(1, 1)                 # host-side injection: the "my update is ready" flag is never written
        g.update(up)
        with pytest.raises(GeePsError) as e:
            for _ in range(4):
                g.clock()              # the expired wait is seen at a clock boundary, at most one clock late
                torch.cuda.synchronize()
                x = g.read(r); b = g.pre_update(u); g.post_read(pr); g.update(up)
        assert e.value.code == 4      # ERR_DEVICE_TIMEOUT
        torch.cuda.synchronize()
        assert float(torch.ones(4, device=dev).sum()) == 4.0
        g.close()
