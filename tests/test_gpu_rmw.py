"""Read-my-updates on the NVLINK transport, and per-stream SSP waits.

The worker's own update of the previous clock has to be visible to its next read at slack 1 even though the
owning shard has not published that clock.  On one GPU the "shard that lags" is made on the host: the worker's
push-ready flag is withheld, so the shard never applies the clock (its bounded wait expires later and reports a
timeout; nothing faults or hangs)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

from geeps_b200.ops import _lib as L
from geeps_b200.ops._lib import lib, ptr, stream_ptr
from geeps_b200.parallel.ps import GeePs
from geeps_b200.utils.config import (DEVICE_CUDA, PARTITION_ROUND_ROBIN, TABLE_SGD_MOMENTUM, TRANSPORT_NVLINK,
                                     GeePsConfig)


def _one_gpu(port, rmw, mode=0, partitioner=0):
    dev = torch.device("cuda:0")
    cfg = GeePsConfig(device=DEVICE_CUDA, cuda_device=0, transport=TRANSPORT_NVLINK, tcp_base_port=port,
                      device_wait_budget_us=300_000, read_my_writes=rmw, table_mode=mode, learning_rate=0.1,
                      momentum=0.9, grad_scale=1.0, partitioner=partitioner)
    with torch.cuda.stream(torch.cuda.Stream(device=dev)):
        g = GeePs(0, cfg)
        rows = list(range(40))
        r = g.virtual_read(0, rows, 1); u = g.virtual_pre_update(0, rows)
        pr = g.virtual_post_read(r); up = g.virtual_update(u); g.virtual_clock()
        g.finish_virtual_iteration()
        g.pre_update(u).fill_(1.0); g.update(up); g.clock(); g.start_iterations()
        x1 = g.read(r).clone()                  # clock 1: initial values (published, or merged from the ring)
        b = g.pre_update(u); g.post_read(pr); b.fill_(2.0)
        g.inject(1, 1)                          # the shard never learns that clock 1 is complete
        g.update(up); g.clock()
        x2 = g.read(r).clone()                  # clock 2: admitted on the bootstrap data
        torch.cuda.current_stream().synchronize()
        plan = g.plan()
        g.close()
    return x1, x2, plan


@pytest.mark.parametrize("partitioner", [0, PARTITION_ROUND_ROBIN])
def test_own_pending_update_is_visible_additive(partitioner):
    x1, x2, plan = _one_gpu(28211 + 40 * partitioner, rmw=1, partitioner=partitioner)
    assert torch.all(x1 == 1.0)
    assert torch.all(x2 == 3.0), (float(x2.min()), float(x2.max()))     # 1.0 + own +2.0 of clock 1
    reads = [op for op in plan["ops"] if op["type"] == "read"]
    assert reads and not any(op["direct"] for op in reads)               # merged into a private copy


def test_without_read_my_updates_the_pending_update_is_not_visible():
    x1, x2, _ = _one_gpu(28311, rmw=0)
    assert torch.all(x1 == 1.0) and torch.all(x2 == 1.0)


def test_own_pending_gradient_is_a_provisional_step_on_optimizer_tables():
    x1, x2, _ = _one_gpu(28351, rmw=1, mode=TABLE_SGD_MOMENTUM)
    assert torch.all(x1 == 1.0)
    assert torch.allclose(x2, torch.full_like(x2, 1.0 - 0.1 * 2.0), atol=1e-6), (float(x2.min()), float(x2.max()))


def test_rmw_gather_retries_while_a_publish_is_in_progress():
    """Kernel-level check of the begin / end stamps: with publish_begin ahead of data_age and nothing completing
    the publish, the bounded wait expires and the kernel reports a timeout instead of returning torn rows; with the
    stamps equal it returns cache + own ring slots."""
    dev = torch.device("cuda:0")
    rows, slots, clock = 16, 2, 3
    cache = torch.full((rows, 128), 5.0, device=dev)
    ring = torch.zeros(slots, rows, 128, device=dev)
    ring[2 % slots] = 0.25                       # own update of clock 2
    ring[1 % slots] = 100.0                      # clock 1: already published (data_age stamp 2), must not be added
    idx = torch.stack([torch.arange(rows), torch.arange(rows)], 1).to(torch.int64).to(dev).contiguous()
    age = torch.full((8,), 2, dtype=torch.int32, device=dev)
    begin = torch.full((8,), 2, dtype=torch.int32, device=dev)
    dst = torch.zeros(rows, 128, device=dev)
    st = L.new_status(dev)
    p = L.RmwReadParams()
    p.dst, p.cache, p.ring, p.index = dst.data_ptr(), cache.data_ptr(), ring.data_ptr(), idx.data_ptr()
    p.data_age, p.publish_begin, p.status = age.data_ptr(), begin.data_ptr(), st.data_ptr()
    p.num_rows, p.num_vals_limit, p.dst_rows, p.total_rows = rows, rows * 128, rows, rows
    p.wait_budget_ns, p.n_ranks, p.partition_kind, p.ring_slots, p.clock = 100_000_000, 1, 0, slots, clock
    p.additive_below_clock, p.alpha = 0, 1.0
    assert lib().geeps_row_gather_rmw(C.byref(p), stream_ptr()) == 0
    torch.cuda.synchronize()
    assert L.read_status(st)["code"] == 0
    assert torch.all(dst == 5.25)
    begin.fill_(3)                               # a publish of clock 2 has begun and never ends
    dst.zero_()
    assert lib().geeps_row_gather_rmw(C.byref(p), stream_ptr()) == 0
    torch.cuda.synchronize()
    assert L.read_status(st)["name"] == "timeout"
    assert torch.all(dst == 0.0)                 # nothing was delivered for the rows in doubt
    assert float(torch.ones(4, device=dev).sum()) == 4.0


def test_second_stream_gets_its_own_wait():
    """A read on stream A followed by a pre-update of the same table on stream B in the same clock: each stream is
    ordered by its own wait kernel (the launch counter of the runtime's flag waits goes up by two)."""
    dev = torch.device("cuda:0")
    cfg = GeePsConfig(device=DEVICE_CUDA, cuda_device=0, transport=TRANSPORT_NVLINK, tcp_base_port=28411)
    sa, sb = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    with torch.cuda.stream(sa):
        g = GeePs(0, cfg)
        rows = list(range(8))
        r = g.virtual_read(0, rows, 0); u = g.virtual_pre_update(0, rows)
        pr = g.virtual_post_read(r); up = g.virtual_update(u); g.virtual_clock()
        g.finish_virtual_iteration()
        g.pre_update(u).fill_(1.0); g.update(up); g.clock(); g.start_iterations()
        for c in range(3):
            w0 = g.get_stats()["client"]["device_waits_enqueued"]
            x = g.read(r, stream=sa)
            b = g.pre_update(u, stream=sb)       # other stream, same table, same clock
            w1 = g.get_stats()["client"]["device_waits_enqueued"]
            assert w1 - w0 == 2, (c, w0, w1)
            g.post_read(pr, stream=sa)
            sb.wait_stream(sa)
            with torch.cuda.stream(sb):
                b.fill_(1.0)
            g.update(up, stream=sb); g.clock()
        torch.cuda.synchronize()
        x = g.read(r, stream=sa, asynchronous=False)
        assert torch.all(x == 4.0)
        assert g.last_error() == 0
        g.close()
