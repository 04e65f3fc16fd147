"""The plan-driven HBM <-> pinned-DRAM swapper on a real GPU: worker-local row batches that do not fit the
GPU budget live in pinned host memory, are fetched into staging buffers (side stream, one access ahead)
and evicted when kept.  Checks data integrity over several clocks and the swap counters."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from geeps_b200.parallel.ps import GeePs
from geeps_b200.utils.config import DEVICE_CUDA, GeePsConfig


def _build(capacity_rows, mm, port):
    cfg = GeePsConfig(device=DEVICE_CUDA, cuda_device=0, tcp_base_port=port, gpu_memory_capacity=capacity_rows * 512,
                      mm_warning_level=mm)
    g = GeePs(0, cfg)
    u = g.virtual_pre_update(0, [0, 1])
    up = g.virtual_update(u)
    n = 6
    rows = [list(range(1000 * (i + 1), 1000 * (i + 1) + 400)) for i in range(n)]     # 6 batches x 400 rows
    # "forward": produce every batch (no fetch, keep); "backward": consume them in reverse (fetch, discard)
    fwd = []
    for i in range(n):
        h = g.virtual_local_access(rows[i], False)
        fwd.append((h, g.virtual_post_local_access(h, True)))
    bwd = []
    for i in reversed(range(n)):
        h = g.virtual_local_access(rows[i], True)
        bwd.append((i, h, g.virtual_post_local_access(h, False)))
    g.virtual_clock()
    g.finish_virtual_iteration()
    return g, u, up, fwd, bwd


@pytest.mark.parametrize("capacity_rows,expect_swap", [(100000, False), (1300, True)])
def test_local_batches_survive_swapping(capacity_rows, expect_swap):
    dev = torch.device("cuda:0")
    with torch.cuda.stream(torch.cuda.Stream(device=dev)):
        g, u, up, fwd, bwd = _build(capacity_rows, 0 if expect_swap else 2, 28300 + capacity_rows % 97)
        plan = g.plan()
        assert plan["ok"]
        assert (plan["cpu_local_rows"] > 0) == expect_swap
        assert plan["gpu_rows_total"] <= capacity_rows
        g.pre_update(u).zero_(); g.update(up); g.clock(); g.start_iterations()
        for clock in range(4):
            g.pre_update(u).zero_(); g.update(up)
            for i, (h, ph) in enumerate(fwd):
                buf = g.local_access(h)
                buf.fill_(float(100 * clock + i))        # device work on the app stream
                buf[:, 0] += 0.5
                g.post_local_access(ph)
            for i, h, ph in bwd:
                buf = g.local_access(h)
                vals = buf.clone()
                g.post_local_access(ph)
                torch.cuda.synchronize()
                assert float(vals[7, 3]) == float(100 * clock + i), (clock, i, float(vals[7, 3]))
                assert float(vals[399, 0]) == float(100 * clock + i) + 0.5
            g.clock()
        st = g.get_stats()["client"]
        if expect_swap:
            assert st["swap_h2d_bytes"] > 0 and st["swap_d2h_bytes"] > 0 and st["rows_fetched"] > 0
        else:
            assert st["swap_h2d_bytes"] == 0 and st["swap_d2h_bytes"] == 0
        assert g.last_error() == 0
        g.shutdown(); g.close()
