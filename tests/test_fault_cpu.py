"""Failure detection with host-made failures (CPU ranks over TCP loopback; no GPU is involved):
a rank that exits between steps, a rank that goes silent, a dropped message."""
import multiprocessing as mp
import os

import pytest

from ps_workers import fault_worker

_port = [26000 + (os.getpid() % 50) * 100]


def _run(mode, kw, expect):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    _port[0] += 100
    procs = [ctx.Process(target=fault_worker, args=(r, 2, _port[0], mode, q, kw)) for r in range(2)]
    for p in procs:
        p.start()
    out = {}
    for _ in range(expect):
        o = q.get(timeout=120)
        out.setdefault(o[0], []).append(o)
    for p in procs:
        p.join(timeout=30)
        if p.is_alive():
            p.kill()
    return out


def test_rank_exit_is_detected_not_hung():
    out = _run("exit", dict(host_wait_budget_ms=20000), 2)
    assert out[1][0][1] == "left"
    rank0 = out[0][-1]
    assert rank0[1] == "error" and rank0[2] == 5, rank0      # ERR_PEER_LOST
    assert rank0[4] < 30                                      # well before any wait budget


def test_silent_rank_is_detected_by_heartbeat():
    out = _run("mute", dict(heartbeat_timeout_ms=1000, host_wait_budget_ms=30000), 2)
    rank0 = out[0][-1]
    assert rank0[1] == "error" and rank0[2] == 5 and "heartbeat" in rank0[3], rank0


def test_dropped_row_batch_times_out_with_an_error():
    out = _run("drop", dict(host_wait_budget_ms=1500, heartbeat_timeout_ms=60000), 2)
    rank0 = out[0][-1]
    assert rank0[1] == "error" and rank0[2] == 3, rank0       # ERR_HOST_TIMEOUT from the bounded read wait
