"""Multi-GPU parameter server over NVLink peer memory: one process per GPU."""
import multiprocessing as mp
import os

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

from ps_workers import nvlink_hello_worker, nvlink_leave_worker, nvlink_pull_gemm_worker, nvlink_train_worker

_port = [15000 + (os.getpid() % 100) * 100]


def _spawn(target, world, args, kw=None):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    _port[0] += 100
    procs = [ctx.Process(target=target, args=(r, world, _port[0]) + args + (q,) + (kw or {},)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for o in out:
        assert o[1] == "ok", o[2]
    return sorted(out)


def _world():
    import torch
    n = torch.cuda.device_count()
    return 8 if n >= 8 else 4 if n >= 4 else 2


@pytest.mark.parametrize("slack", [0, 1])
def test_nvlink_helloworld(slack):
    world, clocks = _world(), 50
    out = _spawn(nvlink_hello_worker, world, (slack, clocks))
    for rank, _, final, seen, _, stats in out:
        assert final == (float(world * clocks),) * 2, final
        for clock, lo, hi in seen:
            need = world * max(0, min(clock - slack - 1, clocks))
            most = min(clock - 1, clocks) + (world - 1) * min(clock + slack, clocks)
            assert lo >= need - 1e-6, (clock, lo, need)
            assert hi <= most + 1e-6, (clock, hi, most)


@pytest.mark.parametrize("slack", [0, 1])
def test_nvlink_helloworld_through_the_multicast_view(slack):
    """Same run with the arena bound to an NVSwitch multicast object: the push kernel reduces with
    multimem.ld_reduce and publishes with multimem.st.  Integer-valued updates, so the in-switch sum is exact."""
    world, clocks = _world(), 40
    out = _spawn(nvlink_hello_worker, world, (slack, clocks), dict(use_multicast=1, _rows=3000))
    for rank, _, final, seen, _, stats in out:
        assert stats["multicast"] is True, "the multicast arena was not used"
        assert final == (float(world * clocks),) * 2, final
        for clock, lo, hi in seen:
            need = world * max(0, min(clock - slack - 1, clocks))
            most = min(clock - 1, clocks) + (world - 1) * min(clock + slack, clocks)
            assert lo >= need - 1e-6, (clock, lo, need)
            assert hi <= most + 1e-6, (clock, hi, most)


def test_nvlink_training_through_the_multicast_view_matches_peer_loads():
    """Data-parallel training with the reduce and the publish going through the switch: every worker reads
    bit-identical parameters, and the losses follow the peer-load run (the sums differ only in the order of the
    additions)."""
    world = _world()
    runs = {}
    for name, kw in (("p2p", {}), ("multicast", dict(use_multicast=1))):
        out = _spawn(nvlink_train_worker, world, (10,), kw)
        digests = [o[3] for o in out]
        for d in digests[1:]:
            assert d == digests[0]
        runs[name] = out[0][2]
    assert runs["multicast"] == pytest.approx(runs["p2p"], rel=5e-3), runs


def test_nvlink_data_parallel_training_is_consistent():
    world = _world()
    out = _spawn(nvlink_train_worker, world, (10,))
    digests = [o[3] for o in out]
    for d in digests[1:]:
        assert d == digests[0]          # every worker reads bit-identical parameters
    for o in out:
        losses = o[2]
        assert all(l == l for l in losses), losses
        if world <= 2:       # with more workers the random-label batches average out within 10 steps
            assert losses[-1] < losses[0], losses


def test_nvlink_training_with_pulled_fc_tables_and_graph_replay_is_consistent():
    """The tables of both fully-connected layers are uncached: every rank's forward GEMM pulls the weight rows from
    all shards over NVLink.  With graph replay on top.  Every worker still reads bit-identical parameters and the run matches the
    published-table run of the same seed."""
    world = _world()
    runs = {}
    for name, mk in (("published", dict(net="fc_net")), ("pulled", dict(net="fc_net", pull_fc=True, use_graph=True))):
        out = _spawn(nvlink_train_worker, world, (10,), dict(_module=mk))
        digests = [o[3] for o in out]
        for d in digests[1:]:
            assert d == digests[0]
        runs[name] = out[0][2]
        for o in out:
            assert all(l == l for l in o[2]), o[2]
    assert runs["pulled"] == pytest.approx(runs["published"], rel=2e-3), runs


def test_pull_gemm_over_peer_memory():
    world = _world()
    out = _spawn(nvlink_pull_gemm_worker, world, (256, 4096, 9216))
    for o in out:
        r = o[2]
        assert r["status"] == 0 and r["w_local_ok"] and r["err"] < 5e-2, r
    print("pull_gemm fc6:", out[0][2])


def test_rank_leaving_between_steps_gives_an_error_not_a_hang():
    """Host-made failure on 2 GPUs: the leaving rank has nothing in flight; no GPU is faulted."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    _port[0] += 100
    procs = [ctx.Process(target=nvlink_leave_worker, args=(r, 2, _port[0], q, {})) for r in range(2)]
    for p in procs:
        p.start()
    out = {}
    for _ in range(2):
        o = q.get(timeout=180)
        out[o[0]] = o
    for p in procs:
        p.join(timeout=30)
    assert out[1][1] == "left"
    assert out[0][1] == "error" and out[0][2] in (4, 5), out[0]     # device wait expired or peer loss seen on the host
    assert out[0][3] < 60 and out[0][4] is True                      # bounded, and the CUDA context still works
