"""Parameter-server semantics on CPU over TCP loopback (no GPU): the helloworld-shaped run with
2 workers + 2 shards, SSP slack 0 and 1, additive and optimizer tables, read-my-writes,
round-robin partitioning, snapshots."""
import multiprocessing as mp
import os
import random

import pytest
import torch

from geeps_b200.parallel.ps import GeePs, GeePsError
from geeps_b200.utils.config import (DEVICE_CPU, PARTITION_ROUND_ROBIN, TABLE_SGD_MOMENTUM, GeePsConfig)

from ps_workers import helloworld_worker, lr_schedule_worker, multitable_worker, rmw_worker

_port = [12000 + (os.getpid() % 300) * 40]   # below the ephemeral port range


def next_port():
    _port[0] += 40
    return _port[0]


def run_workers(target, world, args, timeout=180):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=target, args=(r, world) + args + (q,) + ()) for r in range(world)]
    return ctx, q, procs


def _run_hello(world, slack, clocks, **kw):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = next_port()
    kw.setdefault("device", DEVICE_CPU)
    procs = [ctx.Process(target=helloworld_worker, args=(r, world, port, slack, clocks, q, kw)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for o in out:
        assert o[1] == "ok", o[2]
    return sorted(out)


@pytest.mark.parametrize("slack", [0, 1])
def test_helloworld_two_workers_two_shards(slack):
    clocks = 100
    out = _run_hello(2, slack, clocks)
    for rank, _, final, seen, max_stale, stats in out:
        assert final == (200.0, 200.0), final
        assert max_stale <= slack
        for clock, lo, hi in seen:
            # a read in clock c holds at least every worker's updates of clocks <= c - slack - 1
            # (clock 0 is the zero bootstrap) and at most everything issued so far
            # (its own clocks < c plus a peer that may run up to slack clocks ahead)
            need = 2.0 * max(0, min(clock - slack - 1, clocks))
            most = min(clock - 1, clocks) + min(clock + slack, clocks)
            assert lo >= need - 1e-6, (clock, lo, need)
            assert hi <= most + 1e-6, (clock, hi, most)
        assert stats["server"]["storage"]["nr_errors"] == 0


def test_round_robin_partition_and_read_my_writes():
    out = _run_hello(2, 1, 20, partitioner=PARTITION_ROUND_ROBIN, read_my_writes=1)
    for rank, _, final, seen, max_stale, stats in out:
        assert final == (40.0, 40.0)


def _run_rmw(mode, rmw):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = next_port()
    procs = [ctx.Process(target=rmw_worker, args=(r, 2, port, mode, rmw, q, {})) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for o in out:
        assert o[1] == "ok", o[2]
    return sorted(out)


@pytest.mark.parametrize("rmw", [0, 1])
def test_read_my_updates_additive_with_lagging_peer(rmw):
    """Slack 1, two workers, rank 1 lags before its clock-1 update.  Rank 0's read in clock 2 is admitted on the
    bootstrap data; with read-my-writes it must already contain rank 0's own +1 of clock 1, without it must not
    (the shards cannot have published clock 1 before the lagging worker signalled it)."""
    out = _run_rmw(0, rmw)
    rank0 = out[0]
    by_clock = {c: (lo, hi) for c, lo, hi in rank0[3]}
    assert by_clock[1] == (1.0, 1.0)                       # initial value only
    if rmw:
        assert by_clock[2] == (2.0, 2.0), by_clock         # initial value + own update of clock 1
    else:
        assert by_clock[2] == (1.0, 1.0), by_clock
    for o in out:
        assert o[2] == (11.0, 11.0)                        # 1.0 + 5 clocks x 2 workers, fully applied


def test_read_my_updates_optimizer_table_is_provisional_and_converges():
    """Momentum-SGD table with read-my-writes: the worker's view of its own pending gradient is the plain step
    -lr * g on top of the last published rows; once the shard has stepped, the published rows replace it and the
    final table equals the CPU oracle (the raw gradient is never added to the weights)."""
    out = _run_rmw(TABLE_SGD_MOMENTUM, 1)
    by_clock = {c: (lo, hi) for c, lo, hi in out[0][3]}
    assert by_clock[1] == (1.0, 1.0)
    lo, hi = by_clock[2]
    assert abs(lo - 0.9) < 1e-6 and abs(hi - 0.9) < 1e-6, by_clock     # 1.0 - 0.1 * own gradient of 1.0
    p, v = 1.0, 0.0
    for _ in range(5):                                     # five clocks, summed gradient 2.0
        v = 0.9 * v + 0.1 * 2.0
        p -= v
    for o in out:
        assert abs(o[2][0] - p) < 1e-4 and abs(o[2][1] - p) < 1e-4, (o[2], p)


def _single(cfg_kw, rows=(0, 1, 2, 3)):
    cfg = GeePsConfig(device=DEVICE_CPU, tcp_base_port=next_port(), **cfg_kw)
    return GeePs(0, cfg)


def test_optimizer_table_matches_momentum_sgd():
    g = _single(dict(table_mode=TABLE_SGD_MOMENTUM, learning_rate=0.1, momentum=0.9, weight_decay=0.01))
    rows = [5, 6, 7]
    r = g.virtual_read(0, rows, 0)
    u = g.virtual_pre_update(0, rows)
    pr = g.virtual_post_read(r)
    up = g.virtual_update(u)
    g.virtual_clock()
    g.finish_virtual_iteration()
    torch.manual_seed(0)
    w0 = torch.randn(3, 128)
    g.pre_update(u).copy_(w0)     # bootstrap update = initial values (always additive)
    g.update(up)
    g.clock()
    g.start_iterations()
    p, v = w0.clone(), torch.zeros_like(w0)
    for c in range(6):
        x = g.read(r, asynchronous=False).clone()
        assert torch.allclose(x, p, atol=1e-6), c
        grad = torch.randn(3, 128)
        b = g.pre_update(u)
        g.post_read(pr)
        b.copy_(grad)
        g.update(up)
        g.clock()
        v = 0.9 * v + 0.1 * (grad + 0.01 * p)
        p = p - v
    g.shutdown()
    g.close()


def test_optimizer_table_follows_hyper_parameter_changes():
    """set_hyper_params between iterations: the shard applies the updates of that iteration and all later ones with
    the new learning rate / momentum / weight decay, earlier ones with the old values."""
    g = _single(dict(table_mode=TABLE_SGD_MOMENTUM, learning_rate=0.1, momentum=0.9, weight_decay=0.01))
    rows = [5, 6, 7]
    r = g.virtual_read(0, rows, 0)
    u = g.virtual_pre_update(0, rows)
    pr = g.virtual_post_read(r)
    up = g.virtual_update(u)
    g.virtual_clock()
    g.finish_virtual_iteration()
    torch.manual_seed(0)
    w0 = torch.randn(3, 128)
    g.pre_update(u).copy_(w0)
    g.update(up)
    g.clock()
    g.start_iterations()
    assert g.hyper_params() == pytest.approx((0.1, 0.9, 0.01))
    p, v = w0.clone(), torch.zeros_like(w0)
    lr, mom, wd = 0.1, 0.9, 0.01
    for c in range(8):
        if c == 2:
            lr = 0.02
            g.set_hyper_params(learning_rate=lr)
        if c == 5:
            lr, mom, wd = 0.5, 0.0, 0.0
            g.set_hyper_params(lr, mom, wd)
            g.set_hyper_params(lr, mom, wd)          # repeating a call changes nothing
        assert g.hyper_params() == pytest.approx((lr, mom, wd))
        x = g.read(r, asynchronous=False).clone()
        assert torch.allclose(x, p, atol=1e-5), c
        grad = torch.randn(3, 128)
        b = g.pre_update(u)
        g.post_read(pr)
        b.copy_(grad)
        g.update(up)
        g.clock()
        v = mom * v + lr * (grad + wd * p)
        p = p - v
    g.shutdown()
    g.close()


@pytest.mark.parametrize("slack", [0, 1])
def test_all_shards_switch_hyper_parameters_at_the_same_clock(slack):
    """Two workers, two shards, one worker lagging: the update of clock c is applied with the values that were in
    force for clock c on every shard, so the table equals the single-process recurrence whatever the timing."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = next_port()
    procs = [ctx.Process(target=lr_schedule_worker, args=(rk, 2, port, slack, q, {})) for rk in range(2)]
    for pr in procs:
        pr.start()
    out = sorted(q.get(timeout=240) for _ in procs)
    for pr in procs:
        pr.join(timeout=60)
    p, v = 1.0, 0.0
    lr, mom, wd = 0.1, 0.9, 0.0
    for c in range(1, 9):
        if c == 3:
            lr = 0.05
        if c == 6:
            lr, mom, wd = 0.01, 0.5, 0.1
        v = mom * v + lr * (float(c) + wd * p)
        p -= v
    for o in out:
        assert o[1] == "ok", o[2]
        assert abs(o[2][0] - p) < 1e-4 and abs(o[2][1] - p) < 1e-4, (o[2], p)
        assert o[3][1] == pytest.approx((0.1, 0.9, 0.0)) and o[3][2] == pytest.approx((0.05, 0.9, 0.0))
        assert o[3][7] == pytest.approx((0.01, 0.5, 0.1))


def test_call_order_is_enforced_and_reported():
    g = _single({})
    r = g.virtual_read(0, [0], 0)
    u = g.virtual_pre_update(0, [0])
    pr = g.virtual_post_read(r)
    up = g.virtual_update(u)
    g.virtual_clock()
    g.finish_virtual_iteration()
    g.pre_update(u).zero_()
    g.update(up)
    g.clock()
    g.start_iterations()
    with pytest.raises(GeePsError) as e:
        g.pre_update(u)          # declared order starts with the read
        g.check()
    assert e.value.code == 2
    g.shutdown()
    g.close()


def test_plan_errors_surface():
    g = _single({})
    g.virtual_read(0, [0], 0)
    g.virtual_clock()
    with pytest.raises(GeePsError):
        g.finish_virtual_iteration()   # read never released, table never updated
    g.close()


def test_local_access_keeps_and_discards():
    g = _single({})
    u = g.virtual_pre_update(0, [0])
    up = g.virtual_update(u)
    la = g.virtual_local_access([100, 101], True)
    pla = g.virtual_post_local_access(la, True)
    g.virtual_clock()
    g.finish_virtual_iteration()
    g.pre_update(u).zero_(); g.update(up); g.clock()
    g.start_iterations()
    for c in range(3):
        g.pre_update(u).zero_(); g.update(up)
        buf = g.local_access(la)
        assert float(buf[0, 0]) == float(c)      # survives across clocks
        buf += 1.0
        g.post_local_access(pla)
        g.clock()
    g.shutdown(); g.close()


def test_snapshot_roundtrip(tmp_path):
    def build(port):
        cfg = GeePsConfig(device=DEVICE_CPU, tcp_base_port=port, table_mode=TABLE_SGD_MOMENTUM, learning_rate=0.05)
        g = GeePs(0, cfg)
        rows = list(range(16))
        r = g.virtual_read(0, rows, 0); u = g.virtual_pre_update(0, rows)
        pr = g.virtual_post_read(r); up = g.virtual_update(u); g.virtual_clock()
        g.finish_virtual_iteration()
        return g, r, u, pr, up

    def step(g, r, u, pr, up, seed):
        x = g.read(r, asynchronous=False).clone()
        b = g.pre_update(u); g.post_read(pr)
        b.copy_(torch.randn(16, 128, generator=torch.Generator().manual_seed(seed)))
        g.update(up); g.clock()
        return x

    g, r, u, pr, up = build(next_port())
    g.pre_update(u).copy_(torch.ones(16, 128)); g.update(up); g.clock()
    g.start_iterations()
    for s in range(3):
        if s == 2:
            g.set_hyper_params(learning_rate=0.02)      # in force from this iteration on
        step(g, r, u, pr, up, s)
    assert g.save_snapshot(str(tmp_path))
    import json
    with open(os.path.join(str(tmp_path), "snapshot.4", "MANIFEST.0.json")) as f:
        man = json.load(f)
    assert man["clock"] == 4 and man["learning_rate"] == pytest.approx(0.02) and man["momentum"] == pytest.approx(0.9)
    after = [step(g, r, u, pr, up, 10 + s) for s in range(3)]
    g.shutdown(); g.close()

    g2, r, u, pr, up = build(next_port())
    assert g2.load_snapshot(str(tmp_path))
    g2.start_iterations()
    # rows, momentum and clocks come from the snapshot; the hyper-parameters from the config and later calls
    assert g2.hyper_params()[0] == pytest.approx(0.05)
    g2.set_hyper_params(learning_rate=0.02)
    again = [step(g2, r, u, pr, up, 10 + s) for s in range(3)]
    for a, b in zip(after, again):
        assert torch.equal(a, b)      # parameters AND momentum came back
    g2.shutdown(); g2.close()


def _run_snapshot(world, phase, snap_dir):
    from ps_workers import snapshot_worker
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = next_port()
    procs = [ctx.Process(target=snapshot_worker, args=(r, world, port, phase, snap_dir, q, {})) for r in range(world)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    for o in out:
        assert o[1] == "ok", o[2]
    return [o[2] for o in out]


def test_snapshot_resharded_to_a_smaller_world(tmp_path):
    """Elastic restart: a 2-worker / 2-shard job snapshots, a 1-worker job resumes from it (the rows
    are re-partitioned on load) and continues with the same parameter values."""
    snap = str(tmp_path)
    two = _run_snapshot(2, "save", snap)
    one = _run_snapshot(1, "resume", snap)
    assert two[0] == two[1]
    assert one[0] == two[0]
    expect = (torch.arange(37 * 128, dtype=torch.float32) + 4 * 2 * 1.0 + 2.0).tolist()
    assert two[0] == expect


@pytest.mark.parametrize("policy", [1, 2, 3])
def test_placement_service_policies(policy):
    """The shards' placement service (the reference's MetadataServer: hash / first toucher / most frequent accessor
    with load balance) answers FIND_ROW queries from both workers consistently."""
    from ps_workers import placement_worker
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = next_port()
    procs = [ctx.Process(target=placement_worker, args=(r, 2, port, policy, q, {"device": DEVICE_CPU})) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=240) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    for o in out:
        assert o[1] == "ok", o[2]
    a, b = out[0][2], out[1][2]
    assert a["owners"] == b["owners"]
    if policy == 1:
        assert a["owners"] == [row % 2 for row in range(8)]
    elif policy == 2:
        assert a["owners"] == [(row // 2) % 2 for row in range(8)]
        assert all(v == 0 for v in a["first"].values()) and all(v == 1 for v in b["first"].values())
    else:
        assert a["owners"] == [1, 1, 1, 0]            # rank 1 accesses most; its fair share is 3 of the 4 rows
    assert out[0][3]["policy"] == policy and out[0][3]["nr_requests"] > 0


def test_helloworld_with_two_comm_channels():
    """num_comm_channels = 2: two push workers per process share the tables; same result as one channel."""
    out = _run_hello(2, 1, 30, num_comm_channels=2)
    for rank, _, final, seen, max_stale, stats in out:
        assert final == (60.0, 60.0), final
        assert max_stale <= 1


def test_tables_are_split_over_independent_channels():
    """num_comm_channels = 2 with three tables: tables 0 and 2 travel over channel 0 (port p), table 1 over
    channel 1 (port p + 1) - its own server shard, sockets and threads.  Both channels' shards hold rows and saw
    updates, and every table ends at the right value."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = next_port()
    clocks = 12
    procs = [ctx.Process(target=multitable_worker, args=(r, 2, port, clocks, q, dict(num_comm_channels=2))) for r in range(2)]
    for p in procs:
        p.start()
    out = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for o in sorted(out):
        assert o[1] == "ok", o[2]
        rank, _, vals, channels, nch, _ = o
        assert nch == 2 and len(channels) == 2
        assert vals == [(2.0 * clocks * (t + 1),) * 2 for t in range(3)], vals
        assert channels[0]["port"] + 1 == channels[1]["port"]
        # shard rows: tables 0 and 2 on channel 0, table 1 on channel 1 (range partition over two shards)
        assert channels[0]["storage"]["nr_rows"] in (32 + 9, 32 + 8) and channels[1]["storage"]["nr_rows"] == 100
        for ch in channels:
            assert ch["storage"]["nr_update"] > 0 and ch["storage"]["nr_errors"] == 0
            assert ch["server_router"]["msgs_received"] > 0
