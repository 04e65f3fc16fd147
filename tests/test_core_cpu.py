"""Host-only unit tests of the runtime's core: access-plan compiler, partitioners, allocators and
the CPU row-op oracle (through the C API of the native library)."""
import ctypes as C
import json
import threading
import time

import numpy as np
import pytest

from geeps_b200.parallel.ps import _lib

READ, POST_READ, PRE_UPDATE, UPDATE, LOCAL, POST_LOCAL, CLOCK = range(7)
ROW = 512


class Planner:
    def __init__(self, capacity_rows=-1, mm=1, rmw=0, shards=1, part=0, tables=1, gpu=True, direct=False, ring=False):
        self.l = _lib()
        cap = -1 if capacity_rows < 0 else capacity_rows * ROW
        self.p = C.c_void_p(self.l.geeps_planner_new(C.c_longlong(cap), mm, rmw, shards, part, tables, int(gpu),
                                                     int(direct), int(ring)))

    def rec(self, t, table=0, rows=(), slack=0, prestep=-1, fetch=False, keep=False):
        arr = (C.c_longlong * len(rows))(*rows)
        return self.l.geeps_planner_record(self.p, t, C.c_longlong(table), arr, len(rows), slack, prestep, int(fetch), int(keep))

    def compile(self):
        n = self.l.geeps_planner_compile_json(self.p, None, 0)
        buf = C.create_string_buffer(n + 8)
        self.l.geeps_planner_compile_json(self.p, buf, n + 8)
        return json.loads(buf.value.decode())


def simple_iteration(p, rows=range(10), slack=0):
    r = p.rec(READ, rows=list(rows), slack=slack)
    u = p.rec(PRE_UPDATE, rows=list(rows))
    p.rec(POST_READ, prestep=r)
    p.rec(UPDATE, prestep=u)
    p.rec(CLOCK)


def test_plan_basic_structure_and_last_write():
    p = Planner(tables=2)
    r0 = p.rec(READ, 0, [0, 1, 2]); r1 = p.rec(READ, 1, [5, 6])
    u1 = p.rec(PRE_UPDATE, 1, [5, 6]); p.rec(POST_READ, prestep=r1); w1 = p.rec(UPDATE, prestep=u1)
    u0a = p.rec(PRE_UPDATE, 0, [0]); w0a = p.rec(UPDATE, prestep=u0a)
    u0b = p.rec(PRE_UPDATE, 0, [1, 2]); p.rec(POST_READ, prestep=r0); w0b = p.rec(UPDATE, prestep=u0b)
    c = p.rec(CLOCK)
    plan = p.compile()
    assert plan["ok"] and plan["clock_handle"] == c
    ops = plan["ops"]
    assert ops[w1]["table_last_write"] == 1 and ops[w0b]["table_last_write"] == 1 and ops[w0a]["table_last_write"] == 0
    assert ops[r0]["post"] == 8 and ops[u0a]["post"] == w0a
    assert [t["num_rows"] for t in plan["tables"]] == [3, 2]
    # r0 (3 rows) and r1 (2) are alive together with u1 (2): peak 7 rows, double buffered pool
    assert plan["peak_staging_rows"] == 7 and plan["staging_copies"] == 2
    # buffers alive at the same time never overlap
    live = []
    for i, op in enumerate(ops):
        if op["type"] in ("read", "pre_update") and op["needs_staging"]:
            for (o, n, post) in live:
                if post > i:
                    assert op["staging_offset"] >= o + n or o >= op["staging_offset"] + op["num_rows"]
            live.append((op["staging_offset"], op["num_rows"], op["post"]))


def test_plan_rejects_bad_sequences():
    p = Planner()
    p.rec(READ, rows=[0]); p.rec(CLOCK)
    assert not p.compile()["ok"]                       # read never released
    p = Planner()
    r = p.rec(READ, rows=[0]); p.rec(POST_READ, prestep=r); p.rec(CLOCK)
    assert "never updated" in p.compile()["error"]      # every table needs an update before the clock
    p = Planner()
    simple_iteration(p)
    p2 = Planner(tables=1)
    u = p2.rec(PRE_UPDATE, 3, [0]); p2.rec(UPDATE, prestep=u); p2.rec(CLOCK)
    assert not p2.compile()["ok"]                       # table id out of range


def test_plan_memory_budget_and_warning_levels():
    def proper(cap, mm):
        p = Planner(capacity_rows=cap, mm=mm)
        r = p.rec(READ, rows=list(range(100)))
        la = p.rec(LOCAL, rows=list(range(1000, 1300)), fetch=True)
        lb = p.rec(LOCAL, rows=list(range(2000, 2200)), fetch=False)
        u = p.rec(PRE_UPDATE, rows=list(range(100)))
        p.rec(POST_LOCAL, prestep=lb, keep=True)
        p.rec(POST_LOCAL, prestep=la, keep=False)
        p.rec(POST_READ, prestep=r)
        p.rec(UPDATE, prestep=u)
        p.rec(CLOCK)
        return p.compile()
    big = proper(100000, 3)
    assert big["ok"] and big["cpu_local_rows"] == 0 and big["cpu_param_rows"] == 0 and big["gpu_local_rows"] == 500
    assert big["gpu_rows_total"] <= 100000
    # 1000 rows: local data (500) + double-buffered staging (2 x 200) fit, the parameter cache with its
    # update log (2 x 100) does not: it moves to host memory, which level 3 forbids
    mid = proper(1000, 1)
    assert mid["ok"] and mid["cpu_local_rows"] == 0 and mid["cpu_param_rows"] == 100 and mid["gpu_rows_total"] <= 1000
    assert not proper(1000, 3)["ok"]
    # 800 rows: no choice of resident batches leaves room for 2 x peak staging
    assert not proper(800, 1)["ok"]                     # level 1 insists on double buffering
    low = proper(800, 0)                                # level 0: swap local data, single-buffered staging
    assert low["ok"] and low["cpu_local_rows"] == 500 and low["staging_copies"] == 1 and low["gpu_rows_total"] <= 800
    assert not proper(800, 2)["ok"]                     # level 2: all local data must be resident


def test_plan_direct_access_and_ring():
    p = Planner(direct=True, ring=True, shards=4, part=1)
    simple_iteration(p, range(64), slack=2)
    plan = p.compile()
    assert plan["ok"]
    assert all(op["direct"] == 1 for op in plan["ops"] if op["type"] in ("read", "pre_update"))
    assert plan["staging_rows"] == 0
    t = plan["tables"][0]
    assert t["num_oplog_entries"] == 3                  # slack + 1 ring slots
    assert [s["count"] for s in t["shards"]] == [16] * 4 and [s["stride"] for s in t["shards"]] == [4] * 4
    # a batch that is not one ascending run cannot be served zero-copy
    p = Planner(direct=True, ring=True)
    r = p.rec(READ, rows=[0, 2, 1]); u = p.rec(PRE_UPDATE, rows=[0, 1, 2])
    p.rec(POST_READ, prestep=r); p.rec(UPDATE, prestep=u); p.rec(CLOCK)
    plan = p.compile()
    assert plan["ops"][0]["direct"] == 0 and plan["ops"][1]["direct"] == 1


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("n,s", [(10, 3), (1000, 8), (7, 8), (128, 1)])
def test_partitioner_covers_every_row_once(kind, n, s):
    l = _lib()
    seen = np.zeros(n, dtype=int)
    for shard in range(s):
        out = (C.c_longlong * 3)()
        l.geeps_partition_range(kind, C.c_longlong(n), s, shard, out)
        start, stride, count = out[0], out[1], out[2]
        for k in range(count):
            i = start + k * stride
            seen[i] += 1
            assert l.geeps_partition_shard_of(kind, C.c_longlong(n), s, C.c_longlong(i)) == shard
    assert (seen == 1).all()


def test_multithreaded_cache_helper_blocks_and_wakes():
    l = _lib()
    h = C.c_void_p(l.geeps_mtcache_new(C.c_longlong(100)))
    a = l.geeps_mtcache_get(h, C.c_longlong(60), 0, 1, C.c_longlong(0))
    b = l.geeps_mtcache_get(h, C.c_longlong(40), 0, 2, C.c_longlong(0))
    assert (a, b) == (0, 60) and l.geeps_mtcache_used(h) == 100
    assert l.geeps_mtcache_get(h, C.c_longlong(10), 0, 3, C.c_longlong(0)) == -1          # full, non-blocking
    t0 = time.time()
    assert l.geeps_mtcache_get(h, C.c_longlong(10), 1, 3, C.c_longlong(200)) == -1        # bounded blocking wait
    assert 0.15 < time.time() - t0 < 5
    got = []
    th = threading.Thread(target=lambda: got.append(l.geeps_mtcache_get(h, C.c_longlong(50), 1, 4, C.c_longlong(20000))))
    th.start()
    time.sleep(0.2)
    l.geeps_mtcache_put(h, C.c_longlong(0), C.c_longlong(60))
    th.join(timeout=10)
    assert got == [0]                                   # woke up and reused the freed range
    l.geeps_mtcache_delete(h)


def test_ring_cache_helper_is_fifo():
    l = _lib()
    h = C.c_void_p(l.geeps_ringcache_new(C.c_longlong(10)))
    assert l.geeps_ringcache_get(h, C.c_longlong(4)) == 0
    assert l.geeps_ringcache_get(h, C.c_longlong(4)) == 4
    assert l.geeps_ringcache_get(h, C.c_longlong(4)) == -1
    l.geeps_ringcache_put(h, C.c_longlong(0), C.c_longlong(4))
    assert l.geeps_ringcache_get(h, C.c_longlong(4)) == 0    # wraps past the 2-row tail fragment
    l.geeps_ringcache_delete(h)


def test_cpu_row_ops_and_sgd_oracle():
    l = _lib()
    rng = np.random.default_rng(0)
    cache = rng.standard_normal((50, 128)).astype(np.float32)
    n = 20
    idx = np.stack([np.arange(n), rng.permutation(50)[:n]], 1).astype(np.int64)
    buf = np.full((n, 128), -1, dtype=np.float32)
    fp = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    ip = idx.ctypes.data_as(C.POINTER(C.c_longlong))
    limit = (n - 1) * 128 + 5
    l.geeps_cpu_row_gather(fp(buf), fp(cache), ip, C.c_longlong(n), C.c_longlong(0), C.c_longlong(0), C.c_longlong(limit))
    ref = cache[idx[:, 1]].copy(); ref.reshape(-1)[limit:] = -1
    assert np.array_equal(buf, ref)
    oplog = np.zeros_like(cache)
    l.geeps_cpu_row_scatter_add(fp(oplog), fp(buf), ip, C.c_longlong(n), C.c_longlong(0), C.c_longlong(0), C.c_longlong(1 << 40))
    l.geeps_cpu_row_scatter_add(fp(oplog), fp(buf), ip, C.c_longlong(n), C.c_longlong(0), C.c_longlong(0), C.c_longlong(1 << 40))
    ref2 = np.zeros_like(cache); ref2[idx[:, 1]] = 2 * buf
    assert np.allclose(oplog, ref2)
    p = rng.standard_normal(1000).astype(np.float32); v = np.zeros(1000, np.float32); g = rng.standard_normal(1000).astype(np.float32)
    p0 = p.copy()
    l.geeps_cpu_sgd_momentum(C.c_longlong(1000), fp(p), fp(v), fp(g), C.c_float(0.1), C.c_float(0.9), C.c_float(0.01), C.c_float(0.5))
    v_ref = 0.1 * (g * 0.5 + 0.01 * p0)
    assert np.allclose(v, v_ref, atol=1e-6) and np.allclose(p, p0 - v_ref, atol=1e-6)


def test_plan_staging_pool_reaches_peak_for_a_layer_chain():
    """Activations of a layer chain (each access overlaps only its neighbours) are staged in a pool as large as
    the biggest adjacent pair: lowest / highest gap in turn, where first-fit from the bottom would fragment."""
    sizes = [100, 100, 25, 25, 25, 75, 75, 20, 25, 30]
    p = Planner(capacity_rows=230, mm=0)       # nothing can stay resident next to a 200-row staging pool
    handles, base = [], 0
    prev = None
    for i, n in enumerate(sizes):
        h = p.rec(LOCAL, rows=list(range(1000 * (i + 1), 1000 * (i + 1) + n)), fetch=False)
        if prev is not None:
            p.rec(POST_LOCAL, prestep=prev, keep=True)
        prev = h
    p.rec(POST_LOCAL, prestep=prev, keep=True)
    p.rec(CLOCK)
    plan = p.compile()
    assert plan["ok"], plan.get("error")
    assert plan["peak_staging_rows"] == 200
    assert plan["staging_rows"] == 200
    # no two live accesses overlap in the pool
    live, checked = {}, 0
    for op in plan["ops"]:
        if op["type"] == "local_access" and op["needs_staging"]:
            for off, n in live.values():
                assert op["staging_offset"] + op["num_rows"] <= off or off + n <= op["staging_offset"]
                checked += 1
            live[op["handle"]] = (op["staging_offset"], op["num_rows"])
        elif op["type"] == "post_local_access":
            live.pop(op["prestep"], None)
    assert checked >= len(sizes) - 1


def test_partition_alignment_keeps_row_groups_on_one_shard():
    """Range partition in groups of 72 rows (a 9216-wide weight row = 72 table rows): every shard starts on a
    group boundary, shards cover the table exactly once, and a trailing bias block goes to the last used shard."""
    import ctypes as C
    from geeps_b200 import _native
    lib = _native.load()
    lib.geeps_partition_range_aligned.restype = None
    rows, shards, align = 4096 * 72 + 32, 8, 72
    seen = 0
    for s in range(shards):
        out = (C.c_longlong * 3)()
        lib.geeps_partition_range_aligned(0, C.c_longlong(rows), shards, s, C.c_longlong(align), out)
        start, stride, count = out[0], out[1], out[2]
        assert stride == 1 and start == seen and (start % align == 0 or count == 0)
        seen += count
    assert seen == rows
