"""Host model of the device-flag protocol of the NVLINK transport, run under randomized interleavings.

Every rank is a worker and a shard.  Per clock c a worker (1) waits until data_age[s] >= c - slack for every
shard s (the stamp is clock + 1, so "all updates of clocks <= c - slack - 1 applied"), reads its cache,
(2) writes its update into ring slot c % (slack + 1) and (3) stamps push_ready[me] = c + 1 on every shard.
Shard s (a) waits until push_ready[w] >= c + 1 for every worker w, (b) reads slot c % (slack + 1) of every
worker's ring, applies, writes the fresh value into every worker's cache and (c) stamps data_age[s] = c + 1 on
every worker.  The model executes these micro-steps one at a time in an order drawn from a seeded RNG and checks,
at every step, the properties the kernels rely on:
  * a shard never reads a ring slot that already holds a later clock's update (slot reuse is safe),
  * a read at clock c contains every update of clocks <= c - slack - 1 and nothing newer than the workers
    can have produced,
  * the system always has a runnable step until every rank finished (no deadlock).
The real flags, stamps and ring arithmetic are in csrc/client/clientlib_fabric.cpp and csrc/kernels/ps_fabric.cu.
"""
import random

import pytest


class Model:
    def __init__(self, world, slack, clocks, seed):
        self.W, self.slack, self.clocks = world, slack, clocks
        self.rng = random.Random(seed)
        self.ring = slack + 1
        # per worker: ring slots hold (clock, value); cache[w][s] = (applied_through_clock, value of shard s)
        self.slots = [[None] * self.ring for _ in range(world)]
        self.cache = [[(-1, 0.0) for _ in range(world)] for _ in range(world)]
        self.push_ready = [[0] * world for _ in range(world)]     # [shard][worker]
        self.data_age = [[0] * world for _ in range(world)]       # [worker][shard]
        self.master = [0.0] * world
        self.wclock = [0] * world       # worker's current clock
        self.wphase = [0] * world       # 0 wait+read, 1 write slot, 2 signal
        self.sclock = [0] * world       # shard's current clock
        self.sphase = [0] * world       # 0 wait, 1 reduce+apply+publish, 2 stamp
        self.max_lead = 0

    def worker_step(self, w):
        c = self.wclock[w]
        if c >= self.clocks:
            return False
        if self.wphase[w] == 0:
            if any(self.data_age[w][s] < c - self.slack for s in range(self.W)):
                return False
            for s in range(self.W):
                through, value = self.cache[w][s]
                assert through >= c - self.slack - 1, "read misses an update it must contain"
                assert value == float(self.W * (through + 1)), "cache value does not match its clock stamp"
                assert through <= c + self.slack, "a shard applied a clock no worker can have reached"
            self.wphase[w] = 1
        elif self.wphase[w] == 1:
            self.slots[w][c % self.ring] = (c, 1.0)
            self.wphase[w] = 2
        else:
            for s in range(self.W):
                self.push_ready[s][w] = c + 1
            self.wclock[w], self.wphase[w] = c + 1, 0
            self.max_lead = max(self.max_lead, max(self.wclock) - min(self.wclock))
        return True

    def shard_step(self, s):
        c = self.sclock[s]
        if c >= self.clocks:
            return False
        if self.sphase[s] == 0:
            if any(self.push_ready[s][w] < c + 1 for w in range(self.W)):
                return False
            self.sphase[s] = 1
        elif self.sphase[s] == 1:
            total = 0.0
            for w in range(self.W):
                slot = self.slots[w][c % self.ring]
                assert slot is not None and slot[0] == c, f"shard {s} clock {c}: slot of worker {w} holds {slot}"
                total += slot[1]
            self.master[s] += total
            for w in range(self.W):
                self.cache[w][s] = (c, self.master[s])
            self.sphase[s] = 2
        else:
            for w in range(self.W):
                self.data_age[w][s] = c + 1
            self.sclock[s], self.sphase[s] = c + 1, 0
        return True

    def run(self):
        actors = [("w", i) for i in range(self.W)] + [("s", i) for i in range(self.W)]
        steps = 0
        while any(c < self.clocks for c in self.wclock + self.sclock):
            order = actors[:]
            self.rng.shuffle(order)
            progressed = False
            for kind, i in order:
                if (self.worker_step(i) if kind == "w" else self.shard_step(i)):
                    progressed = True
                    break            # one micro-step, then reshuffle: every interleaving is reachable
            assert progressed, f"deadlock at worker clocks {self.wclock}, shard clocks {self.sclock}"
            steps += 1
        assert all(m == float(self.W * self.clocks) for m in self.master)
        return steps


@pytest.mark.parametrize("world,slack", [(2, 0), (2, 1), (4, 0), (4, 2), (8, 1)])
def test_flag_protocol_holds_under_random_interleavings(world, slack):
    for seed in range(40):
        m = Model(world, slack, clocks=12, seed=seed)
        m.run()
        # bounded staleness also bounds how far workers drift apart
        assert m.max_lead <= slack + 1


def test_model_detects_a_ring_that_is_too_small():
    """Sanity of the model itself: with one slot fewer than slack + 1 the reuse hazard is found."""
    hit = False
    for seed in range(60):
        m = Model(3, 2, clocks=10, seed=seed)
        m.ring = 2
        m.slots = [[None] * 2 for _ in range(3)]
        try:
            m.run()
        except AssertionError:
            hit = True
            break
    assert hit
