"""Training-loop pieces that need no GPU: learning-rate policies, the solver's bookkeeping (when the rate changes,
what is displayed, when snapshots are written, where a resumed run starts) and the data walk of the trainer."""
import math
import os

import numpy as np
import pytest
import torch

from geeps_b200.train import ArraySource, device_batches, synthetic_arrays
from geeps_b200.utils.solver import LrPolicy, Solver


def test_learning_rate_policies_follow_their_formulas():
    assert LrPolicy("fixed", 0.02)(12345) == 0.02
    step = LrPolicy("step", 0.1, gamma=0.5, stepsize=10)
    assert [step(i) for i in (0, 9, 10, 25, 30)] == pytest.approx([0.1, 0.1, 0.05, 0.025, 0.0125])
    multi = LrPolicy("multistep", 1.0, gamma=0.1, stepvalues=(30, 10))
    assert [multi(i) for i in (0, 9, 10, 29, 30, 99)] == pytest.approx([1, 1, 0.1, 0.1, 0.01, 0.01])
    assert LrPolicy("exp", 0.1, gamma=0.99)(100) == pytest.approx(0.1 * 0.99 ** 100)
    assert LrPolicy("inv", 0.01, gamma=1e-4, power=0.75)(5000) == pytest.approx(0.01 * (1 + 0.5) ** -0.75)
    poly = LrPolicy("poly", 0.1, power=2.0, max_iter=100)
    assert [poly(i) for i in (0, 50, 100, 150)] == pytest.approx([0.1, 0.025, 0.0, 0.0])
    sig = LrPolicy("sigmoid", 0.1, gamma=-0.01, stepsize=1000)
    assert sig(1000) == pytest.approx(0.05) and sig(0) == pytest.approx(0.1 / (1 + math.exp(-10)))
    assert step.is_piecewise_constant() and not poly.is_piecewise_constant()
    with pytest.raises(ValueError):
        LrPolicy("cosine")
    with pytest.raises(ValueError):
        LrPolicy("poly", max_iter=0)


class FakeModule:
    """Stands in for PSModule: one reused loss tensor, a log of the calls the solver makes."""

    def __init__(self, steps=0):
        self.steps, self.calls, self.loss = steps, [], torch.zeros(1)

    def step(self, x, labels):
        self.loss.fill_(100.0 - self.steps)          # overwritten every step, like the module's loss buffer
        self.calls.append(("step", self.steps))
        self.steps += 1
        return self.loss

    def set_hyper_params(self, learning_rate=None, momentum=None, weight_decay=None):
        self.calls.append(("hyper", self.steps, learning_rate, momentum, weight_decay))

    def save_snapshot(self, directory):
        self.calls.append(("snapshot", self.steps, directory))


def batches():
    while True:
        yield None, None


def test_solver_changes_the_rate_only_where_the_policy_does_and_snapshots_on_schedule():
    mod, lines = FakeModule(), []
    solver = Solver(mod, LrPolicy("step", 0.1, gamma=0.1, stepsize=4), momentum=0.9, weight_decay=0.0, display=3,
                    snapshot=5, snapshot_dir="snap", log=lines.append)
    hist = solver.run(batches(), max_iter=12)
    hyper = [c for c in mod.calls if c[0] == "hyper"]
    assert [(c[1], round(c[2], 6)) for c in hyper] == [(0, 0.1), (4, 0.01), (8, 0.001)]     # before steps 0, 4, 8
    assert all(c[3] == 0.9 and c[4] == 0.0 for c in hyper)
    for h in hyper:                                 # the call precedes the step of its iteration
        assert mod.calls.index(h) < mod.calls.index(("step", h[1]))
    assert [c[1] for c in mod.calls if c[0] == "snapshot"] == [5, 10, 12]                  # every 5, and at the end
    assert [(it, loss) for it, loss, _ in hist] == [(0, 100.0), (3, 97.0), (6, 94.0), (9, 91.0)]   # each step's own loss
    assert [round(lr, 6) for _, _, lr in hist] == [0.1, 0.1, 0.01, 0.001]
    assert len(lines) == 4 and lines[1].startswith("iteration 3  loss 97.00000  lr 0.1")
    assert solver.iter == 12 and mod.steps == 12


def test_solver_holds_a_continuous_policy_and_resumes_at_the_module_iteration():
    mod = FakeModule(steps=10)                      # a module resumed from a snapshot of iteration 10
    solver = Solver(mod, LrPolicy("poly", 1.0, power=1.0, max_iter=40), lr_hold=8, log=lambda s: None)
    assert solver.iter == 10
    solver.run(batches(), max_iter=30)
    hyper = [(c[1], round(c[2], 6)) for c in mod.calls if c[0] == "hyper"]
    assert hyper == [(10, 0.8), (16, 0.6), (24, 0.4)]         # sampled at iterations 8, 16, 24; held in between
    assert [c[1] for c in mod.calls if c[0] == "step"] == list(range(10, 30))
    assert not [c for c in mod.calls if c[0] == "snapshot"]   # no snapshot directory: nothing written
    exact = Solver(FakeModule(), LrPolicy("poly", 1.0, max_iter=40), lr_hold=1, log=lambda s: None)
    exact.run(batches(), max_iter=5)
    assert len([c for c in exact.mod.calls if c[0] == "hyper"]) == 5
    with pytest.raises(ValueError):
        Solver(FakeModule(), LrPolicy(), snapshot=10)


def test_array_source_gives_every_rank_a_disjoint_share_of_each_epoch():
    images, labels = synthetic_arrays(103, (3, 8, 8), 10, (12, 12), seed=3)
    labels = np.arange(103)                          # the label names the image
    B, world = 5, 2
    srcs = [ArraySource(images, labels, B, r, world, seed=7, pin=False) for r in range(world)]
    per_rank = 103 // (B * world) * B                # 50 images per rank and epoch
    seen = [[], []]
    for r, s in enumerate(srcs):
        for _ in range(per_rank // B):
            x, y = s.next()
            assert x.shape == (B, 3, 12, 12) and x.dtype == torch.uint8 and y.dtype == torch.int64
            for xi, yi in zip(x, y):
                assert torch.equal(xi, torch.from_numpy(images[int(yi)]))
            seen[r] += y.tolist()
    assert len(set(seen[0])) == per_rank and len(set(seen[1])) == per_rank and not set(seen[0]) & set(seen[1])
    assert all(s.epoch == 0 for s in srcs)
    nxt = srcs[0].next()[1].tolist()                 # the next call opens epoch 1 with another permutation
    assert srcs[0].epoch == 1 and nxt != seen[0][:B]
    # skip(n) stands for n calls of next()
    a, b = (ArraySource(images, labels, B, 1, world, seed=7, pin=False) for _ in range(2))
    for _ in range(13):
        a.next()
    b.skip(13)
    assert a.next()[1].tolist() == b.next()[1].tolist()
    with pytest.raises(ValueError):
        ArraySource(images[:6], labels[:6], B, 0, world, pin=False)


class FakeFeeder:
    def __init__(self, depth=2):
        self.depth, self.put_i, self.get_i, self.log, self.slots = depth, 0, 0, [], [None] * depth

    def wait_copied(self, slot):
        self.log.append(("wait", slot))

    def submit(self, x, y):
        s = self.put_i % self.depth
        self.log.append(("submit", s, int(y[0])))
        self.slots[s] = (x.clone(), y.clone())
        self.put_i += 1

    def next(self, stream=None):
        s = self.get_i % self.depth
        self.get_i += 1
        return self.slots[s][0], self.slots[s][1], s

    def release(self, slot, stream=None):
        self.log.append(("release", slot))


def test_device_batches_keep_staging_sets_and_device_slots_in_step():
    images, _ = synthetic_arrays(40, (3, 4, 4), 10, (4, 4), seed=1)
    labels = np.arange(40)
    src = ArraySource(images, labels, 4, pin=False)
    ref = ArraySource(images, labels, 4, pin=False)
    feeder = FakeFeeder()
    gen = device_batches(src, feeder, stream=None)
    for k in range(6):
        x, y = next(gen)
        assert y.tolist() == ref.next()[1].tolist()           # batches arrive in the source's order
        # when batch k is handed out, batch k + 1 has been submitted from staging set (k + 1) % 2 after a wait on it
        subs = [e for e in feeder.log if e[0] == "submit"]
        assert len(subs) == k + 2 and subs[-1][1] == (k + 1) % 2
        i = feeder.log.index(subs[-1])
        assert feeder.log[i - 1] == ("wait", (k + 1) % 2)
    assert [e[1] for e in feeder.log if e[0] == "release"] == [0, 1, 0, 1, 0]


def test_trainer_main_wires_model_data_feeder_and_solver(monkeypatch, tmp_path, capsys):
    """python -m geeps_b200.train end to end with the GPU parts replaced by fakes (the module, the feeder, the CUDA
    stream calls): arguments reach the right places, the data walk feeds the module batch by batch, the policy's
    rate changes arrive before their iterations, snapshots are written, and a resumed run skips the consumed batches."""
    import contextlib

    import geeps_b200.parallel.ps_module as pm
    import geeps_b200.train as train
    import geeps_b200.utils.feeder as fd
    made = []

    class FakeInput:
        def __init__(self):
            self.transform, self.augs = None, 0

        def set_transform(self, mean, scale):
            self.transform = (tuple(mean), scale)

    class FakePS(FakeModule):
        def __init__(self, net, in_shape, cfg, rank=0, world=1, resume_from=None, **kw):
            super().__init__(steps=4 if resume_from else 0)
            self.in_shape, self.cfg, self.kw, self.resume_from = in_shape, cfg, kw, resume_from
            self.net = type("N", (), {"input_layer": FakeInput()})()
            self.labels_seen = []
            made.append(self)

        def step(self, x, labels):
            assert x.dtype == torch.uint8 and tuple(x.shape) == (4, 3, 40, 40)
            self.labels_seen.append(labels.tolist())
            return super().step(x, labels)

        def close(self):
            self.calls.append(("close",))

    class Feeder(FakeFeeder):
        def __init__(self, x_shape, y_shape, device, depth=2, x_dtype=None, timed=False):
            super().__init__(depth)
            assert tuple(x_shape) == (4, 3, 40, 40) and x_dtype == torch.uint8

    monkeypatch.setattr(pm, "PSModule", FakePS)
    monkeypatch.setattr(fd, "HostFeeder", Feeder)
    monkeypatch.setattr(torch.cuda, "set_device", lambda d: None)
    monkeypatch.setattr(torch.cuda, "Stream", lambda **kw: object())
    monkeypatch.setattr(torch.cuda, "stream", lambda s: contextlib.nullcontext())
    monkeypatch.setattr(torch.cuda, "synchronize", lambda d=None: None)
    monkeypatch.setattr(torch.Tensor, "pin_memory", lambda t: t)
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    snap = str(tmp_path / "snap")
    common = ["--model", "inception_bn_small", "--batch", "4", "--synthetic-images", "24", "--source-size", "40",
              "--no-augment", "--lr-policy", "step", "--stepsize", "3", "--base-lr", "0.1", "--display", "2",
              "--snapshot", "4", "--snapshot-dir", snap, "--mean", "1", "2", "3", "--scale", "0.5"]
    train.main(common + ["--max-iter", "8"])
    mod = made[0]
    assert mod.in_shape == (4, 3, 32, 32) and mod.resume_from is None and mod.kw["use_graph"] is True
    assert mod.cfg.learning_rate == pytest.approx(0.1)
    assert mod.net.input_layer.transform == ((1.0, 2.0, 3.0), 0.5)
    assert [c[1] for c in mod.calls if c[0] == "step"] == list(range(8))
    assert [(c[1], round(c[2], 6)) for c in mod.calls if c[0] == "hyper"] == [(0, 0.1), (3, 0.01), (6, 0.001)]
    assert [c[1] for c in mod.calls if c[0] == "snapshot"] == [4, 8] and mod.calls[-1] == ("close",)
    out = capsys.readouterr().out
    assert "iteration 0  loss 100.00000  lr 0.1" in out and "iteration 6  loss 94.00000  lr 0.001" in out
    # a resumed run (the fake resumes at iteration 4) goes on with the batches the first run saw from iteration 4 on
    os.makedirs(snap, exist_ok=True)
    with open(os.path.join(snap, "LATEST"), "w") as f:
        f.write("5")
    train.main(common + ["--max-iter", "8", "--resume"])
    res = made[1]
    assert res.resume_from == snap and [c[1] for c in res.calls if c[0] == "step"] == [4, 5, 6, 7]
    assert res.labels_seen == mod.labels_seen[4:8]
    with pytest.raises(SystemExit):
        train.main(common + ["--max-iter", "8", "--resume", "--snapshot-dir", str(tmp_path / "none")])
