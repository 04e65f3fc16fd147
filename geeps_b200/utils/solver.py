"""Training loop around `PSModule`: learning-rate policies, periodic display, table snapshots and resume.

The reference's training loop was the solver of its Caffe application (absent from the reference tree); the
learning-rate policies here are Caffe's (`lr_policy` of a solver definition), evaluated by every worker on the
iteration number, so all workers hand the shards the same value before the same clock
(`GeePs::SetHyperParams`).

    policy = LrPolicy("step", base_lr=0.01, gamma=0.1, stepsize=100000)
    solver = Solver(mod, policy, display=20, snapshot=5000, snapshot_dir="snap")
    solver.run(batches(), max_iter=450000)          # batches() yields (images, labels) on the device
"""
from __future__ import annotations

import math
import time
from typing import Callable, Iterable, Sequence


class LrPolicy:
    """Learning rate as a function of the iteration number.

    fixed      base_lr
    step       base_lr * gamma ^ floor(iter / stepsize)
    multistep  base_lr * gamma ^ (number of stepvalues <= iter)
    exp        base_lr * gamma ^ iter
    inv        base_lr * (1 + gamma * iter) ^ -power
    poly       base_lr * (1 - iter / max_iter) ^ power
    sigmoid    base_lr / (1 + exp(-gamma * (iter - stepsize)))
    """
    POLICIES = ("fixed", "step", "multistep", "exp", "inv", "poly", "sigmoid")

    def __init__(self, policy: str = "fixed", base_lr: float = 0.01, gamma: float = 0.1, stepsize: int = 100000,
                 stepvalues: Sequence[int] = (), power: float = 1.0, max_iter: int = 0):
        if policy not in self.POLICIES:
            raise ValueError(f"unknown lr policy {policy!r}; one of {', '.join(self.POLICIES)}")
        if policy in ("step", "sigmoid") and stepsize <= 0:
            raise ValueError(f"lr policy {policy} needs stepsize > 0")
        if policy == "poly" and max_iter <= 0:
            raise ValueError("lr policy poly needs max_iter > 0")
        self.policy, self.base_lr, self.gamma, self.stepsize = policy, float(base_lr), float(gamma), int(stepsize)
        self.stepvalues, self.power, self.max_iter = sorted(int(v) for v in stepvalues), float(power), int(max_iter)

    def __call__(self, it: int) -> float:
        p, lr, g = self.policy, self.base_lr, self.gamma
        if p == "fixed":
            return lr
        if p == "step":
            return lr * g ** (it // self.stepsize)
        if p == "multistep":
            return lr * g ** sum(1 for v in self.stepvalues if v <= it)
        if p == "exp":
            return lr * g ** it
        if p == "inv":
            return lr * (1.0 + g * it) ** (-self.power)
        if p == "poly":
            return lr * max(0.0, 1.0 - it / self.max_iter) ** self.power
        return lr / (1.0 + math.exp(-g * (it - self.stepsize)))

    def is_piecewise_constant(self) -> bool:
        return self.policy in ("fixed", "step", "multistep")


class Solver:
    """Runs training steps of a module (`step(x, labels)`, `set_hyper_params(...)`, `save_snapshot(dir)`, `steps`)
    under a learning-rate policy.

    lr_hold: policies that change every iteration (exp, inv, poly, sigmoid) are sampled every lr_hold iterations and
    held in between.  A module that replays captured steps drops and re-captures them whenever the rate changes, so
    with graph replay a hold of a few hundred iterations keeps nearly every step a replay; 1 follows the policy
    exactly.
    display: every `display` iterations the loss of the previous iteration is read back (one iteration late, so the
    launch queue never drains) and a line goes to `log`.
    snapshot: every `snapshot` iterations (and at the end of `run`) the tables are written under snapshot_dir; a
    module built with `resume_from=snapshot_dir` continues at that iteration (`mod.steps`)."""

    def __init__(self, mod, policy: LrPolicy, momentum: float | None = None, weight_decay: float | None = None,
                 display: int = 0, snapshot: int = 0, snapshot_dir: str | None = None, lr_hold: int = 1,
                 log: Callable[[str], None] = print, rank: int = 0):
        if snapshot and not snapshot_dir:
            raise ValueError("snapshot interval without a snapshot_dir")
        self.mod, self.policy, self.momentum, self.weight_decay = mod, policy, momentum, weight_decay
        self.display, self.snapshot, self.snapshot_dir = int(display), int(snapshot), snapshot_dir
        self.lr_hold = 1 if policy.is_piecewise_constant() else max(1, int(lr_hold))
        self.log, self.rank = log, rank
        self.iter = int(getattr(mod, "steps", 0))       # a resumed module starts at its snapshot's iteration
        self.lr = None
        self.history = []                                # (iteration, loss, lr) of every displayed iteration

    def learning_rate(self, it: int) -> float:
        return self.policy(it - it % self.lr_hold)

    def _apply_hyper(self, it: int) -> None:
        lr = self.learning_rate(it)
        if lr != self.lr:
            self.mod.set_hyper_params(learning_rate=lr, momentum=self.momentum, weight_decay=self.weight_decay)
            self.lr = lr

    def step(self, x, labels):
        """One iteration: the policy's rate for this iteration is in force before the step's update is pushed."""
        self._apply_hyper(self.iter)
        loss = self.mod.step(x, labels)
        self.iter += 1
        if self.snapshot and self.iter % self.snapshot == 0:
            self.mod.save_snapshot(self.snapshot_dir)
        return loss

    def run(self, batches: Iterable, max_iter: int, before_step: Callable[[int], None] | None = None) -> list:
        """Train until iteration max_iter on (images, labels) pairs from `batches` (device tensors, or whatever the
        module's step takes).  before_step(iteration) runs first in every iteration (e.g. a new augmentation).
        Returns the displayed (iteration, loss, lr) records."""
        t0, it0, pending = time.time(), self.iter, None
        for x, labels in batches:
            if self.iter >= max_iter:
                break
            if before_step is not None:
                before_step(self.iter)
            it = self.iter
            loss = self.step(x, labels)
            if pending is not None:
                self._show(*pending, t0, it0)
                pending = None
            if self.display and it % self.display == 0:
                # the module reuses its loss tensor: keep this iteration's value in a copy of its own
                pending = (it, loss.clone() if hasattr(loss, "clone") else loss, self.lr)
        if pending is not None:
            self._show(*pending, t0, it0)
        if self.snapshot_dir and self.iter > it0 and not (self.snapshot and self.iter % self.snapshot == 0):
            self.mod.save_snapshot(self.snapshot_dir)
        return self.history

    def _show(self, it, loss, lr, t0, it0):
        value = float(loss.item()) if hasattr(loss, "item") else float(loss)
        self.history.append((it, value, lr))
        if self.rank == 0:
            rate = (self.iter - it0) / max(1e-9, time.time() - t0)
            self.log(f"iteration {it}  loss {value:.5f}  lr {lr:.6g}  {rate:.1f} it/s")
