"""Tracing: NVTX ranges (visible to Nsight tools) and a Chrome-trace (chrome://tracing, Perfetto) JSON of
the host-side schedule.  The reference only keeps wall-clock accumulators per operation
(src/client/stats-tracker.hpp of the reference); the counters live on in GetStats(), this adds a timeline."""
from __future__ import annotations

import contextlib
import json
import os
import threading
import time


class ChromeTrace:
    def __init__(self, process_name: str = "geeps_b200", nvtx: bool = True):
        self.events = []
        self.pid = os.getpid()
        self.process_name = process_name
        self._t0 = time.perf_counter()
        self._nvtx = None
        if nvtx:
            try:
                import torch
                if torch.cuda.is_available():
                    self._nvtx = torch.cuda.nvtx
            except Exception:
                self._nvtx = None

    def _now_us(self) -> float:
        return (time.perf_counter() - self._t0) * 1e6

    @contextlib.contextmanager
    def span(self, name: str, cat: str = "op", **args):
        if self._nvtx is not None:
            self._nvtx.range_push(name)
        t = self._now_us()
        try:
            yield
        finally:
            self.events.append({"name": name, "cat": cat, "ph": "X", "ts": t, "dur": self._now_us() - t,
                                "pid": self.pid, "tid": threading.get_ident() % 100000, "args": args})
            if self._nvtx is not None:
                self._nvtx.range_pop()

    def instant(self, name: str, **args):
        self.events.append({"name": name, "ph": "i", "s": "t", "ts": self._now_us(), "pid": self.pid,
                            "tid": threading.get_ident() % 100000, "args": args})

    def counter(self, name: str, **values):
        self.events.append({"name": name, "ph": "C", "ts": self._now_us(), "pid": self.pid, "args": values})

    def save(self, path: str) -> None:
        meta = [{"name": "process_name", "ph": "M", "pid": self.pid, "args": {"name": self.process_name}}]
        with open(path, "w") as f:
            json.dump({"traceEvents": meta + self.events, "displayTimeUnit": "ms"}, f)


class NullTrace:
    @contextlib.contextmanager
    def span(self, name, cat="op", **args):
        yield

    def instant(self, name, **args):
        pass

    def counter(self, name, **values):
        pass
