"""Python binding of the native parameter-server runtime (the C++ GeePs class).

Method names follow the C++ API (include/geeps.hpp) in snake_case.  Buffers handed out by
read / pre_update / local_access are returned as tensors that alias the runtime's memory:
device memory on a CUDA worker, host memory on a CPU worker.
"""
from __future__ import annotations

import ctypes as C
import json

import numpy as np
import torch

from .. import _native
from ..ops import _lib as _L
from ..utils.config import DEVICE_CUDA, GeePsConfig

ROW_FLOATS = 128

ERRORS = {0: "none", 1: "plan", 2: "order", 3: "host_timeout", 4: "device_timeout", 5: "peer_lost",
          6: "protocol", 7: "transport", 8: "memory", 9: "cuda", 10: "snapshot"}


class GeePsError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"geeps error {code} ({ERRORS.get(code, '?')}): {text}")
        self.code = code


class _CudaView:
    """Minimal __cuda_array_interface__ carrier so torch can alias runtime-owned device memory."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 3, "strides": None}


def _lib():
    lib = _native.load()
    if not getattr(lib, "_geeps_ps_typed", False):
        lib.geeps_config_new.restype = C.c_void_p
        lib.geeps_new.restype = C.c_void_p
        lib.geeps_new.argtypes = [C.c_uint, C.c_void_p]
        lib.geeps_read_bf16.restype = C.c_void_p
        lib.geeps_set_hyper_params.argtypes = [C.c_void_p, C.c_float, C.c_float, C.c_float]
        lib.geeps_set_hyper_params.restype = None
        lib.geeps_get_hyper_params.argtypes = [C.c_void_p, C.POINTER(C.c_float)]
        lib.geeps_get_hyper_params.restype = None
        lib.geeps_planner_new.restype = C.c_void_p
        lib.geeps_mtcache_new.restype = C.c_void_p
        lib.geeps_ringcache_new.restype = C.c_void_p
        for name in ("geeps_mtcache_get", "geeps_mtcache_used", "geeps_ringcache_get"):
            getattr(lib, name).restype = C.c_longlong
        lib._geeps_ps_typed = True
    return lib


def _rows(rows):
    arr = (C.c_longlong * len(rows))(*[int(r) for r in rows])
    return arr, len(rows)


class PullInfo(C.Structure):
    """Mirror of GeePs::PullInfo (include/geeps.hpp)."""
    _fields_ = [("shard_bf16", C.c_void_p * 8), ("shard_fp32", C.c_void_p * 8),
                ("row_start", C.c_longlong * 8), ("row_count", C.c_longlong * 8), ("num_shards", C.c_int),
                ("tail", C.c_void_p), ("tail_from_row", C.c_longlong), ("tail_rows", C.c_longlong)]


class GeePs:
    def __init__(self, process_id: int, config: GeePsConfig):
        self._l = _lib()
        self.config = config
        self.process_id = process_id
        cfg = C.c_void_p(self._l.geeps_config_new())
        for i, h in enumerate(config.host_list):
            port = config.port_list[i] if i < len(config.port_list) else 0
            self._l.geeps_config_add_host(cfg, h.encode(), int(port))
        for k in GeePsConfig._NUMERIC:
            self._l.geeps_config_set(cfg, k.encode(), C.c_double(float(getattr(config, k))))
        for k in GeePsConfig._STRING:
            self._l.geeps_config_set_str(cfg, k.encode(), getattr(config, k).encode())
        for t, m in config.table_modes.items():
            self._l.geeps_config_set_table_mode(cfg, int(t), int(m))
        for t, r in config.table_fp32_from_row.items():
            self._l.geeps_config_set_table_fp32_from_row(cfg, int(t), C.c_longlong(int(r)))
        for t, v in config.table_pull.items():
            self._l.geeps_config_set_table_pull(cfg, int(t), int(v))
        for t, v in config.table_partition_align.items():
            self._l.geeps_config_set_table_partition_align(cfg, int(t), C.c_longlong(int(v)))
        self._g = C.c_void_p(self._l.geeps_new(process_id, cfg))
        self._l.geeps_config_delete(cfg)
        self._ops = {}      # handle -> (kind, num_rows)
        self._views = {}    # (ptr, rows, dtype) -> tensor aliasing runtime memory
        self._cuda = config.device == DEVICE_CUDA and torch.cuda.is_available()
        self.check()

    # ---- errors / info ----
    def last_error(self) -> int:
        return self._l.geeps_last_error(self._g)

    def _string(self, fn) -> str:
        # the text may differ from one call to the next (counters grow): never size the buffer from an earlier call
        cap = 1 << 16
        while True:
            buf = C.create_string_buffer(cap)
            need = fn(self._g, buf, cap)
            if need <= cap:
                return buf.value.decode()
            cap = need + 4096

    def last_error_string(self) -> str:
        return self._string(self._l.geeps_last_error_string)

    def check(self) -> None:
        code = self.last_error()
        if code:
            raise GeePsError(code, self.last_error_string())

    def get_stats(self) -> dict:
        return json.loads(self._string(self._l.geeps_get_stats))

    def locate_row(self, table: int, row: int, metadata_server: int = 0, timeout_ms: int = 5000) -> int:
        """Ask shard `metadata_server` where its placement policy (config pp_policy: 1 hash, 2 first toucher,
        3 most frequent accessor with load balance) puts (table, row); -1 if no answer in time.  The data path
        uses the static partitioner; this is the reference's MetadataServer service
        (src/server/metadata-server.cpp:119-170)."""
        return int(self._l.geeps_locate_row(self._g, C.c_longlong(table), C.c_longlong(row), int(metadata_server),
                                            int(timeout_ms)))

    def report_access(self, table: int, row: int, nread: int = 1, nwrite: int = 0, metadata_server: int = 0) -> None:
        """Feed the placement service with this worker's access counts for (table, row)."""
        self._l.geeps_report_access(self._g, int(metadata_server), C.c_longlong(table), C.c_longlong(row), int(nread),
                                    int(nwrite))

    def plan(self) -> dict:
        return json.loads(self._string(self._l.geeps_plan_json))

    @property
    def clock_value(self) -> int:
        return self._l.geeps_current_clock(self._g)

    def set_hyper_params(self, learning_rate=None, momentum=None, weight_decay=None) -> None:
        """Learning rate, momentum and weight decay of the shard-side optimizer for the updates of the iteration in
        progress and all later ones (None keeps a value).  Every worker makes the same call in the same iteration.
        Iterations captured in a CUDA graph keep the values of the time of capture."""
        lr, mom, wd = self.hyper_params()
        self._l.geeps_set_hyper_params(self._g, lr if learning_rate is None else learning_rate,
                                       mom if momentum is None else momentum, wd if weight_decay is None else weight_decay)

    def hyper_params(self):
        """(learning_rate, momentum, weight_decay) in force for the updates of the iteration in progress."""
        out = (C.c_float * 3)()
        self._l.geeps_get_hyper_params(self._g, out)
        return float(out[0]), float(out[1]), float(out[2])

    # ---- virtual iteration ----
    def virtual_read(self, table: int, rows, slack: int = 0) -> int:
        a, n = _rows(rows)
        h = self._l.geeps_virtual_read(self._g, C.c_longlong(table), a, n, slack)
        self._ops[h] = ("read", n)
        return h

    def virtual_post_read(self, prestep: int) -> int:
        return self._l.geeps_virtual_post_read(self._g, prestep)

    def virtual_pre_update(self, table: int, rows) -> int:
        a, n = _rows(rows)
        h = self._l.geeps_virtual_pre_update(self._g, C.c_longlong(table), a, n)
        self._ops[h] = ("pre_update", n)
        return h

    def virtual_update(self, prestep: int) -> int:
        return self._l.geeps_virtual_update(self._g, prestep)

    def virtual_local_access(self, rows, fetch: bool) -> int:
        a, n = _rows(rows)
        h = self._l.geeps_virtual_local_access(self._g, a, n, int(fetch))
        self._ops[h] = ("local", n)
        return h

    def virtual_post_local_access(self, prestep: int, keep: bool) -> int:
        return self._l.geeps_virtual_post_local_access(self._g, prestep, int(keep))

    def virtual_clock(self) -> int:
        return self._l.geeps_virtual_clock(self._g)

    def finish_virtual_iteration(self) -> None:
        self._l.geeps_finish_virtual_iteration(self._g)
        self.check()

    def start_iterations(self) -> None:
        self._l.geeps_start_iterations(self._g)
        self.check()

    # ---- real access ----
    def _stream(self, stream):
        if not self._cuda:
            return C.c_void_p(0)
        s = stream if stream is not None else torch.cuda.current_stream()
        # handle 0 means "the runtime's own stream" to the C API; CUDA's legacy default stream is 0x1
        return C.c_void_p(s.cuda_stream or 1)

    def _wrap(self, ptr: int, nrows: int, dtype=torch.float32) -> torch.Tensor:
        if not ptr:
            self.check()
            raise GeePsError(-1, "runtime returned no buffer")
        if self._cuda:
            key = (ptr, nrows, dtype)
            t = self._views.get(key)
            if t is None:
                ts = "<f4" if dtype == torch.float32 else "<u2"
                t = torch.as_tensor(_CudaView(ptr, (nrows, ROW_FLOATS), ts), device="cuda")
                t = t.view(torch.bfloat16) if dtype == torch.bfloat16 else t
                self._views[key] = t
            return t
        buf = (C.c_float * (nrows * ROW_FLOATS)).from_address(ptr)
        return torch.from_numpy(np.frombuffer(buf, dtype=np.float32).reshape(nrows, ROW_FLOATS))

    def read(self, handle: int, stream=None, asynchronous: bool = True) -> torch.Tensor:
        p = C.c_void_p()
        ok = _L.record_call(self._l.geeps_read, "read", self._g, handle, C.byref(p), self._stream(stream), int(asynchronous))
        if not ok:
            self.check()
        return self._wrap(p.value, self._ops[handle][1])

    def read_pull(self, handle: int, stream=None) -> "PullInfo":
        """Stands in for read() on an uncached (pull) table: orders the stream after the table's freshness
        condition, fetches the fp32 tail (rows from table_fp32_from_row on) into a private buffer and returns where
        the shards keep the leading rows, for a kernel that reads them in place (ops.functional.pull_gemm)."""
        info = PullInfo()
        ok = _L.record_call(self._l.geeps_read_pull, "read_pull", self._g, handle, C.byref(info), self._stream(stream))
        if not ok:
            self.check()
        info.tail_tensor = self._wrap(info.tail, info.tail_rows) if info.tail else None
        return info

    def read_bf16(self, handle: int):
        p = self._l.geeps_read_bf16(self._g, handle)
        return self._wrap(p, self._ops[handle][1], torch.bfloat16) if p else None

    def post_read(self, handle: int, stream=None) -> None:
        _L.record_call(self._l.geeps_post_read, "post_read", self._g, handle, self._stream(stream))

    def pre_update(self, handle: int, stream=None) -> torch.Tensor:
        p = C.c_void_p()
        _L.record_call(self._l.geeps_pre_update, "pre_update", self._g, handle, C.byref(p), self._stream(stream))
        return self._wrap(p.value, self._ops[handle][1])

    def update(self, handle: int, stream=None, asynchronous: bool = True) -> None:
        _L.record_call(self._l.geeps_update, "update", self._g, handle, self._stream(stream), int(asynchronous))

    def local_access(self, handle: int, stream=None) -> torch.Tensor:
        p = C.c_void_p()
        self._l.geeps_local_access(self._g, handle, C.byref(p), self._stream(stream))
        return self._wrap(p.value, self._ops[handle][1])

    def post_local_access(self, handle: int, stream=None) -> None:
        self._l.geeps_post_local_access(self._g, handle, self._stream(stream))

    def clock(self) -> None:
        _L.record_call(self._l.geeps_clock, "clock", self._g)
        self.check()

    # ---- device-resident clock: iterations replayed from a CUDA graph ----
    def enable_device_clock(self) -> int:
        """Keep the clock in a device word (NVLINK transport) so that one iteration's launches can be captured in a
        CUDA graph; returns the address of the word."""
        if not self._l.geeps_enable_device_clock(self._g):
            self.check()
            raise GeePsError(-1, "device clock not available")
        self._l.geeps_device_clock_ptr.restype = C.c_void_p
        return int(self._l.geeps_device_clock_ptr(self._g))

    def advance_replayed_clock(self) -> None:
        """Host-side bookkeeping of one iteration whose launches were replayed from a captured graph."""
        self._l.geeps_advance_replayed_clock(self._g)

    # ---- snapshots / lifecycle / test hooks ----
    def save_snapshot(self, directory: str) -> bool:
        return bool(self._l.geeps_save_snapshot(self._g, directory.encode()))

    def load_snapshot(self, directory: str) -> bool:
        return bool(self._l.geeps_load_snapshot(self._g, directory.encode()))

    def inject(self, what: int, value: int) -> None:
        self._l.geeps_inject(self._g, what, value)

    def shutdown(self) -> None:
        if self._g:
            self._l.geeps_shutdown(self._g)

    def close(self) -> None:
        if self._g:
            self._l.geeps_delete(self._g)
            self._g = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
