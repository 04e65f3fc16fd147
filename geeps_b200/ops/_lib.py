"""ctypes view of the native kernel ABI (csrc/kernels/kernels.h, nn_ops.h)."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _native

MAX_RANKS = 8
TABLE_ADDITIVE = 0
TABLE_SGD_MOMENTUM = 1

STATUS_CODES = {0: "ok", 1: "timeout", 2: "bounds", 3: "align"}


class GemmParams(C.Structure):
    _fields_ = [
        ("A", C.c_void_p), ("B", C.c_void_p), ("C", C.c_void_p), ("bias", C.c_void_p),
        ("M", C.c_longlong), ("N", C.c_longlong), ("K", C.c_longlong),
        ("lda", C.c_longlong), ("ldb", C.c_longlong), ("ldc", C.c_longlong),
        ("alpha", C.c_float), ("beta", C.c_float),
        ("a_mn_major", C.c_int), ("b_mn_major", C.c_int), ("out_fp32", C.c_int),
        ("bias_mode", C.c_int), ("relu", C.c_int), ("split_k", C.c_int),
        ("block_n", C.c_int), ("status", C.c_void_p),
    ]


class ConvTcParams(C.Structure):
    _fields_ = [
        ("x", C.c_void_p), ("y", C.c_void_p), ("w", C.c_void_p), ("bias", C.c_void_p), ("status", C.c_void_p),
        ("x_pitch", C.c_longlong), ("y_pitch", C.c_longlong), ("ldw", C.c_longlong),
        ("B", C.c_int), ("H", C.c_int), ("W", C.c_int), ("cg", C.c_int), ("OH", C.c_int), ("OW", C.c_int),
        ("og", C.c_int), ("KH", C.c_int), ("KW", C.c_int), ("pad", C.c_int), ("relu", C.c_int),
        ("mode", C.c_int), ("split_k", C.c_int), ("stride", C.c_int),
    ]


class HaloPlanInfo(C.Structure):
    _fields_ = [
        ("ok", C.c_int), ("routed", C.c_int),
        ("PW", C.c_int), ("R", C.c_int), ("row_tiles", C.c_int), ("m_tiles", C.c_int),
        ("positions", C.c_int), ("ncols2", C.c_int), ("ncols1", C.c_int),
        ("TY", C.c_int), ("passes", C.c_int), ("split", C.c_int), ("n_blocks", C.c_int),
        ("stages_x", C.c_int), ("stages_w", C.c_int), ("x_stage_bytes", C.c_int), ("tmem_cols", C.c_int),
        ("smem_bytes", C.c_longlong), ("util", C.c_double),
    ]


class PushApplyParams(C.Structure):
    _fields_ = [
        ("upd", C.c_void_p * MAX_RANKS), ("cache", C.c_void_p * MAX_RANKS),
        ("cache16", C.c_void_p * MAX_RANKS), ("data_age", C.c_void_p * MAX_RANKS),
        ("master", C.c_void_p), ("momentum", C.c_void_p), ("push_ready", C.c_void_p),
        ("global_clock", C.c_void_p), ("cta_counter", C.c_void_p), ("status", C.c_void_p),
        ("n_owned", C.c_longlong), ("row_start", C.c_longlong), ("row_stride", C.c_longlong),
        ("total_rows", C.c_longlong), ("wait_budget_ns", C.c_ulonglong),
        ("n_ranks", C.c_int), ("rank", C.c_int), ("clock_stamp", C.c_int), ("mode", C.c_int),
        ("publish", C.c_int),
        ("lr", C.c_float), ("momentum_coef", C.c_float), ("weight_decay", C.c_float),
        ("grad_scale", C.c_float), ("fp32_from_row", C.c_longlong), ("clock_ref", C.c_void_p),
        ("master16", C.c_void_p), ("upd_mc", C.c_void_p), ("cache_mc", C.c_void_p), ("cache16_mc", C.c_void_p),
    ]


class PullParams(C.Structure):
    _fields_ = [
        ("master", C.c_void_p * MAX_RANKS), ("global_clock", C.c_void_p * MAX_RANKS),
        ("n_owned", C.c_longlong * MAX_RANKS), ("row_start", C.c_longlong * MAX_RANKS),
        ("row_stride", C.c_longlong * MAX_RANKS),
        ("cache", C.c_void_p), ("cache16", C.c_void_p), ("data_age_local", C.c_void_p),
        ("cta_counter", C.c_void_p), ("status", C.c_void_p),
        ("total_rows", C.c_longlong), ("wait_budget_ns", C.c_ulonglong),
        ("n_ranks", C.c_int), ("rank", C.c_int), ("needed_stamp", C.c_int),
        ("row_from", C.c_longlong), ("row_base", C.c_longlong),
    ]


class PullGemmParams(C.Structure):
    _fields_ = [
        ("X", C.c_void_p), ("Y", C.c_void_p), ("bias", C.c_void_p),
        ("w_shard", C.c_void_p * MAX_RANKS), ("ready", C.c_void_p * MAX_RANKS),
        ("n_start", C.c_longlong * (MAX_RANKS + 1)),
        ("w_local", C.c_void_p), ("status", C.c_void_p),
        ("M", C.c_longlong), ("N", C.c_longlong), ("K", C.c_longlong),
        ("ldx", C.c_longlong), ("ldw", C.c_longlong), ("ldy", C.c_longlong),
        ("wait_budget_ns", C.c_ulonglong),
        ("n_shards", C.c_int), ("needed_stamp", C.c_int), ("relu", C.c_int), ("out_fp32", C.c_int),
        ("block_n", C.c_int),
    ]


class RmwReadParams(C.Structure):
    _fields_ = [
        ("dst", C.c_void_p), ("cache", C.c_void_p), ("ring", C.c_void_p), ("index", C.c_void_p),
        ("data_age", C.c_void_p), ("publish_begin", C.c_void_p), ("status", C.c_void_p),
        ("num_rows", C.c_longlong), ("num_vals_limit", C.c_longlong), ("dst_rows", C.c_longlong),
        ("total_rows", C.c_longlong), ("wait_budget_ns", C.c_ulonglong),
        ("n_ranks", C.c_int), ("partition_kind", C.c_int), ("ring_slots", C.c_int), ("clock", C.c_int),
        ("additive_below_clock", C.c_int), ("alpha", C.c_float), ("clock_ref", C.c_void_p),
        ("partition_per", C.c_longlong),
    ]


class FlagList(C.Structure):
    _fields_ = [("ptr", C.c_void_p * MAX_RANKS), ("n", C.c_int)]


class ConvGeom(C.Structure):
    _fields_ = [(n, C.c_int) for n in
                ("B", "H", "W", "C", "c0", "Cg", "KH", "KW", "stride", "pad", "OH", "OW", "ldcol")]


class PoolGeom(C.Structure):
    _fields_ = [(n, C.c_int) for n in
                ("B", "H", "W", "C", "K", "stride", "pad", "OH", "OW", "ldx", "ldy")]


class U8Transform(C.Structure):
    """Mirror of GeepsU8Transform (csrc/kernels/nn_ops.h)."""
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("aug", C.c_void_p)] + [(n, C.c_int) for n in
                ("B", "C", "Hin", "Win", "H", "W", "S", "Hs", "Ws", "Cpad")] + [("mean", C.c_float * 4), ("scale", C.c_float)]


_lib = None
_launches = 0


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = _native.load()
    return _lib


def require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("geeps_b200 kernels need a CUDA device (sm_100a); none is visible")


def stream_ptr(stream=None) -> C.c_void_p:
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def ptr(t) -> C.c_void_p:
    return C.c_void_p(0 if t is None else t.data_ptr())


def check(err: int, what: str) -> None:
    global _launches
    _launches += 1
    if err != 0:
        raise RuntimeError(f"{what}: CUDA launch error {err}")


class Tape:
    """A recorded sequence of native calls (kernel launches and parameter-server calls) with their argument
    objects.  When every pointer a training step uses is static - zero-copy parameter access, slack 0, no
    staged buffers - the step can be replayed by walking the tape, which skips all the Python work between
    launches (argument marshalling, shape logic, view creation)."""

    def __init__(self):
        self.ops = []          # (cfunc, args tuple, label)

    def signature(self):
        sig = []
        for fn, args, label in self.ops:
            row = [label]
            for a in args:
                obj = getattr(a, "_obj", None)       # byref(struct)
                if obj is not None:
                    row.append(bytes(obj))
                elif hasattr(a, "value"):
                    row.append(a.value)
                else:
                    row.append(a)
            sig.append(tuple(row))
        return sig

    def replay(self) -> None:
        global _launches
        for fn, args, label in self.ops:
            err = fn(*args)
            if err:
                raise RuntimeError(f"{label}: native call failed with {err} during tape replay")
        _launches += self.kernel_launches

    @property
    def kernel_launches(self) -> int:
        return sum(1 for _, _, label in self.ops if not label.startswith("ps:"))


class StepGraph:
    """A CUDA graph of one training step: everything a tape enqueues on `stream` (and on the streams that join it
    through events) captured once, then replayed with a single launch."""

    def __init__(self, tape: "Tape", stream):
        self.stream = stream
        self.kernel_launches = tape.kernel_launches
        self.nodes = 0
        self._exec = C.c_void_p()
        l = lib()
        err = l.geeps_graph_begin(C.c_void_p(stream.cuda_stream))
        if err:
            raise RuntimeError(f"cudaStreamBeginCapture failed with {err}")
        global _launches
        counted = _launches
        try:
            tape.replay()            # enqueues into the capture: nothing runs yet
        finally:
            _launches = counted      # the kernels are counted when the graph is launched
            n = C.c_longlong(0)
            err = l.geeps_graph_end(C.c_void_p(stream.cuda_stream), C.byref(self._exec), C.byref(n))
        if err or not self._exec.value:
            raise RuntimeError(f"capturing the step failed with {err}")
        self.nodes = n.value

    def launch(self) -> None:
        global _launches
        err = lib().geeps_graph_launch(self._exec, C.c_void_p(self.stream.cuda_stream))
        if err:
            raise RuntimeError(f"cudaGraphLaunch failed with {err}")
        _launches += self.kernel_launches

    def close(self) -> None:
        if self._exec.value:
            lib().geeps_graph_destroy(self._exec)
            self._exec = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_tape = None


def start_recording() -> Tape:
    global _tape
    _tape = Tape()
    return _tape


def stop_recording() -> Tape:
    global _tape
    t, _tape = _tape, None
    return t


def launch(fn, label: str, *args) -> None:
    """Call a native launcher; record it when a tape is being recorded."""
    if _tape is not None:
        _tape.ops.append((fn, args, label))
    check(fn(*args), label)


def record_call(fn, label: str, *args):
    """Call (and record) a native function whose return value is not an error code."""
    if _tape is not None:
        _tape.ops.append((_ignore_result(fn), args, "ps:" + label))
    return fn(*args)


def _ignore_result(fn):
    def call(*a):
        fn(*a)
        return 0
    return call


def launch_count() -> int:
    """Number of native kernel-launching calls made by this process so far."""
    return _launches


def new_status(device) -> torch.Tensor:
    return torch.zeros(4, dtype=torch.int32, device=device)


def read_status(status: torch.Tensor) -> dict:
    s = status.tolist()
    return {"code": s[0], "name": STATUS_CODES.get(s[0], "?"), "kernel": s[1], "detail": s[2], "seen": s[3]}
