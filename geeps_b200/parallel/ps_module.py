"""PSModule: trains a Net through the parameter server.

Every parameterised layer owns one table (its parameters packed row after row, each padded to
whole 128-float rows).  One fwd/bwd is declared to the runtime as a virtual iteration:
    Read(table_l) before layer l's forward ... then, walking the layers backwards,
    PreUpdate(table_l) -> layer l's backward writes its gradients straight into that buffer ->
    PostRead(table_l) -> Update(table_l) ... Clock.
Because a layer's Update is the last write of its table in the clock, the runtime signals that
table's clock immediately and the push of layer l overlaps the backward pass of layers < l
(the per-table clocks of the reference exist for exactly this: src/client/clientlib-viter.cpp:773-797).

Stands in for the solver glue of the reference's (absent) Caffe application.
"""
from __future__ import annotations

import torch

from ..ops import _lib as L
from ..ops import functional as F
from ..ops.layers import BF
from ..utils.config import TRANSPORT_NVLINK, GeePsConfig
from ..utils.trace import NullTrace
from .ps import ROW_FLOATS, GeePs


def _rows_for(numel: int) -> int:
    return (numel + ROW_FLOATS - 1) // ROW_FLOATS


class _Table:
    def __init__(self, table_id, layer):
        self.table_id = table_id
        self.layer = layer
        self.specs = layer.param_specs()
        self.offsets = []
        off = 0
        for sp in self.specs:
            self.offsets.append(off)
            off += _rows_for(sp.numel) * ROW_FLOATS
        self.rows = off // ROW_FLOATS
        self.h_read = self.h_post = self.h_pre = self.h_upd = -1
        self.p16_buf = None

    def views(self, buf: torch.Tensor) -> dict:
        flat = buf.view(-1)
        return {sp.name: flat[o:o + sp.numel].view(sp.shape) for sp, o in zip(self.specs, self.offsets)}


class PSModule:
    def __init__(self, net, in_shape, ps_config: GeePsConfig, rank: int = 0, world: int = 1, device="cuda:0",
                 slack: int = 0, seed: int = 0, keep_init: bool = False, trace=None, manage_activations: bool = False,
                 cache_fraction: float | None = None, use_tape: bool = False, bf16_weights_only: bool = False,
                 use_graph: bool = False, pull_fc: bool = False, uncached=(), resume_from: str | None = None):
        """bf16_weights_only: with the NVLINK transport and the bf16 compute cache, weight rows are published to
        the workers' bf16 caches only (the layers never read weights in fp32; biases, BatchNorm scale / shift and
        the shard's master rows stay fp32).  The fp32 views of weights (`params_fp32`) then keep their initial
        values.
        use_graph: (NVLINK transport, implies use_tape) once a step's native calls are known to repeat, capture
        them in a CUDA graph per (input buffer, label buffer, update-ring phase) and replay the graph: one launch
        per step instead of one per kernel.  The runtime then keeps its clock in a device word (stamps relative
        to it, dropout seeds derived from it), so nothing in the captured launches changes from step to step.
        pull_fc: (NVLINK transport with the bf16 compute cache) the tables of the fully-connected layers become
        uncached tables: the shards do not publish them, and each layer's forward GEMM pulls the weight rows from
        the owning shards while it computes (ops.functional.pull_gemm), leaving a local bf16 copy for the backward
        pass; the bias rows arrive through the table's fp32 tail.
        uncached: names of further layers whose tables are kept uncached (no worker-side copy; every Read fetches
        the whole table from the shards into the staging pool) - the device-side form of a parameter cache that
        does not fit the GPU budget.
        resume_from: directory of table snapshots (`save_snapshot`): the tables (master rows, momentum, clocks) come
        from its latest snapshot instead of the initial values, and training goes on at the snapshot's clock.  The
        world size may differ from the one that wrote it.  Layer-local state (BatchNorm running statistics) is not
        part of a table snapshot."""
        self.net, self.rank, self.world, self.slack = net, rank, world, slack
        self.device = torch.device(device)
        self.trace = trace or NullTrace()
        net.setup(in_shape, self.device)
        self.tables = [_Table(i, l) for i, l in enumerate(net.param_layers())]
        by_layer = {id(t.layer): t for t in self.tables}
        # tables grouped by top-level layer (a Concat module holds several parameterised layers)
        self.groups = []
        for l in net.layers:
            subs = list(l.sublayers()) if hasattr(l, "sublayers") else [l]
            self.groups.append((l, [by_layer[id(s)] for s in subs if id(s) in by_layer]))
        ps_config.num_tables = len(self.tables)
        # Activations managed by the runtime's memory plan: the output of every large top-level layer becomes a
        # worker-local row batch (produced in forward: no fetch / keep; consumed in backward: fetch / discard), so
        # that under a GPU budget the plan decides which of them stay resident and which are swapped to pinned
        # host memory through the staging pool.
        self.managed = {}
        if manage_activations:
            from ..ops.layers import Dropout, Linear
            for i, (l, _) in enumerate(self.groups):
                nbytes = l.out_numel() * 2
                if isinstance(l, (Linear, Dropout)) or nbytes < (1 << 20):
                    continue
                nrows = (nbytes + 511) // 512
                self.managed[i] = {"rows": range(1_000_000 * (i + 1), 1_000_000 * (i + 1) + nrows), "nrows": nrows}
        direct16 = ps_config.transport == TRANSPORT_NVLINK and ps_config.bf16_compute_cache
        # uncached (pull) tables
        nv = ps_config.transport == TRANSPORT_NVLINK and torch.cuda.is_available()
        from ..ops.layers import Linear as _Linear
        for t in self.tables:
            t.pull = t.fused_pull = False
            l = t.layer
            if not nv:
                continue
            if (pull_fc and isinstance(l, _Linear) and direct16 and l.B <= 256 and l.ld % ROW_FLOATS == 0
                    and len(t.specs) == 2):
                t.pull = t.fused_pull = True
                ps_config.table_partition_align[t.table_id] = l.ld // ROW_FLOATS    # whole weight rows per shard
                ps_config.table_fp32_from_row[t.table_id] = t.offsets[1] // ROW_FLOATS  # the bias rows are the tail
            elif getattr(l, "name", None) in uncached:
                t.pull = True
                ps_config.table_fp32_from_row.pop(t.table_id, None)
            if t.pull:
                ps_config.table_pull[t.table_id] = 1
        self.param_rows = sum(t.rows for t in self.tables)
        self.managed_rows = sum(m["nrows"] for m in self.managed.values())
        if cache_fraction is not None:
            ring = slack + 1 if ps_config.transport == TRANSPORT_NVLINK else 1 + int(bool(ps_config.read_my_writes))
            # rows of parameter state that stay in GPU memory: the update ring of every table, plus the worker's copy
            # of every table that is not uncached
            param_state = sum(t.rows * (ring + (0 if t.pull else 1)) for t in self.tables)
            if ps_config.transport == TRANSPORT_NVLINK:
                # peers read and write the parameter cache and the update ring in place, so that state stays
                # device resident; the cap applies to the activation working set, but never goes below what
                # one forward step needs at once (a layer's input and output)
                sizes = [self.managed.get(i, {"nrows": 0})["nrows"] for i in range(len(self.groups))]
                pair = max([a + b for a, b in zip(sizes, sizes[1:])] + sizes + [0])
                budget_rows = param_state + max(int(cache_fraction * self.managed_rows), int(pair * 1.02) + 16)
            else:
                budget_rows = int(cache_fraction * (param_state + self.managed_rows))
            self.budget_rows = budget_rows
            self.working_set_rows = param_state + self.managed_rows
            ps_config.gpu_memory_capacity = budget_rows * 512
            ps_config.mm_warning_level = 0
        self.direct16 = direct16
        if bf16_weights_only and self.direct16:
            for t in self.tables:
                if t.specs and t.specs[0].name == "weight" and not t.pull:
                    ps_config.table_fp32_from_row[t.table_id] = (t.offsets[1] // ROW_FLOATS) if len(t.specs) > 1 else t.rows
        self.ps = GeePs(rank, ps_config)
        # tape replay: record two consecutive steps; if they issued identical native calls (static pointers),
        # later steps walk the tape instead of re-running the Python layer code
        self.use_graph = (use_graph and not manage_activations and ps_config.transport == TRANSPORT_NVLINK
                          and torch.cuda.is_available())
        self.use_tape = (use_tape or self.use_graph) and not manage_activations
        self._graphs, self._graph_failed = {}, False
        self._period = (slack + 1) if (slack + 1) % 2 == 0 else 2 * (slack + 1)
        self._tapes, self._tape_sigs, self._tape_tries = {}, {}, {}     # keyed by (input ptr, label ptr, clock phase)
        self.tape_mismatch = None
        # diagnostics: set to [] to collect CUDA events (step start, forward end, backward end, clock end) per step
        self.phase_events = None
        # diagnostics: set to [] to collect (tag, CUDA event) at every layer boundary; the markers are part of a
        # recorded tape, so they also fire during tape replay
        self.layer_marks = None
        self.initial_params = {} if keep_init else None
        self.captured = None
        self._declare()
        if resume_from is not None:
            if not self.ps.load_snapshot(resume_from):
                raise RuntimeError(f"resume from {resume_from}: {self.ps.last_error_string()}")
        else:
            self._bootstrap(seed)
        self.ps.start_iterations()
        self.steps = max(0, self.ps.clock_value - 1)      # clock 0 is the bootstrap clock
        if self.use_graph:
            ref = self.ps.enable_device_clock()
            for l in net.all_layers():
                if hasattr(l, "step_ref"):
                    l.step_ref = ref

    # one virtual iteration = the exact call sequence of step()
    def _declare(self):
        ps, M = self.ps, self.managed
        n = len(self.groups)
        for i, (_, tabs) in enumerate(self.groups):
            for t in tabs:
                t.h_read = ps.virtual_read(t.table_id, range(t.rows), self.slack)
            if i in M:
                M[i]["f"] = ps.virtual_local_access(M[i]["rows"], False)
            if i - 1 in M:      # the previous output was this layer's input: release (and keep) it now
                M[i - 1]["pf"] = ps.virtual_post_local_access(M[i - 1]["f"], True)
        if n - 1 in M:
            M[n - 1]["pf"] = ps.virtual_post_local_access(M[n - 1]["f"], True)
            M[n - 1]["b"] = ps.virtual_local_access(M[n - 1]["rows"], True)
        for i, (_, tabs) in reversed(list(enumerate(self.groups))):
            if i - 1 in M:
                M[i - 1]["b"] = ps.virtual_local_access(M[i - 1]["rows"], True)
            for t in reversed(tabs):
                t.h_pre = ps.virtual_pre_update(t.table_id, range(t.rows))
            for t in reversed(tabs):
                t.h_post = ps.virtual_post_read(t.h_read)
                t.h_upd = ps.virtual_update(t.h_pre)
            if i in M:
                M[i]["pb"] = ps.virtual_post_local_access(M[i]["b"], False)
        ps.virtual_clock()
        ps.finish_virtual_iteration()

    def _bootstrap(self, seed):
        # the bootstrap update carries the initial values; updates add up over workers, so only rank 0
        # sends non-zero values
        gen = torch.Generator().manual_seed(seed)
        for t in [t for _, tabs in reversed(self.groups) for t in reversed(tabs)]:
            buf = self.ps.pre_update(t.h_pre)
            buf.zero_()
            views = t.views(buf)
            for sp in t.specs:
                init = sp.initial(gen)
                if self.rank == 0:
                    views[sp.name].copy_(init.to(buf.device))
                if self.initial_params is not None:
                    self.initial_params[f"{t.layer.name}.{sp.name}"] = init.clone()
            self.ps.update(t.h_upd)
        self.ps.clock()

    def _bind_read_pull(self, t):
        """Fully-connected layer on an uncached table: no copy of the weights is made here - the layer's forward
        GEMM reads them from the shards (and leaves a bf16 copy in p16 for its backward)."""
        info = self.ps.read_pull(t.h_read)
        l = t.layer
        rpw = l.ld // ROW_FLOATS                       # table rows per weight row
        wrows = t.offsets[1] // ROW_FLOATS
        shards, n_start = [], []
        for s in range(info.num_shards):
            if info.row_count[s] == 0 or info.row_start[s] >= wrows:
                break
            shards.append(int(info.shard_bf16[s]))
            n_start.append(int(info.row_start[s]) // rpw)
        l.pull = (shards, n_start)
        if t.p16_buf is None:
            t.p16_buf = torch.zeros(t.rows, ROW_FLOATS, dtype=BF, device=self.device)
        l.p16 = t.views(t.p16_buf)
        tail = info.tail_tensor.view(-1)
        l.p32 = {"bias": tail[:t.specs[1].numel].view(t.specs[1].shape)}
        if self.captured is not None:
            self.captured[f"{l.name}.bias"] = l.p32["bias"].clone()

    def _bind_read(self, t):
        if t.fused_pull:
            return self._bind_read_pull(t)
        buf = self.ps.read(t.h_read)
        t.layer.p32 = t.views(buf)
        b16 = self.ps.read_bf16(t.h_read) if self.direct16 else None
        if b16 is None:
            if t.p16_buf is None:
                t.p16_buf = torch.empty(t.rows, ROW_FLOATS, dtype=BF, device=self.device)
            F.f32_to_bf16(buf, t.p16_buf)
            b16 = t.p16_buf
        t.layer.p16 = t.views(b16)
        if self.captured is not None:
            # stream-ordered copy of what this clock's Read delivered (tests)
            for name, v in t.layer.p32.items():
                self.captured[f"{t.layer.name}.{name}"] = v.clone()

    def step(self, x: torch.Tensor, labels: torch.Tensor, capture: bool = False) -> torch.Tensor:
        """One clock: forward, backward, push.  Returns the mean loss as a 1-element device tensor.
        capture=True keeps clones of the parameters this clock read in `self.captured`."""
        net, tr = self.net, self.trace
        # the update ring has slack + 1 slots and staged buffers alternate between two copies, so the pointers a
        # step uses repeat with the least common multiple of the two
        key = (x.data_ptr(), labels.data_ptr(), self.steps % self._period)
        graph = self._graphs.get(key) if self.use_graph and not capture else None
        if graph is not None:
            graph.launch()
            self.ps.advance_replayed_clock()
            self.ps.check()
            self.steps += 1
            return net.loss_layer.loss
        tape = self._tapes.get(key) if self.use_tape and not capture else None
        if tape is not None and self.use_graph and not self._graph_failed:
            # capture this step (the host-side bookkeeping of the iteration happens now, during the capture),
            # then run it by launching the graph once
            try:
                graph = L.StepGraph(tape, torch.cuda.current_stream(self.device))
            except RuntimeError as e:
                self._graph_failed = True
                raise RuntimeError(f"step capture failed: {e}") from e
            self._graphs[key] = graph
            graph.launch()
            self.ps.check()
            self.steps += 1
            return net.loss_layer.loss
        if tape is not None:
            for arg, offset in tape.dropouts:      # the only arguments that change from step to step
                arg.value = offset + self.steps
            tape.replay()
            self.ps.check()
            self.steps += 1
            for l in tape.stepped_layers:
                l.step += 1
            return net.loss_layer.loss
        recording = (self.use_tape and not capture and self.steps >= 2 and self._tape_tries.get(key, 0) < 4
                     and (key in self._tape_tries or len(self._tape_tries) < 24))
        if recording:
            L.start_recording()
        self.captured = {} if capture else None
        ev = self.phase_events
        if ev is not None:
            ev.append([torch.cuda.Event(enable_timing=True) for _ in range(4)])
            ev[-1][0].record()
        self._mark("start")
        with tr.span("input", "fwd"):
            h = net.input_layer.forward(x)
        self._mark("f:input")
        M, n = self.managed, len(self.groups)

        def local(handle):
            return self.ps.local_access(handle).view(BF).view(-1)

        for i, (l, tabs) in enumerate(self.groups):
            name = getattr(l, "name", type(l).__name__)
            if tabs:
                with tr.span(f"read:{name}", "ps"):
                    for t in tabs:
                        self._bind_read(t)
            if i in M:
                l.set_output(local(M[i]["f"]))
            with tr.span(f"fwd:{name}", "fwd"):
                h = l.forward(h)
            self._mark("f:" + name)
            if i - 1 in M:
                self.ps.post_local_access(M[i - 1]["pf"])
        if n - 1 in M:
            self.ps.post_local_access(M[n - 1]["pf"])
            held = local(M[n - 1]["b"])
            self.groups[n - 1][0].set_output(held)
        with tr.span("loss", "fwd"):
            loss = net.loss_layer.forward(h, labels)
            g = net.loss_layer.backward()
        self._mark("loss")
        if ev is not None:
            ev[-1][1].record()
        for i, (l, tabs) in reversed(list(enumerate(self.groups))):
            name = getattr(l, "name", type(l).__name__)
            if i - 1 in M:
                # this layer's input was evicted after forward: fetch it back; it is also the previous
                # layer's output, which that layer's backward (ReLU / BN / LRN) reads
                buf = local(M[i - 1]["b"])
                l.set_input(buf[:self.groups[i - 1][0].out_numel()])
                self.groups[i - 1][0].set_output(buf)
            for t in reversed(tabs):
                t.layer.g32 = t.views(self.ps.pre_update(t.h_pre))
            with tr.span(f"bwd:{name}", "bwd"):
                g = l.backward(g)
            if tabs:
                with tr.span(f"update:{name}", "ps"):
                    for t in reversed(tabs):
                        self.ps.post_read(t.h_post)
                        self.ps.update(t.h_upd)
            if i in M:
                self.ps.post_local_access(M[i]["pb"])
            self._mark("b:" + name)
        if ev is not None:
            ev[-1][2].record()
        with tr.span("clock", "ps", clock=self.steps):
            self.ps.clock()
        if ev is not None:
            ev[-1][3].record()
        if recording:
            self._finish_recording(L.stop_recording(), key)
        self.steps += 1
        return loss

    def is_steady(self, x: torch.Tensor, labels: torch.Tensor) -> bool:
        """True when the next step with these buffers replays a captured graph (or, without graphs, a recorded
        tape): the Python layer code and the capture work are behind us."""
        key = (x.data_ptr(), labels.data_ptr(), self.steps % self._period)
        if self.use_graph and not self._graph_failed:
            return key in self._graphs
        return (not self.use_tape) or key in self._tapes

    def save_snapshot(self, directory: str) -> None:
        """Write every table (master rows, momentum, clocks) under directory/snapshot.<clock>; every rank calls it
        before the same step."""
        if not self.ps.save_snapshot(directory):
            raise RuntimeError(f"snapshot to {directory}: {self.ps.last_error_string()}")

    def set_hyper_params(self, learning_rate=None, momentum=None, weight_decay=None) -> None:
        """Change the optimizer's learning rate / momentum / weight decay from the next step on (every rank makes the
        same call before the same step).  Recorded and captured steps carry the old values in their push launches, so
        they are dropped when a value changes: the next few steps run through the layer code and are captured again."""
        old = self.ps.hyper_params()
        self.ps.set_hyper_params(learning_rate, momentum, weight_decay)
        if self.ps.hyper_params() != old:
            if self.use_graph:
                torch.cuda.synchronize(self.device)      # no replay in flight when its graph is destroyed
            self.invalidate_tapes()

    def invalidate_tapes(self) -> None:
        """Forget the recorded steps (call after anything that changes what a step launches: switching layers
        between training and inference mode, rebinding buffers, changing hyper-parameters baked into arguments)."""
        self._tapes.clear()
        self._tape_sigs.clear()
        self._tape_tries.clear()
        for g in self._graphs.values():
            g.close()
        self._graphs.clear()

    def _mark(self, tag):
        if self.layer_marks is None:
            return

        def fire():
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self.layer_marks.append((tag, e))
            return 0
        L.record_call(fire, "mark:" + tag)

    def _finish_recording(self, tape, key):
        """Keep the tape for this (input, label) buffer pair once two recordings of it issued the same native
        calls with the same arguments (dropout seeds aside, which are re-derived from the step count)."""
        import ctypes
        self._tape_tries[key] = self._tape_tries.get(key, 0) + 1
        tape.dropouts = [(a, a.value - self.steps) for fn, args, label in tape.ops if label == "dropout"
                         for a in args if isinstance(a, ctypes.c_ulonglong)]
        tape.stepped_layers = [l for l in self.net.all_layers() if hasattr(l, "seed") and hasattr(l, "step")]
        sig = [row for row in tape.signature() if row[0] != "dropout"]
        prev = self._tape_sigs.get(key)
        if prev == sig:
            self._tapes[key] = tape
        elif prev is not None:
            # keep the first difference for diagnostics (why a step does not repeat)
            i = next((i for i, (a, b) in enumerate(zip(prev, sig)) if a != b), min(len(prev), len(sig)))
            self.tape_mismatch = (key[2], i, prev[i][0] if i < len(prev) else None, sig[i][0] if i < len(sig) else None,
                                  len(prev), len(sig))
        self._tape_sigs[key] = sig

    def params_fp32(self) -> dict:
        """Current parameter values as seen by this worker's last Read (for tests)."""
        out = {}
        for t in self.tables:
            for name, v in t.layer.p32.items():
                out[f"{t.layer.name}.{name}"] = v
        return out

    def close(self):
        torch.cuda.synchronize(self.device) if self.use_graph else None
        for g in self._graphs.values():
            g.close()
        self._graphs.clear()
        self.ps.shutdown()
        self.ps.close()
