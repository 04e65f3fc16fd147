"""Host -> device input pipeline: double-buffered asynchronous copies from pinned host memory on a
copy stream, so the transfer of batch i+1 overlaps the training step of batch i, and a pinned
mailbox through which the loss of every step is read back without stalling the launch queue."""
from __future__ import annotations

import torch


class HostFeeder:
    def __init__(self, x_shape, y_shape, device, depth: int = 2, x_dtype=torch.float32, timed: bool = False):
        """x_dtype: dtype of the batches on the host and in the device slots (fp32, or bf16 to halve the
        host-to-device bytes; the input layer converts either to bf16 NHWC).  timed: bracket every copy with
        timing events on the copy stream (copy_times_ms() returns their durations)."""
        self.device = torch.device(device)
        self.copy_stream = torch.cuda.Stream(device=self.device)
        self.timed = timed
        self._timing = []          # (begin, end) event pairs of submitted copies
        self.x = [torch.empty(x_shape, dtype=x_dtype, device=self.device) for _ in range(depth)]
        self.y = [torch.empty(y_shape, dtype=torch.int64, device=self.device) for _ in range(depth)]
        self.ready = [torch.cuda.Event() for _ in range(depth)]
        self.free = [torch.cuda.Event() for _ in range(depth)]
        self.depth, self.put_i, self.get_i = depth, 0, 0
        self.bytes_per_batch = self.x[0].numel() * self.x[0].element_size() + self.y[0].numel() * 8
        for e in self.free:
            e.record(torch.cuda.current_stream(self.device))

    def submit(self, x_host: torch.Tensor, y_host: torch.Tensor) -> None:
        """Start copying one batch (pinned host tensors) into the next device slot."""
        s = self.put_i % self.depth
        self.copy_stream.wait_event(self.free[s])      # the step that used this slot has finished with it
        with torch.cuda.stream(self.copy_stream):
            if self.timed:
                t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0.record(self.copy_stream)
            self.x[s].copy_(x_host, non_blocking=True)
            self.y[s].copy_(y_host, non_blocking=True)
            if self.timed:
                t1.record(self.copy_stream)
                self._timing.append((t0, t1))
            self.ready[s].record(self.copy_stream)
        self.put_i += 1

    def wait_copied(self, slot: int) -> None:
        """Host wait until the last copy submitted into `slot` has finished reading its host tensors (call before
        overwriting a staging buffer that was handed to submit)."""
        self.ready[slot].synchronize()

    def copy_times_ms(self, clear: bool = True) -> list:
        """Device time of every completed copy submitted since the last call (needs timed=True)."""
        out, keep = [], []
        for t0, t1 in self._timing:
            if t1.query():
                out.append(t0.elapsed_time(t1))
            else:
                keep.append((t0, t1))
        if clear:
            self._timing = keep
        return out

    def next(self, stream=None):
        """Device tensors of the oldest submitted batch; `stream` waits for its copy."""
        stream = stream or torch.cuda.current_stream(self.device)
        s = self.get_i % self.depth
        stream.wait_event(self.ready[s])
        self.get_i += 1
        return self.x[s], self.y[s], s

    def release(self, slot: int, stream=None) -> None:
        """Call after the step that consumed `slot` has been enqueued."""
        self.free[slot].record(stream or torch.cuda.current_stream(self.device))


class LossMailbox:
    """Reads a 1-element device tensor back every step through pinned memory; `collect` returns the
    value of the previous step (already complete), so the host never waits for the step just launched."""

    def __init__(self, device, depth: int = 2):
        self.host = [torch.zeros(1).pin_memory() for _ in range(depth)]
        self.done = [torch.cuda.Event() for _ in range(depth)]
        self.depth, self.i = depth, 0
        self.bytes_per_step = 4

    def post(self, loss: torch.Tensor, stream=None) -> None:
        s = self.i % self.depth
        self.host[s].copy_(loss, non_blocking=True)
        self.done[s].record(stream or torch.cuda.current_stream(loss.device))
        self.i += 1

    def collect(self, lag: int = 1):
        if self.i - 1 - lag < 0:
            return None
        s = (self.i - 1 - lag) % self.depth
        self.done[s].synchronize()
        return float(self.host[s][0])

    def last(self) -> float:
        s = (self.i - 1) % self.depth
        self.done[s].synchronize()
        return float(self.host[s][0])
