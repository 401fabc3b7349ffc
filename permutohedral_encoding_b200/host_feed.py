"""Double-buffered host-to-device feed for batches of positions.

A training loop that reads its points from (pinned) host memory pays the PCIe copy in front of
every step unless the copy of the next batch runs while the current step computes.  The feeder
keeps ``depth`` device buffers and a copy stream: ``submit`` starts the asynchronous copy of a
host batch, ``next`` hands out the oldest submitted batch after making the current stream wait
for its copy, and a buffer is only overwritten once the work that consumed it (everything
enqueued on the consumer's stream up to the following ``next``/``submit``) has been ordered
before the new copy.  The reference has no counterpart; it is a convenience around the drop-in
module, not part of the encoding itself.
"""
from __future__ import annotations

from collections import deque

import torch


class HostPointFeeder:
    def __init__(self, device, depth: int = 2):
        self.device = torch.device(device)
        self.depth = max(2, int(depth))
        self.copy_stream = torch.cuda.Stream(self.device)
        self._buffers = {}          # (shape, dtype) -> list of device buffers
        self._free = {}             # (shape, dtype) -> deque of (buffer, event after last use | None)
        self._ready = deque()       # (buffer, copy-done event, key)
        self._in_use = None         # (buffer, key) handed out by the last next()

    def _take_buffer(self, key, like):
        free = self._free.setdefault(key, deque())
        if not free and len(self._buffers.setdefault(key, [])) < self.depth:
            buf = torch.empty(like.shape, dtype=like.dtype, device=self.device)
            self._buffers[key].append(buf)
            return buf, None
        if not free:
            raise RuntimeError("HostPointFeeder: more batches submitted than buffers; call next() first")
        return free.popleft()

    def _retire(self):
        if self._in_use is not None:
            buf, key = self._in_use
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.device))   # consumer work enqueued so far
            self._free.setdefault(key, deque()).append((buf, ev))
            self._in_use = None

    def submit(self, host_batch: torch.Tensor) -> None:
        """Start copying ``host_batch`` (pinned memory makes the copy asynchronous)."""
        key = (tuple(host_batch.shape), host_batch.dtype)
        buf, last_use = self._take_buffer(key, host_batch)
        with torch.cuda.stream(self.copy_stream):
            if last_use is not None:
                self.copy_stream.wait_event(last_use)
            buf.copy_(host_batch, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.copy_stream)
        self._ready.append((buf, done, key))

    def next(self) -> torch.Tensor:
        """Oldest submitted batch, on the device; the current stream waits for its copy."""
        if not self._ready:
            raise RuntimeError("HostPointFeeder: nothing submitted")
        self._retire()
        buf, done, key = self._ready.popleft()
        torch.cuda.current_stream(self.device).wait_event(done)
        self._in_use = (buf, key)
        return buf
