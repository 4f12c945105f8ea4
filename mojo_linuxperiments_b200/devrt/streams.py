"""A pool of CUDA streams on one GPU with the reference's pool vocabulary (threading/linux_threading.mojo:103-129):
``launch`` puts work on a free stream, ``wait_all`` joins everything, ``wait_any`` returns the index of a stream
whose work finished.  Work items are callables that enqueue kernels (they run on the calling host thread; the GPU
work is asynchronous), a slot is busy until its completion event has fired."""
from __future__ import annotations

import time

import torch


class StreamPool:
    def __init__(self, capacity: int, device=None):
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.streams = [torch.cuda.Stream(device=self.device) for _ in range(capacity)]
        self.events: list[torch.cuda.Event | None] = [None] * capacity

    def __len__(self): return len(self.streams)
    def __iter__(self): return iter(range(len(self.streams)))

    def _busy(self, i: int) -> bool:
        e = self.events[i]
        return e is not None and not e.query()

    def running(self) -> int:
        return sum(1 for i in self if self._busy(i))

    def launch(self, fn, *args) -> int:
        """Run ``fn(*args)`` with a free stream current; returns the slot index, or -1 when every slot is busy."""
        for i in self:
            if not self._busy(i):
                with torch.cuda.stream(self.streams[i]):
                    fn(*args)
                    ev = torch.cuda.Event()
                    ev.record(self.streams[i])
                self.events[i] = ev
                return i
        return -1

    def wait_all(self, timeout_s: float | None = None) -> int:
        """0 when everything finished, -110 (ETIMEDOUT) otherwise."""
        t0 = time.monotonic()
        for i in self:
            e = self.events[i]
            if e is None:
                continue
            if timeout_s is None:
                e.synchronize()
            else:
                while not e.query():
                    if time.monotonic() - t0 > timeout_s:
                        return -110
                    time.sleep(0.0002)
        return 0

    def wait_any(self, timeout_s: float | None = None) -> int:
        """Index of a slot whose work has finished (it becomes free), -1 when nothing is in flight, -2 on timeout."""
        pending = [i for i in self if self.events[i] is not None]
        if not pending:
            return -1
        t0 = time.monotonic()
        while True:
            for i in pending:
                if self.events[i].query():
                    self.events[i] = None
                    return i
            if timeout_s is not None and time.monotonic() - t0 > timeout_s:
                return -2
            time.sleep(0.0002)
