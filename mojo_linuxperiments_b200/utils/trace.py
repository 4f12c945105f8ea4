"""Timing, tracing and metrics helpers.

The reference only prints (numa/numa.mojo:166-176, test_linux_threading.mojo:11-16).  This module gives the runtime
  * ``cuda_time``  device time of a callable with CUDA events on the launching stream (warm-up, synchronise both sides),
  * ``nvtx_range`` named ranges that show up in Nsight captures,
  * ``MetricsLog`` JSON-lines records (config, world size, tokens/s, arena high-water marks, ...).
"""
from __future__ import annotations

import contextlib
import json
import os
import time


def cuda_time(fn, iters: int = 10, warmup: int = 3) -> float:
    """Mean seconds per call of ``fn`` on the current CUDA stream."""
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / iters


@contextlib.contextmanager
def nvtx_range(name: str):
    try:
        import torch
        torch.cuda.nvtx.range_push(name)
        pushed = True
    except Exception:
        pushed = False
    try:
        yield
    finally:
        if pushed:
            import torch
            torch.cuda.nvtx.range_pop()


class MetricsLog:
    """Append-only JSON-lines file; one dict per record plus a wall-clock stamp."""

    def __init__(self, path: str):
        self.path = path
        d = os.path.dirname(path)
        if d:
            os.makedirs(d, exist_ok=True)

    def write(self, **record) -> dict:
        record = {"t": time.time(), **record}
        with open(self.path, "a") as f:
            f.write(json.dumps(record) + "\n")
        return record

    def read(self) -> list[dict]:
        if not os.path.exists(self.path):
            return []
        with open(self.path) as f:
            return [json.loads(l) for l in f if l.strip()]
