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


def kernel_timeline(fn, iters: int = 3, warmup: int = 2) -> list[list[tuple[str, float, float]]]:
    """Device-side timeline of the kernels ``fn`` launches (also from inside a CUDA-graph replay).

    Returns one list per iteration of ``(kernel name, start_us relative to the iteration's first kernel, duration_us)``
    ordered by start time.  The stamps come from the CUPTI activity records that ``torch.profiler`` collects, so
    kernels that overlap (programmatic dependent launch, several streams) show up with their true overlap.  Use it
    to see where a step spends its time; numbers for a report are taken with ``cuda_time``, never under a profiler.
    """
    import torch
    from torch.profiler import ProfilerActivity, profile
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    per_iter: list[list[tuple[str, float, float]]] = []
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        for _ in range(iters):
            fn()
            torch.cuda.synchronize()
            prof.step() if hasattr(prof, "step") else None
    evs = []
    for e in prof.events():
        if getattr(e, "device_type", None) is not None and "cuda" in str(e.device_type).lower():
            if "memcpy" in e.name.lower() or "memset" in e.name.lower():
                continue
            evs.append((e.name, float(e.time_range.start), float(e.time_range.end - e.time_range.start)))
    evs.sort(key=lambda t: t[1])
    if not evs:
        return per_iter
    n = len(evs) // iters
    for i in range(iters):
        chunk = evs[i * n:(i + 1) * n] if i < iters - 1 else evs[i * n:]
        t0 = chunk[0][1]
        per_iter.append([(name, start - t0, dur) for name, start, dur in chunk])
    return per_iter


def summarize_timeline(per_iter: list[list[tuple[str, float, float]]]) -> str:
    """Text table of a ``kernel_timeline``: per position in the step the kernel, its mean start, duration and the gap
    between the previous kernel's end and this kernel's start (negative: they overlapped), then totals per kernel."""
    if not per_iter:
        return "(no kernels recorded)\n"
    n = min(len(it) for it in per_iter)
    lines = [f"{'#':>4} {'start_us':>10} {'dur_us':>8} {'gap_us':>8}  kernel"]
    by_name: dict[str, list[float]] = {}
    for k in range(n):
        name = per_iter[-1][k][0]
        start = sum(it[k][1] for it in per_iter) / len(per_iter)
        dur = sum(it[k][2] for it in per_iter) / len(per_iter)
        gap = 0.0
        if k:
            gap = sum(it[k][1] - (it[k - 1][1] + it[k - 1][2]) for it in per_iter) / len(per_iter)
        short = name.split("(")[0][-70:]
        lines.append(f"{k:>4} {start:>10.2f} {dur:>8.2f} {gap:>8.2f}  {short}")
        by_name.setdefault(short, []).append(dur)
    end = sum(it[n - 1][1] + it[n - 1][2] for it in per_iter) / len(per_iter)
    lines.append(f"step span: {end:.1f} us over {n} kernels")
    lines.append("")
    lines.append(f"{'count':>6} {'total_us':>10} {'avg_us':>8}  kernel")
    for name, d in sorted(by_name.items(), key=lambda kv: -sum(kv[1])):
        lines.append(f"{len(d):>6} {sum(d):>10.1f} {sum(d) / len(d):>8.2f}  {name}")
    return "\n".join(lines) + "\n"
