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


_NVTX_ON = os.environ.get("B200RT_NVTX", "0") not in ("0", "", "false")


def op_range(name: str):
    """NVTX range around a fused op / layer when B200RT_NVTX=1, else a no-op context: the engine and the decoder wrap
    their steps in these, so a timeline capture shows which launches belong to which layer and phase."""
    return nvtx_range(name) if _NVTX_ON else contextlib.nullcontext()


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


TRACE_KERNELS = {1: "act_quant", 2: "gemm_decode", 3: "gemm_prefill", 4: "rope_kv", 5: "attn_decode", 6: "attn_prefill",
                 7: "peer_allreduce", 8: "gemm_tp", 9: "moe", 10: "argmax"}


class DeviceTrace:
    """Ring of in-kernel ``%globaltimer`` stamps (csrc/kernels/trace.cuh).

    Needs the kernel library built with ``-DB200RT_TRACE`` (``B200RT_KERNELS=trace`` selects it).  ``start()`` hands
    a zeroed device ring to the library, ``records()`` reads it back as dicts ``{t_ns, kernel, phase, sm, cta, grid}``
    sorted by time, ``launches()`` groups them per kernel launch.  Call ``start()`` before the warm-up run that
    precedes a CUDA-graph capture."""

    def __init__(self, capacity: int = 1 << 18, device=None):
        import torch
        from ..ops import _lib
        self._lib = _lib.lib()
        if not self._lib.b200_trace_compiled():
            raise RuntimeError("this kernel library has no time stamps: set B200RT_KERNELS=trace before importing the ops")
        self.capacity = capacity
        self.ring = torch.zeros(2 + 2 * capacity, dtype=torch.int64, device=device or "cuda")

    def start(self) -> None:
        self.ring.zero_()
        import torch
        torch.cuda.synchronize()
        if self._lib.b200_trace_set(self.ring.data_ptr(), self.capacity) != 0:
            raise RuntimeError("b200_trace_set failed")

    def clear(self) -> None:
        self.ring[:2].zero_()

    def stop(self) -> None:
        self._lib.b200_trace_set(None, 0)

    def records(self) -> list[dict]:
        import torch
        torch.cuda.synchronize()
        host = self.ring.cpu()
        n = min(int(host[0].item()) & 0xffffffff, self.capacity)
        out = []
        for i in range(n):
            t, w = int(host[2 + 2 * i].item()), int(host[3 + 2 * i].item()) & 0xffffffffffffffff
            out.append({"t_ns": t & 0xffffffffffffffff, "kernel": (w >> 58) & 63, "phase": (w >> 52) & 63,
                        "sm": (w >> 42) & 1023, "cta": (w >> 21) & 0x1fffff, "grid": w & 0x1fffff})
        out.sort(key=lambda r: r["t_ns"])
        return out

    @staticmethod
    def launches(records: list[dict]) -> list[dict]:
        """Group stamps into launches.  Stamps of one (kernel, grid size, CTA, phase) appear once per launch and in
        launch order, so the n-th such stamp belongs to the n-th launch of that (kernel, grid size)."""
        seen: dict[tuple, int] = {}
        groups: dict[tuple, dict] = {}
        for r in records:
            key = (r["kernel"], r["grid"], r["cta"], r["phase"])
            n = seen.get(key, 0)
            seen[key] = n + 1
            g = groups.setdefault((r["kernel"], r["grid"], n), {"kernel": r["kernel"], "grid": r["grid"], "n": n, "phases": {}})
            g["phases"].setdefault(r["phase"], []).append(r["t_ns"])
        out = list(groups.values())
        for g in out:
            g["t0"] = min(min(v) for v in g["phases"].values())
        out.sort(key=lambda g: g["t0"])
        return out

    @staticmethod
    def summarize(records: list[dict], max_launches: int = 64) -> str:
        """Per launch: for every phase the first / median / last stamp in microseconds relative to the launch's first
        stamp, and the launch's start relative to the first launch."""
        ls = DeviceTrace.launches(records)
        if not ls:
            return "(no stamps)\n"
        base = ls[0]["t0"]
        lines = []
        for g in ls[:max_launches]:
            name = TRACE_KERNELS.get(g["kernel"], str(g["kernel"]))
            lines.append(f"{name} grid {g['grid']} launch #{g['n']} at {(g['t0'] - base) / 1e3:.2f} us")
            for ph in sorted(g["phases"]):
                ts = sorted(g["phases"][ph])
                rel = [(t - g["t0"]) / 1e3 for t in ts]
                lines.append(f"    phase {ph:2d}: n {len(ts):4d}  first {rel[0]:7.2f}  median {rel[len(rel) // 2]:7.2f}  last {rel[-1]:7.2f}")
        return "\n".join(lines) + "\n"
