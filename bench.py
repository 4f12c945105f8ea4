"""Headline benchmark: greedy decode throughput of the Llama-3-8B-shaped W8A8 decoder, tensor-parallel over N GPUs.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torch.distributed.run, one rank per GPU)
    python bench.py --impl reference ...                     (prints why the Mojo reference cannot run here)
    python bench.py --impl torch_baseline ...                (PyTorch + cuBLAS int8 + NCCL build of the same model)

One step = one decode step of the whole batch (32 sequences, 1,024-token prompts already in the paged KV cache), so
the value is tokens/s over all N GPUs.  The timed region is exactly K steps between barrier + synchronize, timed with
CUDA events on the launching stream, max over ranks.  Every step streams this rank's int8 weights (8 GB at N=1, 1 GB at
N=8: larger than the 126 MB L2) from HBM.  Also reported: decode at batch 1, p50 time-to-first-token of a
1,024-token prompt, and the same decode metric end to end through ``Engine.step_from_host`` (pinned host ids in,
sampled ids out, every step).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

METRIC = "decode tokens/sec (bs 32; also bs 1 and p50 TTFT @1024-tok prompt in extra), max over ranks"
MODEL = "llama3-8b-shaped W8A8 (Hadamard int8 weights, bf16 activations and KV)"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch_baseline"])
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt-len", type=int, default=1024)
    ap.add_argument("--model", default="llama3-8b")
    ap.add_argument("--skip-extra", action="store_true", help="only the headline number (no bs-1 / TTFT / e2e runs)")
    ap.add_argument("--layers", type=int, default=0, help="smoke runs only: override the layer count (the line is then marked invalid)")
    return ap.parse_args()


class ClockSampler:
    """Clock / throttle-reason samples of one GPU while the timed region runs (read-only queries).

    ``nvidia-smi -lms 50`` is started before the warm-up steps so that it is already printing when the timed region
    begins; every line carries its own timestamp and only lines between ``mark_start()`` and ``stop()`` count.  A
    second, in-process sampler reads the same values through NVML every 10 ms during the region, which still yields
    samples when the region is shorter than nvidia-smi's period.  If neither saw the region (a very short run), the
    samples taken during the warm-up steps are reported and marked as such."""

    FIELDS = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        import datetime
        import threading
        self._dt = datetime
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None
        self.t_start = None
        self.nvml_samples = []          # (in_region, sm_mhz, max_mhz, reasons bitmask)
        self._stop = threading.Event()
        self._in_region = False
        uuid = None
        try:
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:
            pass
        try:
            self.proc = subprocess.Popen(["nvidia-smi", *(["-i", uuid] if uuid else []), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=self.file, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None
        self._thread = threading.Thread(target=self._nvml_loop, args=(uuid,), daemon=True)
        self._thread.start()

    def _nvml_loop(self, uuid):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if isinstance(uuid, str) else uuid)
            mx = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            while not self._stop.is_set():
                sm = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                try:
                    why = int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                except Exception:
                    why = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                self.nvml_samples.append((self._in_region, float(sm), float(mx), why))
                self._stop.wait(0.01)
        except Exception:
            return

    def mark_start(self):
        self.t_start = self._dt.datetime.now()
        self._in_region = True

    def stop(self) -> dict:
        t_end = self._dt.datetime.now()
        self._in_region = False
        self._stop.set()
        self._thread.join(timeout=2)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        inside, before = [], []
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.file.flush()
            self.file.seek(0)
            for line in self.file.read().splitlines():
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 10:
                    continue
                try:
                    ts = self._dt.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
                    rec = (float(parts[2]), float(parts[3]),
                           {n for n, v in zip(names, parts[6:10]) if v.lower().startswith("active")})
                except ValueError:
                    continue
                (inside if (self.t_start is not None and self.t_start <= ts <= t_end) else before).append(rec)
        try:
            os.unlink(self.file.name)
        except OSError:
            pass
        # NVML reason bits: 0x4 sw_power_cap, 0x8 hw_slowdown, 0x20 sw_thermal, 0x40 hw_thermal
        bits = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
        for in_region, sm, mx, why in self.nvml_samples:
            rec = (sm, mx, {n for b, n in bits.items() if why & b})
            (inside if in_region else before).append(rec)
        window = "timed region"
        use = inside
        if not use:
            use, window = before[-20:], "warm-up steps just before the timed region (the region was shorter than a sample period)"
        if not use:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": ["no clock samples available"]}
        sm = sorted(r[0] for r in use)
        reasons = set().union(*(r[2] for r in use))
        busy = sm[len(sm) // 2:]
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(r[1] for r in use), "samples": len(use),
                "window": window, "reasons": sorted(reasons)}


def dist_setup(n: int):
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world != n:
        raise SystemExit(f"--gpus {n} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {n}")
    return rank, local, world


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def timed_steps(step_fn, k: int, world: int) -> float:
    """Seconds for exactly k calls of step_fn: barrier + sync, event, k steps, event, barrier + sync; max over ranks."""
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(k):
        step_fn()
    e1.record()
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1) * 1e-3, world)


def make_engine(args, world, rank, batch):
    from mojo_linuxperiments_b200.models import config as C
    from mojo_linuxperiments_b200.parallel.comm import Comm
    cfg = C.PRESETS[args.model]()
    if args.layers > 0:
        from dataclasses import replace
        cfg = replace(cfg, n_layers=args.layers)
    total = args.prompt_len + args.warmup + args.steps + 16
    rt = C.RuntimeConfig.from_env(tp=world, ep=world, max_batch=batch, max_seq_len=(total + 127) // 128 * 128,
                                  max_prefill_tokens=16384)
    if args.impl == "torch_baseline":
        from baseline.torch_baseline import BaselineEngine
        return cfg, rt, BaselineEngine(cfg, rt, seed=0, comm=Comm() if world > 1 else Comm.single())
    from mojo_linuxperiments_b200.engine.engine import Engine
    return cfg, rt, Engine(cfg, rt, seed=0, comm=Comm() if world > 1 else Comm.single())


def run(args):
    rank, local, world = dist_setup(args.gpus)
    from mojo_linuxperiments_b200.ops import _lib
    if args.impl == "ours":
        _lib.lib()          # a missing kernel library is an error, never a fallback
    cfg, rt, eng = make_engine(args, world, rank, args.batch)
    g = torch.Generator().manual_seed(1234)
    B, S, K, W = args.batch, args.prompt_len, args.steps, args.warmup

    # ---- headline: decode at batch B, prompts already prefetched into the KV cache -------------------------
    prompts = torch.randint(0, cfg.vocab, (B, S), generator=g).pin_memory()
    eng.start_batch(B, S + W + K + 8)
    eng.prefill(prompts)
    torch.cuda.synchronize()
    if hasattr(eng, "check_status"):
        eng.check_status()          # stop here, not after minutes of timeouts, if a device-side wait ran out
    sampler = ClockSampler(local) if rank == 0 else None      # started early: it is already sampling when timing starts
    for _ in range(W):
        eng.decode_step()
    torch.cuda.synchronize()
    launches_before = _lib.LAUNCHES[0]
    per_step = getattr(eng, "kernels_per_step", None)
    if sampler:
        sampler.mark_start()
    secs = timed_steps(eng.decode_step, K, world)
    clocks = sampler.stop() if sampler else None
    value = B * K / secs
    if per_step is None:
        per_step = (_lib.LAUNCHES[0] - launches_before) // max(K, 1)
    result = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": secs / K * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 weights+activations (W8A8), bf16 residual/KV, fp32 accumulate of scales" if args.impl != "ours" else
                 "int8 W8A8 GEMMs (int32 accumulate), bf16 activations/KV",
        "data": "synthetic (uniform random token ids, random-init weights of the named shape)",
        "impl": args.impl,
        "config": {"model": MODEL if args.model == "llama3-8b" else args.model, "global_batch": B, "seq_len": S,
                   "parallelism": f"tp{world}", "decode_context": f"{S}..{S + W + K}",
                   "l2_note": "every step streams this rank's int8 weights (>= 1 GB) from HBM: inputs larger than the 126 MB L2"},
        "valid": args.layers == 0, "clocks": clocks, "gpu_launches": int(per_step) * K, "kernels_per_step": int(per_step),
    }

    extra = {}
    if not args.skip_extra:
        # ---- end to end through the public API: pinned host ids in, sampled ids out, every step -------------
        host_in = torch.zeros(B, dtype=torch.int64).pin_memory()
        host_out = torch.zeros(B, dtype=torch.int64).pin_memory()
        eng.start_batch(B, S + W + K + 8)
        first = eng.prefill(prompts)
        host_in.copy_(first)
        torch.cuda.synchronize()

        def e2e_step():
            eng.step_from_host(host_in, host_out)      # H2D ids, graph replay, D2H ids, synchronises
            host_in.copy_(host_out)

        for _ in range(W):
            e2e_step()
        barrier(world)
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(K):
            e2e_step()
        e1.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        e2e_secs = max_over_ranks(max(e0.elapsed_time(e1) * 1e-3, wall), world)
        result["e2e"] = {"value": B * K / e2e_secs, "unit": "tokens/s", "h2d_bytes_per_step": B * 8,
                         "d2h_bytes_per_step": B * 8, "ms_per_step": e2e_secs / K * 1e3,
                         "api": "Engine.step_from_host(pinned_ids_in, pinned_ids_out)"}

        # ---- batch 1 decode -------------------------------------------------------------------------------------
        p1 = torch.randint(0, cfg.vocab, (1, S), generator=g).pin_memory()
        eng.start_batch(1, S + W + K + 8)
        eng.prefill(p1)
        for _ in range(W):
            eng.decode_step()
        s1 = timed_steps(eng.decode_step, K, world)
        extra["decode_tokens_per_sec_bs1"] = K / s1
        extra["ms_per_step_bs1"] = s1 / K * 1e3

        # ---- time to first token: H2D of a 1,024-token prompt -> prefill -> first id on the host ------------------
        ttft = []
        for i in range(3 + 7):
            pp = torch.randint(0, cfg.vocab, (1, S), generator=g).pin_memory()
            eng.start_batch(1, S + 8)
            barrier(world)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            first = eng.prefill(pp)
            host_out[:1].copy_(first, non_blocking=True)
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                ttft.append(max_over_ranks(e0.elapsed_time(e1), world))
        extra["ttft_ms_p50_prompt1024_bs1"] = statistics.median(ttft)
        extra["ttft_samples"] = len(ttft)
    result["extra"] = extra
    if args.impl == "ours":
        from mojo_linuxperiments_b200.ops.workspace import default_workspace
        default_workspace(torch.device("cuda", local)).check_status()
    if rank == 0:
        print(json.dumps(result), flush=True)
    if world > 1:
        # Leave without tearing down NCCL / symmetric-memory state: destroying a communicator whose collectives sit in
        # live CUDA graphs has been seen to block for minutes.  Every rank has passed the last barrier and flushed.
        barrier(world)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def main():
    args = parse()
    if args.impl == "reference":
        # The reference is a CPU-only Mojo project with no Python packaging and no GPU code path.
        print(json.dumps({"impl": "reference", "unavailable": "reference is CPU-only Mojo (no setup.py/pyproject.toml: pip reports "
                          "'not installable'; no mojo/pixi toolchain offline) and has no model, decode or GPU path to run this metric"}))
        return
    run(args)


if __name__ == "__main__":
    main()
