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
    ap.add_argument("--skip-baseline", action="store_true", help="do not run the stock-PyTorch comparison arm after the product's own measurement")
    ap.add_argument("--skip-self-check", action="store_true", help="do not decode the miniature model against the oracle before timing")
    ap.add_argument("--metrics-log", default=os.path.join(tempfile.gettempdir(), "b200rt_bench_metrics.jsonl"),
                    help="append the result record to this JSON-lines file (empty: do not)")
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


def make_engine(args, world, rank, batch, impl=None):
    from mojo_linuxperiments_b200.models import config as C
    from mojo_linuxperiments_b200.parallel.comm import Comm
    impl = impl or args.impl
    cfg = C.PRESETS[args.model]()
    if args.layers > 0:
        from dataclasses import replace
        cfg = replace(cfg, n_layers=args.layers)
    total = args.prompt_len + args.warmup + args.steps + 16
    rt = C.RuntimeConfig.from_env(tp=world, ep=world, max_batch=batch, max_seq_len=(total + 127) // 128 * 128,
                                  max_prefill_tokens=16384)
    if impl == "torch_baseline":
        from baseline.torch_baseline import BaselineEngine
        return cfg, rt, BaselineEngine(cfg, rt, seed=0, comm=Comm() if world > 1 else Comm.single())
    from mojo_linuxperiments_b200.engine.engine import Engine
    return cfg, rt, Engine(cfg, rt, seed=0, comm=Comm() if world > 1 else Comm.single())


def measured_hbm_gbs() -> tuple[float, str]:
    """Copy bandwidth this pool's B200s were measured at (MEASURED_PEAKS.json beside this file), else the fallback."""
    try:
        with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "of measured"
    except Exception:
        return 6650.0, "of fallback"


def decode_bytes_per_rank(cfg, world: int, batch: int, context: int) -> dict:
    """Bytes one rank has to stream from HBM per decode step: its int8 weight shards (every linear, the lm_head shard;
    for mixture-of-experts models only an upper bound, all local experts) and the KV cache of the running context."""
    from mojo_linuxperiments_b200.models.config import kv_heads_per_rank
    d, hd = cfg.d_model, cfg.head_dim
    hkv = kv_heads_per_rank(cfg, world)
    per_layer = (cfg.n_heads // world + 2 * hkv) * hd * d + d * (cfg.n_heads // world) * hd
    if cfg.is_moe:
        per_layer += (cfg.n_experts // world) * 3 * cfg.moe_ffn * d + cfg.n_experts * d
    else:
        per_layer += 3 * (cfg.ffn // world) * d
    weights = cfg.n_layers * per_layer + (cfg.vocab // world) * d
    kv = cfg.n_layers * batch * context * 2 * hkv * hd * 2
    return {"weights": int(weights), "kv": int(kv), "total": int(weights + kv)}


def self_check(world: int, rank: int) -> dict:
    """Before anything is timed: a miniature dense model, tensor-parallel over the same ranks and the same fused
    kernels, decodes 8 greedy tokens that every rank compares with the plain PyTorch oracle.  A token may differ only
    where the oracle's own top-2 margin is within rounding noise; anything else aborts the benchmark."""
    from mojo_linuxperiments_b200.engine.engine import Engine
    from mojo_linuxperiments_b200.models import config as C
    from mojo_linuxperiments_b200.models import weights as Wt
    from mojo_linuxperiments_b200.oracle import model as OM
    from mojo_linuxperiments_b200.parallel.comm import Comm
    cfg = C.tiny_dense(n_layers=2, d_model=1024, n_heads=8, n_kv_heads=8 if world > 4 else 4, ffn=2048, vocab=2048)
    rt = C.RuntimeConfig(tp=world, ep=world, max_seq_len=256, max_prefill_tokens=512)
    ck = Wt.quantize_master(Wt.init_master(cfg, 0))
    eng = Engine(cfg, rt, weights=Wt.shard_from_checkpoint(cfg, ck, world, rank, "cuda"), comm=Comm() if world > 1 else Comm.single())
    prompts = torch.randint(0, cfg.vocab, (3, 70), generator=torch.Generator().manual_seed(5))
    new = 8
    out = eng.generate(prompts, new)
    ck_dev = {k: v.cuda() for k, v in ck.items()}
    agree = total = 0
    problems = []
    for b in range(prompts.shape[0]):
        toks, logs = OM.greedy_generate(cfg, ck_dev, prompts[b].cuda(), new, tp=world)
        for i in range(new):
            total += 1
            if int(out[b, i]) == toks[i]:
                agree += 1
                continue
            top2 = logs[i].topk(2).values
            if (top2[0] - top2[1]).item() > 0.05 * logs[i].abs().max().item():
                problems.append(f"rank {rank} sequence {b} step {i}: token {int(out[b, i])} != oracle {toks[i]} with a clear margin")
            break
    if agree < total // 2:
        problems.append(f"rank {rank}: only {agree} of {total} tokens agree with the oracle")
    bad = max_over_ranks(float(len(problems)), world)
    if bad:
        raise SystemExit("self-check failed before timing: " + "; ".join(problems or ["another rank diverged"]))
    del eng
    return {"tokens_compared": total, "tokens_equal": agree, "model": "tiny dense 2x1024, same ranks and kernels"}


def measure(eng, cfg, args, world, local, rank, prompts, g, *, ours: bool, extras: bool):
    """Headline decode number of one engine, plus (extras) the end-to-end, batch-1 and time-to-first-token runs."""
    from mojo_linuxperiments_b200.ops import _lib
    B, S, K, W = args.batch, args.prompt_len, args.steps, args.warmup
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
    per_step = getattr(eng, "kernels_per_step", None) if ours else None
    if sampler:
        sampler.mark_start()
    secs = timed_steps(eng.decode_step, K, world)
    clocks = sampler.stop() if sampler else None
    if ours and not per_step:
        per_step = (_lib.LAUNCHES[0] - launches_before) // max(K, 1)
    res = {"value": B * K / secs, "ms_per_step": secs / K * 1e3, "clocks": clocks, "kernels_per_step": int(per_step or 0)}
    if not extras:
        return res
    host_in = torch.zeros(B, dtype=torch.int64).pin_memory()
    host_out = torch.zeros(B, dtype=torch.int64).pin_memory()
    if ours:
        # ---- end to end through the public API: pinned host ids in, sampled ids out, every step -------------
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
        res["e2e"] = {"value": B * K / e2e_secs, "unit": "tokens/s", "h2d_bytes_per_step": B * 8,
                      "d2h_bytes_per_step": B * 8, "ms_per_step": e2e_secs / K * 1e3,
                      "api": "Engine.step_from_host(pinned_ids_in, pinned_ids_out)"}
    # ---- batch 1 decode -------------------------------------------------------------------------------------
    extra = {}
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
    res["extra"] = extra
    return res


# Stock PyTorch (cuBLASLt int8 + SDPA + NCCL) build of the same model measured earlier on this pool's B200s
# (decode tokens/s at batch 32): used for vs_baseline only when the live baseline arm below cannot run.
RECORDED_BASELINE_TOK_S = {1: 2318.0, 8: 2411.0}


def run(args):
    rank, local, world = dist_setup(args.gpus)
    from mojo_linuxperiments_b200.ops import _lib
    if args.impl == "ours":
        _lib.lib()          # a missing kernel library is an error, never a fallback
    check = None
    if args.impl == "ours" and not args.skip_self_check:
        check = self_check(world, rank)
    cfg, rt, eng = make_engine(args, world, rank, args.batch)
    g = torch.Generator().manual_seed(1234)
    B, S, K, W = args.batch, args.prompt_len, args.steps, args.warmup
    prompts = torch.randint(0, cfg.vocab, (B, S), generator=g).pin_memory()
    m = measure(eng, cfg, args, world, local, rank, prompts, g, ours=args.impl == "ours", extras=not args.skip_extra)
    value = m["value"]
    hbm, hbm_note = measured_hbm_gbs()
    nbytes = decode_bytes_per_rank(cfg, world, B, S + W + K // 2)
    result = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": m["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "int8 weights+activations (W8A8), bf16 residual/KV, fp32 accumulate of scales" if args.impl != "ours" else
                 "int8 W8A8 GEMMs (int32 accumulate), bf16 activations/KV",
        "data": "synthetic (uniform random token ids, random-init weights of the named shape)",
        "impl": args.impl,
        "config": {"model": MODEL if args.model == "llama3-8b" else args.model, "global_batch": B, "seq_len": S,
                   "parallelism": f"tp{world}", "decode_context": f"{S}..{S + W + K}",
                   "l2_note": "every step streams this rank's int8 weights (>= 1 GB) from HBM: inputs larger than the 126 MB L2"},
        "valid": args.layers == 0, "clocks": m["clocks"], "gpu_launches": m["kernels_per_step"] * K,
        "kernels_per_step": m["kernels_per_step"],
        "roofline": {"hbm_bytes_per_rank_per_step": nbytes, "hbm_gbs": hbm,
                     "fraction_of_hbm": nbytes["total"] / (hbm * 1e9) / (m["ms_per_step"] * 1e-3), "note": hbm_note},
    }
    if "e2e" in m:
        result["e2e"] = m["e2e"]
    result["extra"] = m.get("extra", {})
    if check is not None:
        result["self_check"] = check
    if args.impl == "ours":
        eng.check_status()
        result["runtime"] = eng.memory_report()      # rank placement (GPU's NUMA node, pinned CPUs) and arena counters
        # ---- the comparison arm: stock PyTorch ops on the same ranks, same prompts, same step counts --------------
        base = None
        if not args.skip_baseline:
            try:
                eng.kv = None                    # give the KV pages back before the second engine allocates its own
                torch.cuda.empty_cache()
                _, _, beng = make_engine(args, world, rank, args.batch, impl="torch_baseline")
                gb = torch.Generator().manual_seed(1234)
                torch.randint(0, cfg.vocab, (B, S), generator=gb)
                base = measure(beng, cfg, args, world, local, rank, prompts, gb, ours=False, extras=not args.skip_extra)
                beng._graphs.clear()             # graphs with NCCL work in them must not outlive the process group
                del beng
            except Exception as e:  # the product's own line must survive a failing comparison arm
                base = {"error": f"{type(e).__name__}: {e}"[:300]}
        if base and "value" in base:
            bx = base.get("extra", {})
            ex = result["extra"]
            result["vs_baseline"] = value / base["value"]
            result["baseline"] = {
                "impl": "torch_baseline (cuBLASLt int8 torch._int_mm, SDPA, NCCL, CUDA-graph decode), measured in this run",
                "decode_tokens_per_sec_bs32": base["value"], "ms_per_step": base["ms_per_step"], "clocks": base["clocks"],
                **{k: bx[k] for k in ("decode_tokens_per_sec_bs1", "ttft_ms_p50_prompt1024_bs1") if k in bx},
                "ratios": {"decode_bs32": value / base["value"],
                           **({"decode_bs1": ex["decode_tokens_per_sec_bs1"] / bx["decode_tokens_per_sec_bs1"],
                               "ttft": bx["ttft_ms_p50_prompt1024_bs1"] / ex["ttft_ms_p50_prompt1024_bs1"]}
                              if "decode_tokens_per_sec_bs1" in bx and "decode_tokens_per_sec_bs1" in ex else {})}}
        else:
            rec = RECORDED_BASELINE_TOK_S.get(world)
            if rec and args.model == "llama3-8b" and B == 32:
                result["vs_baseline"] = value / rec
                result["baseline"] = {"impl": "torch_baseline, recorded earlier on this pool",
                                      "decode_tokens_per_sec_bs32": rec, **({"live_run": base} if base else {})}
            elif base:
                result["baseline"] = base
        try:
            from mojo_linuxperiments_b200.utils.trace import MetricsLog
            if rank == 0 and args.metrics_log:
                MetricsLog(args.metrics_log).write(**result)
        except Exception:
            pass
    if rank == 0:
        print(json.dumps(result), flush=True)
    if world > 1:
        # Orderly teardown: first everything that pins the communicator (captured graphs with NCCL / symmetric-memory
        # work in them, the symmetric heaps), then the process group.  Destroying the group while such graphs were alive
        # has blocked for minutes; should the orderly path ever block too, a watchdog ends the process (the result
        # line is already out and every rank is past the last barrier).
        import threading
        barrier(world)
        sys.stdout.flush()
        sys.stderr.flush()
        threading.Timer(30.0, lambda: os._exit(0)).start()
        try:
            if hasattr(eng, "close"):
                eng.close()
            del eng
            import gc
            gc.collect()
            torch.cuda.synchronize()
            import torch.distributed as dist
            dist.destroy_process_group()
            if rank == 0:
                print("teardown: process group destroyed after the graphs and heaps were released", file=sys.stderr, flush=True)
        finally:
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
