"""Device-timed W8A8 GEMM sweep: this package's tcgen05 kernel vs torch._int_mm (cuBLASLt) on the same shapes.

Timing: CUDA events around one CUDA graph of `iters` back-to-back launches that rotate through enough distinct weight / activation
buffers to exceed the 126 MB L2 (so every launch streams its operands from HBM), after warm-up.
Usage: python benchmarks/bench_gemm.py [--out gemm.json]
"""
import argparse
import json

import torch

import os
import sys as _sys
_sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.ops import linear as L

SHAPES = [  # (M, N, K, tag)
    (1, 6144, 4096, "llama qkv tp1 bs1"), (32, 6144, 4096, "llama qkv tp1 bs32"),
    (1, 28672, 4096, "llama gate_up tp1 bs1"), (32, 28672, 4096, "llama gate_up tp1 bs32"),
    (32, 4096, 14336, "llama down tp1 bs32"), (32, 4096, 4096, "llama o tp1 bs32"),
    (32, 128256, 4096, "llama lm_head tp1 bs32"),
    (32, 768, 4096, "llama qkv tp8 bs32"), (32, 3584, 4096, "llama gate_up tp8 bs32"),
    (32, 4096, 1792, "llama down tp8 bs32"), (32, 4096, 512, "llama o tp8 bs32"),
    (256, 14336, 4096, "cfg2 M256"), (1024, 28672, 4096, "prefill gate_up tp1 1k"),
    (1024, 6144, 4096, "prefill qkv tp1 1k"), (1024, 4096, 14336, "prefill down tp1 1k"),
    (4096, 1792, 4096, "cfg2 col tp8 M4096"), (4096, 4096, 1792, "cfg2 row tp8 M4096"),
    (4096, 14336, 4096, "cfg2 M4096 tp1"), (8192, 8192, 8192, "square 8k"),
]


def time_fn(fn, n_bufs, iters, warmup=3):
    """Seconds per launch; the launches are captured in one CUDA graph so host launch cost is not in the number."""
    for i in range(warmup):
        fn(i % n_bufs)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            for i in range(iters):
                fn(i % n_bufs)
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=None)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    rows = []
    for (M, N, K, tag) in SHAPES:
        per = N * K + M * K + M * N * 2
        n_bufs = max(2, min(16, (300 << 20) // per + 1))
        ws = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev) for _ in range(n_bufs)]
        xs = [torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev) for _ in range(n_bufs)]
        sx = torch.rand(M, device=dev) * 0.01
        sw = torch.rand(N, device=dev) * 0.01
        out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
        t = time_fn(lambda i: L.w8a8_gemm(xs[i], sx, ws[i], sw, out=out), n_bufs, args.iters)
        row = {"tag": tag, "M": M, "N": N, "K": K, "ours_us": t * 1e6,
               "ours_tops": 2.0 * M * N * K / t / 1e12, "ours_gbs": per / t / 1e9}
        if M > 16:
            try:
                wts = [w.t() for w in ws]
                Mp = (M + 7) // 8 * 8
                xp = [torch.nn.functional.pad(x, (0, 0, 0, Mp - M)) for x in xs]
                tb = time_fn(lambda i: torch._int_mm(xp[i], wts[i]), n_bufs, args.iters)
                row["int_mm_us"] = tb * 1e6
                row["int_mm_tops"] = 2.0 * M * N * K / tb / 1e12
            except Exception as e:  # shape constraints of _int_mm
                row["int_mm_err"] = str(e)[:80]
        rows.append(row)
        print(json.dumps(row), flush=True)
        del ws, xs
        torch.cuda.empty_cache()
    if args.out:
        with open(args.out, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
