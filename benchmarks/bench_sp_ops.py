"""Per-kernel cost of the fused tensor-parallel prefill linears against the plain GEMM of the same shape, on ONE GPU with
a single virtual rank (every "peer" store lands in local memory): isolates what the gather / scatter machinery itself
costs (flag waits, comm warps, epilogue re-layout, reduction tail) from what NVLink costs.

python benchmarks/bench_sp_ops.py [M] [world_shapes]
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.ops import linear as L  # noqa: E402
from mojo_linuxperiments_b200.parallel import sp as SP  # noqa: E402


def graph_time(fn, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for _ in range(iters):
                fn()
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def main():
    M = int(sys.argv[1]) if len(sys.argv) > 1 else 4096
    tp = int(sys.argv[2]) if len(sys.argv) > 2 else 8          # shard shapes of this tensor-parallel degree
    d, ffn = 4096, 14336
    link = SP.virtual_links(1, max(M, 128), d, d)[0]
    for (name, N, K) in (("qkv", 6144 // tp, d), ("gate_up", 2 * ffn // tp, d)):
        xq = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda")
        sx = torch.rand(M, device="cuda") * 0.01
        wq = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda")
        sw = torch.rand(N, device="cuda") * 0.01
        out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        r = {"op": "ag_linear", "case": name, "M": M, "N": N, "K": K}
        r["plain_gemm_us"] = graph_time(lambda: L.w8a8_gemm(xq, sx, wq, sw, out=out))
        r["ag_gemm_us"] = graph_time(lambda: link.ag_linear(xq, sx, wq, sw, M, out=out))
        print(json.dumps(r), flush=True)
    for (name, N, K) in (("o", d, d // tp), ("down", d, ffn // tp)):
        xq = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda")
        sx = torch.rand(M, device="cuda") * 0.01
        wq = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda")
        sw = torch.rand(N, device="cuda") * 0.01
        out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        r = {"op": "rs_linear", "case": name, "M": M, "N": N, "K": K}
        r["plain_gemm_us"] = graph_time(lambda: L.w8a8_gemm(xq, sx, wq, sw, out=out))
        r["rs_gemm_us"] = graph_time(lambda: link.rs_linear(xq, sx, wq, sw, out=out))
        print(json.dumps(r), flush=True)
    link.check_status()


if __name__ == "__main__":
    main()
