"""CPU point of the W8A8 Hadamard linear benchmark (K=4096 -> N=14336 -> 4096): the host runtime's pinned worker pools
run rotate + quantise + int8 GEMM (AMX int8 tiles or AVX-512 VNNI, whichever the CPU offers) for M in {1, 32, 256}.  No GPU needed.

python benchmarks/bench_config2_host.py [--reps 3]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200 import hostrt as H  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--sizes", type=int, nargs="*", default=[1, 32, 256])
    a = ap.parse_args()
    K, N = 4096, 14336
    g = torch.Generator().manual_seed(0)
    w1 = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    s1 = torch.rand((N,), generator=g) * 9e-3 + 1e-3
    w2 = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    s2 = torch.rand((K,), generator=g) * 9e-3 + 1e-3
    info = H.NumaInfo()
    for M in a.sizes:
        x = torch.randn((M, K), generator=g)
        x = torch.where(torch.rand((M, K), generator=g) < 1e-3, x * 50, x).to(torch.bfloat16)
        for isa in ("best", "vnni"):
            best = None
            for _ in range(a.reps):
                r1 = H.w8a8_linear(info, x, w1, s1, isa=isa)
                r2 = H.w8a8_linear(info, r1["y"], w2, s2, isa=isa)
                assert r1["status"] == 0 and r2["status"] == 0
                t = (r1["quant_ns"] + r1["gemm_ns"] + r2["quant_ns"] + r2["gemm_ns"]) * 1e-6
                best = t if best is None else min(best, t)
            ops = 2 * 2.0 * M * N * K
            print(json.dumps({"op": "config2 W8A8 linear pair (host CPUs)", "M": M, "K": K, "N": N, "workers": r1["workers"],
                              "isa": r1["isa"], "ms": best, "gops": ops / (best * 1e-3) / 1e9}), flush=True)


if __name__ == "__main__":
    main()
