"""Launch the W8A8 GEMM a few times on one shape (for profiler captures): python benchmarks/run_gemm_once.py M N K [reps]"""
import sys

import torch

import os
import sys as _sys
_sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.ops import linear as L
from mojo_linuxperiments_b200.ops.workspace import default_workspace

M, N, K = (int(a) for a in sys.argv[1:4])
reps = int(sys.argv[4]) if len(sys.argv) > 4 else 3
dev = torch.device("cuda", 0)
x = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev)
sx = torch.rand(M, device=dev) * 0.01
sw = torch.rand(N, device=dev) * 0.01
out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
for _ in range(reps):
    L.w8a8_gemm(x, sx, w, sw, out=out)
torch.cuda.synchronize()
default_workspace(dev).check_status()
print("ok", float(out.float().abs().mean()))
