"""Launch the fused tensor-parallel GEMM kernels a few times on ONE GPU with a single virtual rank (every peer store
lands in local memory), for profiler captures of the kernels themselves:

    python benchmarks/run_tp_gemm_once.py ag  M N K [reps]     all-gather -> GEMM      (w8a8_gemm_tp_kernel, gather form)
    python benchmarks/run_tp_gemm_once.py rs  M N K [reps]     GEMM -> reduce-scatter  (w8a8_gemm_tp_kernel, scatter form)
    python benchmarks/run_tp_gemm_once.py ar  M N K [reps]     decode GEMM + all-reduce (w8a8_gemm_decode_kernel, low-latency tail)
"""
import ctypes
import sys

import torch

import os
import sys as _sys
_sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.ops import _lib
from mojo_linuxperiments_b200.parallel import sp as SP

kind = sys.argv[1]
M, N, K = (int(a) for a in sys.argv[2:5])
reps = int(sys.argv[5]) if len(sys.argv) > 5 else 3
dev = torch.device("cuda", 0)
x = torch.randint(-127, 128, (M, K), dtype=torch.int8, device=dev)
w = torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev)
sx = torch.rand(M, device=dev) * 0.01
sw = torch.rand(N, device=dev) * 0.01
out = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
if kind in ("ag", "rs"):
    link = SP.virtual_links(1, max(M, 128), max(K, 128), max(N, 128))[0]
    for _ in range(reps):
        if kind == "ag":
            link.ag_linear(x, sx, w, sw, M, out=out)
        else:
            link.rs_linear(x, sx, w, sw, out=out)
    torch.cuda.synchronize()
    link.check_status()
else:
    small = 64 * N * 2
    recv = M * (N // 2) * 8
    heap = torch.zeros(2 * small + 2 * recv + 4096, dtype=torch.uint8, device=dev)
    flags = torch.zeros(1024, dtype=torch.int32, device=dev)
    words = torch.zeros(8, dtype=torch.int32, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    data = (ctypes.c_void_p * 1)(heap.data_ptr())
    fl = (ctypes.c_void_p * 1)(flags.data_ptr())
    for _ in range(reps):
        rc = _lib.lib().b200_w8a8_gemm_decode_ar(
            x.data_ptr(), sx.data_ptr(), w.data_ptr(), sw.data_ptr(), out.data_ptr(), None, M, N, K, N,
            status.data_ptr(), _lib.num_sms(0), data, fl, None, 1, 0, 0, small, words.data_ptr(), 200, 1,
            2 * small, 2 * small + recv, recv, 0, 0, 0, 0, _lib.stream())
        _lib.check(rc, "w8a8_gemm_decode_ar")
    torch.cuda.synchronize()
    assert int(status[0].item()) == 0, int(status[0].item())
print("ok", float(out.float().abs().mean()))
