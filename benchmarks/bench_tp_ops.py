"""Row-parallel linear + all-reduce at decode and prefill sizes, per rank group (launch with torch.distributed.run):
this package's fused GEMM+all-reduce kernel vs GEMM followed by its peer all-reduce kernel vs GEMM followed by NCCL,
and the all-reduce kernels alone against NCCL.  Device-timed (CUDA graph of `iters` calls, events), max over ranks.

python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_tp_ops.py
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.models.weights import LinearW  # noqa: E402
from mojo_linuxperiments_b200.ops import linear as L  # noqa: E402
from mojo_linuxperiments_b200.parallel import symm as S  # noqa: E402
from mojo_linuxperiments_b200.parallel.tp import TPContext  # noqa: E402


def graph_time(fn, iters=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for _ in range(iters):
                fn()
    torch.cuda.synchronize()
    dist.barrier()
    g.replay()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())       # microseconds


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    d = 4096
    tp = TPContext(d, max_tokens=4096)
    rows = []
    for (M, K_full, tag) in [(1, 4096, "o bs1"), (32, 4096, "o bs32"), (1, 14336, "down bs1"), (32, 14336, "down bs32"),
                             (1024, 4096, "o prefill 1k"), (1024, 14336, "down prefill 1k"), (4096, 14336, "cfg2 row M4096")]:
        K = K_full // world
        xq = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda")
        sx = torch.rand(M, device="cuda") * 0.01
        lw = LinearW(torch.randint(-127, 128, (d, K), dtype=torch.int8, device="cuda"), torch.rand(d, device="cuda") * 0.01)
        out = torch.empty((M, d), dtype=torch.bfloat16, device="cuda")
        r = {"op": "row_parallel_linear", "case": tag, "M": M, "N": d, "K_shard": K, "world": world}
        r["gemm_only_us"] = graph_time(lambda: L.w8a8_gemm(xq, sx, lw.qweight, lw.scale, out=out))
        r["ours_us"] = graph_time(lambda: tp.row_parallel(xq, sx, lw))        # fused for M <= 64, GEMM + peer AR above
        def nccl():
            y = L.w8a8_gemm(xq, sx, lw.qweight, lw.scale, out=out)
            dist.all_reduce(y)
        r["gemm_plus_nccl_us"] = graph_time(nccl)
        # roofline: the slower of the weight stream from HBM and the partials over NVLink (770 GB/s per direction)
        hbm_us = (d * K + M * K) / 6539.5e9 * 1e6
        link_us = (M * d * 2) * (world - 1) / world / 770e9 * 1e6
        r["roofline_us"] = max(hbm_us, link_us)
        rows.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)
    heap = tp.heap
    for nbytes in (8 << 10, 256 << 10, 8 << 20, 64 << 20):
        n = nbytes // 2
        if n * 2 > heap.remaining():
            continue
        mark = heap.mark()
        off, x = heap.alloc_tensor((n,), torch.bfloat16)
        x.normal_()
        out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        r = {"op": "all_reduce bf16", "bytes": nbytes, "world": world}
        ll_recv = tp.ll_recv_off
        algos = ([("low_latency", S.AR_LOW_LATENCY)] if nbytes <= (512 << 10) else []) + [("p2p_one_shot", S.AR_ONE_SHOT_P2P)] + ([("nvls_one_shot", S.AR_ONE_SHOT_NVLS), ("nvls_two_shot", S.AR_TWO_SHOT_NVLS)] if heap.has_multicast else [])
        for name, algo in algos:
            if algo == S.AR_ONE_SHOT_P2P and nbytes > (8 << 20):
                continue
            r[name + "_us"] = graph_time(lambda: heap.all_reduce(off, n, torch.bfloat16, out if algo != S.AR_TWO_SHOT_NVLS else None,
                                                                 algo=algo, scratch_offset=ll_recv, max_ctas=128,
                                                                 trailing_barrier=algo not in (S.AR_LOW_LATENCY, S.AR_TWO_SHOT_NVLS)), iters=10)
        y = x.clone()
        r["nccl_us"] = graph_time(lambda: dist.all_reduce(y), iters=10)
        r["busbw_gbs_best_ours"] = 2 * (world - 1) / world * nbytes / (min(v for k, v in r.items() if k.endswith("_us") and k != "nccl_us") * 1e-6) / 1e9
        r["busbw_gbs_nccl"] = 2 * (world - 1) / world * nbytes / (r["nccl_us"] * 1e-6) / 1e9
        if rank == 0:
            print(json.dumps(r), flush=True)
        heap.reset_to(mark)
    tp.heap.check_status()
    dist.barrier()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
