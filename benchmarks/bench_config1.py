"""Config-1 workload: fill 64 MiB of float32 with uniform[-1,1) from a counter RNG (seed 0, keyed on the global element
index) and reduce it to one sum.

  host  : the C++ host runtime - NUMA topology query, one pinned clone3 worker per CPU per node, node-local arenas,
          pairwise tree reduce (`hostrt::fill_reduce`), plus the chain / butterfly collectives between rank threads
  GPU   : `fill_uniform_reduce` on each GPU's slice of the index space, then a peer-memory all-reduce of the
          per-GPU sums (one process per GPU under torch.distributed.run; a single process uses one GPU)

python benchmarks/bench_config1.py [--host-only]
python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_config1.py
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

N_ELEMS = 16 * 1024 * 1024


def host_part():
    from mojo_linuxperiments_b200 import hostrt as H
    info = H.NumaInfo()
    best = None
    for _ in range(5):
        r = H.fill_reduce(info, N_ELEMS, 0)
        if best is None or r["elapsed_ns"] < best["elapsed_ns"]:
            best = r
    import time
    t0 = time.perf_counter()
    st, v = H.chain_reduce(info, max(2, info.num_nodes))
    chain_us = (time.perf_counter() - t0) * 1e6
    t0 = time.perf_counter()
    st2, out = H.butterfly_allreduce(info, 4)
    bfly_us = (time.perf_counter() - t0) * 1e6
    return {"where": "host", "nodes": info.num_nodes, "cpus": info.total_cpus(), "workers": best["workers"], "sum": best["sum"],
            "fill_reduce_ms": best["elapsed_ns"] / 1e6, "gbs": N_ELEMS * 4 / best["elapsed_ns"],
            "misplaced": best["misplaced"], "chain_reduce_us_incl_spawn": chain_us, "butterfly_allreduce_us_incl_spawn": bfly_us}


def gpu_part():
    import torch
    import torch.distributed as dist
    from mojo_linuxperiments_b200.ops.workload import FillReduce
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    heap = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        from mojo_linuxperiments_b200.parallel import symm as S
        heap = S.SymmetricHeap(1 << 20)
        off, slot = heap.alloc_tensor((2,), torch.float64)
        scratch = heap.alloc(4096)
    fr = FillReduce(N_ELEMS, world, rank)
    total = torch.zeros(2, dtype=torch.float64, device="cuda")

    def step():
        fr.run(0)
        if heap is not None:
            slot[0:1].copy_(fr.result)
            heap.all_reduce(off, 2, torch.float64, total, algo=S.AR_ONE_SHOT_P2P)
        else:
            total[0:1].copy_(fr.result)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = 20
    e0.record()
    for _ in range(iters):
        step()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    # fill alone (HBM-write roofline: 4 bytes per element)
    e0.record()
    for _ in range(iters):
        fr.run(0)
    e1.record()
    torch.cuda.synchronize()
    fill_ms = e0.elapsed_time(e1) / iters
    res = {"where": "gpu", "n_gpus": world, "sum": float(total[0].item()), "ms_fill_plus_allreduce": float(t.item()),
           "ms_fill_only_this_rank": fill_ms, "fill_gbs_this_rank": (fr.end - fr.begin) * 4 / (fill_ms * 1e-3) / 1e9,
           "frac_of_measured_hbm_copy_bw": (fr.end - fr.begin) * 4 / (fill_ms * 1e-3) / 1e9 / 6539.5}
    if heap is not None:
        heap.check_status()
    return rank, world, res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--host-only", action="store_true")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    if rank == 0:
        print(json.dumps(host_part()), flush=True)
    if a.host_only:
        return
    rank, world, res = gpu_part()
    if rank == 0:
        print(json.dumps(res), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        sys.stdout.flush()
        os._exit(0)


if __name__ == "__main__":
    main()
