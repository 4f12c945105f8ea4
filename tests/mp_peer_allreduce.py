"""Worker for tests/test_multigpu.py: one process per GPU (launched by torch.distributed.run)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.parallel import symm as S  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    heap = S.SymmetricHeap(64 << 20)
    results = {"multicast": heap.has_multicast}
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    failures = []

    def check(name, cond):
        if not cond:
            failures.append(name)

    ll_recv = heap.alloc(2 * world * (512 << 10) * 2)      # receive area of the low-latency algorithm
    # bf16 messages of several sizes, every algorithm that applies
    for n in (8, 4096, 32 * 4096, 1024 * 4096 + 8):
        off, x = heap.alloc_tensor((n,), torch.bfloat16)
        scratch = heap.alloc(1 << 16)
        for rep in range(3):        # repeated use of the same flags: epochs keep increasing
            x.copy_(torch.randn(n, device="cuda", generator=g).to(torch.bfloat16))
            ref = x.float().clone()
            dist.all_reduce(ref)
            res = torch.randn(n, device="cuda", generator=g).to(torch.bfloat16)
            algos = [S.AR_ONE_SHOT_P2P] + ([S.AR_ONE_SHOT_NVLS, S.AR_TWO_SHOT_NVLS] if heap.has_multicast else [])
            if n % 2 == 0 and n * 2 <= (512 << 10):
                algos.append(S.AR_LOW_LATENCY)
            for algo in algos:
                if algo == S.AR_TWO_SHOT_NVLS:
                    keep = x.clone()
                out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
                heap.all_reduce(off, n, torch.bfloat16, out, algo=algo, residual=res, scratch_offset=ll_recv)
                torch.cuda.synchronize()
                heap.check_status()
                want = ref + res.float()
                tol = 0.02 * max(1.0, float(want.abs().max()))
                check(f"bf16 n={n} algo={algo} rep={rep}", bool((out.float() - want).abs().max() <= tol))
                if algo == S.AR_TWO_SHOT_NVLS:
                    dist.barrier()
                    x.copy_(keep)
                    torch.cuda.synchronize()
                    dist.barrier()
    # fp32 / fp64 scalars-to-vectors: one-shot, chain (result on rank 0), butterfly
    for dtype in (torch.float32, torch.float64):
        for n in (1, 5, 1024):
            off, x = heap.alloc_tensor((n,), dtype, align=256)
            scratch = heap.alloc(8 * n * 8 + 256)
            x.copy_((torch.arange(n, device="cuda", dtype=torch.float64) + rank + 1).to(dtype))
            want = (torch.arange(n, device="cuda", dtype=torch.float64) * world + world * (world + 1) / 2).to(dtype)
            dist.barrier()
            for algo in (S.AR_ONE_SHOT_P2P, S.AR_CHAIN, S.AR_BUTTERFLY):
                out = torch.zeros(n, dtype=dtype, device="cuda")
                heap.all_reduce(off, n, dtype, out, algo=algo, scratch_offset=scratch)
                torch.cuda.synchronize()
                heap.check_status()
                if algo == S.AR_CHAIN and rank != 0:
                    continue
                check(f"{dtype} n={n} algo={algo}", bool(torch.allclose(out, want)))
    # graph replay: epochs advance on the device, no host clean-up between replays
    n = 4096
    off, x = heap.alloc_tensor((n,), torch.bfloat16)
    out = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    x.fill_(float(rank + 1))
    heap.all_reduce(off, n, torch.bfloat16, out)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.stream(s):
        with torch.cuda.graph(gr, stream=s):
            heap.all_reduce(off, n, torch.bfloat16, out)
    for rep in range(5):
        gr.replay()
    torch.cuda.synchronize()
    heap.check_status()
    check("graph replay", bool((out.float() == world * (world + 1) / 2).all()))
    dist.barrier()
    bad = torch.tensor([len(failures)], device="cuda")
    dist.all_reduce(bad)
    if rank == 0:
        print("MULTICAST", heap.has_multicast)
        print("symm backend", heap.backend, "multicast", heap.has_multicast)
        print("FAILURES", int(bad.item()), failures)
    dist.barrier()
    sys.stdout.flush()
    os._exit(1 if failures else 0)      # skip communicator / symmetric-memory teardown (can block with live graphs)


if __name__ == "__main__":
    main()
