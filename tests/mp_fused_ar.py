"""Worker for tests/test_multigpu.py: the decode GEMM fused with its all-reduce, one-trip and two-hop tails.

Every rank multiplies its own K-shard; the fused launch must return, on every rank, the sum over ranks of the bf16-rounded
partial products (the partials travel as bf16), bit-identical across ranks, for token counts on both sides of the
two-hop threshold, replayed from a CUDA graph (epochs and slot parity must survive replays)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.models.weights import LinearW  # noqa: E402
from mojo_linuxperiments_b200.ops import linear as L  # noqa: E402
from mojo_linuxperiments_b200.parallel.tp import TPContext  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    d = 4096
    tp = TPContext(d, max_tokens=256)
    failures = []
    timing = {}
    for two_hop_min in (0, 1):
        tp.two_hop_min = two_hop_min
        for M, K in [(1, 512), (3, 1792), (8, 512), (32, 1792), (32, 512), (64, 512), (32, 128)]:
            g = torch.Generator().manual_seed(100 * rank + M + K)
            xq = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8).cuda()
            sx = (torch.rand(M, generator=g) * 0.01 + 0.001).cuda()
            lw = LinearW(torch.randint(-127, 128, (d, K), generator=g, dtype=torch.int8).cuda(), (torch.rand(d, generator=g) * 0.01).cuda())
            # reference: every rank's bf16 partial, summed in rank order in fp32, rounded once
            part = L.w8a8_gemm(xq, sx, lw.qweight, lw.scale).float()
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
            ref = torch.zeros_like(part)
            for p in parts:
                ref += p
            ref = ref.to(torch.bfloat16)
            outs = []
            for it in range(3):                       # consecutive launches alternate the slot parity
                outs.append(tp.row_parallel(xq, sx, lw).clone())
            gr = torch.cuda.CUDAGraph()
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                with torch.cuda.graph(gr, stream=s):
                    for _ in range(5):
                        y = tp.row_parallel(xq, sx, lw)
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            gr.replay()
            torch.cuda.synchronize()
            dist.barrier()
            e0.record()
            for _ in range(4):
                gr.replay()
            e1.record()
            torch.cuda.synchronize()
            outs.append(y.clone())
            t = torch.tensor([e0.elapsed_time(e1) / 20 * 1e3], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            timing[(two_hop_min, M, K)] = float(t.item())
            tag = f"two_hop_min={two_hop_min} M={M} K={K}"
            for i, o in enumerate(outs):
                if not torch.allclose(o.float(), ref.float(), rtol=2e-2, atol=2e-2 * ref.float().abs().max().item()):
                    failures.append(f"{tag} launch {i}: max error {(o.float() - ref.float()).abs().max().item():.4g}")
                    break
                same = o.clone()
                dist.broadcast(same, 0)
                if not torch.equal(same, o):
                    failures.append(f"{tag} launch {i}: ranks hold different bits")
                    break
    tp.heap.check_status()
    bad = torch.tensor([len(failures)], device="cuda")
    dist.all_reduce(bad)
    if rank == 0:
        for k, v in timing.items():
            print("TIMING two_hop_min=%d M=%d K_shard=%d: %.2f us per fused GEMM+all-reduce" % (*k, v))
        print("symm backend", tp.heap.backend, "multicast", tp.heap.has_multicast)
        print("FAILURES", int(bad.item()), failures)
    else:
        if failures:
            print(f"rank {rank}:", failures)
    dist.barrier()
    sys.stdout.flush()
    os._exit(1 if failures else 0)


if __name__ == "__main__":
    main()
