"""Worker for tests/test_multigpu.py: fused all-gather->GEMM and GEMM->reduce-scatter over real peer memory."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.ops import linear as L  # noqa: E402
from mojo_linuxperiments_b200.parallel import sp as SP  # noqa: E402
from mojo_linuxperiments_b200.parallel import symm as S  # noqa: E402


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    m_cap, k_cap, n_cap = 4096, 1024, 1024
    lay = SP.SPLayout(world, m_cap, k_cap, n_cap)
    heap = S.SymmetricHeap(2 * lay.nbytes + (4 << 20))
    links = {"nvls": SP.SPLink.on_heap(heap, m_cap, k_cap, n_cap, use_nvls=True),
             "p2p": SP.SPLink.on_heap(heap, m_cap, k_cap, n_cap, use_nvls=False)}
    failures = []

    def check(name, cond):
        if not cond:
            failures.append(name)

    def gen(seed):
        return torch.Generator(device="cuda").manual_seed(seed)

    for name, ln in links.items():
        if name == "nvls" and not heap.has_multicast:
            continue
        for (M, K, N, Ks) in ((1024, 512, 768, 256), (520, 256, 320, 128), (4096, 1024, 512, 384), (130, 128, 64, 128)):
            for rep in range(3):
                # the same full activation on every rank (seeded), this rank's own weights
                x = torch.randn((M, K), device="cuda", generator=gen(7 + rep)).to(torch.bfloat16)
                wq = torch.randint(-127, 128, (N, K), device="cuda", generator=gen(100 + rank), dtype=torch.int8)
                sw = torch.rand((N,), device="cuda", generator=gen(200 + rank)) * 9e-3 + 1e-3
                xq, sx = L.act_quant(x)
                a, b = ln.my_rows(M)
                y = ln.ag_linear(xq[a:b].contiguous(), sx[a:b].contiguous(), wq, sw, M)
                torch.cuda.synchronize()
                ln.check_status()
                check(f"{name} ag M={M} rep={rep}", torch.equal(y, L.w8a8_gemm(xq, sx, wq, sw)))

                # row-parallel: this rank's K-shard activations and weights, sum over ranks, keep my rows
                x2 = torch.randn((M, Ks), device="cuda", generator=gen(1000 + 10 * rep + rank)).to(torch.bfloat16)
                w2 = torch.randint(-127, 128, (K, Ks), device="cuda", generator=gen(300 + rank), dtype=torch.int8)
                s2 = torch.rand((K,), device="cuda", generator=gen(400 + rank)) * 9e-3 + 1e-3
                x2q, s2x = L.act_quant(x2)
                R = ln.rows_per_rank(M)
                res = torch.randn((R, K), device="cuda", generator=gen(500 + rank)).to(torch.bfloat16)
                out = ln.rs_linear(x2q, s2x, w2, s2, residual=res)
                torch.cuda.synchronize()
                ln.check_status()
                part = L.w8a8_gemm(x2q, s2x, w2, s2)
                gathered = [torch.empty_like(part) for _ in range(world)]
                dist.all_gather(gathered, part)
                total = gathered[0].float()
                for r in range(1, world):
                    total += gathered[r].float()
                want = (total[a:b] + res[: b - a].float()).to(torch.bfloat16)
                check(f"{name} rs M={M} rep={rep}", torch.equal(out[: b - a], want))

    # back-to-back calls without host synchronisation (epoch parity, acknowledgements, counters under skew)
    ln = links["nvls"] if heap.has_multicast else links["p2p"]
    M, K, N = 2048, 1024, 1024
    x = torch.randn((M, K), device="cuda", generator=gen(9)).to(torch.bfloat16)
    wq = torch.randint(-127, 128, (N, K), device="cuda", generator=gen(600 + rank), dtype=torch.int8)
    sw = torch.rand((N,), device="cuda", generator=gen(700 + rank)) * 9e-3 + 1e-3
    xq, sx = L.act_quant(x)
    a, b = ln.my_rows(M)
    xl, sl = xq[a:b].contiguous(), sx[a:b].contiguous()
    want_y = L.w8a8_gemm(xq, sx, wq, sw)
    ys, outs = [], []
    for it in range(12):
        if it % 3 == rank % 3:
            torch.cuda._sleep(2_000_000)          # skew the ranks against each other
        y = ln.ag_linear(xl, sl, wq, sw, M)
        yq, ysx = L.act_quant(y)
        outs.append(ln.rs_linear(yq, ysx, wq, sw))
        ys.append(y)
    torch.cuda.synchronize()
    ln.check_status()
    check("chain ag", all(torch.equal(y, want_y) for y in ys))
    check("chain rs", all(torch.equal(o, outs[0]) for o in outs))

    fl = torch.tensor([len(failures)], device="cuda")
    dist.all_reduce(fl)
    if failures:
        print(f"rank {rank} failed: {failures[:8]}", flush=True)
    dist.barrier()
    torch.cuda.synchronize()
    if rank == 0:
        print(f"FAILURES {int(fl.item())}", flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
