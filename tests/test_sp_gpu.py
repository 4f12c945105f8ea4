"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels on ONE GPU: several virtual ranks share the device, their
kernels run one after another with phase masks (all pushes, then all consumers), and every result is compared with
the plain GEMM kernel / the PyTorch fp32 reference of the same op."""
import pytest
import torch

from mojo_linuxperiments_b200.oracle import quant as Q

pytestmark = pytest.mark.gpu


def _mk_x(m, k, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((m, k), generator=g)
    x = torch.where(torch.rand((m, k), generator=g) < 1e-3, x * 50, x)
    return x.to(torch.bfloat16).cuda()


def _mk_w(n, k, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    wq = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8).cuda()
    sw = (torch.rand((n,), generator=g) * 9e-3 + 1e-3).cuda()
    return wq, sw


@pytest.mark.parametrize("world,M,K,N", [(4, 1024, 512, 768), (4, 520, 256, 320), (8, 256, 512, 256), (2, 200, 128, 64)])
def test_ag_linear_virtual_ranks(world, M, K, N):
    from mojo_linuxperiments_b200.ops import linear as L
    from mojo_linuxperiments_b200.parallel import sp as SP
    links = SP.virtual_links(world, m_cap=1024, k_cap=512, n_cap=1024)
    ws = [_mk_w(N, K, 10 + r) for r in range(world)]
    for epoch in range(3):                        # both parities and the wait for the call-before-last acknowledgement
        x = _mk_x(M, K, 100 + epoch)
        xq, sx = L.act_quant(x)
        outs = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        parts = []
        for r, ln in enumerate(links):
            a, b = ln.my_rows(M)
            parts.append((xq[a:b].contiguous(), sx[a:b].contiguous()))
        for r, ln in enumerate(links):
            ln.ag_linear(parts[r][0], parts[r][1], ws[r][0], ws[r][1], M, out=outs[r], phase=SP.PHASE_PUSH)
        for r, ln in enumerate(links):
            ln.ag_linear(parts[r][0], parts[r][1], ws[r][0], ws[r][1], M, out=outs[r], phase=SP.PHASE_TILES)
        torch.cuda.synchronize()
        for r, ln in enumerate(links):
            ln.check_status()
            want = L.w8a8_gemm(xq, sx, ws[r][0], ws[r][1])
            assert torch.equal(outs[r], want), f"rank {r} epoch {epoch}"
            ref = Q.w8a8_linear(xq, sx, ws[r][0], ws[r][1])
            assert torch.allclose(outs[r].float(), ref.float(), rtol=1e-2, atol=1e-2 * float(ref.abs().max()))
            assert int(ln.ag_words[0].item()) == epoch + 1


@pytest.mark.parametrize("world,M,K,N", [(4, 1024, 256, 512), (4, 520, 128, 320), (8, 256, 384, 256), (2, 200, 128, 64)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_rs_linear_virtual_ranks(world, M, K, N, with_residual):
    from mojo_linuxperiments_b200.ops import linear as L
    from mojo_linuxperiments_b200.parallel import sp as SP
    links = SP.virtual_links(world, m_cap=1024, k_cap=512, n_cap=512)
    ws = [_mk_w(N, K, 20 + r) for r in range(world)]
    R = links[0].rows_per_rank(M)
    for epoch in range(3):
        xs = [L.act_quant(_mk_x(M, K, 200 + 10 * epoch + r)) for r in range(world)]
        res = [_mk_x(R, N, 300 + r) if with_residual else None for r in range(world)]
        outs = [torch.full((R, N), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        for r, ln in enumerate(links):
            ln.rs_linear(xs[r][0], xs[r][1], ws[r][0], ws[r][1], residual=res[r], out=outs[r], phase=SP.PHASE_TILES)
        for r, ln in enumerate(links):
            ln.rs_linear(xs[r][0], xs[r][1], ws[r][0], ws[r][1], residual=res[r], out=outs[r], phase=SP.PHASE_TAIL)
        torch.cuda.synchronize()
        partial = [L.w8a8_gemm(xs[r][0], xs[r][1], ws[r][0], ws[r][1]).float() for r in range(world)]
        total = partial[0].clone()
        for r in range(1, world):
            total += partial[r]                    # same rank order as the kernel
        exact = sum(Q.w8a8_linear(xs[r][0], xs[r][1], ws[r][0], ws[r][1]).float() for r in range(world))
        for r, ln in enumerate(links):
            ln.check_status()
            a, b = ln.my_rows(M)
            want = total[a:b]
            if with_residual:
                want = want + res[r][: b - a].float()
            got = outs[r][: b - a]
            assert torch.equal(got, want.to(torch.bfloat16)), f"rank {r} epoch {epoch}"
            tol = 2e-2 * float(exact.abs().max())
            ref = exact[a:b] + (res[r][: b - a].float() if with_residual else 0)
            assert torch.allclose(got.float(), ref, rtol=2e-2, atol=tol)
            assert int(ln.rs_words[0].item()) == epoch + 1


@pytest.mark.parametrize("world,M,d,E,k", [(4, 520, 256, 16, 4), (8, 1024, 512, 128, 8), (2, 200, 128, 8, 2)])
def test_ep_dispatch_and_combine_virtual_ranks(world, M, d, E, k):
    """Expert all-to-all over virtual ranks: rows reach exactly the ranks that own one of their experts, the routing
    reaches everyone, and the weighted expert outputs come back summed at the owners."""
    from mojo_linuxperiments_b200.ops import moe as MO
    from mojo_linuxperiments_b200.parallel import sp as SP
    links = SP.virtual_links(world, m_cap=1024, k_cap=512, n_cap=512)
    epr = E // world
    g = torch.Generator(device="cpu").manual_seed(11)
    for epoch in range(3):
        xq = torch.randint(-127, 128, (M, d), generator=g, dtype=torch.int8).cuda()
        sx = (torch.rand((M,), generator=g) + 0.1).cuda()
        ids = torch.rand((M, E), generator=g).topk(k, dim=1).indices.to(torch.int32).cuda()
        wts = torch.rand((M, k), generator=g).cuda()
        rows = [ln.my_rows(M) for ln in links]
        for r, ln in enumerate(links):
            a, b = rows[r]
            ln.ep_dispatch(xq[a:b].contiguous(), sx[a:b].contiguous(), ids[a:b].contiguous(), wts[a:b].contiguous(), M, epr)
        works, ys = [], []
        for r, ln in enumerate(links):
            ids_all, wts_all = ln.ep_wait(M, k)
            assert torch.equal(ids_all, ids) and torch.equal(wts_all, wts), f"routing on rank {r}"
            work = MO.moe_align(ids_all, r * epr, epr)
            xp, sp_scale = ln.ep_gather(work, d)
            ln.ag_sync(M, wait=False, finish=True)
            torch.cuda.synchronize()
            n = int(work.meta[0].item())
            tok = work.slot_token[:n].long()
            assert torch.equal(xp[:n], xq[tok]) and torch.equal(sp_scale[:n], sx[tok]), f"gathered rows on rank {r}"
            y = torch.randn((work.max_slots, d), generator=torch.Generator(device="cpu").manual_seed(100 * epoch + r)).to(torch.bfloat16).cuda()
            works.append((work, wts_all))
            ys.append(y)
        R = links[0].rows_per_rank(M)
        outs = [torch.full((R, d), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        for r, ln in enumerate(links):
            a, b = rows[r]
            ln.ep_combine(ys[r], works[r][0], works[r][1], ids[a:b].contiguous(), M, epr, out=outs[r], phase=SP.PHASE_TILES)
        for r, ln in enumerate(links):
            a, b = rows[r]
            ln.ep_combine(ys[r], works[r][0], works[r][1], ids[a:b].contiguous(), M, epr, out=outs[r], phase=SP.PHASE_TAIL)
        torch.cuda.synchronize()
        # reference: per rank the plain combine kernel (bf16 partial per token), summed in rank order over the ranks
        # that own one of the token's experts
        partial = [MO.moe_combine(ys[r], works[r][0], works[r][1]).float() for r in range(world)]
        owner_of = (ids // epr).long()
        total = torch.zeros((M, d), device="cuda")
        for r in range(world):
            has = (owner_of == r).any(dim=1, keepdim=True)
            total += torch.where(has, partial[r], torch.zeros((), device="cuda"))
        for r, ln in enumerate(links):
            ln.check_status()
            a, b = rows[r]
            assert torch.equal(outs[r][: b - a], total[a:b].to(torch.bfloat16)), f"combine on rank {r} epoch {epoch}"
            assert int(ln.rs_words[0].item()) == epoch + 1 and int(ln.ag_words[0].item()) == epoch + 1
