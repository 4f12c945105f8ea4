"""Mixture-of-experts kernels and the miniature MoE model against PyTorch references."""
import pytest
import torch

from mojo_linuxperiments_b200.models import config as C
from mojo_linuxperiments_b200.models import weights as Wt
from mojo_linuxperiments_b200.oracle import model as OM
from mojo_linuxperiments_b200.oracle import quant as Q

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,E,k", [(1, 128, 8), (37, 128, 8), (5, 16, 4), (300, 64, 2)])
def test_router_topk(M, E, k):
    from mojo_linuxperiments_b200.ops import moe as MO
    logits = torch.randn((M, E), generator=torch.Generator().manual_seed(M)).cuda()
    ids, wts = MO.router_topk(logits, k, True)
    probs = logits.softmax(-1)
    tv, ti = probs.topk(k, dim=-1)
    tv = tv / tv.sum(-1, keepdim=True)
    assert torch.equal(ids.long().sort(-1).values, ti.sort(-1).values)
    order = ids.long().argsort(-1)
    assert torch.allclose(wts.gather(-1, order), tv.gather(-1, ti.argsort(-1)), rtol=1e-4, atol=1e-6)
    ids2, wts2 = MO.router_topk(logits, k, False)
    assert torch.allclose(wts2.sum(-1), tv.new_tensor(1.0) * probs.topk(k, -1).values.sum(-1), rtol=1e-4)


@pytest.mark.parametrize("M,d,E,k,F,e0,n_local", [(8, 512, 16, 4, 256, 0, 16), (33, 512, 16, 4, 256, 8, 8),
                                                  (300, 1024, 32, 4, 512, 0, 32), (1000, 512, 16, 2, 256, 4, 4)])
def test_grouped_expert_pipeline(M, d, E, k, F, e0, n_local):
    """align -> gather -> grouped gate_up -> swiglu+quant -> grouped down -> combine, against per-expert references."""
    from mojo_linuxperiments_b200.ops import linear as L
    from mojo_linuxperiments_b200.ops import moe as MO
    from mojo_linuxperiments_b200.ops.workspace import default_workspace
    g = torch.Generator().manual_seed(M + d)
    x = torch.randn((M, d), generator=g).to(torch.bfloat16).cuda()
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(M)]).to(torch.int32).cuda()
    wts = torch.rand((M, k), generator=g).cuda()
    gu_q = torch.randint(-127, 128, (n_local, 2 * F, d), generator=g, dtype=torch.int8).cuda()
    gu_s = (torch.rand((n_local, 2 * F), generator=g) * 2e-4 + 1e-4).cuda()
    dn_q = torch.randint(-127, 128, (n_local, d, F), generator=g, dtype=torch.int8).cuda()
    dn_s = (torch.rand((n_local, d), generator=g) * 2e-4 + 1e-4).cuda()
    xq, sx = L.act_quant(x)
    work = MO.moe_align(ids, e0, n_local)
    xp, sp = MO.moe_gather(xq, sx, work)
    gu = MO.grouped_gemm(xp, sp, gu_q, gu_s, work)
    hq, sh = L.act_quant(gu, mode=L.AQ_SWIGLU)
    yd = MO.grouped_gemm(hq, sh, dn_q, dn_s, work)
    out = MO.moe_combine(yd, work, wts)
    torch.cuda.synchronize()
    default_workspace(x.device).check_status()
    counts = torch.stack([(ids == e0 + e).sum() for e in range(n_local)]).int()
    assert torch.equal(work.counts, counts) and int(work.meta[0]) == int(counts.sum())
    ref = torch.zeros((M, d), dtype=torch.float32, device="cuda")
    for e in range(n_local):
        sel = ids == (e0 + e)
        rows = sel.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        gu_ref = Q.w8a8_linear(xq[rows], sx[rows], gu_q[e], gu_s[e]).to(torch.bfloat16)
        hmid = Q.swiglu(gu_ref)
        hq_r, sh_r = Q.quantize_rows(Q.rotate(hmid))
        y = Q.w8a8_linear(hq_r, sh_r, dn_q[e], dn_s[e]).to(torch.bfloat16).float()
        ref[rows] += (wts * sel)[rows].sum(-1, keepdim=True) * y
    tol = 0.03 * float(ref.abs().max())
    assert (out.float() - ref).abs().max().item() <= tol


def test_tiny_moe_model_matches_oracle():
    from mojo_linuxperiments_b200.engine.engine import Engine
    cfg = C.tiny_moe()
    rt = C.RuntimeConfig(max_seq_len=256)
    ck = Wt.quantize_master(Wt.init_master(cfg, 1))
    ck_dev = {k: v.cuda() for k, v in ck.items()}
    w = Wt.shard_from_checkpoint(cfg, ck, 1, 0, "cuda")
    eng = Engine(cfg, rt, weights=w)
    B, S, NEW = 2, 150, 8
    prompts = torch.randint(0, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(4))
    out = eng.generate(prompts, NEW)
    out_eager = eng.generate(prompts, NEW, use_graph=False)
    assert torch.equal(out, out_eager)
    eng.start_batch(B, S + NEW)
    eng.prefill(prompts, use_graph=False)      # eager: `last_logits` is then this call's tensor, not a captured one
    torch.cuda.synchronize()
    got = eng.model.last_logits.float()
    agree = 0
    for b in range(B):
        ref = OM.forward_sequence(cfg, ck_dev, prompts[b].cuda())[-1]
        assert (got[b] - ref).abs().max().item() <= 0.08 * ref.abs().max().item()
        toks, logs = OM.greedy_generate(cfg, ck_dev, prompts[b].cuda(), NEW)
        for t in range(NEW):
            if int(out[b, t]) == toks[t]:
                agree += 1
                continue
            top2 = logs[t].topk(2).values
            assert (top2[0] - top2[1]).item() < 0.08 * logs[t].abs().max().item()
            break
    assert agree >= B * NEW // 2
