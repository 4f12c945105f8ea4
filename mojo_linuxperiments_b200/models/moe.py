"""Mixture-of-experts block with expert parallelism over replicated tokens.

After the attention all-reduce every rank holds the same normalised, rotated, int8-quantised tokens.  Each rank routes
all tokens (same result everywhere), keeps the (token, expert) pairs whose expert it owns, runs the two grouped expert
GEMMs on them and produces a partial output per token; the partials are summed across ranks by the same peer-memory
all-reduce the dense row-parallel layers use.  With one rank this degenerates to a plain local MoE.

Token-sharded prefill (``forward_sharded``) replaces the replication by the expert all-to-all: each rank routes only
the rows it owns, ``ep_dispatch`` stores a row into the heaps of exactly the ranks that own one of its experts,
the grouped expert GEMMs run on what arrived, and ``ep_combine`` sends each token's weighted local outputs back to its
owner, which sums the contributions (``csrc/kernels/moe_ep.cu``).
"""
from __future__ import annotations

import torch

from ..ops import linear as L
from ..ops import moe as MO


class MoEBlock:
    def __init__(self, cfg, rt, comm, device, tp_ctx=None):
        self.cfg, self.rt, self.comm, self.device, self.tp_ctx = cfg, rt, comm, device, tp_ctx
        self.n_local = cfg.n_experts // max(rt.ep, 1)
        self.e0 = comm.rank * self.n_local if rt.ep > 1 else 0

    def forward(self, W: dict, xq: torch.Tensor, sx: torch.Tensor, xn=None) -> torch.Tensor:
        cfg = self.cfg
        M = xq.shape[0]
        logits = L.w8a8_gemm(xq, sx, W["router"].qweight, W["router"].scale, out_dtype=torch.float32, narrow=True)
        ids, wts = MO.router_topk(logits, cfg.top_k, cfg.norm_topk_prob)
        work = MO.moe_align(ids, self.e0, self.n_local)
        xp, sp = MO.moe_gather(xq, sx, work)
        gu = MO.grouped_gemm(xp, sp, W["experts_gate_up"].qweight, W["experts_gate_up"].scale, work)
        hq, sh = L.act_quant(gu, mode=L.AQ_SWIGLU)
        yd = MO.grouped_gemm(hq, sh, W["experts_down"].qweight, W["experts_down"].scale, work)
        if self.tp_ctx is not None:
            return self.tp_ctx.reduce_partial(lambda out: MO.moe_combine(yd, work, wts, out=out), M, cfg.d_model)
        out = MO.moe_combine(yd, work, wts)
        return self.comm.all_reduce(out)

    def forward_sharded(self, W: dict, xq_loc: torch.Tensor, sx_loc: torch.Tensor, M: int) -> torch.Tensor:
        """xq_loc / sx_loc: the normalised, quantised rows this rank owns of an M-token call; returns the MoE output of
        those rows (bf16 [rows_per_rank, d], the first ``my_rows`` valid)."""
        cfg, sp = self.cfg, self.tp_ctx.sp
        logits = L.w8a8_gemm(xq_loc, sx_loc, W["router"].qweight, W["router"].scale, out_dtype=torch.float32)
        ids_loc, wts_loc = MO.router_topk(logits, cfg.top_k, cfg.norm_topk_prob)
        sp.ep_dispatch(xq_loc, sx_loc, ids_loc, wts_loc, M, self.n_local)
        ids, wts = sp.ep_wait(M, cfg.top_k)
        work = MO.moe_align(ids, self.e0, self.n_local)
        xp, sp_scale = sp.ep_gather(work, cfg.d_model)
        sp.ag_sync(M, wait=False, finish=True)        # the gather buffer of this epoch has been consumed
        gu = MO.grouped_gemm(xp, sp_scale, W["experts_gate_up"].qweight, W["experts_gate_up"].scale, work)
        hq, sh = L.act_quant(gu, mode=L.AQ_SWIGLU)
        yd = MO.grouped_gemm(hq, sh, W["experts_down"].qweight, W["experts_down"].scale, work)
        return sp.ep_combine(yd, work, wts, ids_loc, M, self.n_local)
