"""Plain PyTorch statement of the decoder forward pass (dense and MoE), used as the numerical oracle for the
miniature models.  It applies the same definitions (Hadamard rotation, per-token int8, int32 accumulation,
bf16 rounding of every tensor the kernels materialise) with ordinary tensor ops, one sequence at a time."""
from __future__ import annotations

import math

import torch

from . import attention as OA
from . import quant as Q

BF = torch.bfloat16


def _linear(x_bf16: torch.Tensor, qweight: torch.Tensor, scale: torch.Tensor, tp: int = 1) -> torch.Tensor:
    return Q.hadamard_linear(x_bf16, qweight, scale, tp=tp).to(BF)


def _norm(x_bf16, gamma, eps):
    return Q.rmsnorm(x_bf16, gamma, eps)       # fp32; rotated / quantised by the following linear


def _linear_from_f32(x_f32, lw_q, lw_s, tp=1):
    """Linear whose input is an fp32 tensor that the kernels never round to bf16 (norm output, SwiGLU output)."""
    k = x_f32.shape[-1]
    ks = k // tp
    y = None
    for r in range(tp):
        xq, sx = Q.quantize_rows(Q.rotate(x_f32[..., r * ks:(r + 1) * ks]))
        part = Q.w8a8_linear(xq, sx, lw_q[:, r * ks:(r + 1) * ks], lw_s)
        y = part if y is None else y + part
    return y.to(BF)


def moe_block(cfg, ck, p, xn_f32):
    """xn fp32 [T, d] (normalised) -> bf16 [T, d].  The router is a W8A8 linear like every other projection (it
    consumes the same rotated int8 activations); its logits stay in fp32."""
    T = xn_f32.shape[0]
    xq, sx = Q.quantize_rows(Q.rotate(xn_f32))
    logits = Q.w8a8_linear(xq, sx, ck[p + "router.qweight"], ck[p + "router.scale"])
    probs = logits.softmax(-1)
    topv, topi = probs.topk(cfg.top_k, dim=-1)
    if cfg.norm_topk_prob:
        topv = topv / topv.sum(-1, keepdim=True)
    out = torch.zeros((T, cfg.d_model), dtype=torch.float32, device=xn_f32.device)
    for e in range(cfg.n_experts):
        sel = (topi == e)
        rows = sel.any(-1).nonzero().flatten()
        if rows.numel() == 0:
            continue
        gq = torch.cat([ck[p + f"experts.{e}.gate.qweight"], ck[p + f"experts.{e}.up.qweight"]], 0)
        gs = torch.cat([ck[p + f"experts.{e}.gate.scale"], ck[p + f"experts.{e}.up.scale"]], 0)
        gu = Q.w8a8_linear(xq[rows], sx[rows], gq, gs).to(BF)
        hmid = Q.swiglu(gu)
        y = _linear_from_f32(hmid, ck[p + f"experts.{e}.down.qweight"], ck[p + f"experts.{e}.down.scale"]).float()
        wgt = (topv * sel)[rows].sum(-1, keepdim=True)
        out[rows] += wgt * y          # y is bf16-rounded (the expert GEMM's output), the weighted sum is fp32
    return out.to(BF)


def forward_sequence(cfg, ck: dict, ids: torch.Tensor, tp: int = 1) -> torch.Tensor:
    """Full causal forward of one sequence: ids int64 [T] -> logits fp32 [T, vocab] (bf16-rounded values).
    ``ck`` is the quantised checkpoint dict; ``tp`` mirrors the K-sharded quantisation of row-parallel layers."""
    dev = ids.device
    T = ids.numel()
    pos = torch.arange(T, device=dev)
    hd = cfg.head_dim
    h = ck["embed"][ids].to(BF)
    delta = None
    for l in range(cfg.n_layers):
        p = f"layers.{l}."
        if delta is not None:
            h = (h.float() + delta.float()).to(BF)
        xn = _norm(h, ck[p + "attn_norm"], cfg.eps)
        q = _linear_from_f32(xn, ck[p + "wq.qweight"], ck[p + "wq.scale"]).view(T, cfg.n_heads, hd)
        k = _linear_from_f32(xn, ck[p + "wk.qweight"], ck[p + "wk.scale"]).view(T, cfg.n_kv_heads, hd)
        v = _linear_from_f32(xn, ck[p + "wv.qweight"], ck[p + "wv.scale"]).view(T, cfg.n_kv_heads, hd)
        if cfg.qk_norm:
            q = OA.head_rmsnorm(q, ck[p + "q_norm"], cfg.eps)
            k = OA.head_rmsnorm(k, ck[p + "k_norm"], cfg.eps)
        q = OA.rope(q, pos, cfg.rope_theta).to(BF)
        k = OA.rope(k, pos, cfg.rope_theta).to(BF)
        attn = OA.causal_gqa(q, k, v, 1.0 / math.sqrt(hd)).to(BF).reshape(T, -1)
        delta = _linear(attn, ck[p + "wo.qweight"], ck[p + "wo.scale"], tp=tp)
        h = (h.float() + delta.float()).to(BF)
        xn = _norm(h, ck[p + "mlp_norm"], cfg.eps)
        if cfg.is_moe:
            delta = moe_block(cfg, ck, p, xn)
        else:
            g = _linear_from_f32(xn, ck[p + "gate.qweight"], ck[p + "gate.scale"])
            u = _linear_from_f32(xn, ck[p + "up.qweight"], ck[p + "up.scale"])
            hmid = Q.swiglu(torch.cat([g, u], -1))
            delta = _linear_from_f32(hmid, ck[p + "down.qweight"], ck[p + "down.scale"], tp=tp)
    h = (h.float() + delta.float()).to(BF)
    xn = _norm(h, ck["final_norm"], cfg.eps)
    return _linear_from_f32(xn, ck["lm_head.qweight"], ck["lm_head.scale"]).float()


def greedy_generate(cfg, ck, prompt: torch.Tensor, n_new: int, tp: int = 1):
    """Greedy decoding by full re-computation (no cache): returns (tokens [n_new], logits of each step)."""
    ids = prompt.clone()
    toks, logs = [], []
    for _ in range(n_new):
        lg = forward_sequence(cfg, ck, ids, tp)[-1]
        t = int(lg.argmax())
        toks.append(t)
        logs.append(lg)
        ids = torch.cat([ids, torch.tensor([t], device=ids.device)])
    return toks, logs
