"""Plain PyTorch fp32 references: rotary embedding (rotate-half), causal GQA attention, paged decode attention."""
from __future__ import annotations

import math

import torch


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x [..., T, H, D] with positions [T]: pairs (i, i + D/2) rotated by pos * theta^(-2i/D)."""
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float64, device=x.device) / d))
    ang = positions.to(torch.float64)[:, None] * inv[None, :]
    cos, sin = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]
    xf = x.float()
    a, b = xf[..., : d // 2], xf[..., d // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


def head_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def causal_gqa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None) -> torch.Tensor:
    """One sequence: q [T, hq, D], k/v [T, hkv, D] -> [T, hq, D] fp32."""
    T, hq, d = q.shape
    g = hq // k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    kf = k.float().repeat_interleave(g, dim=1)
    vf = v.float().repeat_interleave(g, dim=1)
    s = torch.einsum("thd,shd->hts", q.float(), kf) * scale
    mask = torch.ones(T, T, dtype=torch.bool, device=q.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    return torch.einsum("hts,shd->thd", s.softmax(-1), vf)


def decode_gqa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float | None = None) -> torch.Tensor:
    """One sequence, one query token: q [hq, D], k/v [L, hkv, D] -> [hq, D] fp32."""
    hq, d = q.shape
    g = hq // k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    kf = k.float().repeat_interleave(g, dim=1)
    vf = v.float().repeat_interleave(g, dim=1)
    s = torch.einsum("hd,lhd->hl", q.float(), kf) * scale
    return torch.einsum("hl,lhd->hd", s.softmax(-1), vf)
