"""Plain PyTorch reference (fp32/fp64, runs on CPU or GPU) of the W8A8 Hadamard linear.

Definitions used everywhere in the package:
  H128      128x128 Sylvester-Hadamard matrix scaled by 1/sqrt(128) (orthogonal and symmetric)
  rotate    Xr = X . blockdiag(H128, ...) over blocks of 128 along the last dim
  quantise  sx[m] = max_k |Xr[m,k]| / 127 (1 when the row is all zero); Xq = clamp(rint(Xr / sx), -127, 127)
  linear    Y[m,n] = (sum_k Xq[m,k] Wq[n,k]) * sx[m] * sw[n]; W is stored already rotated
  tp        a row-parallel (K-sharded) layer rotates / quantises each K-shard with its own per-token scale
            and sums the dequantised partial outputs
"""
from __future__ import annotations

import math

import torch

HADAMARD_BLOCK = 128


def hadamard_matrix(n: int = HADAMARD_BLOCK, dtype=torch.float32, device="cpu") -> torch.Tensor:
    assert n & (n - 1) == 0
    h = torch.ones((1, 1), dtype=torch.float64)
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    return (h / math.sqrt(n)).to(dtype=dtype, device=device)


def rotate(x: torch.Tensor, block: int = HADAMARD_BLOCK) -> torch.Tensor:
    """Block-diagonal Hadamard rotation of the last dim, fp32 math."""
    k = x.shape[-1]
    assert k % block == 0
    h = hadamard_matrix(block, torch.float32, x.device)
    xr = x.to(torch.float32).reshape(*x.shape[:-1], k // block, block) @ h
    return xr.reshape(*x.shape)


def quantize_rows(xr: torch.Tensor):
    """Per-row symmetric int8 quantisation of already-rotated fp32 rows -> (int8, fp32 scale)."""
    amax = xr.abs().amax(dim=-1)
    s = torch.where(amax > 0, amax / 127.0, torch.ones_like(amax))
    q = torch.clamp(torch.round(xr / s.unsqueeze(-1)), -127, 127).to(torch.int8)
    return q, s.to(torch.float32)


def rotate_quantize(x: torch.Tensor):
    return quantize_rows(rotate(x))


def quantize_weight(w: torch.Tensor):
    """fp32 weight [N,K] -> (rotated int8 [N,K], per-output-channel fp32 scale [N])."""
    return quantize_rows(rotate(w))


def int_gemm(xq: torch.Tensor, wq: torch.Tensor) -> torch.Tensor:
    """Exact integer product (float64 carries it exactly for K < 2^37 / 127^2)."""
    return (xq.to(torch.float64) @ wq.to(torch.float64).t())


def w8a8_linear(xq, sx, wq, sw, residual=None) -> torch.Tensor:
    y = int_gemm(xq, wq) * sx.to(torch.float64).unsqueeze(1) * sw.to(torch.float64).unsqueeze(0)
    if residual is not None:
        y = y + residual.to(torch.float64)
    return y.to(torch.float32)


def hadamard_linear(x: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor, tp: int = 1) -> torch.Tensor:
    """Full op from bf16 activations, mirroring K-sharded (row-parallel) execution when tp > 1."""
    k = x.shape[-1]
    assert k % (tp * HADAMARD_BLOCK) == 0
    ks = k // tp
    y = None
    for r in range(tp):
        xq, sx = rotate_quantize(x[..., r * ks:(r + 1) * ks])
        part = w8a8_linear(xq, sx, wq[:, r * ks:(r + 1) * ks], sw)
        y = part if y is None else y + part
    return y


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.to(torch.float32)
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.to(torch.float32)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    f = gate_up.shape[-1] // 2
    g = gate_up[..., :f].to(torch.float32)
    u = gate_up[..., f:].to(torch.float32)
    return g * torch.sigmoid(g) * u
