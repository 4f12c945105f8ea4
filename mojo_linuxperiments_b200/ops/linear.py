"""W8A8 Hadamard linear: activation prologue (rotate + per-token int8) and the tcgen05 int8 GEMM."""
from __future__ import annotations

import os

import torch

from . import _lib
from .workspace import Workspace, default_workspace

AQ_PLAIN, AQ_NORM, AQ_ADD_NORM, AQ_SWIGLU = 0, 1, 2, 3


def act_quant(x: torch.Tensor, *, mode: int = AQ_PLAIN, gamma: torch.Tensor | None = None, eps: float = 1e-5,
              residual: torch.Tensor | None = None, want_normed: bool = False,
              out_q: torch.Tensor | None = None, out_scale: torch.Tensor | None = None):
    """Rotate (block-128 Hadamard) and quantise rows of ``x`` (bf16 [M, K], last dim contiguous).

    mode AQ_NORM applies RMSNorm(gamma) first; AQ_ADD_NORM first adds ``x`` into ``residual`` (in place);
    AQ_SWIGLU treats ``x`` as [M, 2K] = gate | up and quantises silu(gate) * up.
    Returns (q int8 [M,K], scale fp32 [M]) and, if ``want_normed``, the normalised bf16 rows.
    """
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    M = x.shape[0]
    K = x.shape[1] // 2 if mode == AQ_SWIGLU else x.shape[1]
    q = out_q if out_q is not None else torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = out_scale if out_scale is not None else torch.empty((M,), dtype=torch.float32, device=x.device)
    xn = torch.empty((M, K), dtype=torch.bfloat16, device=x.device) if want_normed else None
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.stride(1) == 1
    rc = _lib.lib().b200_act_quant(
        x.data_ptr(), x.stride(0), _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
        _lib.ptr(gamma), float(eps), q.data_ptr(), q.stride(0), s.data_ptr(), _lib.ptr(xn),
        xn.stride(0) if xn is not None else 0, M, K, mode, _lib.stream())
    _lib.check(rc, "act_quant")
    return (q, s, xn) if want_normed else (q, s)


DECODE_MAX_M = 64


def w8a8_gemm(xq: torch.Tensor, sx: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor, *,
              residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
              out_dtype: torch.dtype = torch.bfloat16, workspace: Workspace | None = None,
              force_mode: int = -1, force_splits: int = 0, narrow: bool = False) -> torch.Tensor:
    """y[m,n] = (sum_k xq[m,k] wq[n,k]) * sx[m] * sw[n] (+ residual); int8 operands, int32 accumulate in TMEM.

    Up to 64 tokens the cluster split-K weight-streaming kernel runs (``force_mode`` -1) unless the problem has
    enough tiles for the persistent kernel; ``force_mode`` 0 / 1 select the persistent kernel's whole-tile / stream-K
    schedules, ``force_mode`` 2 the cluster kernel with ``force_splits`` CTAs per cluster."""
    assert xq.is_cuda and xq.dtype == torch.int8 and wq.dtype == torch.int8
    assert xq.is_contiguous() and wq.is_contiguous()
    M, K = xq.shape
    N, K2 = wq.shape
    assert K == K2
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=xq.device)
    assert out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.stride(0) == out.stride(0) and residual.stride(1) == 1
    w = workspace or default_workspace(xq.device)
    n_tiles = (N + 127) // 128
    use_cluster = M <= DECODE_MAX_M and (force_mode == 2 or (force_mode == -1 and n_tiles < _DECODE_TILE_WAVES * _lib.num_sms(xq.device.index)))
    # a narrow output (a router: one channel tile) for up to 256 tokens is still a weight stream: the persistent
    # kernel would walk its whole K loop on one or two CTAs, the cluster kernel splits K and takes 64 tokens per grid layer
    # (one channel tile only: wider outputs stay on the persistent kernel, whose results the token-sharded paths are
    # compared with bit for bit - the two kernels multiply the scales in a different order)
    # The caller asks for it (``narrow=True``) because the two kernels multiply the scales in a different order and
    # other callers compare this function's persistent-kernel results bit for bit with the token-sharded paths.
    if not use_cluster and force_mode in (-1, 2) and M <= 4 * DECODE_MAX_M and (force_mode == 2 or (narrow and n_tiles == 1)):
        use_cluster = True
    if use_cluster:
        rc = _lib.lib().b200_w8a8_gemm_decode(
            xq.data_ptr(), sx.data_ptr(), wq.data_ptr(), sw.data_ptr(), out.data_ptr(), _lib.ptr(residual),
            M, N, K, out.stride(0), 1 if out.dtype == torch.float32 else 0, w.status.data_ptr(),
            _lib.num_sms(xq.device.index), force_splits, _lib.stream())
        _lib.check(rc, "w8a8_gemm_decode")
        return out
    if force_mode == 2:
        force_mode = -1
    rc = _lib.lib().b200_w8a8_gemm(
        xq.data_ptr(), sx.data_ptr(), wq.data_ptr(), sw.data_ptr(), out.data_ptr(), _lib.ptr(residual),
        M, N, K, out.stride(0), 1 if out.dtype == torch.float32 else 0,
        w.ws.data_ptr(), w.ws_bytes, w.counters.data_ptr(), w.counters.numel(), w.status.data_ptr(),
        _lib.num_sms(xq.device.index), force_mode, _lib.stream())
    _lib.check(rc, "w8a8_gemm")
    return out


# up to this many 128-channel tiles per SM a small-M GEMM goes to the weight-streaming cluster kernel
_DECODE_TILE_WAVES = int(os.environ.get("B200RT_DECODE_TILE_WAVES", "4"))

QR_PLAIN, QR_NORM, QR_ADD_NORM, QR_SWIGLU = 1, 2, 3, 4
FUSED_PROLOG_MAX_K = 20480          # a row is parked as floats in the GEMM's stage memory (80 KiB)


INLINE_PROLOG_MAX_M = 4             # up to this many tokens the GEMM CTAs quantise their own operand (no quantiser CTAs)


def make_prolog(x: torch.Tensor, mode: int, *, gamma: torch.Tensor | None = None, eps: float = 1e-5,
                residual: torch.Tensor | None = None, residual_out: torch.Tensor | None = None,
                inline: bool = False, workspace: Workspace | None = None):
    """Describe the activation prologue a decode GEMM launch should run itself (see ``fused_linear``).

    Returns ``(struct, keep)``: the ctypes struct for the C entry points and the tensors it points at (int8 rows,
    scales), which the caller keeps alive until the launch has run."""
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1
    M = x.shape[0]
    K = x.shape[1] // 2 if mode == QR_SWIGLU else x.shape[1]
    assert M <= DECODE_MAX_M and K % 128 == 0 and K <= FUSED_PROLOG_MAX_K
    w = workspace or default_workspace(x.device)
    q = torch.empty((M, K), dtype=torch.int8, device=x.device)
    s = torch.empty((M,), dtype=torch.float32, device=x.device)
    if residual is not None:
        assert residual.dtype == torch.bfloat16 and residual.stride(1) == 1
    if residual_out is not None:
        assert residual is not None and residual_out.dtype == torch.bfloat16 and residual_out.stride(1) == 1
        assert residual_out.shape == residual.shape
    st = _lib.QuantProlog(mode, x.data_ptr(), x.stride(0), _lib.ptr(residual), residual.stride(0) if residual is not None else 0,
                          _lib.ptr(gamma), float(eps), q.data_ptr(), s.data_ptr(), w.qflags.data_ptr(), w.step.data_ptr(),
                          _lib.ptr(residual_out), residual_out.stride(0) if residual_out is not None else 0,
                          1 if inline else 0)
    return st, (q, s)


def fused_linear(x: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor, *, mode: int = QR_PLAIN,
                 gamma: torch.Tensor | None = None, eps: float = 1e-5, residual: torch.Tensor | None = None,
                 residual_out: torch.Tensor | None = None, inline: bool = False,
                 out_dtype: torch.dtype = torch.bfloat16, workspace: Workspace | None = None) -> torch.Tensor:
    """bf16 activations in, bf16 (or fp32) result out, in ONE launch for up to 64 tokens: the activation prologue
    (``mode``: QR_PLAIN rotate + int8; QR_NORM RMSNorm first; QR_ADD_NORM ``residual += x`` in place, then RMSNorm of
    the residual; QR_SWIGLU x = gate | up) runs in quantiser CTAs of the GEMM's own grid, which publish a flag per
    token row; the GEMM CTAs stream their first weight tiles meanwhile and wait for the flags, not for a kernel.

    With ``inline`` and up to ``INLINE_PROLOG_MAX_M`` tokens there are no quantiser CTAs: every GEMM CTA quantises its own K slice of the
    rows into its operand stages and the cluster exchanges the row statistics (sum of squares, maximum) through
    distributed shared memory.  Because every cluster then reads the old residual, QR_ADD_NORM needs ``residual_out``
    (a second buffer that receives ``residual + x``; without it the sum is written in place and quantiser CTAs run)."""
    import ctypes
    N, K = wq.shape
    M = x.shape[0]
    w = workspace or default_workspace(x.device)
    st, keep = make_prolog(x, mode, gamma=gamma, eps=eps, residual=residual, residual_out=residual_out, inline=inline, workspace=w)
    assert keep[0].shape[1] == K
    out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    rc = _lib.lib().b200_w8a8_gemm_decode_p(
        ctypes.byref(st), wq.data_ptr(), sw.data_ptr(), out.data_ptr(), None, M, N, K, out.stride(0),
        1 if out_dtype == torch.float32 else 0, w.status.data_ptr(), _lib.num_sms(x.device.index), _lib.stream())
    _lib.check(rc, "w8a8_gemm_decode_p")
    return out
