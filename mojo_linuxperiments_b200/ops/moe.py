"""Mixture-of-experts ops: router top-k, work-list construction, token gather, grouped expert GEMMs, combine."""
from __future__ import annotations

import torch

from . import _lib
from . import linear as L
from .workspace import default_workspace


def router_topk(logits: torch.Tensor, k: int, renorm: bool = True):
    """fp32 logits [M, E] -> (ids int32 [M, k], weights fp32 [M, k]) of softmax top-k (ties: lowest expert id)."""
    M, E = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    ids = torch.empty((M, k), dtype=torch.int32, device=logits.device)
    wts = torch.empty((M, k), dtype=torch.float32, device=logits.device)
    _lib.check(_lib.lib().b200_router_topk(logits.data_ptr(), logits.stride(0), M, E, k, 1 if renorm else 0,
                                           ids.data_ptr(), wts.data_ptr(), _lib.stream()), "router_topk")
    return ids, wts


class MoEWorkList:
    """Device-side description of which (token, k) pairs this rank's experts process, in slot order."""

    def __init__(self, M: int, k: int, n_local: int, device):
        self.M, self.k, self.n_local = M, k, n_local
        self.max_slots = M * k
        self.max_tiles = (self.max_slots + 127) // 128 + n_local
        i32 = dict(dtype=torch.int32, device=device)
        self.counts = torch.empty(n_local, **i32)
        self.offsets = torch.empty(n_local + 1, **i32)
        self.slot_token = torch.empty(self.max_slots, **i32)
        self.inv = torch.empty((M, k), **i32)
        self.tiles = torch.empty((self.max_tiles, 4), **i32)
        self.meta = torch.empty(2, **i32)


def moe_align(ids: torch.Tensor, e0: int, n_local: int, work: MoEWorkList | None = None) -> MoEWorkList:
    M, k = ids.shape
    w = work or MoEWorkList(M, k, n_local, ids.device)
    _lib.check(_lib.lib().b200_moe_align(ids.data_ptr(), M, k, e0, n_local, w.counts.data_ptr(), w.offsets.data_ptr(),
                                         w.slot_token.data_ptr(), w.inv.data_ptr(), w.tiles.data_ptr(), w.meta.data_ptr(),
                                         _lib.stream()), "moe_align")
    return w


def moe_gather(xq: torch.Tensor, sx: torch.Tensor, w: MoEWorkList):
    M, d = xq.shape
    xp = torch.empty((w.max_slots, d), dtype=torch.int8, device=xq.device)
    sp = torch.empty((w.max_slots,), dtype=torch.float32, device=xq.device)
    _lib.check(_lib.lib().b200_moe_gather(xq.data_ptr(), sx.data_ptr(), d, w.slot_token.data_ptr(), w.meta.data_ptr(),
                                          w.max_slots, xp.data_ptr(), sp.data_ptr(), _lib.stream()), "moe_gather")
    return xp, sp


def grouped_gemm(xp: torch.Tensor, sp: torch.Tensor, wq: torch.Tensor, sw: torch.Tensor, w: MoEWorkList) -> torch.Tensor:
    """Per local expert e: y[slots of e] = xp[slots of e] . wq[e]^T * sp * sw[e].  wq int8 [E_local, N, K]."""
    E, N, K = wq.shape
    assert wq.is_contiguous() and sw.is_contiguous() and xp.is_contiguous()
    y = torch.empty((w.max_slots, N), dtype=torch.bfloat16, device=xp.device)
    ws = default_workspace(xp.device)
    sms = _lib.num_sms(xp.device.index)
    if w.M <= L.DECODE_MAX_M:
        rc = _lib.lib().b200_w8a8_gemm_decode_grouped(
            xp.data_ptr(), sp.data_ptr(), wq.data_ptr(), sw.data_ptr(), y.data_ptr(), w.M, w.max_slots, N, K,
            y.stride(0), E, w.offsets.data_ptr(), w.counts.data_ptr(), ws.status.data_ptr(), sms, _lib.stream())
        _lib.check(rc, "w8a8_gemm_decode_grouped")
    else:
        rc = _lib.lib().b200_w8a8_gemm_grouped(
            xp.data_ptr(), sp.data_ptr(), wq.data_ptr(), sw.data_ptr(), y.data_ptr(), w.max_slots, N, K, y.stride(0), E,
            w.tiles.data_ptr(), w.meta[1:].data_ptr(), w.max_tiles, ws.status.data_ptr(), sms, _lib.stream())
        _lib.check(rc, "w8a8_gemm_grouped")
    return y


def moe_combine(y: torch.Tensor, w: MoEWorkList, wts: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[token] = sum_k wts[token, k] * y[slot(token, k)] over the pairs whose expert is local (bf16 [M, d])."""
    d = y.shape[1]
    if out is None:
        out = torch.empty((w.M, d), dtype=torch.bfloat16, device=y.device)
    _lib.check(_lib.lib().b200_moe_combine(y.data_ptr(), y.stride(0), w.inv.data_ptr(), wts.data_ptr(), w.M, w.k, d,
                                           out.data_ptr(), out.stride(0), _lib.stream()), "moe_combine")
    return out
