"""Tensor-parallel execution context of one rank: the symmetric heap plus the fused compute+collective ops.

Row-parallel linears (o_proj, down) produce partial sums that have to be added across ranks:
  * up to 64 tokens (decode) the GEMM kernel itself performs the all-reduce over peer memory (one launch);
  * above that the GEMM writes its bf16 partial straight into the symmetric heap and this package's NVLS two-shot
    all-reduce kernel finishes it (two launches, no NCCL, no extra copy);
  * dense prefill (at least ``SP_MIN_TOKENS_PER_RANK`` tokens per rank) leaves the replicated layout altogether:
    ``self.sp`` (``parallel.sp.SPLink``) keeps the residual stream sharded by token and runs all-gather->GEMM and
    GEMM->reduce-scatter as single kernels.
Greedy sampling merges per-rank arg-max candidates through the heap as well.
"""
from __future__ import annotations

import torch

from ..ops import _lib
from ..ops import attention as A
from ..ops import linear as L
from ..ops.workspace import default_workspace
from .symm import SymmetricHeap, AR_LOW_LATENCY, AR_ONE_SHOT_NVLS, AR_ONE_SHOT_P2P, AR_TWO_SHOT_NVLS

FUSED_MAX_M = 64
SP_MIN_TOKENS_PER_RANK = 16


class TPContext:
    def __init__(self, d_model: int, max_tokens: int, group=None, device=None, use_nvls: bool | None = None,
                 wait_limit_ms: int = 2000):
        self.d_model = d_model
        self.max_tokens = max_tokens
        import os
        import torch.distributed as dist
        world = dist.get_world_size(group)
        small = FUSED_MAX_M * d_model * 2
        big = max(FUSED_MAX_M, max_tokens) * d_model * 2
        # low-latency all-reduce: per slot, one [M, N/2] array of 8-byte {2 x bf16, epoch} words per source rank
        self.recv_bytes = world * FUSED_MAX_M * (d_model // 2) * 8
        self.recv2_bytes = FUSED_MAX_M * (d_model // 2) * 8                  # two-hop form: the owners' broadcast lands here
        cand_bytes = 2 * world * 1024 * 16                                   # arg-max exchange: up to 1,024 rows
        self.ll_recv_bytes = 2 * world * (512 << 10) * 2                     # low-latency all-reduce of <= 512 KiB
        total = 2 * small + big + 2 * self.recv_bytes + 2 * self.recv2_bytes + cand_bytes + self.ll_recv_bytes
        from .sp import SPLayout, SPLink
        want_sp = os.environ.get("B200RT_SP", "1") != "0" and max_tokens >= SP_MIN_TOKENS_PER_RANK * world
        if want_sp:
            total += SPLayout(world, max_tokens, d_model, d_model).nbytes + 4096
        self.heap = SymmetricHeap(total + (1 << 20), group=group, device=device)
        self.world, self.rank = self.heap.world, self.heap.rank
        self.recv_off = [self.heap.alloc(self.recv_bytes), self.heap.alloc(self.recv_bytes)]
        self.recv2_off = [self.heap.alloc(self.recv2_bytes), self.heap.alloc(self.recv2_bytes)]
        # above this many tokens the fused all-reduce goes through the slice owners (two NVLink trips, 1/4 of the bytes
        # at 8 ranks); below, one trip wins.  B200RT_AR_TWO_HOP_MIN overrides (0: never).
        self.two_hop_min = int(os.environ.get("B200RT_AR_TWO_HOP_MIN", "8"))
        self.low_latency = os.environ.get("B200RT_AR", "ll") != "barrier"
        # Fused launches alternate between two small slots by the parity of the device-side epoch, so a rank that runs
        # ahead never overwrites a partial a slower rank is still summing.  The unfused path owns a third slot and its
        # all-reduce ends with a barrier, so that slot is free again as soon as the call returns.
        self.part_off = [self.heap.alloc(small), self.heap.alloc(small)]
        self.big_off = self.heap.alloc(big)
        self.cand_recv_off = self.heap.alloc(cand_bytes)
        self.ll_recv_off = self.heap.alloc(self.ll_recv_bytes)
        self.use_nvls = self.heap.has_multicast if use_nvls is None else (use_nvls and self.heap.has_multicast)
        self.limit_ms = wait_limit_ms
        self.sp = SPLink.on_heap(self.heap, max_tokens, d_model, d_model, use_nvls=self.use_nvls,
                                 limit_ms=wait_limit_ms) if want_sp else None

    def sp_ok(self, M: int, moe: bool = False) -> bool:
        """Whether an M-token prefill call should use the token-sharded path.  Dense models do.  Mixture-of-experts
        models do only when B200RT_SP_MOE=1: their dispatch / combine path is correct at 2 and 8 GPUs but measured
        slower than the replicated-token path it would replace (Qwen3-30B-A3B shape, 1,024-token prompt: 12.3 ms vs
        11.2 ms to first token on 8 GPUs, 14.2 ms vs 13.5 ms on 2), because it adds eight small launches per layer."""
        if self.sp is None or not (SP_MIN_TOKENS_PER_RANK * self.world <= M <= self.sp.layout.m_cap and M > FUSED_MAX_M):
            return False
        if moe:
            import os
            want = os.environ.get("B200RT_SP_MOE")
            return want == "1"
        return True

    def row_parallel_fused(self, x: torch.Tensor, lw, mode: int, inline: bool = False):
        """Row-parallel linear from bf16 activations: activation prologue (``mode`` as in ``ops.linear.fused_linear``),
        K-shard product and all-reduce in ONE launch.  Returns None when the grid would not be co-resident (the caller
        then quantises with the stand-alone kernel and calls ``row_parallel``)."""
        import ctypes
        M = x.shape[0]
        N, K = lw.qweight.shape
        if M > FUSED_MAX_M or K % 128 or K > L.FUSED_PROLOG_MAX_K:
            return None
        h = self.heap
        ws = default_workspace(x.device)
        st, keep = L.make_prolog(x, mode, inline=inline, workspace=ws)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        rc = _lib.lib().b200_w8a8_gemm_decode_ar_p(
            ctypes.byref(st), lw.qweight.data_ptr(), lw.scale.data_ptr(), out.data_ptr(), None, M, N, K, out.stride(0),
            ws.status.data_ptr(), _lib.num_sms(x.device.index), h._c_data, h._c_flags,
            (h.mc_data_ptr or None) if self.use_nvls else None, h.world, h.rank, self.part_off[0], self.part_off[1],
            h.epoch_words.data_ptr(), self.limit_ms, 1 if self.low_latency else 0, self.recv_off[0], self.recv_off[1],
            self.recv_bytes, 1 if (self.two_hop_min > 0 and M >= self.two_hop_min) else 0, self.recv2_off[0],
            self.recv2_off[1], self.recv2_bytes, _lib.stream())
        if rc == -20:
            return None
        _lib.check(rc, "w8a8_gemm_decode_ar_p")
        return out

    def row_parallel(self, xq: torch.Tensor, sx: torch.Tensor, lw, residual: torch.Tensor | None = None) -> torch.Tensor:
        """Sum over ranks of this rank's K-shard product; returns the full [M, N] bf16 result on every rank."""
        M, K = xq.shape
        N = lw.qweight.shape[0]
        out = torch.empty((M, N), dtype=torch.bfloat16, device=xq.device)
        h = self.heap
        ws = default_workspace(xq.device)
        if M <= FUSED_MAX_M:
            rc = _lib.lib().b200_w8a8_gemm_decode_ar(
                xq.data_ptr(), sx.data_ptr(), lw.qweight.data_ptr(), lw.scale.data_ptr(), out.data_ptr(),
                _lib.ptr(residual), M, N, K, out.stride(0), ws.status.data_ptr(), _lib.num_sms(xq.device.index),
                h._c_data, h._c_flags, (h.mc_data_ptr or None) if self.use_nvls else None, h.world, h.rank,
                self.part_off[0], self.part_off[1], h.epoch_words.data_ptr(), self.limit_ms,
                1 if self.low_latency else 0, self.recv_off[0], self.recv_off[1], self.recv_bytes,
                1 if (self.two_hop_min > 0 and M >= self.two_hop_min) else 0, self.recv2_off[0], self.recv2_off[1],
                self.recv2_bytes, _lib.stream())
            if rc != -20:
                _lib.check(rc, "w8a8_gemm_decode_ar")
                return out
        # unfused: partial into the heap, then the peer all-reduce kernel
        assert M <= max(self.max_tokens, FUSED_MAX_M), f"{M} tokens exceed the symmetric buffer sized for {self.max_tokens}"
        off = self.big_off
        part = h.tensor(off, (M, N), torch.bfloat16)
        L.w8a8_gemm(xq, sx, lw.qweight, lw.scale, out=part)
        return self._reduce_slot(off, part, M, N, out, residual)

    def _reduce_slot(self, off, part, M, N, out, residual):
        """All-reduce the bf16 [M, N] partial every rank holds at ``off``.  Large messages are reduced in place through
        the switch (two-shot NVLS) and the heap view itself is returned - no copy; the view stays valid until the next
        unfused collective of this context, which in a decoder is after its consumer ran."""
        h = self.heap
        nbytes = M * N * 2
        if self.use_nvls and nbytes % 16 == 0 and nbytes > (512 << 10) and residual is None:
            h.all_reduce(off, M * N, torch.bfloat16, None, algo=AR_TWO_SHOT_NVLS, trailing_barrier=False,
                         limit_ms=self.limit_ms, max_ctas=128)
            return part
        if self.low_latency and nbytes <= (16 << 10) and (M * N) % 2 == 0:
            h.all_reduce(off, M * N, torch.bfloat16, out, algo=AR_LOW_LATENCY, residual=residual, scratch_offset=self.ll_recv_off,
                         trailing_barrier=False, limit_ms=self.limit_ms, max_ctas=128)
            return out
        algo = AR_ONE_SHOT_NVLS if (self.use_nvls and nbytes % 16 == 0) else AR_ONE_SHOT_P2P
        h.all_reduce(off, M * N, torch.bfloat16, out, algo=algo, residual=residual, trailing_barrier=True,
                     limit_ms=self.limit_ms, max_ctas=128)
        return out

    def reduce_partial(self, produce, M: int, N: int) -> torch.Tensor:
        """``produce(out)`` writes this rank's bf16 [M, N] partial into the symmetric heap; returns the sum over ranks."""
        h = self.heap
        part = h.tensor(self.big_off, (M, N), torch.bfloat16)
        produce(part)
        out = torch.empty((M, N), dtype=torch.bfloat16, device=part.device)
        return self._reduce_slot(self.big_off, part, M, N, out, None)

    def argmax(self, cand_val: torch.Tensor, cand_idx: torch.Tensor) -> torch.Tensor:
        """cand_* [ncand, rows] of this rank's vocabulary shard -> global greedy token per row (same on all ranks)."""
        ncand, rows = cand_val.shape
        assert rows <= 1024 and cand_val.is_contiguous() and cand_idx.is_contiguous()
        h = self.heap
        out = torch.empty(rows, dtype=torch.int64, device=cand_val.device)
        rc = _lib.lib().b200_peer_argmax(h._c_data, h._c_flags, h.world, h.rank, self.cand_recv_off, cand_val.data_ptr(),
                                         cand_idx.data_ptr(), ncand, rows, out.data_ptr(), h.epoch_words.data_ptr(),
                                         h.status.data_ptr(), self.limit_ms, _lib.stream())
        _lib.check(rc, "peer_argmax")
        return out
