"""Decoder forward pass (Llama-shaped dense and Qwen3-shaped MoE) as a sequence of sm_100a kernels.

Residual stream convention: ``h`` is the bf16 residual; every block produces a ``delta`` that is folded into ``h``
by the *next* norm kernel (residual add + RMSNorm + Hadamard rotation + int8 quantisation are one launch).
With tensor parallelism the delta of a row-parallel linear is a partial sum that is all-reduced first, either
inside the GEMM kernel over peer memory (fused) or by NCCL between kernels (baseline wiring).
"""
from __future__ import annotations

import math

import torch

from ..ops import attention as A
from ..ops import linear as L
from ..parallel.comm import Comm
from ..utils.trace import op_range
from .config import ModelConfig, RuntimeConfig, kv_heads_per_rank


class KVState:
    """Paged KV cache of all layers of one rank plus the page table / lengths of the running batch."""

    @staticmethod
    def nbytes(cfg: ModelConfig, rt: RuntimeConfig, num_seqs: int, max_seq_len: int) -> int:
        """Device bytes of a cache for ``num_seqs`` sequences of up to ``max_seq_len`` tokens (storage + tables)."""
        max_pages = (max_seq_len + rt.page_size - 1) // rt.page_size
        hkv = kv_heads_per_rank(cfg, rt.tp)
        return (cfg.n_layers * (num_seqs * max_pages + 1) * 2 * hkv * rt.page_size * cfg.head_dim * 2
                + num_seqs * max_pages * 4 + num_seqs * 4 + 3 * 1024)

    def __init__(self, cfg: ModelConfig, rt: RuntimeConfig, device, num_seqs: int, max_seq_len: int, alloc=None):
        """``alloc(shape, dtype) -> zeroed tensor``: where the cache lives (the rank's HBM arena); default torch.zeros.

        Pages are handed out on demand (``admit`` as a sequence grows) from a host-side free list.  The last page is
        a scratch page no sequence owns: the page-table rows of empty slots point at it, so a kernel that runs over
        an empty slot of the batch has somewhere harmless to write."""
        if alloc is None:
            def alloc(shape, dtype):
                return torch.zeros(shape, dtype=dtype, device=device)
        self.page_size = rt.page_size
        self.max_pages = (max_seq_len + rt.page_size - 1) // rt.page_size
        self.num_pages = num_seqs * self.max_pages + 1
        self.scratch_page = self.num_pages - 1
        hkv = kv_heads_per_rank(cfg, rt.tp)
        self.storage = alloc((cfg.n_layers, self.num_pages, 2, hkv, rt.page_size, cfg.head_dim), torch.bfloat16)
        self.layers = [A.PagedKVCache(self.num_pages, hkv, rt.page_size, device, storage=self.storage[l])
                       for l in range(cfg.n_layers)]
        self.page_table = alloc((num_seqs, self.max_pages), torch.int32)
        self.seq_lens = alloc((num_seqs,), torch.int32)
        self.free_pages = list(range(self.num_pages - 2, -1, -1))
        self.owned: dict[int, list[int]] = {}
        # host mirror of the page table (pinned where possible): rows are edited here and copied over when they changed
        self.table_host = torch.full((num_seqs, self.max_pages), self.scratch_page, dtype=torch.int32)
        if torch.cuda.is_available() and torch.device(device).type == "cuda":
            self.table_host = self.table_host.pin_memory()
        self._dirty = True
        self.pages_high_water = 0

    def admit(self, seq: int, n_tokens: int) -> None:
        """Make sure sequence slot ``seq`` owns pages for ``n_tokens`` tokens (grows, never shrinks)."""
        need = (n_tokens + self.page_size - 1) // self.page_size
        if need > self.max_pages:
            raise RuntimeError(f"{n_tokens} tokens exceed the {self.max_pages * self.page_size} a page-table row can describe")
        have = self.owned.setdefault(seq, [])
        if need - len(have) > len(self.free_pages):
            raise RuntimeError("KV cache exhausted")
        while len(have) < need:
            self.table_host[seq, len(have)] = self.free_pages[-1]
            have.append(self.free_pages.pop())
            self._dirty = True
        self.pages_high_water = max(self.pages_high_water, self.num_pages - 1 - len(self.free_pages))

    def release(self, seq: int) -> None:
        """Give the pages of slot ``seq`` back; its page-table row points at the scratch page again."""
        pages = self.owned.pop(seq, [])
        if pages:
            self.free_pages.extend(reversed(pages))
            self.table_host[seq].fill_(self.scratch_page)
            self._dirty = True

    def flush(self) -> None:
        """Copy the page table to the device if a row changed since the last flush (asynchronous, stream-ordered)."""
        if self._dirty:
            self.page_table.copy_(self.table_host, non_blocking=True)
            self._dirty = False

    def pages_in_use(self) -> int:
        return self.num_pages - 1 - len(self.free_pages)


def own_last_rows(last_idx: torch.Tensor, a: int, b: int):
    """For a rank that owns token rows [a, b): which of the sequences' last rows (global indices ``last_idx``) it holds
    (bool [n, 1]) and where they sit in its local tensors (clamped so that the gather is always in range)."""
    mine = ((last_idx >= a) & (last_idx < b)).unsqueeze(1)
    loc = (last_idx - a).clamp(0, max(b - a - 1, 0))
    return mine, loc


class Decoder:
    def __init__(self, cfg: ModelConfig, rt: RuntimeConfig, weights: dict, comm: Comm | None = None, device=None,
                 tp_ctx=None):
        self.cfg, self.rt, self.w = cfg, rt, weights
        self.comm = comm or Comm.single()
        self.tp_ctx = tp_ctx          # parallel.tp.TPContext: peer-memory collectives (None: NCCL between kernels)
        self.device = device or weights["embed"].device
        self.hq = cfg.n_heads // rt.tp
        self.hkv = kv_heads_per_rank(cfg, rt.tp)
        self.cos, self.sin = A.rope_tables(rt.max_seq_len, cfg.rope_theta, self.device, cfg.head_dim)
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        self.moe = None
        if cfg.is_moe:
            from .moe import MoEBlock
            self.moe = MoEBlock(cfg, rt, self.comm, self.device, tp_ctx=tp_ctx)
        self._decode_scratch: dict[int, A.DecodeAttnScratch] = {}
        import os
        # decode attention with rope / KV append / output quantisation folded in (B200RT_FUSED_ATTN=0: three launches)
        self.fused_attention = os.environ.get("B200RT_FUSED_ATTN", "1") not in ("0", "false")
        # fused decode attention may give a CTA up to 9 blocks of 128 cached tokens (no KV split at batch 32 x 1,024)
        self.long_attention = os.environ.get("B200RT_ATTN_LONG", "1") not in ("0", "false")
        # decode linears that run their own activation prologue (norm / SwiGLU + rotation + int8) in quantiser CTAs of
        # the GEMM launch.  Opt-in (B200RT_FUSED_QUANT=1): the hand-over of the int8 rows between CTAs of one launch (flag
        # in L2, acquire, proxy fence) measured slower than the kernel boundary it replaces (programmatic dependent
        # launch already overlaps that boundary): 5 instead of 8 launches per layer but +10..15 us per layer.
        self.fused_quant = os.environ.get("B200RT_FUSED_QUANT", "0") not in ("0", "false")
        # Up to four tokens the GEMM CTAs can quantise their own K slice of the rows (no extra CTAs, no flags: the row
        # statistics cross the split-K cluster through distributed shared memory).  Opt-in as well: 5 launches per layer
        # instead of 8, but measured slower at batch 1 (4 layers of the 1/8 shard: 227 us against 177 us) - the
        # prologue's serial steps (load, two reductions, cluster exchange, pack, proxy fence) run on four warps of every
        # CTA and cost more than the stand-alone kernel plus its boundary.
        self.inline_quant = os.environ.get("B200RT_INLINE_QUANT", "0") not in ("0", "false")

    # -- building blocks ------------------------------------------------------------------------------------
    def _norm_quant(self, h, delta, gamma, want_normed=False):
        if delta is None:
            return L.act_quant(h, mode=L.AQ_NORM, gamma=gamma, eps=self.cfg.eps, want_normed=want_normed)
        return L.act_quant(delta, mode=L.AQ_ADD_NORM, gamma=gamma, eps=self.cfg.eps, residual=h, want_normed=want_normed)

    def _row_parallel(self, xq, sx, lw):
        """Row-parallel linear: local partial product, then the cross-rank sum."""
        if self.tp_ctx is not None:
            return self.tp_ctx.row_parallel(xq, sx, lw)
        y = L.w8a8_gemm(xq, sx, lw.qweight, lw.scale)
        return self.comm.all_reduce(y)

    def _attention(self, l, qkv, positions, kv: KVState, mode, cu_seqlens, max_len, seq_ids):
        W = self.w["layers"][l]
        M = qkv.shape[0]
        cache = kv.layers[l]
        if mode == "prefill":
            k_rot = torch.empty((M, self.hkv, self.cfg.head_dim), dtype=torch.bfloat16, device=qkv.device)
            q = A.rope_kv_write(qkv, positions, self.cos, self.sin, self.hq, self.hkv, k_out=k_rot, cache=cache,
                                page_table=kv.page_table, seq_ids=seq_ids, q_norm_w=W.get("q_norm"),
                                k_norm_w=W.get("k_norm"), eps=self.cfg.eps)
            v = qkv.view(M, self.hq + 2 * self.hkv, self.cfg.head_dim)[:, self.hq + self.hkv:]
            return A.attn_prefill(q, k_rot, v, cu_seqlens, max_len, scale=self.scale)
        impl = A.decode_impl(cache.page_size, self.hq // self.hkv)
        if impl in ("tc", "tcp"):
            splits = A.pick_decode_splits_tc(M, self.hkv, kv.page_table.shape[1] * cache.page_size,
                                             fused=(impl == "tc" and self.fused_attention and self.long_attention
                                                    and self.hq // self.hkv <= 8))
        else:
            splits = A.pick_decode_splits(M, self.hkv, max_len)
        fused = impl == "tc" and self.fused_attention
        sc = None
        if splits > 1 or fused:
            sc = self._decode_scratch.get((M, splits))
            if sc is None:
                sc = A.DecodeAttnScratch(M, self.hq, self.hkv, splits, qkv.device)
                self._decode_scratch[(M, splits)] = sc
        if fused:
            # one launch: per-head norm + rotary embedding + KV append + attention + rotation / int8 of the output
            xq, sx, _ = A.attn_decode_fused(qkv, positions, self.cos, self.sin, self.hq, self.hkv, cache, kv.page_table,
                                            kv.seq_lens, scratch=sc, splits=splits, scale=self.scale,
                                            q_norm_w=W.get("q_norm"), k_norm_w=W.get("k_norm"), eps=self.cfg.eps,
                                            next_weights=W["o"].qweight)
            return xq, sx
        q = A.rope_kv_write(qkv, positions, self.cos, self.sin, self.hq, self.hkv, cache=cache,
                            page_table=kv.page_table, seq_ids=None, q_norm_w=W.get("q_norm"),
                            k_norm_w=W.get("k_norm"), eps=self.cfg.eps)
        return A.attn_decode(q, cache, kv.page_table, kv.seq_lens, scratch=sc, splits=splits, scale=self.scale)

    def _fused_norm_linear(self, h, delta, gamma, lw, h_out=None):
        """(residual add +) RMSNorm + rotation + int8 + column-parallel linear as one launch (decode, <= 64 tokens).
        With ``h_out`` the updated residual stream ``h + delta`` is written there instead of in place."""
        if delta is None:
            return L.fused_linear(h, lw.qweight, lw.scale, mode=L.QR_NORM, gamma=gamma, eps=self.cfg.eps, inline=self.inline_quant)
        return L.fused_linear(delta, lw.qweight, lw.scale, mode=L.QR_ADD_NORM, gamma=gamma, eps=self.cfg.eps, residual=h,
                              residual_out=h_out, inline=self.inline_quant)

    def _fused_swiglu_down(self, gu, lw):
        """SwiGLU + rotation + int8 + row-parallel down projection (+ all-reduce under tensor parallelism): one launch."""
        if self.tp_ctx is not None:
            y = self.tp_ctx.row_parallel_fused(gu, lw, L.QR_SWIGLU, inline=self.inline_quant)
            if y is not None:
                return y
        if self.comm.world > 1:
            hq, sh = L.act_quant(gu, mode=L.AQ_SWIGLU)
            return self._row_parallel(hq, sh, lw)
        return L.fused_linear(gu, lw.qweight, lw.scale, mode=L.QR_SWIGLU, inline=self.inline_quant)

    def _mlp(self, l, xq, sx, xn):
        W = self.w["layers"][l]
        if self.moe is not None:
            return self.moe.forward(W, xq, sx, xn)
        gu = L.w8a8_gemm(xq, sx, W["gate_up"].qweight, W["gate_up"].scale)
        hq, sh = L.act_quant(gu, mode=L.AQ_SWIGLU)
        return self._row_parallel(hq, sh, W["down"])

    # -- full forward ------------------------------------------------------------------------------------------
    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor, kv: KVState, *, mode: str,
                cu_seqlens: torch.Tensor | None = None, max_len: int = 0, seq_ids: torch.Tensor | None = None,
                last_idx: torch.Tensor | None = None) -> torch.Tensor:
        """token_ids int64 [M], positions int32 [M] -> greedy next token per sequence (int64).

        mode "prefill": M = all prompt tokens (concatenated), ``last_idx`` selects each sequence's last row;
        mode "decode":  M = batch, one token per sequence, kv.seq_lens already counts the current token.
        """
        cfg = self.cfg
        if (mode == "prefill" and self.tp_ctx is not None and last_idx is not None
                and self.tp_ctx.sp_ok(token_ids.shape[0], moe=self.moe is not None)):
            return self._forward_prefill_sharded(token_ids, positions, kv, cu_seqlens, max_len, seq_ids, last_idx)
        h = A.embed_gather(token_ids, self.w["embed"])
        delta = None
        d_ok = cfg.d_model % 128 == 0 and cfg.d_model <= L.FUSED_PROLOG_MAX_K
        M = token_ids.shape[0]
        # a few tokens: the linears quantise their own operand inside the GEMM CTAs (always on); more: quantiser CTAs
        # in the launch (opt-in)
        fq = ((self.fused_quant and M <= L.DECODE_MAX_M) or (self.inline_quant and M <= L.INLINE_PROLOG_MAX_M)) and mode == "decode" and d_ok
        # The inline form reads the old residual in every cluster, so the sum goes to a second buffer and the two swap.
        h_alt = torch.empty_like(h) if fq else None
        for l in range(cfg.n_layers):
            W = self.w["layers"][l]
            if fq:
                qkv = self._fused_norm_linear(h, delta, W["attn_norm"], W["qkv"], h_alt)
                if delta is not None:
                    h, h_alt = h_alt, h
            else:
                xq, sx = self._norm_quant(h, delta, W["attn_norm"])
                qkv = L.w8a8_gemm(xq, sx, W["qkv"].qweight, W["qkv"].scale)
            with op_range(f"layer{l}.attention.{mode}"):
                attn = self._attention(l, qkv, positions, kv, mode, cu_seqlens, max_len, seq_ids)
            aq, sa = attn if isinstance(attn, tuple) else L.act_quant(attn.view(attn.shape[0], -1))
            with op_range(f"layer{l}.o_proj+allreduce"):
                delta = self._row_parallel(aq, sa, W["o"])
            if fq and self.moe is None:
                gu = self._fused_norm_linear(h, delta, W["mlp_norm"], W["gate_up"], h_alt)
                h, h_alt = h_alt, h
                delta = self._fused_swiglu_down(gu, W["down"])
                continue
            xq, sx = self._norm_quant(h, delta, W["mlp_norm"])      # the router, too, consumes the quantised rows
            with op_range(f"layer{l}.mlp"):
                delta = self._mlp(l, xq, sx, None)
        if last_idx is not None:
            h = h.index_select(0, last_idx)
            delta = delta.index_select(0, last_idx)
        return self._sample(h, delta)

    def _forward_prefill_sharded(self, token_ids, positions, kv, cu_seqlens, max_len, seq_ids, last_idx):
        """Tensor-parallel prefill with the residual stream sharded by token: this rank normalises and quantises only
        the rows it owns, column-parallel linears gather the int8 rows inside the GEMM kernel, row-parallel linears
        reduce-scatter their partial sums from the GEMM epilogue, and mixture-of-experts layers dispatch rows to the
        experts' ranks and combine the outputs back at the owners.  Attention sees all tokens of its own heads exactly
        as in the replicated path."""
        cfg, sp = self.cfg, self.tp_ctx.sp
        M = token_ids.shape[0]
        a, b = sp.my_rows(M)
        h = A.embed_gather(token_ids[a:b], self.w["embed"])
        delta = None
        for l in range(cfg.n_layers):
            W = self.w["layers"][l]
            xq, sx = self._norm_quant(h, delta, W["attn_norm"])
            qkv = sp.ag_linear(xq, sx, W["qkv"].qweight, W["qkv"].scale, M)
            attn = self._attention(l, qkv, positions, kv, "prefill", cu_seqlens, max_len, seq_ids)
            aq, sa = L.act_quant(attn.view(M, -1))
            delta = sp.rs_linear(aq, sa, W["o"].qweight, W["o"].scale)[: b - a]
            xq, sx = self._norm_quant(h, delta, W["mlp_norm"])
            if self.moe is not None:
                delta = self.moe.forward_sharded(W, xq, sx, M)[: b - a]
                continue
            gu = sp.ag_linear(xq, sx, W["gate_up"].qweight, W["gate_up"].scale, M)
            hq, sh = L.act_quant(gu, mode=L.AQ_SWIGLU)
            delta = sp.rs_linear(hq, sh, W["down"].qweight, W["down"].scale)[: b - a]
        # each sequence's last row lives on exactly one rank: the others contribute zeros to a small all-reduce
        mine, loc = own_last_rows(last_idx, a, b)
        d = cfg.d_model
        nb = last_idx.shape[0]

        def produce(buf):
            buf[:, :d] = torch.where(mine, h.index_select(0, loc), torch.zeros((), dtype=h.dtype, device=h.device))
            buf[:, d:] = torch.where(mine, delta.index_select(0, loc), torch.zeros((), dtype=h.dtype, device=h.device))
        both = self.tp_ctx.reduce_partial(produce, nb, 2 * d).clone()
        return self._sample(both[:, :d].contiguous(), both[:, d:].contiguous())

    def _sample(self, h, delta):
        with op_range("lm_head+argmax"):
            return self._sample_body(h, delta)

    def _sample_body(self, h, delta):
        xq, sx = self._norm_quant(h, delta, self.w["final_norm"])
        lm = self.w["lm_head"]
        logits = L.w8a8_gemm(xq, sx, lm.qweight, lm.scale)
        val, idx = A.argmax_rows(logits, index_offset=self.w["vocab_offset"])
        self.last_logits = logits
        if self.tp_ctx is not None:
            return self.tp_ctx.argmax(val, idx)
        if self.comm.world > 1:
            val, idx = self.comm.all_gather(val), self.comm.all_gather(idx)
        return A.argmax_merge(val, idx)
