"""GPU baseline: the same W8A8 Hadamard decoder (dense and mixture-of-experts) written with stock PyTorch ops only -
cuBLASLt int8 GEMMs (torch._int_mm), a matmul with H128 for the rotation, scaled_dot_product_attention, NCCL all-reduce
between ops - with the same engine interface as the product so bench.py can time both.  None of this package's kernels
run here.  Experts use replicated tokens like the product: prefill gathers each local expert's rows (data-dependent
shapes, eager only); decode evaluates every local expert on all rows and masks, which is what makes the step
capturable in a CUDA graph.  The engine also runs on the CPU (eager), which is how the tests check it against the oracle."""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F

from mojo_linuxperiments_b200.models import weights as Wt
from mojo_linuxperiments_b200.models.config import ModelConfig, RuntimeConfig, kv_heads_per_rank
from mojo_linuxperiments_b200.oracle.quant import hadamard_matrix
from mojo_linuxperiments_b200.parallel.comm import Comm


class BaselineEngine:
    def __init__(self, cfg: ModelConfig, rt: RuntimeConfig, weights: dict | None = None, seed: int = 0, comm: Comm | None = None,
                 device=None):
        self.cfg, self.rt = cfg, rt
        self.comm = comm or Comm.single()
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.w = weights or Wt.random_shard(cfg, rt.tp, self.comm.rank, self.device, seed)
        for L in self.w["layers"]:
            for k in ("qkv", "o", "gate_up", "down", "router"):
                if k in L:
                    L[k + "_t"] = L[k].qweight.t()      # _int_mm wants [K, N] (column-major view is fine)
            if cfg.is_moe:
                L["experts_gate_up_t"] = L["experts_gate_up"].qweight.transpose(1, 2)     # [E_local, d, 2F]
                L["experts_down_t"] = L["experts_down"].qweight.transpose(1, 2)           # [E_local, F, d]
        self.n_local = cfg.n_experts // max(rt.ep, 1) if cfg.is_moe else 0
        self.e0 = self.comm.rank * self.n_local if rt.ep > 1 else 0
        self.w["lm_head_t"] = self.w["lm_head"].qweight.t()
        self.H = hadamard_matrix(128, torch.bfloat16, self.device)
        self.hq = cfg.n_heads // rt.tp
        self.hkv = kv_heads_per_rank(cfg, rt.tp)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float64) / cfg.head_dim))
        ang = torch.arange(rt.max_seq_len, dtype=torch.float64)[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos().float().to(self.device), ang.sin().float().to(self.device)
        self._graphs = {}
        self._stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self.kernels_per_step = 0

    # ---- ops -------------------------------------------------------------------------------------------------
    def _quant(self, x):
        M, K = x.shape
        xr = (x.view(M, K // 128, 128) @ self.H).view(M, K).float()
        s = xr.abs().amax(dim=1).clamp_min(1e-20) / 127.0
        q = torch.clamp(torch.round(xr / s[:, None]), -127, 127).to(torch.int8)
        return q, s

    def _int_linear(self, q, s, wt, sw, out_dtype=torch.bfloat16):
        M = q.shape[0]
        if M <= 16:
            q = F.pad(q, (0, 0, 0, 32 - M))             # cuBLASLt's int8 path wants more than 16 rows
        acc = torch._int_mm(q, wt)[:M]
        return (acc.float() * s[:, None] * sw[None, :]).to(out_dtype)

    def _linear(self, x, wt, sw):
        q, s = self._quant(x)
        return self._int_linear(q, s, wt, sw)

    def _head_norm(self, x, g):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * g.float()).to(torch.bfloat16)

    def _moe(self, x, L, decode: bool):
        """x bf16 [T, d] (normalised) -> this rank's partial MoE output bf16 [T, d] (summed over ranks by the caller)."""
        cfg = self.cfg
        q, s = self._quant(x)
        logits = self._int_linear(q, s, L["router_t"], L["router"].scale, out_dtype=torch.float32)
        topv, topi = logits.softmax(-1).topk(cfg.top_k, dim=-1)
        if cfg.norm_topk_prob:
            topv = topv / topv.sum(-1, keepdim=True)
        out = torch.zeros((x.shape[0], cfg.d_model), dtype=torch.float32, device=x.device)
        gu_s, dn_s = L["experts_gate_up"].scale, L["experts_down"].scale
        for j in range(self.n_local):
            sel = topi == (self.e0 + j)
            wgt = (topv * sel).sum(-1, keepdim=True)                  # 0 for rows that did not pick this expert
            if decode:
                qe, se, rows = q, s, None                             # all rows, masked by the zero weight
            else:
                rows = sel.any(-1).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                qe, se, wgt = q[rows], s[rows], wgt[rows]
            gu = self._int_linear(qe, se, L["experts_gate_up_t"][j], gu_s[j])
            f = gu.shape[1] // 2
            act = (F.silu(gu[:, :f].float()) * gu[:, f:].float()).to(torch.bfloat16)
            y = self._linear(act, L["experts_down_t"][j], dn_s[j]).float()
            if rows is None:
                out += wgt * y
            else:
                out.index_add_(0, rows, wgt * y)
        return out.to(torch.bfloat16)

    def _norm(self, x, g):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.eps) * g.float()).to(torch.bfloat16)

    def _rope(self, x, pos):
        d = x.shape[-1]
        cos, sin = self.cos[pos][:, None, :], self.sin[pos][:, None, :]
        xf = x.float()
        a, b = xf[..., : d // 2], xf[..., d // 2:]
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1).to(torch.bfloat16)

    def _forward(self, ids, pos, B, S, decode: bool):
        cfg = self.cfg
        hd = cfg.head_dim
        h = self.w["embed"][ids]
        for l, L in enumerate(self.w["layers"]):
            x = self._norm(h, L["attn_norm"])
            qkv = self._linear(x, L["qkv_t"], L["qkv"].scale).view(-1, self.hq + 2 * self.hkv, hd)
            q, k, v = qkv[:, : self.hq], qkv[:, self.hq: self.hq + self.hkv], qkv[:, self.hq + self.hkv:]
            if cfg.qk_norm:
                q, k = self._head_norm(q, L["q_norm"]), self._head_norm(k, L["k_norm"])
            q, k = self._rope(q, pos), self._rope(k, pos)
            if decode:
                self.k_cache[l].scatter_(2, self.pos_idx[:, None, None, None].expand(B, self.hkv, 1, hd), k.view(B, self.hkv, 1, hd))
                self.v_cache[l].scatter_(2, self.pos_idx[:, None, None, None].expand(B, self.hkv, 1, hd), v.view(B, self.hkv, 1, hd))
                kk, vv = self.k_cache[l][:, :, : self.ctx_cap], self.v_cache[l][:, :, : self.ctx_cap]
                attn = F.scaled_dot_product_attention(q.view(B, self.hq, 1, hd), kk, vv, attn_mask=self.mask, enable_gqa=True)
                attn = attn.reshape(B, self.hq * hd)
            else:
                qb = q.view(B, S, self.hq, hd).transpose(1, 2)
                kb = k.view(B, S, self.hkv, hd).transpose(1, 2)
                vb = v.view(B, S, self.hkv, hd).transpose(1, 2)
                self.k_cache[l][:, :, :S] = kb
                self.v_cache[l][:, :, :S] = vb
                attn = F.scaled_dot_product_attention(qb, kb, vb, is_causal=True, enable_gqa=True)
                attn = attn.transpose(1, 2).reshape(B * S, self.hq * hd)
            o = self._linear(attn, L["o_t"], L["o"].scale)
            h = h + self.comm.all_reduce(o)
            x = self._norm(h, L["mlp_norm"])
            if cfg.is_moe:
                d = self._moe(x, L, decode)
            else:
                gu = self._linear(x, L["gate_up_t"], L["gate_up"].scale)
                f = gu.shape[1] // 2
                act = (F.silu(gu[:, :f].float()) * gu[:, f:].float()).to(torch.bfloat16)
                d = self._linear(act, L["down_t"], L["down"].scale)
            h = h + self.comm.all_reduce(d)
        if not decode:
            h = h.view(B, S, -1)[:, -1]
        x = self._norm(h, self.w["final_norm"])
        logits = self._linear(x, self.w["lm_head_t"], self.w["lm_head"].scale)
        val, idx = logits.float().max(dim=1)
        idx = idx + self.w["vocab_offset"]
        if self.comm.world > 1:
            vals, idxs = self.comm.all_gather(val), self.comm.all_gather(idx)
            idx = idxs.gather(0, vals.argmax(dim=0, keepdim=True))[0]
        return idx

    # ---- engine interface ------------------------------------------------------------------------------------------
    def start_batch(self, batch: int, max_total_len: int) -> None:
        cfg = self.cfg
        self.batch = batch
        self.ctx_cap = (max_total_len + 63) // 64 * 64
        shape = (cfg.n_layers, batch, self.hkv, self.ctx_cap, cfg.head_dim)
        if getattr(self, "k_cache", None) is None or tuple(self.k_cache.shape) != shape:
            self.k_cache = torch.zeros(shape, dtype=torch.bfloat16, device=self.device)
            self.v_cache = torch.zeros(shape, dtype=torch.bfloat16, device=self.device)
        self.tokens = torch.zeros(batch, dtype=torch.int64, device=self.device)
        self.pos_idx = torch.zeros(batch, dtype=torch.int64, device=self.device)
        self.mask = torch.zeros((batch, 1, 1, self.ctx_cap), dtype=torch.bool, device=self.device)
        self._graphs.clear()

    def prefill(self, prompts: torch.Tensor) -> torch.Tensor:
        B, S = prompts.shape
        ids = prompts.to(self.device, non_blocking=True).reshape(-1)
        pos = torch.arange(S, device=self.device).repeat(B)
        nxt = self._forward(ids, pos, B, S, decode=False)
        self.tokens.copy_(nxt)
        self.pos_idx.fill_(S)
        self.mask.zero_()
        self.mask[..., : S + 1] = True
        return nxt

    def _decode_body(self):
        nxt = self._forward(self.tokens, self.pos_idx, self.batch, 1, decode=True)
        self.tokens.copy_(nxt)
        self.pos_idx.add_(1)
        self.mask.scatter_(3, self.pos_idx[:, None, None, None], True)

    def decode_step(self, use_graph: bool = True) -> torch.Tensor:
        if not use_graph or self.device.type != "cuda":
            self._decode_body()
            return self.tokens
        g = self._graphs.get(self.batch)
        if g is None:
            saved = (self.tokens.clone(), self.pos_idx.clone(), self.mask.clone())
            self._stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._stream):
                self._decode_body()
            torch.cuda.current_stream().wait_stream(self._stream)
            torch.cuda.synchronize()
            self.tokens.copy_(saved[0]); self.pos_idx.copy_(saved[1]); self.mask.copy_(saved[2])
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self._stream):
                self._decode_body()
            self.tokens.copy_(saved[0]); self.pos_idx.copy_(saved[1]); self.mask.copy_(saved[2])
            self._graphs[self.batch] = g
        g.replay()
        return self.tokens

    def step_from_host(self, ids_in: torch.Tensor, ids_out: torch.Tensor) -> torch.Tensor:
        self.tokens.copy_(ids_in, non_blocking=True)
        nxt = self.decode_step()
        ids_out.copy_(nxt, non_blocking=True)
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        return ids_out

    def generate(self, prompts: torch.Tensor, max_new_tokens: int, use_graph: bool = True) -> torch.Tensor:
        """Greedy generation. prompts int64 [B, S] -> int64 [B, max_new_tokens] on the host."""
        B, S = prompts.shape
        self.start_batch(B, S + max_new_tokens)
        out = [self.prefill(prompts).cpu()]
        for _ in range(1, max_new_tokens):
            out.append(self.decode_step(use_graph).cpu().clone())
        return torch.stack(out, 1)
