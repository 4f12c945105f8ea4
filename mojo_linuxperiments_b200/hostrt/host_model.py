"""Decoder forward pass on the host CPUs: every W8A8 Hadamard linear runs on the host runtime's pinned worker pools
(AMX int8 tiles / AVX-512 VNNI, ``csrc/hostrt/w8a8_host.cpp``), the glue around them (RMSNorm, RoPE, attention over a
contiguous KV cache, SwiGLU, expert routing) is PyTorch on the CPU.  It consumes the same checkpoint dictionary as the GPU
engine's ``shard_from_checkpoint`` and the oracle, so it doubles as an end-to-end check of the host linear against the
oracle and as the CPU point of the decode benchmark.  The reference itself has no model code
(test_linux_threading.mojo only exercises pools, arenas and two reductions)."""
from __future__ import annotations

import torch

from . import HostWeights, NumaInfo, WorkerTeam, w8a8_linear
from ..oracle import attention as OA
from ..oracle import quant as Q

BF = torch.bfloat16


class HostDecoder:
    def __init__(self, cfg, ck: dict, info: NumaInfo | None = None, isa: str = "best"):
        self.cfg, self.ck = cfg, ck
        self.info = info or NumaInfo()
        self.team = WorkerTeam(self.info)          # parked workers: a decode step is ~7 linears per layer
        self.isa = isa
        self.linear_ns = 0
        # every dense linear's weights go into the NUMA arena of the node whose workers stream them (fused where the
        # GPU engine fuses them); expert weights stay in the checkpoint tensors
        self._w = {}
        for l in range(cfg.n_layers):
            p = f"layers.{l}."
            self._w[p + "qkv"] = self._place(p, ("wq", "wk", "wv"))
            self._w[p + "wo"] = self._place(p, ("wo",))
            if not cfg.is_moe:
                self._w[p + "gate_up"] = self._place(p, ("gate", "up"))
                self._w[p + "down"] = self._place(p, ("down",))
        self._w["lm_head"] = HostWeights(self.team, ck["lm_head.qweight"].contiguous(), ck["lm_head.scale"])
        self.reset()

    def _place(self, p, names) -> HostWeights:
        q = torch.cat([self.ck[p + n + ".qweight"] for n in names], 0).contiguous()
        s = torch.cat([self.ck[p + n + ".scale"] for n in names], 0).contiguous()
        return HostWeights(self.team, q, s)          # the concatenated copy is dropped once it sits in the arenas

    def reset(self):
        self.k_cache = [None] * self.cfg.n_layers
        self.v_cache = [None] * self.cfg.n_layers
        self.pos = 0

    # ---- linears on the worker pools ----------------------------------------------------------------------------
    def _lin(self, x: torch.Tensor, qweight, scale=None, fp32_out: bool = False) -> torch.Tensor:
        """``qweight``: a ``HostWeights`` (node-local shards) or an int8 tensor with its ``scale``."""
        if isinstance(qweight, HostWeights):
            r = w8a8_linear(self.info, x.to(BF).contiguous(), None, None, isa=self.isa, weights=qweight)
            scale = qweight.sw
        else:
            r = w8a8_linear(self.info, x.to(BF).contiguous(), qweight, scale, isa=self.isa, team=self.team)
        if r["status"] != 0:
            raise RuntimeError(f"host linear failed with status {r['status']}")
        self.linear_ns += r["quant_ns"] + r["gemm_ns"]
        if fp32_out:       # the exact accumulators, scaled without the bf16 rounding of the output
            return r["acc"].float() * r["sx"][:, None] * scale[None, :]
        return r["y"]

    def _moe(self, p: str, xn: torch.Tensor) -> torch.Tensor:
        cfg, ck = self.cfg, self.ck
        logits = self._lin(xn, ck[p + "router.qweight"], ck[p + "router.scale"], fp32_out=True)
        topv, topi = logits.softmax(-1).topk(cfg.top_k, dim=-1)
        if cfg.norm_topk_prob:
            topv = topv / topv.sum(-1, keepdim=True)
        out = torch.zeros((xn.shape[0], cfg.d_model), dtype=torch.float32)
        for e in range(cfg.n_experts):
            sel = topi == e
            rows = sel.any(-1).nonzero().flatten()
            if rows.numel() == 0:
                continue
            gq = torch.cat([ck[p + f"experts.{e}.gate.qweight"], ck[p + f"experts.{e}.up.qweight"]], 0).contiguous()
            gs = torch.cat([ck[p + f"experts.{e}.gate.scale"], ck[p + f"experts.{e}.up.scale"]], 0).contiguous()
            gu = self._lin(xn[rows], gq, gs)
            y = self._lin(Q.swiglu(gu), ck[p + f"experts.{e}.down.qweight"], ck[p + f"experts.{e}.down.scale"]).float()
            out[rows] += (topv * sel)[rows].sum(-1, keepdim=True) * y
        return out.to(BF)

    # ---- one forward step over T new tokens of a single sequence ------------------------------------------------
    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        """ids int64 [T] appended at the current position -> fp32 logits [vocab] of the last token."""
        cfg, ck = self.cfg, self.ck
        T, hd = ids.numel(), cfg.head_dim
        pos = torch.arange(self.pos, self.pos + T)
        h = ck["embed"][ids].to(BF)
        for l in range(cfg.n_layers):
            p = f"layers.{l}."
            xn = Q.rmsnorm(h, ck[p + "attn_norm"], cfg.eps)
            qkv = self._lin(xn, self._w[p + "qkv"]).view(T, cfg.n_heads + 2 * cfg.n_kv_heads, hd)
            q, k, v = qkv[:, : cfg.n_heads], qkv[:, cfg.n_heads: cfg.n_heads + cfg.n_kv_heads], qkv[:, cfg.n_heads + cfg.n_kv_heads:]
            if cfg.qk_norm:
                q = OA.head_rmsnorm(q, ck[p + "q_norm"], cfg.eps)
                k = OA.head_rmsnorm(k, ck[p + "k_norm"], cfg.eps)
            q = OA.rope(q, pos, cfg.rope_theta).to(BF)
            k = OA.rope(k, pos, cfg.rope_theta).to(BF)
            self.k_cache[l] = k if self.k_cache[l] is None else torch.cat([self.k_cache[l], k], 0)
            self.v_cache[l] = v.to(BF) if self.v_cache[l] is None else torch.cat([self.v_cache[l], v.to(BF)], 0)
            attn = self._attend(q, self.k_cache[l], self.v_cache[l]).to(BF).reshape(T, -1)
            h = (h.float() + self._lin(attn, self._w[p + "wo"]).float()).to(BF)
            xn = Q.rmsnorm(h, ck[p + "mlp_norm"], cfg.eps)
            if cfg.is_moe:
                delta = self._moe(p, xn)
            else:
                gu = self._lin(xn, self._w[p + "gate_up"])
                delta = self._lin(Q.swiglu(gu), self._w[p + "down"])
            h = (h.float() + delta.float()).to(BF)
        self.pos += T
        xn = Q.rmsnorm(h[-1:], ck["final_norm"], cfg.eps)
        return self._lin(xn, self._w["lm_head"]).float()[0]

    def _attend(self, q, k_all, v_all):
        """q [T, hq, D] (the last T positions), k_all / v_all [S, hkv, D] -> [T, hq, D] fp32, causal."""
        T, S = q.shape[0], k_all.shape[0]
        qpos = torch.arange(S - T, S)[:, None]
        mask = torch.arange(S)[None, :] <= qpos                       # [T, S]: key s visible to query t
        out = torch.nn.functional.scaled_dot_product_attention(
            q.float().transpose(0, 1)[None], k_all.float().transpose(0, 1)[None], v_all.float().transpose(0, 1)[None],
            attn_mask=mask, enable_gqa=True)
        return out[0].transpose(0, 1)

    def generate(self, prompt: torch.Tensor, n_new: int):
        """Greedy tokens after ``prompt`` (int64 [S]); returns (tokens, per-step logits)."""
        self.reset()
        toks, logs = [], []
        lg = self.forward(prompt)
        for i in range(n_new):
            t = int(lg.argmax())
            toks.append(t)
            logs.append(lg)
            if i + 1 < n_new:
                lg = self.forward(torch.tensor([t]))
        return toks, logs
