"""Weights of the W8A8 models: int8 rotated weight + fp32 per-output-channel scale per linear, bf16 elsewhere.

Checkpoint layout (safetensors): ``<name>.qweight`` int8 [N, K] (K contiguous, already Hadamard-rotated along K in
blocks of 128), ``<name>.scale`` fp32 [N]; norms, embeddings and the router in bf16; the metadata carries the
ModelConfig, ``hadamard_block`` and ``rotated``.  Tensor-parallel ranks slice the same tensors:
  column-parallel (qkv, gate_up, lm_head, experts' gate_up): rows of [N, K]
  row-parallel    (o_proj, down, experts' down):              columns of [N, K] in multiples of 128, scale shared
"""
from __future__ import annotations

import json
from dataclasses import dataclass

import torch

from ..oracle import quant as Q
from .config import ModelConfig, kv_head_of_rank, kv_heads_per_rank


@dataclass
class LinearW:
    qweight: torch.Tensor     # int8 [N, K]
    scale: torch.Tensor       # fp32 [N]

    @property
    def out_features(self) -> int: return self.qweight.shape[0]
    @property
    def in_features(self) -> int: return self.qweight.shape[1]

    def to(self, device) -> "LinearW":
        return LinearW(self.qweight.to(device).contiguous(), self.scale.to(device).contiguous())


def quantize_linear(w_fp32: torch.Tensor) -> LinearW:
    q, s = Q.quantize_weight(w_fp32)
    return LinearW(q.contiguous(), s.contiguous())


def random_linear(n: int, k: int, device, gen: torch.Generator, std: float = 0.02) -> LinearW:
    """Random int8 weight generated in place on the device (no fp32 master): uniform int8, scale set so that the
    dequantised weight has standard deviation ~``std``."""
    q = torch.randint(-127, 128, (n, k), dtype=torch.int8, device=device, generator=gen)
    s = (torch.rand((n,), device=device, generator=gen) * 0.5 + 0.75) * (std / 73.3)
    return LinearW(q, s.float())


# ---------------------------------------------------------------------------------------------------------
# full-precision master weights (small models: tests, oracles, checkpoints)
# ---------------------------------------------------------------------------------------------------------
def init_master(cfg: ModelConfig, seed: int = 0) -> dict:
    """fp32 weights of the whole model on the CPU, keyed like the checkpoint."""
    g = torch.Generator().manual_seed(seed)
    d, hd = cfg.d_model, cfg.head_dim

    def w(n, k, std=None):
        return torch.randn((n, k), generator=g) * (std if std is not None else k ** -0.5)

    def gamma(n):
        return 1.0 + 0.1 * torch.randn((n,), generator=g)

    m = {"embed": torch.randn((cfg.vocab, d), generator=g) * 1.0, "final_norm": gamma(d), "lm_head": w(cfg.vocab, d)}
    for l in range(cfg.n_layers):
        p = f"layers.{l}."
        m[p + "attn_norm"] = gamma(d)
        m[p + "wq"] = w(cfg.n_heads * hd, d)
        m[p + "wk"] = w(cfg.n_kv_heads * hd, d)
        m[p + "wv"] = w(cfg.n_kv_heads * hd, d)
        m[p + "wo"] = w(d, cfg.n_heads * hd)
        if cfg.qk_norm:
            m[p + "q_norm"] = gamma(hd)
            m[p + "k_norm"] = gamma(hd)
        m[p + "mlp_norm"] = gamma(d)
        if cfg.is_moe:
            m[p + "router"] = torch.randn((cfg.n_experts, d), generator=g) * 0.02 * 8
            for e in range(cfg.n_experts):
                m[p + f"experts.{e}.gate"] = w(cfg.moe_ffn, d)
                m[p + f"experts.{e}.up"] = w(cfg.moe_ffn, d)
                m[p + f"experts.{e}.down"] = w(d, cfg.moe_ffn)
        else:
            m[p + "gate"] = w(cfg.ffn, d)
            m[p + "up"] = w(cfg.ffn, d)
            m[p + "down"] = w(d, cfg.ffn)
    return m


LINEAR_SUFFIXES = ("wq", "wk", "wv", "wo", "gate", "up", "down", "lm_head", "router")


def quantize_master(master: dict) -> dict:
    """checkpoint-layout dict: linears -> .qweight/.scale (int8 rotated + fp32), everything else bf16."""
    out = {}
    for name, t in master.items():
        if name.split(".")[-1] in LINEAR_SUFFIXES:
            lw = quantize_linear(t)
            out[name + ".qweight"] = lw.qweight
            out[name + ".scale"] = lw.scale
        else:
            out[name] = t.to(torch.bfloat16)
    return out


def save_checkpoint(path: str, cfg: ModelConfig, tensors: dict) -> None:
    from safetensors.torch import save_file
    meta = {"config": cfg.to_json(), "hadamard_block": str(cfg.hadamard_block), "rotated": "true", "format": "w8a8-hadamard-v1"}
    save_file({k: v.contiguous().cpu() for k, v in tensors.items()}, path, metadata=meta)


def load_checkpoint(path: str):
    from safetensors import safe_open
    tensors = {}
    with safe_open(path, framework="pt") as f:
        meta = f.metadata()
        for k in f.keys():
            tensors[k] = f.get_tensor(k)
    if meta.get("rotated") != "true" or int(meta.get("hadamard_block", "0")) != 128:
        raise ValueError("checkpoint is not in the rotated block-128 W8A8 layout")
    return ModelConfig.from_json(meta["config"]), tensors


class _LazyTensor:
    """A tensor of an open safetensors file that is only read where it is sliced: ``t[a:b]`` / ``t[:, a:b]`` read
    those rows / columns, ``t.to(device)`` reads all of it."""

    def __init__(self, reader: "ShardReader", name: str):
        self.reader, self.name = reader, name

    def _count(self, t: torch.Tensor) -> torch.Tensor:
        self.reader.bytes_read += t.numel() * t.element_size()
        return t

    def __getitem__(self, idx) -> torch.Tensor:
        return self._count(self.reader.file.get_slice(self.name)[idx])

    def full(self) -> torch.Tensor:
        return self._count(self.reader.file.get_tensor(self.name))

    def to(self, *args, **kw) -> torch.Tensor:
        return self.full().to(*args, **kw)


class ShardReader:
    """Dict-like view of a checkpoint file whose tensors are read slice by slice (``shard_from_checkpoint`` then pulls
    only this rank's rows / columns of every linear from the file instead of materialising the whole model per rank)."""

    def __init__(self, path: str):
        from safetensors import safe_open
        self._ctx = safe_open(path, framework="pt")
        self.file = self._ctx.__enter__()
        self.meta = self.file.metadata()
        self.names = set(self.file.keys())
        self.bytes_read = 0
        if self.meta.get("rotated") != "true" or int(self.meta.get("hadamard_block", "0")) != 128:
            self.close()
            raise ValueError("checkpoint is not in the rotated block-128 W8A8 layout")

    def __getitem__(self, name: str) -> _LazyTensor:
        if name not in self.names:
            raise KeyError(name)
        return _LazyTensor(self, name)

    def config(self) -> ModelConfig:
        return ModelConfig.from_json(self.meta["config"])

    def close(self) -> None:
        if self._ctx is not None:
            self._ctx.__exit__(None, None, None)
            self._ctx = None


def load_shard(path: str, tp: int, rank: int, device):
    """(config, this rank's weights) read from a checkpoint file without loading the other ranks' shards."""
    rd = ShardReader(path)
    try:
        cfg = rd.config()
        w = shard_from_checkpoint(cfg, rd, tp, rank, device)
        w["checkpoint_bytes_read"] = rd.bytes_read
        return cfg, w
    finally:
        rd.close()


def _full(t):
    return t.full() if isinstance(t, _LazyTensor) else t


# ---------------------------------------------------------------------------------------------------------
# per-rank model weights
# ---------------------------------------------------------------------------------------------------------
def _lin(ck: dict, name: str) -> LinearW:
    return LinearW(ck[name + ".qweight"], ck[name + ".scale"])


def _rows(lw: LinearW, a: int, b: int) -> LinearW:
    return LinearW(lw.qweight[a:b], lw.scale[a:b])


def _cols(lw: LinearW, a: int, b: int) -> LinearW:
    return LinearW(lw.qweight[:, a:b], _full(lw.scale))


def _cat_rows(*ls: LinearW) -> LinearW:
    return LinearW(torch.cat([_full(l.qweight) for l in ls], 0), torch.cat([_full(l.scale) for l in ls], 0))


def shard_from_checkpoint(cfg: ModelConfig, ck: dict, tp: int, rank: int, device) -> dict:
    """This rank's weights (fused qkv / gate_up layouts the kernels consume) cut from a full checkpoint dict."""
    hd, d = cfg.head_dim, cfg.d_model
    hq_l = cfg.n_heads // tp
    hkv_l = kv_heads_per_rank(cfg, tp)
    kv0 = kv_head_of_rank(cfg, tp, rank)
    vs = (cfg.vocab + tp - 1) // tp
    w = {"embed": ck["embed"].to(device), "final_norm": ck["final_norm"].to(device),
         "lm_head": _rows(_lin(ck, "lm_head"), rank * vs, min(cfg.vocab, (rank + 1) * vs)).to(device),
         "vocab_offset": rank * vs, "layers": []}
    for l in range(cfg.n_layers):
        p = f"layers.{l}."
        q = _rows(_lin(ck, p + "wq"), rank * hq_l * hd, (rank + 1) * hq_l * hd)
        k = _rows(_lin(ck, p + "wk"), kv0 * hd, (kv0 + hkv_l) * hd)
        v = _rows(_lin(ck, p + "wv"), kv0 * hd, (kv0 + hkv_l) * hd)
        L = {"attn_norm": ck[p + "attn_norm"].to(device), "mlp_norm": ck[p + "mlp_norm"].to(device),
             "qkv": _cat_rows(q, k, v).to(device),
             "o": _cols(_lin(ck, p + "wo"), rank * hq_l * hd, (rank + 1) * hq_l * hd).to(device)}
        if cfg.qk_norm:
            L["q_norm"] = ck[p + "q_norm"].to(device)
            L["k_norm"] = ck[p + "k_norm"].to(device)
        if cfg.is_moe:
            L["router"] = _lin(ck, p + "router").to(device)        # replicated: every rank routes identically
            epr = cfg.n_experts // tp
            gu, dn = [], []
            for e in range(rank * epr, (rank + 1) * epr):
                gu.append(_cat_rows(_lin(ck, p + f"experts.{e}.gate"), _lin(ck, p + f"experts.{e}.up")))
                dn.append(_lin(ck, p + f"experts.{e}.down"))
            L["experts_gate_up"] = LinearW(torch.stack([x.qweight for x in gu]).to(device).contiguous(),
                                           torch.stack([x.scale for x in gu]).to(device).contiguous())
            L["experts_down"] = LinearW(torch.stack([_full(x.qweight) for x in dn]).to(device).contiguous(),
                                        torch.stack([_full(x.scale) for x in dn]).to(device).contiguous())
        else:
            fs = cfg.ffn // tp
            L["gate_up"] = _cat_rows(_rows(_lin(ck, p + "gate"), rank * fs, (rank + 1) * fs),
                                     _rows(_lin(ck, p + "up"), rank * fs, (rank + 1) * fs)).to(device)
            L["down"] = _cols(_lin(ck, p + "down"), rank * fs, (rank + 1) * fs).to(device)
        w["layers"].append(L)
    return w


def random_shard(cfg: ModelConfig, tp: int, rank: int, device, seed: int = 0) -> dict:
    """Random-init weights of this rank's shard generated directly on the device (benchmarks: no checkpoint, no
    host copy; a 235B-parameter shape never exists in one place)."""
    gen = torch.Generator(device=device).manual_seed(seed * 1000 + rank)
    shared = torch.Generator(device=device).manual_seed(seed * 1000 + 999)      # replicated tensors: same on all ranks
    hd, d = cfg.head_dim, cfg.d_model
    hq_l = cfg.n_heads // tp
    hkv_l = kv_heads_per_rank(cfg, tp)
    vs = (cfg.vocab + tp - 1) // tp

    def gamma(n):
        return (1.0 + 0.05 * torch.randn((n,), device=device, generator=shared)).to(torch.bfloat16)

    w = {"embed": (torch.randn((cfg.vocab, d), device=device, generator=shared)).to(torch.bfloat16),
         "final_norm": gamma(d),
         "lm_head": random_linear(min(cfg.vocab, (rank + 1) * vs) - rank * vs, d, device, gen, std=d ** -0.5),
         "vocab_offset": rank * vs, "layers": []}
    for _ in range(cfg.n_layers):
        L = {"attn_norm": gamma(d), "mlp_norm": gamma(d),
             "qkv": random_linear((hq_l + 2 * hkv_l) * hd, d, device, gen, std=d ** -0.5),
             "o": random_linear(d, hq_l * hd, device, gen, std=(cfg.n_heads * hd) ** -0.5)}
        if cfg.qk_norm:
            L["q_norm"], L["k_norm"] = gamma(hd), gamma(hd)
        if cfg.is_moe:
            epr = cfg.n_experts // tp
            L["router"] = random_linear(cfg.n_experts, d, device, shared, std=0.02)
            gu = random_linear(epr * 2 * cfg.moe_ffn, d, device, gen, std=d ** -0.5)
            dn = random_linear(epr * d, cfg.moe_ffn, device, gen, std=cfg.moe_ffn ** -0.5)
            L["experts_gate_up"] = LinearW(gu.qweight.view(epr, 2 * cfg.moe_ffn, d), gu.scale.view(epr, 2 * cfg.moe_ffn))
            L["experts_down"] = LinearW(dn.qweight.view(epr, d, cfg.moe_ffn), dn.scale.view(epr, d))
        else:
            fs = cfg.ffn // tp
            L["gate_up"] = random_linear(2 * fs, d, device, gen, std=d ** -0.5)
            L["down"] = random_linear(d, fs, device, gen, std=cfg.ffn ** -0.5)
        w["layers"].append(L)
    return w
