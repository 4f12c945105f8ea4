"""Model and runtime configuration.

The reference configures everything through compile-time parameters (ThreadPool[stack_size, mask_size],
NumaArena[alignment, page_size], threading/linux_threading.mojo:44, threading/numa_arena.mojo:6); the inference
layer here is configured by two small dataclasses plus ``B200RT_*`` environment overrides for debugging.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field, replace


@dataclass(frozen=True)
class ModelConfig:
    name: str
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    ffn: int                      # dense SwiGLU width (0 for pure-MoE models)
    vocab: int
    head_dim: int = 128
    rope_theta: float = 500000.0
    eps: float = 1e-5
    n_experts: int = 0
    top_k: int = 0
    moe_ffn: int = 0              # per-expert SwiGLU width
    qk_norm: bool = False         # per-head RMSNorm on q and k before RoPE (Qwen3)
    norm_topk_prob: bool = True   # renormalise the top-k router weights
    hadamard_block: int = 128

    @property
    def is_moe(self) -> bool:
        return self.n_experts > 0

    def to_json(self) -> str:
        return json.dumps(asdict(self))

    @staticmethod
    def from_json(text: str) -> "ModelConfig":
        return ModelConfig(**json.loads(text))

    def weight_bytes(self) -> int:
        """int8 linear weights + bf16 embedding (what one full replica stores)."""
        d, hd = self.d_model, self.head_dim
        attn = d * (self.n_heads + 2 * self.n_kv_heads) * hd + self.n_heads * hd * d
        mlp = 3 * d * self.ffn if not self.is_moe else self.n_experts * 3 * d * self.moe_ffn + d * self.n_experts * 2
        return self.n_layers * (attn + mlp) + self.vocab * d * (1 + 2)


def llama3_8b() -> ModelConfig:
    return ModelConfig("llama3-8b", 32, 4096, 32, 8, 14336, 128256, rope_theta=500000.0, eps=1e-5)


def qwen3_30b_a3b() -> ModelConfig:
    return ModelConfig("qwen3-30b-a3b", 48, 2048, 32, 4, 0, 151936, rope_theta=1000000.0, eps=1e-6,
                       n_experts=128, top_k=8, moe_ffn=768, qk_norm=True)


def qwen3_235b_a22b() -> ModelConfig:
    return ModelConfig("qwen3-235b-a22b", 94, 4096, 64, 4, 0, 151936, rope_theta=1000000.0, eps=1e-6,
                       n_experts=128, top_k=8, moe_ffn=1536, qk_norm=True)


def tiny_dense(n_layers: int = 2, d_model: int = 512, n_heads: int = 4, n_kv_heads: int = 2, ffn: int = 1024,
               vocab: int = 1024) -> ModelConfig:
    """Miniature with the same code path as the Llama shape, small enough for a fp32 oracle."""
    return ModelConfig("tiny-dense", n_layers, d_model, n_heads, n_kv_heads, ffn, vocab)


def tiny_moe(n_layers: int = 2, d_model: int = 512, n_heads: int = 4, n_kv_heads: int = 2, n_experts: int = 16,
             top_k: int = 4, moe_ffn: int = 256, vocab: int = 1024) -> ModelConfig:
    return ModelConfig("tiny-moe", n_layers, d_model, n_heads, n_kv_heads, 0, vocab, rope_theta=1000000.0, eps=1e-6,
                       n_experts=n_experts, top_k=top_k, moe_ffn=moe_ffn, qk_norm=True)


PRESETS = {"llama3-8b": llama3_8b, "qwen3-30b-a3b": qwen3_30b_a3b, "qwen3-235b-a22b": qwen3_235b_a22b,
           "tiny-dense": tiny_dense, "tiny-moe": tiny_moe}


@dataclass(frozen=True)
class RuntimeConfig:
    tp: int = 1                   # tensor-parallel ranks (attention + dense MLP)
    ep: int = 1                   # expert-parallel ranks (MoE experts); equals tp in this runtime
    dp: int = 1                   # kept for completeness; data parallelism is not built
    page_size: int = 16
    max_batch: int = 32
    max_seq_len: int = 2048
    max_prefill_tokens: int = 32768     # most tokens one prefill call may carry (sizes the symmetric TP buffers)
    fused_collectives: bool = True      # in-kernel peer-memory collectives; False = NCCL between kernels
    wait_limit_ms: int = 2000           # bound of every device-side wait
    debug: bool = False

    @staticmethod
    def from_env(**kw) -> "RuntimeConfig":
        cfg = RuntimeConfig(**kw)
        env = os.environ
        if "B200RT_FUSED" in env:
            cfg = replace(cfg, fused_collectives=env["B200RT_FUSED"] not in ("0", "false"))
        if "B200RT_WAIT_LIMIT_MS" in env:
            cfg = replace(cfg, wait_limit_ms=int(env["B200RT_WAIT_LIMIT_MS"]))
        if "B200RT_DEBUG" in env:
            cfg = replace(cfg, debug=env["B200RT_DEBUG"] not in ("0", "false"))
        return cfg


def kv_heads_per_rank(cfg: ModelConfig, tp: int) -> int:
    """KV heads are sharded across ranks; with fewer KV heads than ranks each head is replicated on tp/kv ranks."""
    return max(1, cfg.n_kv_heads // tp)


def kv_head_of_rank(cfg: ModelConfig, tp: int, rank: int) -> int:
    """First global KV head held by ``rank``."""
    if cfg.n_kv_heads >= tp:
        return rank * (cfg.n_kv_heads // tp)
    return rank // (tp // cfg.n_kv_heads)
