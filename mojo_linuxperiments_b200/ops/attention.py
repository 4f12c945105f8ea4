"""RoPE + paged-KV write, prefill (tcgen05) and decode (split-KV) attention, embedding gather, greedy argmax."""
from __future__ import annotations

import math

import torch

from . import _lib
from .workspace import default_workspace

HEAD_DIM = 128


def rope_tables(max_pos: int, theta: float, device, head_dim: int = HEAD_DIM):
    """cos/sin tables [max_pos, head_dim/2] fp32 for the rotate-half convention (pairs i, i + head_dim/2)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    ang = torch.arange(max_pos, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device).contiguous(), ang.sin().float().to(device).contiguous()


class PagedKVCache:
    """One layer's paged KV storage: [num_pages][2][kv_heads][page_size][128] bf16."""

    def __init__(self, num_pages: int, kv_heads: int, page_size: int, device, storage: torch.Tensor | None = None):
        shape = (num_pages, 2, kv_heads, page_size, HEAD_DIM)
        self.data = storage if storage is not None else torch.zeros(shape, dtype=torch.bfloat16, device=device)
        assert tuple(self.data.shape) == shape
        self.num_pages, self.kv_heads, self.page_size = num_pages, kv_heads, page_size


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, hq: int, hkv: int, *,
                  q_out: torch.Tensor | None = None, k_out: torch.Tensor | None = None, v_out: torch.Tensor | None = None,
                  cache: PagedKVCache | None = None, page_table: torch.Tensor | None = None,
                  seq_ids: torch.Tensor | None = None, q_norm_w=None, k_norm_w=None, eps: float = 1e-6):
    """qkv bf16 [M, (hq + 2 hkv) * 128] -> rotated q [M, hq, 128]; k, v appended to ``cache`` at (sequence, position)."""
    M = qkv.shape[0]
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[1] == (hq + 2 * hkv) * HEAD_DIM
    assert positions.dtype == torch.int32
    if q_out is None:
        q_out = torch.empty((M, hq, HEAD_DIM), dtype=torch.bfloat16, device=qkv.device)
    rc = _lib.lib().b200_rope_kv_write(
        qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), _lib.ptr(seq_ids), cos.data_ptr(), sin.data_ptr(),
        _lib.ptr(q_norm_w), _lib.ptr(k_norm_w), float(eps), q_out.data_ptr(), _lib.ptr(k_out), _lib.ptr(v_out),
        cache.data.data_ptr() if cache is not None else None, _lib.ptr(page_table),
        page_table.shape[1] if page_table is not None else 0, cache.page_size if cache is not None else 0,
        hq, hkv, M, cos.shape[0], cache.num_pages if cache is not None else 0,
        default_workspace(qkv.device).status.data_ptr(), _lib.stream())
    _lib.check(rc, "rope_kv_write")
    return q_out


_PREFILL_SPLIT_SCRATCH: dict = {}


def attn_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor, max_len: int,
                 scale: float | None = None, out: torch.Tensor | None = None, kv_chunk: int | None = None) -> torch.Tensor:
    """Causal GQA attention over concatenated sequences. q [T, hq, 128], k/v [T, hkv, 128] (token stride free).

    ``kv_chunk`` > 0 selects the split-KV form: every ``kv_chunk`` KV tiles of 128 tokens of a query tile are a CTA of
    their own and a merge kernel combines them - more parallelism when there are few (sequence, head) pairs.  Default
    (``None``): B200RT_PREFILL_SPLIT if set, else split exactly when the un-split grid would not fill the GPU."""
    T, hq, d = q.shape
    hkv = k.shape[1]
    assert d == HEAD_DIM and q.dtype == torch.bfloat16 and q.stride(2) == 1 and q.stride(1) == d
    assert k.stride(2) == 1 and k.stride(1) == d and v.stride(2) == 1 and v.stride(1) == d
    assert cu_seqlens.dtype == torch.int32
    if out is None:
        out = torch.empty((T, hq, d), dtype=torch.bfloat16, device=q.device)
    ws = default_workspace(q.device)
    if kv_chunk is None:
        import os
        env = os.environ.get("B200RT_PREFILL_SPLIT", "")
        if env != "":
            kv_chunk = int(env)
        else:
            # Few (sequence, head, query tile) CTAs leave most SMs idle while the last query tiles walk their KV tiles
            # alone: split the KV range then (measured on B200: 1 x 1,024 tokens x 4 heads 33 -> 16 us, 1 x 4,096 x 4
            # heads 143 -> 103 us; with >= 148 CTAs the un-split kernel is faster).
            B_ = cu_seqlens.numel() - 1
            n_q = (int(max_len) + 127) // 128
            sms = _lib.num_sms(q.device.index)
            kv_chunk = 0
            if B_ * hq * n_q < sms and n_q > 1:
                kv_chunk = max(1, min(8, B_ * hq * n_q * (n_q + 1) // 2 // sms))
    if kv_chunk > 0:
        B = cu_seqlens.numel() - 1
        n = _lib.lib().b200_attn_prefill_split_scratch_floats(B, hq, int(max_len), kv_chunk)
        key = (q.device.index, n)
        scratch = _PREFILL_SPLIT_SCRATCH.get(key)
        if scratch is None:
            scratch = _PREFILL_SPLIT_SCRATCH[key] = torch.empty(max(n, 4), dtype=torch.float32, device=q.device)
        rc = _lib.lib().b200_attn_prefill_split(
            q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), out.data_ptr(),
            cu_seqlens.data_ptr(), B, T, int(max_len), hq, hkv,
            float(scale if scale is not None else 1.0 / math.sqrt(d)), kv_chunk, scratch.data_ptr(), ws.status.data_ptr(),
            _lib.stream())
        _lib.check(rc, "attn_prefill_split")
        return out
    rc = _lib.lib().b200_attn_prefill(
        q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0), out.data_ptr(),
        cu_seqlens.data_ptr(), cu_seqlens.numel() - 1, T, int(max_len), hq, hkv,
        float(scale if scale is not None else 1.0 / math.sqrt(d)), ws.status.data_ptr(), _lib.stream())
    _lib.check(rc, "attn_prefill")
    return out


class DecodeAttnScratch:
    def __init__(self, B: int, hq: int, hkv: int, splits: int, device):
        n = _lib.lib().b200_attn_decode_scratch_floats(B, hq, splits)
        self.buf = torch.empty(max(n, 1), dtype=torch.float32, device=device)
        self.counters = torch.zeros(B * hkv, dtype=torch.int32, device=device)
        self.splits = splits
        # the fused kernel's quantising epilogue, when a token's heads span several CTAs (hkv > 1)
        self.rot = torch.empty(B * hq * HEAD_DIM, dtype=torch.float32, device=device) if hkv > 1 else None
        self.blk_amax = torch.zeros(B * hkv, dtype=torch.float32, device=device) if hkv > 1 else None
        self.seq_counters = torch.zeros(B, dtype=torch.int32, device=device) if hkv > 1 else None


TC_BLOCKS_PER_CTA = 4          # the tensor-core decode kernel holds at most 4 x 128 cached tokens per CTA
TC_BLOCKS_PER_CTA_FUSED = 9    # its fused form has a variant without the cluster-merge zone that holds 9 x 128


def tc_min_splits(max_len: int, fused: bool = False) -> int:
    """Fewest KV splits the tensor-core decode kernel accepts for sequences of up to ``max_len`` tokens."""
    blocks = (max_len + 127) // 128
    return max(1, -(-blocks // (TC_BLOCKS_PER_CTA_FUSED if fused else TC_BLOCKS_PER_CTA)))


def decode_impl(page_size: int, group: int) -> str:
    """Which decode-attention kernel "auto" means: the tcgen05 one where it applies (B200RT_ATTN=tma|simple overrides)."""
    import os
    want = os.environ.get("B200RT_ATTN", "tc")
    if page_size == 16 and group in (1, 2, 4, 8, 16):
        return want if want in ("tc", "tcp", "tma", "simple") else "tc"
    return "simple"


def pick_decode_splits_tc(B: int, hkv: int, max_len: int, num_sms: int = 148, fused: bool = False) -> int:
    """KV splits for the tensor-core decode kernel.  Measured on B200 its time is close to
    waves x (128-token blocks per CTA + 1.6) x 2.7 us with two CTAs per SM (the 1.6 is the per-CTA set-up, softmax
    exchange and partial write), plus a little per split for the merge: few, long CTAs win once the grid fills the GPU."""
    blocks = max(1, (max_len + 127) // 128)
    smin = tc_min_splits(max_len, fused)     # fused: a CTA may take a whole sequence (one wave of long CTAs beats three
                                             # of short ones: every CTA pays ~1.6 blocks' worth of set-up and epilogue)
    slots = 2 * num_sms
    best, best_cost = smin, None
    # up to eight splits are one thread-block cluster that merges in shared memory: stay there when that is possible
    cap = 8 if smin <= 8 else 32
    for s in range(smin, max(smin, min(cap, blocks)) + 1):
        cost = -(-(max(1, B * hkv) * s) // slots) * (-(-blocks // s) + 1.6) + 0.15 * s
        if best_cost is None or cost < best_cost - 1e-9:
            best, best_cost = s, cost
    return best


def pick_decode_splits(B: int, hkv: int, max_len: int, num_sms: int = 148, ctas_per_sm: int = 3,
                       min_splits: int = 1) -> int:
    """Number of KV splits: the grid is B * hkv * splits CTAs on num_sms * ctas_per_sm slots, and each CTA's work is
    ~1/splits, so the time is ~ceil(grid / slots) / splits; pick the smallest split count within 5 % of the best,
    keeping at least 64 tokens per split (and at least ``min_splits``)."""
    slots = num_sms * ctas_per_sm
    pairs = max(1, B * hkv)
    max_splits = max(min_splits, min(32, max_len // 64))
    best_cost = min(-(-(pairs * s) // slots) / s for s in range(min_splits, max_splits + 1))
    for s in range(min_splits, max_splits + 1):
        if -(-(pairs * s) // slots) / s <= best_cost * 1.05:
            return s
    return min_splits


def attn_decode(q: torch.Tensor, cache: PagedKVCache, page_table: torch.Tensor, seq_lens: torch.Tensor, *,
                scratch: DecodeAttnScratch | None = None, splits: int = 1, scale: float | None = None,
                out: torch.Tensor | None = None, impl: str = "auto") -> torch.Tensor:
    """q [B, hq, 128] against the first seq_lens[b] cached tokens of sequence b.

    impl "tc" (page size 16, group size 1/2/4/8/16): tcgen05 MMAs for Q.K^T and P.V, scores in TMEM, pages by TMA
    (raises ``splits`` to what the longest representable sequence needs); "tcp": the same as a persistent grid whose
    producer runs ahead into the next work item; "tma": TMA-fed ring with CUDA-core dot
    products; "simple": the general kernel; "auto" picks the first that applies."""
    B, hq, d = q.shape
    assert d == HEAD_DIM and q.is_contiguous() and page_table.dtype == torch.int32 and seq_lens.dtype == torch.int32
    if out is None:
        out = torch.empty_like(q)
    G = hq // cache.kv_heads
    if impl == "auto":
        impl = decode_impl(cache.page_size, G)
    if impl in ("tc", "tcp"):
        splits = max(splits, tc_min_splits(page_table.shape[1] * cache.page_size))
    if splits > 1 and (scratch is None or scratch.splits != splits):
        scratch = DecodeAttnScratch(B, hq, cache.kv_heads, splits, q.device)
    if impl in ("tc", "tcp", "tma"):
        fn = {"tc": _lib.lib().b200_attn_decode_tc, "tcp": _lib.lib().b200_attn_decode_tcp,
              "tma": _lib.lib().b200_attn_decode_tma}[impl]
        extra = (_lib.num_sms(q.device.index),) if impl == "tcp" else ()
        rc = fn(
            q.data_ptr(), cache.data.data_ptr(), cache.num_pages, page_table.data_ptr(), seq_lens.data_ptr(), out.data_ptr(),
            scratch.buf.data_ptr() if scratch is not None else None,
            scratch.counters.data_ptr() if scratch is not None else None,
            B, hq, cache.kv_heads, cache.page_size, page_table.shape[1], splits,
            float(scale if scale is not None else 1.0 / math.sqrt(d)), default_workspace(q.device).status.data_ptr(),
            *extra, _lib.stream())
        _lib.check(rc, "attn_decode_" + impl)
        return out
    rc = _lib.lib().b200_attn_decode(
        q.data_ptr(), cache.data.data_ptr(), page_table.data_ptr(), seq_lens.data_ptr(), out.data_ptr(),
        scratch.buf.data_ptr() if scratch is not None else None,
        scratch.counters.data_ptr() if scratch is not None else None,
        B, hq, cache.kv_heads, cache.page_size, page_table.shape[1], splits,
        float(scale if scale is not None else 1.0 / math.sqrt(d)), default_workspace(q.device).status.data_ptr(),
        _lib.stream())
    _lib.check(rc, "attn_decode")
    return out


def attn_decode_fused(qkv: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, hq: int, hkv: int,
                      cache: PagedKVCache, page_table: torch.Tensor, seq_lens: torch.Tensor, *,
                      scratch: DecodeAttnScratch | None = None, splits: int = 1, scale: float | None = None,
                      q_norm_w=None, k_norm_w=None, eps: float = 1e-6, quantize: bool = True, want_out: bool = False,
                      next_weights: torch.Tensor | None = None):
    """One launch for rope_kv_write + decode attention + the activation prologue of o_proj.

    qkv bf16 [B, (hq + 2 hkv) * 128]: the new token's raw projections; ``positions[b]`` is where it goes in the cache and
    ``seq_lens[b]`` counts it.  Returns ``(xq int8 [B, hq*128], sx fp32 [B], out bf16 [B, hq, 128] or None)``; with
    ``quantize=False`` only ``out``.  Needs page size 16 and a group size of 1/2/4/8/16 (the tcgen05 kernel).
    ``next_weights``: a constant tensor the following kernel streams (the o-projection's int8 weights); the kernel's CTAs
    ask for it to be brought into L2 meanwhile."""
    B = qkv.shape[0]
    d = HEAD_DIM
    assert qkv.dtype == torch.bfloat16 and qkv.stride(1) == 1 and qkv.shape[1] == (hq + 2 * hkv) * d
    assert positions.dtype == torch.int32 and page_table.dtype == torch.int32 and seq_lens.dtype == torch.int32
    assert cache.page_size == 16 and cache.kv_heads == hkv and hq // hkv in (1, 2, 4, 8, 16)
    # nine blocks per CTA only up to eight heads per KV head (the scores stay in registers)
    splits = max(splits, tc_min_splits(page_table.shape[1] * cache.page_size, fused=hq // hkv <= 8))
    if scratch is None or scratch.splits != splits:
        scratch = DecodeAttnScratch(B, hq, hkv, splits, qkv.device)
    out = torch.empty((B, hq, d), dtype=torch.bfloat16, device=qkv.device) if (want_out or not quantize) else None
    xq = torch.empty((B, hq * d), dtype=torch.int8, device=qkv.device) if quantize else None
    sx = torch.empty((B,), dtype=torch.float32, device=qkv.device) if quantize else None
    rc = _lib.lib().b200_attn_decode_fused(
        qkv.data_ptr(), qkv.stride(0), positions.data_ptr(), cos.data_ptr(), sin.data_ptr(), cos.shape[0],
        _lib.ptr(q_norm_w), _lib.ptr(k_norm_w), float(eps), cache.data.data_ptr(), cache.num_pages, page_table.data_ptr(),
        seq_lens.data_ptr(), _lib.ptr(out), _lib.ptr(xq), xq.stride(0) if xq is not None else 0, _lib.ptr(sx),
        scratch.buf.data_ptr(), scratch.counters.data_ptr(), _lib.ptr(scratch.rot), _lib.ptr(scratch.blk_amax),
        _lib.ptr(scratch.seq_counters), B, hq, hkv, cache.page_size, page_table.shape[1], splits,
        float(scale if scale is not None else 1.0 / math.sqrt(d)), default_workspace(qkv.device).status.data_ptr(),
        _lib.ptr(next_weights), next_weights.numel() * next_weights.element_size() if next_weights is not None else 0,
        _lib.stream())
    _lib.check(rc, "attn_decode_fused")
    return (xq, sx, out) if quantize else out


def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    assert ids.dtype == torch.int64 and table.dtype == torch.bfloat16 and table.is_contiguous()
    M, d = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty((M, d), dtype=torch.bfloat16, device=table.device)
    _lib.check(_lib.lib().b200_embed_gather(ids.data_ptr(), table.data_ptr(), out.data_ptr(), M, d, table.shape[0],
                                            _lib.stream()), "embed_gather")
    return out


def argmax_rows(logits: torch.Tensor, index_offset: int = 0, chunks: int | None = None):
    """Candidates (max value fp32, index int64 + offset) per row of bf16 logits [rows, n], one per column chunk:
    returns ([chunks, rows], [chunks, rows]); ``argmax_merge`` picks the winner (lowest index wins ties)."""
    rows, n = logits.shape
    assert logits.dtype == torch.bfloat16 and logits.stride(1) == 1
    if chunks is None:
        chunks = max(1, min(64, n // 2048, 296 // max(rows, 1) + 1))
    out_val = torch.empty((chunks, rows), dtype=torch.float32, device=logits.device)
    out_idx = torch.empty((chunks, rows), dtype=torch.int64, device=logits.device)
    _lib.check(_lib.lib().b200_argmax_rows(logits.data_ptr(), logits.stride(0), rows, n, index_offset, chunks,
                                           out_val.data_ptr(), out_idx.data_ptr(), _lib.stream()), "argmax_rows")
    return out_val, out_idx


def argmax_merge(cand_val: torch.Tensor, cand_idx: torch.Tensor, out_idx: torch.Tensor | None = None) -> torch.Tensor:
    """cand_* [..., rows] (any number of leading candidate dims) -> global argmax index per row."""
    rows = cand_val.shape[-1]
    cand_val = cand_val.reshape(-1, rows)
    cand_idx = cand_idx.reshape(-1, rows)
    world = cand_val.shape[0]
    if out_idx is None:
        out_idx = torch.empty(rows, dtype=torch.int64, device=cand_val.device)
    _lib.check(_lib.lib().b200_argmax_merge(cand_val.data_ptr(), cand_idx.data_ptr(), world, rows, out_idx.data_ptr(),
                                            _lib.stream()), "argmax_merge")
    return out_idx
