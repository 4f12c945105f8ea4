"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some hosts of the kernel library may never call the CUDA allocator (all HBM already belongs to their own arena, or they
are plain C programs without any pooling allocator), so ``b200_attn_decode_noalloc`` keeps its split-KV scratch in a
fixed device array inside the library.  This file checks it against the regular entry point (caller-owned scratch) on
two calls in a row, and that oversize requests are refused.  It is named to be collected last."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
D = 128


def _setup(B, hq, hkv, lens, seed):
    from mojo_linuxperiments_b200.ops import attention as A
    ps = 16
    max_pages = (max(lens) + ps - 1) // ps
    g = torch.Generator().manual_seed(seed)
    page_table = torch.randperm(B * max_pages, generator=g).to(torch.int32).view(B, max_pages).cuda()
    cache = A.PagedKVCache(B * max_pages, hkv, ps, "cuda")
    cache.data.copy_(torch.randn(tuple(cache.data.shape), generator=g).to(torch.bfloat16))
    q = torch.randn((B, hq, D), generator=g).to(torch.bfloat16).cuda()
    seq_lens = torch.tensor(lens, dtype=torch.int32).cuda()
    return cache, page_table, seq_lens, q


def _noalloc(lib, q, cache, page_table, seq_lens, splits):
    B, hq, _ = q.shape
    out = torch.empty_like(q)
    torch.cuda.synchronize()
    held = torch.cuda.memory_allocated()
    rc = lib.b200_attn_decode_noalloc(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(cache.data.data_ptr()), ctypes.c_void_p(page_table.data_ptr()),
        ctypes.c_void_p(seq_lens.data_ptr()), ctypes.c_void_p(out.data_ptr()), B, hq, cache.kv_heads, cache.page_size,
        page_table.shape[1], splits, ctypes.c_float(1.0 / math.sqrt(D)),
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == held        # nothing was taken from (or returned to) torch's allocator
    return rc, out


def test_noalloc_entry_point_matches_regular_one_twice_in_a_row():
    from mojo_linuxperiments_b200.ops import _lib
    from mojo_linuxperiments_b200.ops import attention as A
    lib = _lib.lib()
    for call, (lens, hq, hkv, splits, seed) in enumerate([([700, 33, 1280, 5], 32, 8, 4, 1), ([64, 900, 1, 257], 8, 2, 6, 2)]):
        cache, page_table, seq_lens, q = _setup(len(lens), hq, hkv, lens, seed)
        ref = A.attn_decode(q, cache, page_table, seq_lens, splits=splits, impl="simple")
        rc, out = _noalloc(lib, q, cache, page_table, seq_lens, splits)
        assert rc == 0, f"call {call}: rc {rc}"
        assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=2e-2), (out.float() - ref.float()).abs().max().item()


def test_noalloc_entry_point_takes_any_batch_when_nothing_is_split():
    """With one split the kernel needs neither partials nor counters, so the built-in array's limits do not apply:
    B * hkv = 5,000 (sequence, head) pairs is beyond the 4,096 counters and must still be served."""
    from mojo_linuxperiments_b200.ops import _lib
    from mojo_linuxperiments_b200.ops import attention as A
    lib = _lib.lib()
    B, hq, hkv = 2500, 4, 2
    lens = [1 + (i * 7) % 48 for i in range(B)]
    cache, page_table, seq_lens, q = _setup(B, hq, hkv, lens, 4)
    ref = A.attn_decode(q, cache, page_table, seq_lens, splits=1, impl="simple")
    rc, out = _noalloc(lib, q, cache, page_table, seq_lens, 1)
    assert rc == 0
    assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


def test_noalloc_entry_point_rejects_requests_beyond_its_scratch(capfd):
    from mojo_linuxperiments_b200.ops import _lib
    lib = _lib.lib()
    cache, page_table, seq_lens, q = _setup(2, 8, 2, [40, 50], 3)
    # 32 splits x 64 heads x 4097 sequences of partials would need far more than the built-in 1 Mi floats
    out = torch.empty_like(q)
    rc = lib.b200_attn_decode_noalloc(
        ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(cache.data.data_ptr()), ctypes.c_void_p(page_table.data_ptr()),
        ctypes.c_void_p(seq_lens.data_ptr()), ctypes.c_void_p(out.data_ptr()), 4097, 64, 8, 16, page_table.shape[1], 32,
        ctypes.c_float(0.1), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -30
    assert "built-in" in capfd.readouterr().err
    torch.cuda.synchronize()
