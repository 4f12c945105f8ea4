"""Attention-side kernels on the GPU against plain PyTorch fp32 references."""
import math

import os

import pytest
import torch

from mojo_linuxperiments_b200.oracle import attention as OA

pytestmark = pytest.mark.gpu
D = 128


def _rand(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).cuda()


@pytest.mark.parametrize("hq,hkv,qk_norm", [(32, 8, False), (4, 1, False), (8, 1, True)])
def test_rope_kv_write_and_cache_layout(hq, hkv, qk_norm):
    from mojo_linuxperiments_b200.ops import attention as A
    B, S, ps = 3, 37, 16
    theta = 500000.0
    M = B * S
    qkv = _rand((M, (hq + 2 * hkv) * D), 1)
    pos = torch.arange(S, dtype=torch.int32).repeat(B).cuda()
    seq = torch.arange(B, dtype=torch.int32).repeat_interleave(S).cuda()
    max_pages = (S + ps - 1) // ps
    perm = torch.randperm(B * max_pages, generator=torch.Generator().manual_seed(0)).to(torch.int32)
    page_table = perm.view(B, max_pages).cuda()
    cache = A.PagedKVCache(B * max_pages, hkv, ps, qkv.device)
    cos, sin = A.rope_tables(64, theta, qkv.device)
    qw = (torch.rand(D) + 0.5).to(torch.bfloat16).cuda() if qk_norm else None
    kw = (torch.rand(D) + 0.5).to(torch.bfloat16).cuda() if qk_norm else None
    k_out = torch.empty((M, hkv, D), dtype=torch.bfloat16, device=qkv.device)
    q = A.rope_kv_write(qkv, pos, cos, sin, hq, hkv, k_out=k_out, cache=cache, page_table=page_table, seq_ids=seq,
                        q_norm_w=qw, k_norm_w=kw, eps=1e-6)
    torch.cuda.synchronize()
    x = qkv.view(M, hq + 2 * hkv, D)
    q_in, k_in, v_in = x[:, :hq], x[:, hq:hq + hkv], x[:, hq + hkv:]
    if qk_norm:
        q_in, k_in = OA.head_rmsnorm(q_in, qw, 1e-6), OA.head_rmsnorm(k_in, kw, 1e-6)
    q_ref, k_ref = OA.rope(q_in, pos, theta), OA.rope(k_in, pos, theta)
    assert torch.allclose(q.float(), q_ref, rtol=2e-2, atol=2e-2)
    assert torch.allclose(k_out.float(), k_ref, rtol=2e-2, atol=2e-2)
    for b in range(B):
        for t in (0, 15, 16, S - 1):
            page = int(page_table[b, t // ps])
            kc = cache.data[page, 0, :, t % ps]
            vc = cache.data[page, 1, :, t % ps]
            assert torch.equal(kc, k_out[b * S + t])
            assert torch.equal(vc, v_in[b * S + t])


@pytest.mark.parametrize("lens,hq,hkv", [([128], 4, 1), ([256], 8, 2), ([1024], 4, 1), ([100, 333, 128], 4, 1), ([1, 129], 8, 1)])
def test_attn_prefill_matches_reference(lens, hq, hkv):
    from mojo_linuxperiments_b200.ops import attention as A
    from mojo_linuxperiments_b200.ops.workspace import default_workspace
    T = sum(lens)
    q, k, v = _rand((T, hq, D), 1), _rand((T, hkv, D), 2), _rand((T, hkv, D), 3)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32).cuda()
    out = A.attn_prefill(q, k, v, cu, max(lens))
    torch.cuda.synchronize()
    default_workspace(q.device).check_status()
    o = 0
    for L in lens:
        ref = OA.causal_gqa(q[o:o + L], k[o:o + L], v[o:o + L])
        got = out[o:o + L].float()
        assert torch.allclose(got, ref, rtol=3e-2, atol=3e-2), (got - ref).abs().max().item()
        o += L


@pytest.mark.parametrize("lens,hq,hkv", [([128], 4, 1), ([1024], 4, 1), ([100, 333, 128], 4, 1), ([1, 129], 8, 1), ([640], 8, 2)])
@pytest.mark.parametrize("chunk", [1, 2, 3])
def test_attn_prefill_split_kv_matches_reference(lens, hq, hkv, chunk):
    from mojo_linuxperiments_b200.ops import attention as A
    from mojo_linuxperiments_b200.ops.workspace import default_workspace
    T = sum(lens)
    q, k, v = _rand((T, hq, D), 1), _rand((T, hkv, D), 2), _rand((T, hkv, D), 3)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32).cuda()
    out = A.attn_prefill(q, k, v, cu, max(lens), kv_chunk=chunk)
    base = A.attn_prefill(q, k, v, cu, max(lens), kv_chunk=0)
    torch.cuda.synchronize()
    default_workspace(q.device).check_status()
    o = 0
    for L in lens:
        ref = OA.causal_gqa(q[o:o + L], k[o:o + L], v[o:o + L])
        got = out[o:o + L].float()
        assert torch.allclose(got, ref, rtol=3e-2, atol=3e-2), (got - ref).abs().max().item()
        assert torch.allclose(got, base[o:o + L].float(), rtol=2e-2, atol=2e-2)
        o += L


def test_attn_prefill_reads_strided_qkv():
    """K and V can be consumed in place from the fused qkv buffer."""
    from mojo_linuxperiments_b200.ops import attention as A
    T, hq, hkv = 256, 4, 1
    qkv = _rand((T, (hq + 2 * hkv) * D), 7)
    x = qkv.view(T, hq + 2 * hkv, D)
    q, k, v = x[:, :hq], x[:, hq:hq + hkv], x[:, hq + hkv:]
    cu = torch.tensor([0, T], dtype=torch.int32).cuda()
    out = A.attn_prefill(q, k, v, cu, T)
    torch.cuda.synchronize()
    ref = OA.causal_gqa(q, k, v)
    assert torch.allclose(out.float(), ref, rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("hq,hkv", [(32, 8), (4, 1), (8, 1), (16, 1), (2, 2)])
@pytest.mark.parametrize("splits", [1, 4])
@pytest.mark.parametrize("impl", ["simple", "tma", "tc", "tcp"])
def test_attn_decode_paged(hq, hkv, splits, impl):
    from mojo_linuxperiments_b200.ops import attention as A
    if impl in ("tma", "tcp") and hq // hkv == 16:
        pytest.skip("these forms cover group sizes up to 8 (the one-item tcgen05 kernel takes 16)")
    ps = 16
    lens = [1, 17, 300, 1280, 64]
    B = len(lens)
    max_pages = (max(lens) + ps - 1) // ps
    n_pages = B * max_pages
    g = torch.Generator().manual_seed(3)
    page_table = torch.randperm(n_pages, generator=g).to(torch.int32).view(B, max_pages).cuda()
    cache = A.PagedKVCache(n_pages, hkv, ps, "cuda")
    cache.data.copy_(_rand(tuple(cache.data.shape), 5))
    q = _rand((B, hq, D), 6)
    seq_lens = torch.tensor(lens, dtype=torch.int32).cuda()
    out = A.attn_decode(q, cache, page_table, seq_lens, splits=splits, impl=impl)
    out2 = A.attn_decode(q, cache, page_table, seq_lens, splits=splits, impl=impl)     # scratch counters must self-reset
    torch.cuda.synchronize()
    for b, L in enumerate(lens):
        pages = page_table[b, : (L + ps - 1) // ps].long()
        kk = cache.data[pages, 0].permute(0, 2, 1, 3).reshape(-1, hkv, D)[:L]
        vv = cache.data[pages, 1].permute(0, 2, 1, 3).reshape(-1, hkv, D)[:L]
        ref = OA.decode_gqa(q[b], kk, vv)
        assert torch.allclose(out[b].float(), ref, rtol=2e-2, atol=2e-2), (out[b].float() - ref).abs().max().item()
    assert torch.equal(out, out2)


def test_embed_and_argmax():
    from mojo_linuxperiments_b200.ops import attention as A
    table = _rand((1000, 256), 1)
    ids = torch.tensor([0, 999, 5, 5, 123], dtype=torch.int64).cuda()
    assert torch.equal(A.embed_gather(ids, table), table[ids])
    logits = _rand((7, 16032), 2)
    logits[3, 77] = 100.0
    logits[3, 9000] = 100.0       # tie: lowest index wins
    for chunks in (1, 7, None):
        cv, ci = A.argmax_rows(logits, index_offset=1000, chunks=chunks)
        idx = A.argmax_merge(cv, ci)
        torch.cuda.synchronize()
        assert torch.equal(idx - 1000, logits.float().argmax(dim=1))
        assert idx[3].item() == 1077
    val = cv.max(dim=0).values
    cv3 = torch.stack([val, val + 1.0, val - 1.0])
    ci3 = torch.stack([idx, idx + 5, idx + 9])
    assert torch.equal(A.argmax_merge(cv3, ci3), idx + 5)


def test_rope_kv_write_skips_positions_outside_the_admitted_pages():
    """One token past the pages of its sequence (and one past the rotary tables) must be refused with a status code,
    not written to whatever page id lies behind the row of the page table."""
    from mojo_linuxperiments_b200.ops import attention as A
    from mojo_linuxperiments_b200.ops.workspace import default_workspace
    hq, hkv, ps, B = 4, 1, 16, 3
    max_pages = 2                                          # 32 tokens per sequence
    page_table = torch.arange(B * max_pages, dtype=torch.int32).view(B, max_pages).cuda()
    cache = A.PagedKVCache(B * max_pages, hkv, ps, "cuda")
    cos, sin = A.rope_tables(64, 10000.0, "cuda")
    qkv = _rand((B, (hq + 2 * hkv) * D), 7)
    ws = default_workspace(qkv.device)
    ws.status.zero_()
    # sequence 0 in range, sequence 1 one token past its pages, sequence 2 past the tables
    pos = torch.tensor([31, 32, 64], dtype=torch.int32).cuda()
    q_out = torch.full((B, hq, D), 7.0, dtype=torch.bfloat16, device="cuda")
    A.rope_kv_write(qkv, pos, cos, sin, hq, hkv, q_out=q_out, cache=cache, page_table=page_table)
    torch.cuda.synchronize()
    code = int(ws.status[0].item())
    assert code & 255 == 6 and code >> 8 == 7, code          # bad argument, reported by rope_kv_write
    ws.status.zero_()
    assert cache.data[1, :, :, 15].abs().sum().item() > 0    # sequence 0 wrote token 31 (page 1, slot 15)
    assert cache.data[2:].abs().sum().item() == 0             # nothing else was touched
    assert torch.all(q_out[1:] == 7.0) and not torch.all(q_out[0] == 7.0)


@pytest.mark.parametrize("impl", ["simple", "tma", "tc"])
def test_attn_decode_clamps_lengths_beyond_the_page_table_row(impl):
    from mojo_linuxperiments_b200.ops import attention as A
    from mojo_linuxperiments_b200.ops.workspace import default_workspace
    hq, hkv, ps, B = 4, 1, 16, 2
    max_pages = 8                                          # 128 tokens per sequence
    page_table = torch.arange(B * max_pages, dtype=torch.int32).view(B, max_pages).cuda()
    cache = A.PagedKVCache(B * max_pages, hkv, ps, "cuda")
    cache.data.copy_(_rand(tuple(cache.data.shape), 8))
    q = _rand((B, hq, D), 9)
    ws = default_workspace(q.device)
    ws.status.zero_()
    ok = A.attn_decode(q, cache, page_table, torch.tensor([128, 128], dtype=torch.int32).cuda(), impl=impl)
    over = A.attn_decode(q, cache, page_table, torch.tensor([128, 129], dtype=torch.int32).cuda(), impl=impl)
    torch.cuda.synchronize()
    code = int(ws.status[0].item())
    ws.status.zero_()
    assert code & 255 == 6, code
    assert torch.equal(ok, over)                             # the over-long sequence was read as its 128 admitted tokens


@pytest.mark.parametrize("hq,hkv,qk_norm", [(32, 8, False), (4, 1, False), (8, 1, True), (8, 4, True), (2, 2, False),
                                            (16, 1, True), (32, 2, False)])
@pytest.mark.parametrize("splits,longest", [(1, 1280), (4, 1280), (1, 1150), (2, 1025)])
def test_attn_decode_fused_matches_the_three_kernels_it_replaces(hq, hkv, qk_norm, splits, longest):
    """rope_kv_write + attn_decode + act_quant in one launch: same cache contents, same attention output (against the
    fp32 oracle), and exactly the int8 rows / scales the stand-alone prologue makes of that output."""
    from mojo_linuxperiments_b200.ops import attention as A
    from mojo_linuxperiments_b200.ops import linear as L
    from mojo_linuxperiments_b200.ops.workspace import default_workspace
    ps, theta = 16, 500000.0
    # tokens per sequence including the new one; up to 1,152 a CTA of the fused kernel may take a whole sequence (nine
    # blocks of 128, no split), beyond that the splits merge through global memory, with four splits as a cluster
    lens = [1, 17, 300, longest, 64, 128, 513, 1024, min(longest, 1025)]
    B = len(lens)
    max_pages = (max(lens) + ps - 1) // ps
    n_pages = B * max_pages
    g = torch.Generator().manual_seed(11)
    page_table = torch.randperm(n_pages, generator=g).to(torch.int32).view(B, max_pages).cuda()
    cache_a = A.PagedKVCache(n_pages, hkv, ps, "cuda")
    cache_a.data.copy_(_rand(tuple(cache_a.data.shape), 12))
    cache_b = A.PagedKVCache(n_pages, hkv, ps, "cuda")
    cache_b.data.copy_(cache_a.data)
    qkv = _rand((B, (hq + 2 * hkv) * D), 13)
    seq_lens = torch.tensor(lens, dtype=torch.int32).cuda()
    pos = (seq_lens - 1).contiguous()
    cos, sin = A.rope_tables(2048, theta, "cuda")
    qw = (torch.rand(D) + 0.5).to(torch.bfloat16).cuda() if qk_norm else None
    kw = (torch.rand(D) + 0.5).to(torch.bfloat16).cuda() if qk_norm else None
    ws = default_workspace(qkv.device)
    ws.status.zero_()
    # the three separate kernels
    q = A.rope_kv_write(qkv, pos, cos, sin, hq, hkv, cache=cache_a, page_table=page_table, q_norm_w=qw, k_norm_w=kw, eps=1e-6)
    ref_out = A.attn_decode(q, cache_a, page_table, seq_lens, splits=max(splits, 3), impl="tc")
    # the fused kernel, twice (its counters must reset themselves)
    xq, sx, out = A.attn_decode_fused(qkv, pos, cos, sin, hq, hkv, cache_b, page_table, seq_lens, splits=splits,
                                      q_norm_w=qw, k_norm_w=kw, eps=1e-6, want_out=True)
    xq2, sx2, out2 = A.attn_decode_fused(qkv, pos, cos, sin, hq, hkv, cache_b, page_table, seq_lens, splits=splits,
                                         q_norm_w=qw, k_norm_w=kw, eps=1e-6, want_out=True)
    torch.cuda.synchronize()
    assert int(ws.status[0].item()) == 0
    # the cache received the same new rows (one bf16 ulp of slack: the two kernels may contract a*b-c*d differently)
    assert torch.allclose(cache_b.data.float(), cache_a.data.float(), rtol=1e-2, atol=1e-2)
    assert (cache_b.data != cache_a.data).float().mean().item() < 1e-3
    # attention output against the fp32 oracle over the cache that now holds the new token
    for b, Ln in enumerate(lens):
        pages = page_table[b, : (Ln + ps - 1) // ps].long()
        kk = cache_a.data[pages, 0].permute(0, 2, 1, 3).reshape(-1, hkv, D)[:Ln]
        vv = cache_a.data[pages, 1].permute(0, 2, 1, 3).reshape(-1, hkv, D)[:Ln]
        ref = OA.decode_gqa(q[b], kk, vv)
        assert torch.allclose(out[b].float(), ref, rtol=2e-2, atol=2e-2), (b, (out[b].float() - ref).abs().max().item())
        assert torch.allclose(out[b].float(), ref_out[b].float(), rtol=2e-2, atol=2e-2)
    # the quantised rows are exactly what the stand-alone prologue makes of the kernel's own bf16 output
    q_ref, s_ref = L.act_quant(out.view(B, hq * D))
    assert torch.equal(sx, s_ref) and torch.equal(xq, q_ref)
    assert torch.equal(xq, xq2) and torch.equal(sx, sx2) and torch.equal(out, out2)


def test_attn_decode_fused_refuses_a_position_outside_the_pages():
    from mojo_linuxperiments_b200.ops import attention as A
    from mojo_linuxperiments_b200.ops.workspace import default_workspace
    hq, hkv, ps, B = 4, 1, 16, 2
    max_pages = 2
    page_table = torch.arange(B * max_pages, dtype=torch.int32).view(B, max_pages).cuda()
    cache = A.PagedKVCache(B * max_pages, hkv, ps, "cuda")
    cos, sin = A.rope_tables(64, 10000.0, "cuda")
    qkv = _rand((B, (hq + 2 * hkv) * D), 7)
    ws = default_workspace(qkv.device)
    ws.status.zero_()
    seq_lens = torch.tensor([32, 33], dtype=torch.int32).cuda()       # sequence 1 is one token past its two pages
    A.attn_decode_fused(qkv, (seq_lens - 1).contiguous(), cos, sin, hq, hkv, cache, page_table, seq_lens)
    torch.cuda.synchronize()
    code = int(ws.status[0].item())
    ws.status.zero_()
    assert code & 255 == 6, code
    assert cache.data[1, :, :, 15].abs().sum().item() > 0             # sequence 0 appended token 31
    assert cache.data[2:].abs().sum().item() == 0                      # nothing was written for sequence 1
