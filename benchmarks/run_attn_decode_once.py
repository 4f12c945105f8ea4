"""Launch paged decode attention a few times on one shape (for profiler captures).
python benchmarks/run_attn_decode_once.py [impl=fused|tcp|tc|tma|simple] [B=32] [ctx=1024] [hq=32] [hkv=8] [splits=0(auto)]"""
import sys

import torch

import os
import sys as _sys
_sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.ops import attention as A

impl = sys.argv[1] if len(sys.argv) > 1 else "tma"
B, ctx, hq, hkv, splits = [int(a) for a in (sys.argv[2:7] + ["32", "1024", "32", "8", "0"][len(sys.argv) - 2:])][:5] if len(sys.argv) > 2 else (32, 1024, 32, 8, 0)
dev = torch.device("cuda", 0)
ps = 16
max_pages = (ctx + 64 + ps - 1) // ps
n_layers = 3
caches = [A.PagedKVCache(B * max_pages, hkv, ps, dev) for _ in range(n_layers)]
for c in caches:
    c.data.normal_()
pt = torch.arange(B * max_pages, dtype=torch.int32, device=dev).view(B, max_pages)
lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
q = torch.randn((B, hq, 128), device=dev).to(torch.bfloat16)
if splits <= 0 and impl != "fused":
    if impl in ("tc", "tcp"):
        splits = A.pick_decode_splits_tc(B, hkv, max_pages * ps)
    else:
        splits = A.pick_decode_splits(B, hkv, ctx + 64)
sc = A.DecodeAttnScratch(B, hq, hkv, max(splits, 1), dev)
out = torch.empty_like(q)
if impl == "fused":
    # the decoder's form: RoPE + KV append + attention + rotate / quantise of the output in one launch
    qkv = torch.randn((B, (hq + 2 * hkv) * 128), device=dev).to(torch.bfloat16)
    pos = (lens - 1).contiguous()
    cos, sin = A.rope_tables(ctx + 64, 500000.0, dev)
    if len(sys.argv) <= 6 or int(sys.argv[6]) <= 0:
        splits = A.pick_decode_splits_tc(B, hkv, max_pages * ps, fused=True)
    sc = A.DecodeAttnScratch(B, hq, hkv, splits, dev)
    for i in range(3):
        xq, sx, _ = A.attn_decode_fused(qkv, pos, cos, sin, hq, hkv, caches[i % n_layers], pt, lens, scratch=sc, splits=splits)
    torch.cuda.synchronize()
    print("ok", impl, B, ctx, hq, hkv, splits, float(sx.mean()))
    sys.exit(0)
for i in range(3):
    A.attn_decode(q, caches[i % n_layers], pt, lens, scratch=sc, splits=splits, out=out, impl=impl)
torch.cuda.synchronize()
print("ok", impl, B, ctx, hq, hkv, splits, float(out.float().abs().mean()))
