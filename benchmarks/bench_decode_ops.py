"""Device-timed decode-side kernels (attention over the paged KV cache, activation prologues, RoPE + KV write) at the
Llama-3-8B shapes, each as a CUDA graph of back-to-back launches over rotating buffers larger than L2.
Prints one JSON line per case with the achieved fraction of the measured HBM copy bandwidth.

python benchmarks/bench_decode_ops.py [--hbm-gbs 6539.5]
"""
import argparse
import json
import os

import torch

import os
import sys as _sys
_sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.ops import attention as A
from mojo_linuxperiments_b200.ops import linear as L


def graph_time(fn, iters=20):
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        with torch.cuda.graph(g, stream=s):
            for i in range(iters):
                fn(i)
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters * 1e-3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hbm-gbs", type=float, default=None)
    a = ap.parse_args()
    hbm = a.hbm_gbs
    if hbm is None:
        try:
            hbm = json.load(open(os.path.join(os.path.dirname(__file__), "..", "MEASURED_PEAKS.json")))["hbm_gbs"]
        except Exception:
            hbm = 6650.0
    dev = torch.device("cuda", 0)
    ps = 16
    for (B, ctx, hq, hkv, tag) in [(32, 1024, 32, 8, "tp1 bs32"), (1, 1024, 32, 8, "tp1 bs1"), (32, 1024, 4, 1, "tp8 bs32"),
                                   (1, 1024, 4, 1, "tp8 bs1"), (128, 1024, 8, 1, "qwen235 tp8 bs128")]:
        max_pages = (ctx + 64 + ps - 1) // ps
        n_layers = max(2, min(16, (300 << 20) // (B * max_pages * ps * hkv * 512) + 1))
        caches = [A.PagedKVCache(B * max_pages, hkv, ps, dev) for _ in range(n_layers)]
        for c in caches:
            c.data.normal_()
        pt = torch.arange(B * max_pages, dtype=torch.int32, device=dev).view(B, max_pages)
        lens = torch.full((B,), ctx, dtype=torch.int32, device=dev)
        q = torch.randn((B, hq, 128), device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        byts = B * ctx * hkv * 512
        for impl in ("tcp", "tc", "tma"):
            if impl in ("tc", "tcp"):
                splits = A.pick_decode_splits_tc(B, hkv, max_pages * ps)
            else:
                splits = A.pick_decode_splits(B, hkv, ctx + 64)
            sc = A.DecodeAttnScratch(B, hq, hkv, splits, dev)
            t = graph_time(lambda i: A.attn_decode(q, caches[i % n_layers], pt, lens, scratch=sc, splits=splits, out=out, impl=impl))
            print(json.dumps({"op": "attn_decode", "impl": impl, "case": tag, "splits": splits, "us": t * 1e6,
                              "gbs": byts / t / 1e9, "frac_of_measured_hbm": byts / t / 1e9 / hbm}), flush=True)
        # the fused form the decoder runs (RoPE + KV append + attention + rotate / quantise of the output in one launch);
        # `lens` counts the new token, so the cached part is ctx - 1 tokens
        qkv = torch.randn((B, (hq + 2 * hkv) * 128), device=dev).to(torch.bfloat16)
        pos = (lens - 1).contiguous()
        cos, sin = A.rope_tables(ctx + 64, 500000.0, dev)
        for long_form in (True, False):
            splits = A.pick_decode_splits_tc(B, hkv, max_pages * ps, fused=long_form)
            sc = A.DecodeAttnScratch(B, hq, hkv, splits, dev)
            t = graph_time(lambda i: A.attn_decode_fused(qkv, pos, cos, sin, hq, hkv, caches[i % n_layers], pt, lens, scratch=sc, splits=splits))
            print(json.dumps({"op": "attn_decode_fused", "blocks_per_cta": 9 if long_form else 4, "case": tag, "splits": splits,
                              "us": t * 1e6, "gbs": byts / t / 1e9, "frac_of_measured_hbm": byts / t / 1e9 / hbm}), flush=True)
        if os.environ.get("SWEEP_SPLITS"):
            for splits in range(A.tc_min_splits(max_pages * ps), 10):
                sc = A.DecodeAttnScratch(B, hq, hkv, splits, dev)
                t = graph_time(lambda i: A.attn_decode(q, caches[i % n_layers], pt, lens, scratch=sc, splits=splits, out=out, impl="tcp"))
                print(json.dumps({"op": "attn_decode", "impl": "tcp", "case": tag, "splits": splits, "us": t * 1e6}), flush=True)
        del caches
    for (M, K, mode, tag) in [(32, 4096, L.AQ_ADD_NORM, "add_norm bs32"), (1, 4096, L.AQ_ADD_NORM, "add_norm bs1"),
                              (32, 14336, L.AQ_SWIGLU, "swiglu bs32"), (32, 4096, L.AQ_PLAIN, "plain bs32"),
                              (32768, 4096, L.AQ_ADD_NORM, "add_norm prefill 32k tokens"),
                              (32768, 14336, L.AQ_SWIGLU, "swiglu prefill 32k tokens")]:
        nb = 2 if M > 1000 else 8
        width = 2 * K if mode == L.AQ_SWIGLU else K
        xs = [torch.randn((M, width), device=dev).to(torch.bfloat16) for _ in range(nb)]
        res = torch.randn((M, K), device=dev).to(torch.bfloat16) if mode == L.AQ_ADD_NORM else None
        gamma = torch.ones(K, device=dev, dtype=torch.bfloat16)
        oq = torch.empty((M, K), dtype=torch.int8, device=dev)
        osc = torch.empty((M,), dtype=torch.float32, device=dev)
        t = graph_time(lambda i: L.act_quant(xs[i % nb], mode=mode, gamma=gamma, residual=res, out_q=oq, out_scale=osc),
                       iters=10 if M > 1000 else 20)
        byts = M * width * 2 + M * K + (M * K * 4 if mode == L.AQ_ADD_NORM else 0)
        print(json.dumps({"op": "act_quant", "case": tag, "us": t * 1e6, "gbs": byts / t / 1e9,
                          "frac_of_measured_hbm": byts / t / 1e9 / hbm}), flush=True)
    for (M, tag) in [(32, "bs32"), (1, "bs1")]:
        hq, hkv = 32, 8
        qkv = torch.randn((M, (hq + 2 * hkv) * 128), device=dev).to(torch.bfloat16)
        pos = torch.full((M,), 1000, dtype=torch.int32, device=dev)
        cos, sin = A.rope_tables(2048, 500000.0, dev)
        cache = A.PagedKVCache(M * 80, hkv, ps, dev)
        pt = torch.arange(M * 80, dtype=torch.int32, device=dev).view(M, 80)
        qo = torch.empty((M, hq, 128), dtype=torch.bfloat16, device=dev)
        t = graph_time(lambda i: A.rope_kv_write(qkv, pos, cos, sin, hq, hkv, q_out=qo, cache=cache, page_table=pt))
        print(json.dumps({"op": "rope_kv_write", "case": tag, "us": t * 1e6}), flush=True)


if __name__ == "__main__":
    main()
