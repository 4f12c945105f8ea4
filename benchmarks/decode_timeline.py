"""Device-side timeline of one graph-replayed decode step (kernel starts, durations, overlaps, gaps).

    python benchmarks/decode_timeline.py [--batch 32] [--layers 4] [--shard-of 1] [--model llama3-8b] [--out FILE]

The stamps are CUPTI activity records collected by torch.profiler during replays of the captured decode graph, so
kernels overlapped by programmatic dependent launch appear overlapped.  This shows shares and gaps; throughput
numbers come from bench.py (CUDA events, no profiler).
"""
import argparse
import os
import sys
from dataclasses import replace

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.engine.engine import Engine
from mojo_linuxperiments_b200.models import config as C
from mojo_linuxperiments_b200.utils.trace import kernel_timeline, summarize_timeline

ap = argparse.ArgumentParser()
ap.add_argument("--batch", type=int, default=32)
ap.add_argument("--prompt-len", type=int, default=1024)
ap.add_argument("--layers", type=int, default=4)
ap.add_argument("--model", default="llama3-8b")
ap.add_argument("--shard-of", type=int, default=1)
ap.add_argument("--iters", type=int, default=3)
ap.add_argument("--out", default="")
a = ap.parse_args()
cfg = replace(C.PRESETS[a.model](), n_layers=a.layers)
eng = Engine(cfg, C.RuntimeConfig(tp=a.shard_of, ep=a.shard_of, max_batch=a.batch, max_seq_len=a.prompt_len + 128), seed=0)
prompts = torch.randint(0, cfg.vocab, (a.batch, a.prompt_len))
eng.start_batch(a.batch, a.prompt_len + 64)
eng.prefill(prompts)
eng.decode_step()
torch.cuda.synchronize()
tl = kernel_timeline(eng.decode_step, iters=a.iters, warmup=2)
eng.check_status()
text = (f"decode step timeline: model {a.model}, {a.layers} layers, batch {a.batch}, context {a.prompt_len}, "
        f"shard 1/{a.shard_of}, {eng.kernels_per_step} kernels per step\n" + summarize_timeline(tl))
print(text)
if a.out:
    os.makedirs(os.path.dirname(a.out) or ".", exist_ok=True)
    with open(a.out, "w") as f:
        f.write(text)
