"""Prefill a batch and run a few eager (un-graphed) decode steps of the Llama-3-8B-shaped model, for profiler captures.

python benchmarks/decode_once.py [--batch 32] [--prompt-len 1024] [--steps 2] [--layers 32]
"""
import argparse
from dataclasses import replace

import torch

import os
import sys as _sys
_sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.engine.engine import Engine
from mojo_linuxperiments_b200.models import config as C
from mojo_linuxperiments_b200.ops import _lib

ap = argparse.ArgumentParser()
ap.add_argument("--batch", type=int, default=32)
ap.add_argument("--prompt-len", type=int, default=1024)
ap.add_argument("--steps", type=int, default=2)
ap.add_argument("--layers", type=int, default=32)
ap.add_argument("--model", default="llama3-8b")
ap.add_argument("--shard-of", type=int, default=1, help="run rank 0's shard of a tensor-parallel group of this size on one GPU "
                "(same kernel shapes as that group, partial sums are simply not reduced)")
a = ap.parse_args()
cfg = replace(C.PRESETS[a.model](), n_layers=a.layers)
eng = Engine(cfg, C.RuntimeConfig(tp=a.shard_of, ep=a.shard_of, max_batch=a.batch, max_seq_len=a.prompt_len + 128), seed=0)
prompts = torch.randint(0, cfg.vocab, (a.batch, a.prompt_len))
eng.start_batch(a.batch, a.prompt_len + a.steps + 9)
eng.prefill(prompts)
eng.decode_step(use_graph=False)      # warm-up step (lazy kernel attributes, allocator)
torch.cuda.synchronize()
n0 = _lib.LAUNCHES[0]
torch.cuda.profiler.start()           # with `ncu --profile-from-start off` only the steps below are captured
for _ in range(a.steps):
    eng.decode_step(use_graph=False)
torch.cuda.synchronize()
torch.cuda.profiler.stop()
eng.check_status()
print("launches before decode:", n0, "per step:", (_lib.LAUNCHES[0] - n0) // a.steps)
