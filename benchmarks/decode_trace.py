"""In-kernel phase stamps of a graph-replayed decode step (needs the kernel library built with -DB200RT_TRACE).

    B200RT_KERNELS=trace python benchmarks/decode_trace.py [--batch 32] [--layers 2] [--shard-of 1] [--out FILE]

Prints, per kernel launch of one step, when its CTAs started, passed their dependency wait, got their first operand
tile, finished the tensor-core work, passed their cluster barriers and left: which part of a launch overlaps the
previous one and where a launch waits.  Stamps perturb the kernels a little; throughput numbers come from bench.py.
"""
import argparse
import os
import sys
from dataclasses import replace

os.environ.setdefault("B200RT_KERNELS", "trace")
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.engine.engine import Engine
from mojo_linuxperiments_b200.models import config as C
from mojo_linuxperiments_b200.utils.trace import DeviceTrace

ap = argparse.ArgumentParser()
ap.add_argument("--batch", type=int, default=32)
ap.add_argument("--prompt-len", type=int, default=1024)
ap.add_argument("--layers", type=int, default=2)
ap.add_argument("--model", default="llama3-8b")
ap.add_argument("--shard-of", type=int, default=1)
ap.add_argument("--out", default="")
a = ap.parse_args()
cfg = replace(C.PRESETS[a.model](), n_layers=a.layers)
tr = DeviceTrace()
tr.start()
eng = Engine(cfg, C.RuntimeConfig(tp=a.shard_of, ep=a.shard_of, max_batch=a.batch, max_seq_len=a.prompt_len + 128), seed=0)
prompts = torch.randint(0, cfg.vocab, (a.batch, a.prompt_len))
eng.start_batch(a.batch, a.prompt_len + 64)
eng.prefill(prompts)
for _ in range(3):
    eng.decode_step()
torch.cuda.synchronize()
tr.clear()
eng.decode_step()
recs = tr.records()
tr.stop()
eng.check_status()
text = (f"decode step phase stamps: model {a.model}, {a.layers} layers, batch {a.batch}, context {a.prompt_len}, "
        f"shard 1/{a.shard_of}; {len(recs)} stamps\n"
        "gemm_decode phases: 0 start, 1 producer past dependency wait, 2 first stage landed, 3 last MMA issued, "
        "4 accumulator complete, 5 cluster is running, 10 partials sent, 6 cluster barrier passed, 11 slice reduced and stored, "
        "7 CTA past its last barrier, 8 pushed to peers, 9 peers summed; quantiser CTAs of a fused launch: 20 start, "
        "21 dependency wait passed, 22 row stored and flagged (GEMM CTAs: phase 1 = all row flags seen)\n"
        "attn_decode phases: 0 start, 1 dependency wait passed, 2 scores in registers, 3 maxima exchanged, 5 P.V read, "
        "6 partial written, 7 merge begins (last CTA of a head), 63 merge done, 62 output quantised\n"
        "act_quant phases: 0 start, 1 dependency wait passed, 2 row rotated, 63 row stored\n" + DeviceTrace.summarize(recs, 400))
print(text)
if a.out:
    os.makedirs(os.path.dirname(a.out) or ".", exist_ok=True)
    with open(a.out, "w") as f:
        f.write(text)
