"""The stock-PyTorch baseline engine (dense and mixture-of-experts) on the CPU against the oracle: it is the comparison
arm of the GPU benchmarks, so it has to compute the same model."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from baseline.torch_baseline import BaselineEngine  # noqa: E402
from mojo_linuxperiments_b200.models import config as C  # noqa: E402
from mojo_linuxperiments_b200.models import weights as Wt  # noqa: E402
from mojo_linuxperiments_b200.oracle import model as OM  # noqa: E402


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_baseline_engine_follows_the_oracle_on_cpu(kind):
    torch.manual_seed(0)
    if kind == "moe":
        cfg = C.tiny_moe(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, n_experts=8, top_k=2, moe_ffn=128, vocab=512)
    else:
        cfg = C.tiny_dense(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=512)
    rt = C.RuntimeConfig(max_seq_len=64)
    ck = Wt.quantize_master(Wt.init_master(cfg, 0))
    w = Wt.shard_from_checkpoint(cfg, ck, 1, 0, "cpu")
    eng = BaselineEngine(cfg, rt, weights=w, device="cpu")
    B, S, NEW = 2, 12, 5
    prompts = torch.randint(0, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(3))
    out = eng.generate(prompts, NEW, use_graph=False)
    assert out.shape == (B, NEW)
    agree = total = 0
    for b in range(B):
        toks, logs = OM.greedy_generate(cfg, ck, prompts[b], NEW)
        for t in range(NEW):
            total += 1
            if int(out[b, t]) == toks[t]:
                agree += 1
                continue
            top2 = logs[t].topk(2).values
            assert (top2[0] - top2[1]).item() < 0.05 * logs[t].abs().max().item(), f"seq {b} step {t} diverged with a clear margin"
            break
    assert agree >= total // 2
