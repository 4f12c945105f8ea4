"""End-to-end miniature models through the engine (prefill + CUDA-graph decode) against the PyTorch oracle."""
import pytest
import torch

from mojo_linuxperiments_b200.models import config as C
from mojo_linuxperiments_b200.models import weights as Wt
from mojo_linuxperiments_b200.oracle import model as OM

pytestmark = pytest.mark.gpu


def _setup(cfg, seed=0):
    master = Wt.init_master(cfg, seed)
    ck = Wt.quantize_master(master)
    ck_dev = {k: v.cuda() for k, v in ck.items()}
    return ck, ck_dev


def test_tiny_dense_prefill_logits_and_greedy_decode():
    from mojo_linuxperiments_b200.engine.engine import Engine
    cfg = C.tiny_dense()
    rt = C.RuntimeConfig(max_seq_len=256)
    ck, ck_dev = _setup(cfg)
    w = Wt.shard_from_checkpoint(cfg, ck, 1, 0, "cuda")
    eng = Engine(cfg, rt, weights=w)
    g = torch.Generator().manual_seed(1)
    B, S, NEW = 3, 40, 12
    prompts = torch.randint(0, cfg.vocab, (B, S), generator=g)
    out = eng.generate(prompts, NEW)
    assert out.shape == (B, NEW)
    # prefill logits of the last prompt token against the oracle
    eng.start_batch(B, S + NEW)
    eng.prefill(prompts, use_graph=False)      # eager: `last_logits` is then this call's tensor, not a captured one
    torch.cuda.synchronize()
    got = eng.model.last_logits.float()
    agree = 0
    for b in range(B):
        ref = OM.forward_sequence(cfg, ck_dev, prompts[b].cuda())[-1]
        assert torch.allclose(got[b], ref, rtol=5e-2, atol=5e-2 * ref.abs().max().item()), (got[b] - ref).abs().max().item()
        toks, logs = OM.greedy_generate(cfg, ck_dev, prompts[b].cuda(), NEW)
        # token-for-token unless the oracle's own top-2 margin is within rounding noise
        for t in range(NEW):
            if int(out[b, t]) == toks[t]:
                agree += 1
                continue
            top2 = logs[t].topk(2).values
            assert (top2[0] - top2[1]).item() < 0.05 * logs[t].abs().max().item(), f"seq {b} step {t} diverged with a clear margin"
            break
        else:
            continue
    assert agree >= B * NEW // 2


def test_graph_and_eager_decode_agree():
    from mojo_linuxperiments_b200.engine.engine import Engine
    cfg = C.tiny_dense()
    rt = C.RuntimeConfig(max_seq_len=128)
    ck, _ = _setup(cfg, 3)
    w = Wt.shard_from_checkpoint(cfg, ck, 1, 0, "cuda")
    eng = Engine(cfg, rt, weights=w)
    prompts = torch.randint(0, cfg.vocab, (2, 17), generator=torch.Generator().manual_seed(2))
    a = eng.generate(prompts, 10, use_graph=True)
    b = eng.generate(prompts, 10, use_graph=False)
    assert torch.equal(a, b)


def test_decode_past_the_admitted_length_is_refused_on_the_host():
    from mojo_linuxperiments_b200.engine.engine import Engine
    cfg = C.tiny_dense()
    rt = C.RuntimeConfig(max_seq_len=128)
    ck, _ = _setup(cfg, 4)
    eng = Engine(cfg, rt, weights=Wt.shard_from_checkpoint(cfg, ck, 1, 0, "cuda"))
    prompts = torch.randint(0, cfg.vocab, (2, 20), generator=torch.Generator().manual_seed(5))
    eng.start_batch(2, 22)
    eng.prefill(prompts)
    eng.decode_step()
    eng.decode_step()                # positions 20 and 21 fit the 22 admitted tokens
    with pytest.raises(RuntimeError, match="admitted"):
        eng.decode_step()
    torch.cuda.synchronize()
    eng.check_status()               # and nothing on the device went out of range either
