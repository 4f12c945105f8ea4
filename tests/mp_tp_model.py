"""Worker for tests/test_multigpu.py: tensor-parallel miniature model against the single-process oracle."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.engine.engine import Engine  # noqa: E402
from mojo_linuxperiments_b200.models import config as C  # noqa: E402
from mojo_linuxperiments_b200.models import weights as Wt  # noqa: E402
from mojo_linuxperiments_b200.oracle import model as OM  # noqa: E402
from mojo_linuxperiments_b200.parallel.comm import Comm  # noqa: E402


def main():
    fused = sys.argv[1] == "fused"
    kind = sys.argv[2] if len(sys.argv) > 2 else "dense"
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    if kind == "moe":
        os.environ.setdefault("B200RT_SP_MOE", "1")      # exercise the expert dispatch / combine kernels at any rank count
        # 4 KV heads on up to 8 ranks (heads replicated on rank pairs), 16 experts sharded over the ranks
        cfg = C.tiny_moe(n_layers=2, d_model=1024, n_heads=8, n_kv_heads=4, n_experts=16, top_k=4, moe_ffn=256, vocab=2048)
    else:
        cfg = C.tiny_dense(n_layers=2, d_model=1024, n_heads=8, n_kv_heads=8 if world > 4 else 4, ffn=2048, vocab=2048)
    rt = C.RuntimeConfig(tp=world, ep=world, max_seq_len=256, max_prefill_tokens=512, fused_collectives=fused)
    ck = Wt.quantize_master(Wt.init_master(cfg, 0))
    w = Wt.shard_from_checkpoint(cfg, ck, world, rank, "cuda")
    eng = Engine(cfg, rt, weights=w, comm=Comm())
    prompts = torch.randint(0, cfg.vocab, (3, 70), generator=torch.Generator().manual_seed(5))
    NEW = 8
    out = eng.generate(prompts, NEW)
    out_eager = eng.generate(prompts, NEW, use_graph=False)
    failures = []
    if not torch.equal(out, out_eager):
        failures.append("graph != eager")
    # every rank must have produced the same tokens
    t = out.cuda()
    ref = t.clone()
    dist.broadcast(ref, 0)
    if not torch.equal(t, ref):
        failures.append("ranks disagree")
    if rank == 0:
        ck_dev = {k: v.cuda() for k, v in ck.items()}
        agree = total = 0
        for b in range(prompts.shape[0]):
            toks, logs = OM.greedy_generate(cfg, ck_dev, prompts[b].cuda(), NEW, tp=world)
            for i in range(NEW):
                total += 1
                if int(out[b, i]) == toks[i]:
                    agree += 1
                    continue
                top2 = logs[i].topk(2).values
                if (top2[0] - top2[1]).item() > 0.05 * logs[i].abs().max().item():
                    failures.append(f"seq {b} step {i}: diverged from the oracle with a clear margin")
                break
        print("AGREE", agree, "of", total)
        if agree < total // 2:
            failures.append("too few tokens agree with the oracle")
    bad = torch.tensor([len(failures)], device="cuda")
    dist.all_reduce(bad)
    if rank == 0:
        print("FAILURES", int(bad.item()), failures)
    dist.barrier()
    sys.stdout.flush()
    os._exit(1 if failures else 0)      # skip communicator / symmetric-memory teardown (can block with live graphs)


if __name__ == "__main__":
    main()
