"""CPU checks of the model-side bookkeeping: configs, sharding, the checkpoint layout and the oracles themselves."""
import math

import pytest
import torch

from mojo_linuxperiments_b200.models import config as C
from mojo_linuxperiments_b200.models import weights as Wt
from mojo_linuxperiments_b200.oracle import attention as OA
from mojo_linuxperiments_b200.oracle import model as OM
from mojo_linuxperiments_b200.oracle import quant as Q


def test_presets_match_the_named_shapes():
    l = C.llama3_8b()
    assert (l.n_layers, l.d_model, l.n_heads, l.n_kv_heads, l.ffn, l.vocab, l.rope_theta, l.eps) == \
        (32, 4096, 32, 8, 14336, 128256, 500000.0, 1e-5)
    q = C.qwen3_30b_a3b()
    assert (q.n_layers, q.d_model, q.n_heads, q.n_kv_heads, q.n_experts, q.top_k, q.moe_ffn, q.vocab) == \
        (48, 2048, 32, 4, 128, 8, 768, 151936)
    b = C.qwen3_235b_a22b()
    assert (b.n_layers, b.d_model, b.n_heads, b.n_kv_heads, b.moe_ffn) == (94, 4096, 64, 4, 1536)
    assert 7.5e9 < l.weight_bytes() < 9.5e9 and 2.2e11 < b.weight_bytes() < 2.5e11
    assert C.ModelConfig.from_json(q.to_json()) == q


def test_kv_head_placement_with_fewer_heads_than_ranks():
    q = C.qwen3_30b_a3b()
    assert C.kv_heads_per_rank(q, 8) == 1
    assert [C.kv_head_of_rank(q, 8, r) for r in range(8)] == [0, 0, 1, 1, 2, 2, 3, 3]
    l = C.llama3_8b()
    assert C.kv_heads_per_rank(l, 2) == 4 and [C.kv_head_of_rank(l, 2, r) for r in range(2)] == [0, 4]


def test_runtime_config_env_overrides(monkeypatch):
    monkeypatch.setenv("B200RT_FUSED", "0")
    monkeypatch.setenv("B200RT_WAIT_LIMIT_MS", "150")
    rt = C.RuntimeConfig.from_env(tp=2)
    assert rt.tp == 2 and rt.fused_collectives is False and rt.wait_limit_ms == 150


def test_hadamard_is_orthogonal_and_symmetric():
    h = Q.hadamard_matrix(128, torch.float64)
    assert torch.allclose(h @ h.t(), torch.eye(128, dtype=torch.float64), atol=1e-12)
    assert torch.equal(h, h.t())
    x = torch.randn(5, 256)
    assert torch.allclose(Q.rotate(Q.rotate(x)), x, atol=1e-5)          # H is an involution per block


def test_quantisation_definitions():
    x = torch.tensor([[0.0] * 128, [1.0] + [0.0] * 127])
    q, s = Q.quantize_rows(x)
    assert s[0].item() == 1.0 and q[0].abs().max().item() == 0          # all-zero row: scale 1
    assert q[1, 0].item() == 127 and abs(s[1].item() - 1 / 127) < 1e-9
    xr = torch.randn(7, 384) * 3
    q, s = Q.quantize_rows(xr)
    assert q.abs().max().item() <= 127 and (q.float() * s[:, None] - xr).abs().max() <= s.max() * 0.5 + 1e-6


def test_rotated_weights_reproduce_the_unrotated_product():
    torch.manual_seed(0)
    x, w = torch.randn(6, 512).to(torch.bfloat16), torch.randn(32, 512) * 0.05
    wq, sw = Q.quantize_weight(w)
    y = Q.hadamard_linear(x, wq, sw)
    exact = x.float() @ w.t()
    assert (y - exact).norm() / exact.norm() < 0.03
    y2 = Q.hadamard_linear(x, wq, sw, tp=4)                            # K-sharded: per-shard scales, partial sums
    assert (y2 - exact).norm() / exact.norm() < 0.03


def test_checkpoint_roundtrip_and_sharding(tmp_path):
    cfg = C.tiny_moe(n_layers=1, d_model=256, n_heads=2, n_kv_heads=2, n_experts=4, top_k=2, moe_ffn=128, vocab=256)
    ck = Wt.quantize_master(Wt.init_master(cfg, 0))
    assert ck["layers.0.wq.qweight"].dtype == torch.int8 and ck["layers.0.wq.scale"].dtype == torch.float32
    assert ck["layers.0.attn_norm"].dtype == torch.bfloat16
    path = str(tmp_path / "m.safetensors")
    Wt.save_checkpoint(path, cfg, ck)
    cfg2, ck2 = Wt.load_checkpoint(path)
    assert cfg2 == cfg and set(ck2) == set(ck)
    assert all(torch.equal(ck[k], ck2[k]) for k in ck)
    w0 = Wt.shard_from_checkpoint(cfg, ck2, 2, 0, "cpu")
    w1 = Wt.shard_from_checkpoint(cfg, ck2, 2, 1, "cpu")
    L0, L1 = w0["layers"][0], w1["layers"][0]
    hd = cfg.head_dim
    assert L0["qkv"].qweight.shape == ((1 + 2) * hd, 256) and L0["o"].qweight.shape == (256, hd)
    assert torch.equal(torch.cat([L0["o"].qweight, L1["o"].qweight], 1), ck["layers.0.wo.qweight"])
    assert torch.equal(L0["o"].scale, L1["o"].scale)                    # row-parallel shards share the channel scale
    assert L0["experts_gate_up"].qweight.shape == (2, 2 * 128, 256) and L1["experts_down"].qweight.shape == (2, 256, 128)
    assert torch.equal(L1["experts_gate_up"].qweight[0, :128], ck["layers.0.experts.2.gate.qweight"])
    assert w0["vocab_offset"] == 0 and w1["vocab_offset"] == 128
    assert torch.equal(L0["router"].qweight, L1["router"].qweight)      # replicated


def test_checkpoint_rejects_unrotated_layout(tmp_path):
    from safetensors.torch import save_file
    path = str(tmp_path / "bad.safetensors")
    save_file({"x": torch.zeros(1)}, path, metadata={"config": C.tiny_dense().to_json(), "rotated": "false", "hadamard_block": "128"})
    with pytest.raises(ValueError):
        Wt.load_checkpoint(path)


def test_attention_oracles_agree_with_each_other():
    torch.manual_seed(1)
    T, hq, hkv, d = 9, 4, 2, 128
    q, k, v = torch.randn(T, hq, d), torch.randn(T, hkv, d), torch.randn(T, hkv, d)
    full = OA.causal_gqa(q, k, v)
    last = OA.decode_gqa(q[-1], k, v)
    assert torch.allclose(full[-1], last, atol=1e-5)
    r = OA.rope(q, torch.arange(T), 500000.0)
    assert torch.allclose(r.norm(dim=-1), q.norm(dim=-1), rtol=1e-4)    # rotations keep the norm
    assert torch.allclose(r[0], q[0], atol=1e-6)                        # position 0 is the identity


def test_oracle_model_is_causal_and_tp_consistent():
    cfg = C.tiny_dense(n_layers=1, d_model=256, n_heads=2, n_kv_heads=1, ffn=256, vocab=128)
    ck = Wt.quantize_master(Wt.init_master(cfg, 0))
    ids = torch.randint(0, cfg.vocab, (12,), generator=torch.Generator().manual_seed(0))
    a = OM.forward_sequence(cfg, ck, ids)
    b = OM.forward_sequence(cfg, ck, ids[:7])
    assert torch.allclose(a[:7], b, atol=1e-3)                          # a prefix sees the same logits
    c = OM.forward_sequence(cfg, ck, ids, tp=2)
    assert (a - c).abs().max() < 0.1 * a.abs().max()                    # K-sharded quantisation only perturbs


def test_last_token_rows_of_a_token_sharded_prefill_sum_to_the_replicated_rows():
    """Each sequence's last row lives on exactly one rank: summing every rank's masked gather reproduces the rows."""
    import torch
    from mojo_linuxperiments_b200.models.decoder import own_last_rows
    g = torch.Generator().manual_seed(0)
    for world, lens in ((2, [70, 70, 70]), (8, [70, 70, 70]), (4, [1024]), (8, [5, 300, 33, 129]), (3, [16, 16])):
        M = sum(lens)
        last = torch.tensor([sum(lens[: i + 1]) - 1 for i in range(len(lens))])
        h = torch.randn((M, 8), generator=g)
        R = (M + world - 1) // world
        total = torch.zeros((len(lens), 8))
        owners = torch.zeros(len(lens))
        for r in range(world):
            a = min(M, r * R)
            b = min(M, a + R)
            mine, loc = own_last_rows(last, a, b)
            owners += mine.squeeze(1).float()
            if b > a:
                total += torch.where(mine, h[a:b].index_select(0, loc), torch.zeros(()))
        assert torch.equal(owners, torch.ones(len(lens))) and torch.equal(total, h[last])


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_load_shard_reads_only_this_ranks_part_of_the_file(tmp_path, kind):
    """``load_shard`` cuts a rank's rows / columns out of the checkpoint file slice by slice: the result equals sharding
    a fully loaded checkpoint, and what was read from the file is well below the whole model."""
    import os

    def same(a, b):
        if isinstance(a, Wt.LinearW):
            return torch.equal(a.qweight, b.qweight) and torch.equal(a.scale, b.scale)
        return torch.equal(a, b) if isinstance(a, torch.Tensor) else a == b

    if kind == "dense":
        cfg = C.tiny_dense(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=512)
    else:
        cfg = C.tiny_moe(n_layers=1, d_model=256, n_heads=4, n_kv_heads=2, n_experts=8, top_k=2, moe_ffn=128, vocab=512)
    ck = Wt.quantize_master(Wt.init_master(cfg, 1))
    path = str(tmp_path / "m.safetensors")
    Wt.save_checkpoint(path, cfg, ck)
    size = os.path.getsize(path)
    tp = 4 if kind == "moe" else 2
    total_read = 0
    for rank in range(tp):
        cfg2, w = Wt.load_shard(path, tp, rank, "cpu")
        ref = Wt.shard_from_checkpoint(cfg, ck, tp, rank, "cpu")
        assert cfg2 == cfg
        read = w.pop("checkpoint_bytes_read")
        total_read += read
        for k in ("embed", "final_norm", "lm_head", "vocab_offset"):
            assert same(w[k], ref[k]), k
        for La, Lb in zip(w["layers"], ref["layers"]):
            assert set(La) == set(Lb)
            for k in La:
                assert same(La[k], Lb[k]), k
        # the linears are sharded; only the replicated tensors (embedding, norms, router) are read by every rank
        assert read < 0.8 * size
    with pytest.raises(ValueError):
        from safetensors.torch import save_file
        bad = str(tmp_path / "bad.safetensors")
        save_file({"x": torch.zeros(1)}, bad, metadata={"config": cfg.to_json(), "rotated": "false", "hadamard_block": "128"})
        Wt.load_shard(bad, 2, 0, "cpu")
