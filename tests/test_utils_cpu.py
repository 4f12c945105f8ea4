import json

from mojo_linuxperiments_b200.utils.trace import MetricsLog, nvtx_range


def test_metrics_log_roundtrip(tmp_path):
    log = MetricsLog(str(tmp_path / "m" / "run.jsonl"))
    log.write(kind="bench", tokens_per_s=1234.5, world=8)
    log.write(kind="arena", used=10, remaining=90)
    recs = log.read()
    assert [r["kind"] for r in recs] == ["bench", "arena"] and recs[0]["world"] == 8 and "t" in recs[1]
    assert json.loads(open(log.path).readline())["tokens_per_s"] == 1234.5


def test_nvtx_range_is_harmless_without_a_gpu():
    with nvtx_range("unit-test"):
        x = 1 + 1
    assert x == 2


def test_decode_attention_split_policy_and_sp_layout():
    """Host-side policies of the tensor-core decode attention and the token-sharded exchange layout (no GPU needed)."""
    from mojo_linuxperiments_b200.ops import attention as A
    from mojo_linuxperiments_b200.parallel import sp as SP
    # at most 4 x 128 tokens per CTA
    assert [A.tc_min_splits(n) for n in (1, 128, 512, 513, 1024, 1088, 2048, 4096)] == [1, 1, 1, 2, 2, 3, 4, 8]
    for B, hkv, max_len in ((1, 1, 64), (32, 8, 1088), (1, 8, 2048), (128, 1, 1280), (4, 2, 8192)):
        s = A.pick_decode_splits_tc(B, hkv, max_len)
        assert s >= A.tc_min_splits(max_len) and s <= max(A.tc_min_splits(max_len), min(32, (max_len + 127) // 128))
    assert A.pick_decode_splits_tc(32, 8, 1088) == 3            # a full GPU prefers few, long CTAs
    assert A.pick_decode_splits_tc(1, 1, 1088) > 3              # a nearly empty one prefers many short ones
    assert A.decode_impl(16, 4) in ("tc", "tcp", "tma", "simple") and A.decode_impl(32, 4) == "simple"
    assert A.decode_impl(16, 16) == "simple"
    # exchange layout: every area aligned, nothing overlaps, rows per rank cover the tokens
    for world, m_cap, d in ((2, 512, 1024), (8, 16384, 4096), (3, 1000, 256)):
        lay = SP.SPLayout(world, m_cap, d, d)
        areas = sorted([(lay.q_off[0], m_cap * d), (lay.q_off[1], m_cap * d), (lay.s_off[0], m_cap * 4),
                        (lay.s_off[1], m_cap * 4), (lay.flag_off, world * lay.blk_cap * 4), (lay.done_off, world * 4),
                        (lay.recv_off[0], world * lay.r_cap * d * 2), (lay.recv_off[1], world * lay.r_cap * d * 2),
                        (lay.ctr_off, 16), (lay.ids_off[0], m_cap * 32), (lay.ids_off[1], m_cap * 32),
                        (lay.wts_off[0], m_cap * 32), (lay.wts_off[1], m_cap * 32)])
        for (a, n), (b, _) in zip(areas, areas[1:]):
            assert a % 1024 == 0 and a + n <= b
        assert areas[-1][0] + areas[-1][1] <= lay.nbytes
        assert lay.r_cap * world >= m_cap and lay.blk_cap * 128 >= lay.r_cap
