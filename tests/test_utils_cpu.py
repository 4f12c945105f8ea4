import json
import time

import pytest

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
    # the fused form may hold 9 x 128 tokens per CTA: whole sequences when that makes one wave of CTAs
    assert [A.tc_min_splits(n, fused=True) for n in (1, 1152, 1153, 2304, 4096)] == [1, 1, 2, 2, 4]
    assert A.pick_decode_splits_tc(32, 8, 1152, fused=True) == 1   # 256 CTAs of nine blocks: one wave
    assert A.pick_decode_splits_tc(32, 8, 1280, fused=True) == 2   # ten blocks do not fit one CTA
    # a 1/8 shard keeps its many short CTAs (they merge as a cluster)
    assert A.pick_decode_splits_tc(32, 1, 1152, fused=True) == A.pick_decode_splits_tc(32, 1, 1152) > 1
    assert A.pick_decode_splits_tc(32, 2, 1152, fused=True) * 64 <= 296
    assert A.decode_impl(16, 4) in ("tc", "tcp", "tma", "simple") and A.decode_impl(32, 4) == "simple"
    assert A.decode_impl(16, 16) in ("tc", "tcp", "tma", "simple") and A.decode_impl(16, 32) == "simple"   # up to 16 heads per KV head
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


def test_index_arithmetic_of_the_fused_tp_gemms():
    """Python restatement of the integer bookkeeping in csrc/kernels/w8a8_gemm_tp.cu, swept over awkward shapes:
    (a) scatter form: the row counts the epilogue warps report to each owner add up to rows_owner x column tiles;
    (b) gather form: every (source, block) flag a tile waits for is one the source publishes, and the grouped push
        covers each of a rank's 16-byte vectors exactly once with `members` arrivals per block."""
    def ceil_div(a, b): return -(-a // b)
    for world in (1, 2, 3, 4, 8):
        for M in (65, 128, 130, 200, 256, 520, 1000, 1024, 4096 + 17):
            R = ceil_div(M, world)
            m_tiles = ceil_div(M, 128)
            for n_tiles in (1, 3):
                # (a) arrival counts per owner
                got = [0] * world
                for m_tile in range(m_tiles):
                    for _ in range(n_tiles):
                        for q in range(4):
                            m0, m1 = m_tile * 128 + q * 32, min(m_tile * 128 + q * 32 + 32, M)
                            if m0 >= m1:
                                continue
                            for o in range(m0 // R, (m1 - 1) // R + 1):
                                got[o] += min(m1, (o + 1) * R) - max(m0, o * R)
                want = [max(0, min(R, M - o * R)) * n_tiles for o in range(world)]
                assert got == want, (world, M, n_tiles)
            # (b) flags a consumer tile needs vs flags a source publishes
            for m_tile in range(m_tiles):
                r_lo, r_hi = m_tile * 128, min(m_tile * 128 + 128, M) - 1
                for s in range(r_lo // R, r_hi // R + 1):
                    assert s < world
                    rows_s = max(0, min(R, M - s * R))
                    a, b = max(r_lo, s * R) - s * R, min(r_hi, (s + 1) * R - 1) - s * R
                    for blk in range(a >> 7, (b >> 7) + 1):
                        assert blk * 128 < rows_s, (world, M, m_tile, s, blk)       # published by the push
            # grouped push of one rank's rows: CTA groups, members per block, vector coverage
            G, K = 148, 256
            for rank in range(world):
                my_rows = max(0, min(R, M - rank * R))
                nblk = ceil_div(my_rows, 128)
                members = G // nblk if 0 < nblk <= G else 1
                arrivals = [0] * nblk
                covered = [0] * (my_rows * (K // 16))
                for cta in range(G):
                    first = cta // members if nblk <= G else cta
                    step = nblk if nblk <= G else G
                    mtid0 = (cta % members if nblk <= G else 0) * 64
                    blk = first
                    while blk < nblk:
                        rows_b = min(128, my_rows - blk * 128)
                        for ct in range(64):
                            v = mtid0 + ct
                            while v < rows_b * (K // 16):
                                covered[blk * 128 * (K // 16) + v] += 1
                                v += members * 64
                        arrivals[blk] += 1
                        blk += step
                assert all(c == 1 for c in covered), (world, M, rank)
                assert all(a == members for a in arrivals), (world, M, rank, arrivals, members)


def test_split_prefill_attention_work_decomposition():
    """Python restatement of the (query tile, KV chunk) enumeration of csrc/kernels/attn_prefill_split.cu: every pair is
    visited exactly once, heavy query tiles first, and the chunks of a tile cover KV tiles 0..qt without overlap."""
    for n_q in (1, 2, 3, 8, 13):
        for chunk in (1, 2, 3, 5):
            total = sum((qt + chunk) // chunk for qt in range(n_q))
            seen = {}
            order = []
            for bx in range(total):
                qt, rem = n_q - 1, bx
                while qt > 0 and rem >= (qt + chunk) // chunk:
                    rem -= (qt + chunk) // chunk
                    qt -= 1
                nchunks = (qt + chunk) // chunk
                assert 0 <= rem < nchunks
                j_lo = rem * chunk
                n_tiles = min(qt + 1, j_lo + chunk) - j_lo
                assert n_tiles >= 1
                seen.setdefault(qt, []).extend(range(j_lo, j_lo + n_tiles))
                order.append(qt)
            assert order == sorted(order, reverse=True)
            assert sorted(seen) == list(range(n_q))
            for qt, tiles in seen.items():
                assert sorted(tiles) == list(range(qt + 1)), (n_q, chunk, qt)
            max_chunks = (n_q + chunk - 1) // chunk
            assert all((qt + chunk) // chunk <= max_chunks for qt in range(n_q))


def test_decode_attention_split_geometry_covers_every_block_once():
    """Python restatement of the per-CTA geometry of csrc/kernels/attn_decode_tc.cu: with at least ``tc_min_splits`` splits
    no CTA gets more than four 128-token blocks, and the splits cover blocks 0..ceil(len/128)-1 exactly once."""
    from mojo_linuxperiments_b200.ops import attention as A
    for max_len in (64, 128, 512, 513, 1088, 2048, 5000):
        smin = A.tc_min_splits(max_len)
        for splits in (smin, smin + 1, 2 * smin + 3):
            for length in sorted({1, 17, 127, 128, 129, 640, max_len // 2, max_len - 1, max_len}):
                if length < 1 or length > max_len:
                    continue
                total_blocks = (length + 127) // 128
                per = -(-total_blocks // splits)
                covered = []
                for split in range(splits):
                    blk0 = split * per
                    nb = max(0, min(total_blocks, blk0 + per) - blk0)
                    assert nb <= A.TC_BLOCKS_PER_CTA, (max_len, splits, length, nb)
                    covered += list(range(blk0, blk0 + nb))
                    total_pages = (length + 15) // 16
                    for lane in range(32):                       # page-id prefetch stays inside the sequence's pages
                        assert 0 <= min(blk0 * 8 + lane, total_pages - 1) < total_pages
                assert covered == list(range(total_blocks)), (max_len, splits, length)


def test_heartbeat_monitor_thread_feeds_the_fast_check():
    """With ``start(monitor=True)`` the beating thread also watches the peers; ``check_fast`` is then a memory read
    that raises once a peer has been silent for the timeout."""
    from mojo_linuxperiments_b200.utils.health import Heartbeat, RankFailure

    class DictStore:
        def __init__(self): self.d = {}
        def set(self, k, v): self.d[k] = v
        def get(self, k): return self.d[k].encode() if isinstance(self.d[k], str) else self.d[k]
        def check(self, keys): return all(k in self.d for k in keys)

    store = DictStore()
    a = Heartbeat(store, 0, 2, interval_s=0.02, timeout_s=0.15, prefix="t").start(monitor=True)
    b = Heartbeat(store, 1, 2, interval_s=0.02, timeout_s=0.15, prefix="t").start()
    time.sleep(0.3)
    a.check_fast()                      # both alive: nothing raised
    b.stop()                            # rank 1 leaves between steps
    time.sleep(0.5)
    with pytest.raises(RankFailure) as e:
        a.check_fast()
    assert e.value.ranks == [1]
    a.stop()
