"""Host runtime (C++): the reference's behaviours (test_linux_threading.mojo) plus unit checks of each component."""
import ctypes
import os
import re
import subprocess
import time
from pathlib import Path

import numpy as np
import pytest

from mojo_linuxperiments_b200 import hostrt as H
from mojo_linuxperiments_b200.oracle import philox as P

S = 1_000_000_000


def test_syscall_numbers_match_kernel_headers():
    hdr = Path("/usr/include/x86_64-linux-gnu/asm/unistd_64.h")
    if not hdr.exists():
        pytest.skip("no kernel headers")
    text = hdr.read_text()
    for name in ["mmap", "mprotect", "munmap", "madvise", "exit", "gettid", "sched_setaffinity", "mbind", "move_pages",
                 "rseq", "clone3", "futex_waitv", "futex_wake", "futex_wait", "getcpu"]:
        m = re.search(rf"#define __NR_{name}\s+(\d+)", text)
        assert m, name
        assert H.lib().hostrt_syscall_nr(name.encode()) == int(m.group(1)), name


def test_abi_struct_sizes_and_flags():
    L = H.lib()
    assert L.hostrt_struct_size(b"FutexNuma32") == 8
    assert L.hostrt_struct_size(b"FutexWaitv") == 24
    assert L.hostrt_struct_size(b"Clone3Args") == 88
    assert L.hostrt_struct_size(b"Rseq") == 32
    flags = L.hostrt_thread_clone_flags()
    for bit in (0x100, 0x200, 0x400, 0x800, 0x10000, 0x40000, 0x80000, 0x100000):   # VM FS FILES SIGHAND THREAD SYSVSEM SETTLS PARENT_SETTID
        assert flags & bit
    assert L.hostrt_slot_total_size(64 * 1024) == 73728     # same slot footprint as the reference's default


def test_cpumask_semantics():
    m = H.CpuMask()
    assert m.count() == 0 and m.byte_size() == 128
    m.set(0); m.set(9); m.set(1023); m.set(1024); m.set(-1)          # out of range ignored
    assert m.count() == 3 and m.test(9) and not m.test(8) and not m.test(1024)
    raw = m.to_bytes()
    assert raw[0] == 1 and raw[1] == 2 and raw[127] == 0x80        # cpu_set_t layout
    m.clear(9)
    assert not m.test(9) and m.count() == 2
    m.set_all(); assert m.count() == 1024
    m.clear_all(); assert m.count() == 0
    assert H.CpuMask.from_cpu_list([3, 5]).cpus() == [3, 5]


def test_cpulist_and_meminfo_parsers():
    assert H.parse_cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert H.parse_cpulist("5") == [5]
    assert H.parse_cpulist("") == []
    txt = "Node 0 MemTotal:       65842380 kB\nNode 0 MemFree:        1234 kB\n"
    assert H.parse_meminfo(txt, "MemTotal") == 65842380
    assert H.parse_meminfo(txt, "MemFree") == 1234
    assert H.parse_meminfo(txt, "Nope") == -1


def _fake_sysfs(tmp_path, nodes):
    """nodes: {id: (cpulist, distances, total_kb, free_kb)}"""
    root = tmp_path / "node"
    root.mkdir()
    ids = sorted(nodes)
    (root / "online").write_text(",".join(str(i) for i in ids) + "\n")
    for i, (cpus, dist, tot, free) in nodes.items():
        d = root / f"node{i}"
        d.mkdir()
        (d / "cpulist").write_text(cpus + "\n")
        (d / "distance").write_text(" ".join(map(str, dist)) + "\n")
        (d / "meminfo").write_text(f"Node {i} MemTotal:  {tot} kB\nNode {i} MemFree:   {free} kB\n")
    return str(root)


def test_numa_info_on_fixture_trees(tmp_path):
    two = _fake_sysfs(tmp_path, {0: ("0-3", [10, 21], 1000, 500), 1: ("4-7", [21, 10], 2000, 700)})
    info = H.NumaInfo(two)
    assert info.ok and info.num_nodes == 2 and info.node_ids == [0, 1]
    assert info.get_node_cpus(1) == [4, 5, 6, 7]
    assert info.distance(0, 1) == 21 and info.distance(1, 1) == 10 and info.distance(0, 7) == -1
    assert info.cpus_per_node() == 4 and info.total_cpus() == 8 and info.cpus_on_node(1) == 4
    assert info.mem_total_kb(1) == 2000 and info.mem_free_kb(0) == 500
    assert info.get_node_mask(1).cpus() == [4, 5, 6, 7]
    assert "node 1" in info.debug_string()


def test_numa_info_eight_nodes_many_cpus(tmp_path):
    """An 8-socket tree with 256 CPUs: wide masks, symmetric distances, per-node memory."""
    nodes = {}
    for n in range(8):
        dist = [10 if m == n else (21 if m // 4 == n // 4 else 32) for m in range(8)]
        nodes[n] = (f"{32 * n}-{32 * n + 31}", dist, 1000 * (n + 1), 100 * (n + 1))
    info = H.NumaInfo(_fake_sysfs(tmp_path, nodes))
    assert info.ok and info.num_nodes == 8 and info.node_ids == list(range(8))
    assert info.total_cpus() == 256 and info.cpus_per_node() == 32
    assert info.get_node_cpus(7) == list(range(224, 256)) and info.get_node_mask(7).cpus() == list(range(224, 256))
    assert info.distance(0, 3) == 21 and info.distance(0, 4) == 32 and info.distance(5, 5) == 10
    assert [info.mem_total_kb(n) for n in range(8)] == [1000 * (n + 1) for n in range(8)]
    assert info.mem_free_kb(7) == 800


def test_numa_info_sparse_ids_and_missing_tree(tmp_path):
    (tmp_path / "a").mkdir()
    sparse = _fake_sysfs(tmp_path / "a", {0: ("0-1", [10, 40], 10, 5), 2: ("8-9,12", [40, 10], 20, 6)})
    info = H.NumaInfo(sparse)
    assert info.node_ids == [0, 2]
    assert info.get_node_cpus(2) == [8, 9, 12]          # looked up by id, not by position
    assert info.distance(2, 0) == 40 and info.get_node_cpus(1) == []
    bad = H.NumaInfo(str(tmp_path / "does-not-exist"))
    assert not bad.ok and bad.num_nodes == 0


def test_live_topology_and_where_am_i():
    info = H.NumaInfo()
    assert info.ok and info.num_nodes >= 1 and info.total_cpus() >= 1
    cpu, node = H.get_current_cpu_and_node()
    assert node in info.node_ids and cpu in info.get_node_cpus(node)
    saved = H.get_thread_affinity()
    try:
        target = info.get_node_cpus(info.node_ids[0])[0]
        assert H.set_thread_affinity(H.CpuMask([target])) == 0
        assert H.get_current_cpu_and_node()[0] == target
        rc, rn = H.get_cpu_and_node_rseq()
        if rc >= 0:      # libc registered an rseq area for this thread
            assert (rc, rn) == H.get_current_cpu_and_node()
    finally:
        H.set_thread_affinity(saved)


def test_arena_bump_mark_reset_exhaustion():
    info = H.NumaInfo()
    a = H.NumaArena(info.node_ids[0], 4096, alignment=64, page_size=H.PAGE_STANDARD)
    assert a and a.used() == 0 and a.remaining() == 4096 and a.verify_placement()
    p1 = a.alloc(10)
    p2 = a.alloc(10)
    assert p1 == a.base() and p2 == a.base() + 64            # aligned bump
    m = a.mark()
    assert a.alloc(1000) is not None
    assert a.alloc(4096) is None                              # would overflow: refused, state unchanged
    used = a.used()
    a.reset_to(used + 100)                                    # forward resets are ignored
    assert a.used() == used
    a.reset_to(m)
    assert a.used() == m
    H.lib().hostrt_poke(p1, 42)                               # first touch
    assert H.lib().hostrt_peek(p1) == 42
    assert a.verify_placement()
    assert H.lib().hostrt_move_pages_query(p1) == info.node_ids[0]
    a.reset()
    assert a.used() == 0 and a.remaining() == 4096


def test_arena_failure_is_a_null_arena():
    a = H.NumaArena(1000, 4096, page_size=H.PAGE_STANDARD)     # node 1000 cannot be bound
    assert not a and a.alloc(8) is None and not a.verify_placement()


def test_pool_launch_join_and_refusal_when_full():
    pool = H.ThreadPool(2, stack_size=8192)
    assert pool and len(pool) == 2
    buf = (ctypes.c_ulonglong * 4)()
    base = ctypes.addressof(buf)
    slow = H.worker_address("hostrt_worker_sleep_store")
    assert pool.launch(slow, 100, base, 11)
    assert pool.launch(slow, 100, base + 8, 22)
    assert not pool.launch(slow, 1, base + 16, 33)             # both slots busy
    assert pool.wait_all(10 * S) == 0
    assert list(buf)[:3] == [11, 22, 0]
    assert pool.launch(H.worker_address("hostrt_worker_store"), base + 16, 33) and pool.wait_all(10 * S) == 0
    assert buf[2] == 33
    pool.close()


def test_pool_wait_any_order_and_timeouts():
    pool = H.ThreadPool(3)
    slow = H.worker_address("hostrt_worker_sleep_store")
    assert pool.wait_any(S) == H.WAIT_NOTHING_RUNNING
    for ms in (300, 200, 100):
        assert pool.launch(slow, ms, 0, 0)
    assert pool.wait_any(1_000_000) == H.WAIT_TIMED_OUT        # 1 ms: nothing has finished yet
    assert pool.wait_all(1_000_000) == -H.ETIMEDOUT
    assert [pool.wait_any(10 * S) for _ in range(3)] == [2, 1, 0]
    assert pool.wait_all(10 * S) == 0
    pool.close()


def test_pinned_pool_runs_where_asked_and_rseq_agrees():
    info = H.NumaInfo()
    node = info.node_ids[0]
    cpu = info.get_node_cpus(node)[-1]
    pool = H.ThreadPool(1, H.CpuMask([cpu]), node)
    out = (ctypes.c_int * 4)()
    assert pool.launch(H.worker_address("hostrt_worker_where"), ctypes.addressof(out))
    assert pool.wait_all(10 * S) == 0
    assert out[0] == cpu and out[1] == node and out[2] == cpu and out[3] == node
    pool.close()


def test_gate_release_wakes_worker_and_timeout_is_reported():
    info = H.NumaInfo()
    arena = H.NumaArena(info.node_ids[0], 4096, page_size=H.PAGE_STANDARD)
    gate_addr = arena.alloc(4)
    res = (ctypes.c_longlong * 2)()
    pool = H.ThreadPool(2)
    waiter = H.worker_address("hostrt_worker_gate_wait_store")
    assert pool.launch(waiter, gate_addr, 5 * S, ctypes.addressof(res))
    gate = H.MutexGate.from_addr(gate_addr)
    assert gate.wait(2_000_000) == -H.ETIMEDOUT                 # nobody released it yet
    gate.release()
    assert pool.wait_all(10 * S) == 0 and res[0] == 1
    assert gate.wait(S) == 0                                     # stays open
    gate.reset()
    assert pool.launch(waiter, gate_addr, 20_000_000, ctypes.addressof(res) + 8)   # 20 ms bound, never released
    assert pool.wait_all(10 * S) == 0 and res[1] == -H.ETIMEDOUT
    pool.close()


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_chain_reduce(world):
    st, v = H.chain_reduce(H.NumaInfo(), world)
    assert st == 0 and v == world * (world + 1) // 2


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_butterfly_allreduce(world):
    st, out = H.butterfly_allreduce(H.NumaInfo(), world)
    assert st == 0 and out == [world * (world + 1) // 2] * world


def test_butterfly_rejects_non_power_of_two():
    st, _ = H.butterfly_allreduce(H.NumaInfo(), 3)
    assert st == -22


@pytest.mark.parametrize("world,rounds", [(2, 1), (4, 3), (8, 2)])
def test_fabric_allreduce_epochs(world, rounds):
    vals = [float(i) + 0.25 for i in range(world)]
    st, out = H.fabric_allreduce(H.NumaInfo(), vals, rounds=rounds)
    want = sum(vals) * (world ** (rounds - 1))
    assert st == 0 and all(abs(o - want) < 1e-9 * abs(want) for o in out)
    assert len(set(out)) == 1                                    # bitwise identical on every rank


def test_fabric_allreduce_silent_rank_times_out_cleanly():
    st, _ = H.fabric_allreduce(H.NumaInfo(), [1.0, 2.0, 3.0, 4.0], timeout_ns=50_000_000, drop_rank=2)
    assert st == -H.ETIMEDOUT


def test_philox_matches_numpy_oracle():
    ref = P.uniform_pm1(64, seed=0)
    got = np.array([H.philox_uniform(i, 0) for i in range(64)], dtype=np.float32)
    assert np.array_equal(ref, got)
    assert ref.min() >= -1.0 and ref.max() < 1.0
    blk = (ctypes.c_uint * 4)()
    H.lib().hostrt_philox_block(7, 123456789123, blk)
    assert list(blk) == P.philox4x32_10(np.array([7], dtype=np.uint64), 123456789123)[0].tolist()


def test_fill_reduce_matches_oracle_and_is_split_invariant():
    info = H.NumaInfo()
    n = 1 << 20
    want = float(P.uniform_pm1(n, 0).astype(np.float64).sum())
    r_all = H.fill_reduce(info, n, 0)
    r_two = H.fill_reduce(info, n, 0, max_workers_per_node=2)
    for r in (r_all, r_two):
        assert r["status"] == 0 and r["misplaced"] == 0
        assert abs(r["sum"] - want) < 1e-6 * n ** 0.5 + 1e-6
    assert r_two["workers"] == 2 * info.num_nodes


def test_reference_scenarios_all_pass():
    for name, result, detail in H.run_scenarios():
        assert result in (H.SC_PASS, H.SC_SKIP), f"{name}: {detail}"


def test_selftest_executable_exit_code():
    from mojo_linuxperiments_b200 import _build
    exe = _build.build_hostrt_selftest()
    p = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0, p.stdout
    assert p.stdout.count("[PASS]") + p.stdout.count("[SKIP]") == 12 and "[FAIL]" not in p.stdout


@pytest.mark.parametrize("M,K,N", [(1, 128, 64), (5, 512, 130), (32, 1024, 257), (37, 256, 96)])
@pytest.mark.parametrize("force_scalar", [False, True])
def test_w8a8_linear_on_the_worker_pools_matches_the_oracle(M, K, N, force_scalar):
    """Host W8A8 Hadamard linear (rotate + quantise + int8 GEMM over the pinned pools): the integer accumulators are
    exact, the quantisation matches the PyTorch reference up to rounding ties, VNNI and scalar paths agree."""
    import torch
    from mojo_linuxperiments_b200.oracle import quant as Q
    g = torch.Generator().manual_seed(M * 1000 + K + N)
    x = torch.randn((M, K), generator=g)
    x = torch.where(torch.rand((M, K), generator=g) < 1e-2, x * 50, x).to(torch.bfloat16)
    if M > 2:
        x[2].zero_()                                  # an all-zero row quantises with scale 1
    wq = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    sw = torch.rand((N,), generator=g) * 9e-3 + 1e-3
    info = H.NumaInfo()
    r = H.w8a8_linear(info, x, wq, sw, force_scalar=force_scalar)
    assert r["status"] == 0 and r["workers"] >= 1
    q_ref, s_ref = Q.rotate_quantize(x)
    assert torch.allclose(r["sx"], s_ref, rtol=1e-5, atol=0)
    d = (r["q"].int() - q_ref.int()).abs()
    assert d.max().item() <= 1 and (d > 0).float().mean().item() < 5e-3
    # exact integer product of what the host itself quantised
    assert torch.equal(r["acc"].double(), Q.int_gemm(r["q"], wq))
    want = Q.w8a8_linear(r["q"], r["sx"], wq, sw)
    assert torch.allclose(r["y"].float(), want, rtol=1e-2, atol=1e-2 * float(want.abs().max()))
    if not force_scalar:
        for isa in ("scalar", "vnni"):            # every instruction-set path gives the same bits
            r2 = H.w8a8_linear(info, x, wq, sw, isa=isa)
            assert torch.equal(r["acc"], r2["acc"]) and torch.equal(r["y"], r2["y"]) and torch.equal(r["q"], r2["q"]), (r["isa"], r2["isa"])


@pytest.mark.parametrize("kind", ["dense", "moe"])
def test_host_decoder_on_the_worker_pools_follows_the_oracle(kind):
    """A whole miniature decoder with every linear on the pinned pools (prefill + cached decode) against the oracle's
    re-computation: token for token unless the oracle's own top-2 margin is within rounding noise."""
    import torch
    from mojo_linuxperiments_b200.hostrt.host_model import HostDecoder
    from mojo_linuxperiments_b200.models import config as C
    from mojo_linuxperiments_b200.models import weights as Wt
    from mojo_linuxperiments_b200.oracle import model as OM
    if kind == "moe":
        cfg = C.tiny_moe(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, n_experts=8, top_k=2, moe_ffn=128, vocab=512)
    else:
        cfg = C.tiny_dense(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, ffn=512, vocab=512)
    ck = Wt.quantize_master(Wt.init_master(cfg, 0))
    dec = HostDecoder(cfg, ck)
    prompt = torch.randint(0, cfg.vocab, (11,), generator=torch.Generator().manual_seed(7))
    NEW = 5
    toks, _ = dec.generate(prompt, NEW)
    ref, logs = OM.greedy_generate(cfg, ck, prompt, NEW)
    agree = 0
    for t in range(NEW):
        if toks[t] == ref[t]:
            agree += 1
            continue
        top2 = logs[t].topk(2).values
        assert (top2[0] - top2[1]).item() < 0.05 * logs[t].abs().max().item(), f"step {t} diverged with a clear margin"
        break
    assert agree >= NEW // 2 and dec.linear_ns > 0


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_token_exchange_protocol_on_the_thread_fabric(world):
    """The all-gather / reduce-scatter protocol of the GPU kernels (epoch parity, per-block flags, done acknowledgements,
    owner-reset arrival counters) run by skewed threads-as-ranks: no payload word may ever differ from its expectation,
    and the harness must notice when one of the two buffers is taken away."""
    info = H.NumaInfo()
    for mode in (1, 2, 3):
        st, mis = H.fabric_token_exchange(info, world, rows_per_rank=48, blocks=3, iters=200, skew_seed=world + mode, mode=mode)
        assert (st, mis) == (0, 0), (mode, st, mis)
    st, mis = H.fabric_token_exchange(info, world, iters=200, mode=1, fault=1)      # acknowledgements are belt and braces here
    assert (st, mis) == (0, 0)
    if world > 1:
        st, mis = H.fabric_token_exchange(info, world, iters=300, mode=1, fault=2)  # single buffer: must be caught
        assert st == 0 and mis > 0


def test_worker_team_runs_many_jobs_on_the_same_parked_threads():
    """The parked-worker team gives the same bits as thread-per-job pools, job after job, and shuts down cleanly."""
    import torch
    info = H.NumaInfo()
    team = H.WorkerTeam(info)
    assert team.size >= 1
    g = torch.Generator().manual_seed(5)
    wq = torch.randint(-127, 128, (96, 256), generator=g, dtype=torch.int8)
    sw = torch.rand((96,), generator=g) * 9e-3 + 1e-3
    before = team.jobs_run
    for i in range(20):
        x = torch.randn((1 + i % 7, 256), generator=g).to(torch.bfloat16)
        a = H.w8a8_linear(info, x, wq, sw, team=team)
        b = H.w8a8_linear(info, x, wq, sw)
        assert a["status"] == 0 and a["workers"] == team.size
        assert torch.equal(a["y"], b["y"]) and torch.equal(a["acc"], b["acc"]) and torch.equal(a["q"], b["q"])
    assert team.jobs_run == before + 40            # two phases per linear
    team.close()


def test_node_sharded_weights_live_where_their_readers_run():
    """Weights copied into per-node arenas: every shard's pages are on the node of the worker that streams them, and the
    linear over them gives the same bits as the linear over the original tensor."""
    import torch
    info = H.NumaInfo()
    team = H.WorkerTeam(info)
    g = torch.Generator().manual_seed(9)
    wq = torch.randint(-127, 128, (203, 384), generator=g, dtype=torch.int8)
    sw = torch.rand((203,), generator=g) * 9e-3 + 1e-3
    hw = H.HostWeights(team, wq, sw)
    assert hw.misplaced in (0, -1)                 # -1: move_pages is not permitted in this sandbox
    for m in (1, 9, 40):
        x = torch.randn((m, 384), generator=g).to(torch.bfloat16)
        a = H.w8a8_linear(info, x, None, None, weights=hw)
        b = H.w8a8_linear(info, x, wq, sw)
        assert a["status"] == 0 and torch.equal(a["y"], b["y"]) and torch.equal(a["acc"], b["acc"])
    del hw
    team.close()


def test_arena_unmaps_exactly_what_it_mapped():
    """The mapped length is the size rounded up to the page size of the mode, and that is what munmap gets back."""
    info = H.NumaInfo()
    a = H.NumaArena(info.node_ids[0], 5000, page_size=H.PAGE_STANDARD)
    assert a and a.mapped_bytes() == 8192 and a.unmap() == 0
    huge = H.NumaArena(info.node_ids[0], (2 << 20) + 4096, page_size=H.PAGE_EXPLICIT_2MB)
    if not huge:
        pytest.skip("no hugetlb pool on this machine: the explicit 2 MiB mapping cannot be made")
    assert huge.mapped_bytes() == 4 << 20
    assert huge.unmap() == 0              # a 4 KiB-rounded length would be refused with EINVAL and leak the huge pages


def test_worker_team_skips_nodes_without_cpus(tmp_path):
    """A memory-only node (online, empty cpulist) gets no pool and no workers; the team on the other node works."""
    live = H.NumaInfo()
    node0 = live.node_ids[0]
    cpus = live.get_node_cpus(node0)[:2]
    nodes = {node0: (",".join(map(str, cpus)), [10, 80], 1000, 500), node0 + 1: ("", [80, 10], 4000, 4000)}
    info = H.NumaInfo(_fake_sysfs(tmp_path, nodes))
    assert info.num_nodes == 2 and info.get_node_cpus(node0 + 1) == []
    assert info.cpus_per_node() == len(cpus) and info.total_cpus() == len(cpus)
    team = H.WorkerTeam(info)
    assert team.valid and team.size == len(cpus)
    assert {team.node_of(i) for i in range(team.size)} == {node0}
    assert team.run_sleep(1, 5000) == 0
    team.close()
    # the memory-only node in front of the CPU node
    (tmp_path / "b").mkdir()
    info2 = H.NumaInfo(_fake_sysfs(tmp_path / "b", {node0: ("", [10, 80], 10, 10), node0 + 1: (",".join(map(str, cpus)), [80, 10], 10, 10)}))
    assert info2.cpus_per_node() == len(cpus)


def test_worker_team_timeout_kills_the_team_instead_of_racing_on_the_job():
    """A job that overruns its timeout: run() reports -ETIMEDOUT, waits (bounded) for the stragglers so that the job's
    storage is not freed under them, and the team refuses every later job."""
    info = H.NumaInfo()
    team = H.WorkerTeam(info, max_workers_per_node=2)
    assert team.run_sleep(1, 5000) == 0 and team.valid
    t0 = time.monotonic()
    assert team.run_sleep(300, 30) == -110            # -ETIMEDOUT
    waited = time.monotonic() - t0
    assert 0.25 < waited < 2.5                         # it stayed until the sleepers were done, not just 30 ms
    assert not team.valid and not team.stragglers
    assert team.run_sleep(1, 5000) == -22             # -EINVAL: fail fast from now on
    team.close()


def test_fabric_protocols_are_race_free_under_the_thread_sanitizer():
    """The collective protocols (epoch all-reduce, token exchange in all three modes) compiled with -fsanitize=thread
    and the ranks as std::threads: right values, and no data race reported."""
    from mojo_linuxperiments_b200 import _build
    try:
        exe = _build.build_hostrt_tsan()
    except RuntimeError as e:
        pytest.skip(f"no thread-sanitizer runtime on this machine: {str(e)[-200:]}")
    # address-space randomisation with very high entropy can break the sanitizer's shadow mapping: run without it
    cmd = (["setarch", "-R"] if subprocess.run(["setarch", "-R", "true"], capture_output=True).returncode == 0 else []) + [str(exe)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert "ThreadSanitizer" not in p.stderr, p.stderr[-3000:]
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert p.stdout.count("[PASS]") == 8


def test_heap_range_check_reports_and_refuses_out_of_range_offsets():
    """The check the range-checked ("debug") GPU kernels apply before touching a symmetric heap, exercised on the host
    with bad offsets (on a GPU only valid cases ever run): in range passes, anything else is refused and the first
    violation is what the report keeps."""
    RC = 0x52430001
    rep = (ctypes.c_int * 3)()
    chk = H.lib().hostrt_range_check
    ext = 1 << 20
    assert chk(0, 16, ext, rep) == 1 and chk(ext - 16, 16, ext, rep) == 1 and chk(123, 0, ext, rep) == 1
    assert list(rep) == [0, 0, 0]
    assert chk(ext - 15, 16, ext, rep) == 0                       # one byte past the end
    assert list(rep) == [RC, (ext - 15) & 0xffffffff, 0]
    assert chk((5 << 32) + 8, 8, ext, rep) == 0                   # far outside: refused, first report kept
    assert list(rep) == [RC, (ext - 15) & 0xffffffff, 0]
    rep2 = (ctypes.c_int * 3)()
    assert chk((5 << 32) + 8, 8, ext, rep2) == 0 and list(rep2) == [RC, 8, 5]
    assert chk(2**64 - 8, 16, ext, rep2) == 0                     # offset + length would wrap around
    assert chk(0, ext + 1, ext, rep2) == 0
    assert chk(1 << 40, 1 << 40, 0, rep2) == 1                    # extent 0 = unknown: nothing is checked
