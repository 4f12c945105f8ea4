"""Python face of the C++ host runtime (``csrc/hostrt``): NUMA topology, CPU masks, NUMA-bound bump arenas,
a clone3/futex2 worker pool, futex gates, thread-rank collectives and the fill+reduce workload.

Capability parity with the reference's ``numa/``, ``threading/`` and ``notstdcollections/`` packages; the
heavy lifting (raw syscalls, child trampoline, futex waits) is native.  Workers launched on the pool must be
native functions (pass their address): a raw kernel thread has no Python thread state.
"""
from __future__ import annotations

import ctypes
from ctypes import (POINTER, byref, c_char_p, c_double, c_float, c_int, c_long, c_longlong, c_uint, c_ulong,
                    c_ulonglong, c_void_p, create_string_buffer)
from functools import lru_cache
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "libb200_hostrt.so"

ETIMEDOUT = 110
WAIT_FOREVER = -1
WAIT_NOTHING_RUNNING = -1
WAIT_TIMED_OUT = -2
PAGE_STANDARD, PAGE_THP_2MB, PAGE_EXPLICIT_2MB, PAGE_EXPLICIT_1GB = 4096, 2 << 20, -2, -1
SC_PASS, SC_FAIL, SC_SKIP = 0, 1, 2


@lru_cache(maxsize=None)
def lib() -> ctypes.CDLL:
    if not _LIB_PATH.exists():
        from .. import _build
        _build.build_hostrt()
    L = ctypes.CDLL(str(_LIB_PATH))
    sig = {
        "hostrt_syscall_nr": (c_long, [c_char_p]), "hostrt_thread_clone_flags": (c_ulonglong, []),
        "hostrt_struct_size": (c_long, [c_char_p]), "hostrt_slot_total_size": (c_long, [c_ulong]),
        "hostrt_gettid": (c_long, []), "hostrt_monotonic_ns": (c_long, []),
        "hostrt_mmap_numa": (c_void_p, [c_ulong, c_int, c_long]), "hostrt_munmap": (c_long, [c_void_p, c_ulong]),
        "hostrt_move_pages_query": (c_long, [c_void_p]), "hostrt_mprotect": (c_long, [c_void_p, c_ulong, c_long]),
        "hostrt_poke": (None, [c_void_p, c_longlong]), "hostrt_peek": (c_longlong, [c_void_p]),
        "hostrt_numa_create": (c_void_p, [c_char_p]), "hostrt_numa_destroy": (None, [c_void_p]),
        "hostrt_numa_ok": (c_int, [c_void_p]), "hostrt_numa_num_nodes": (c_int, [c_void_p]),
        "hostrt_numa_node_id": (c_int, [c_void_p, c_int]),
        "hostrt_numa_node_cpus": (c_int, [c_void_p, c_int, POINTER(c_int), c_int]),
        "hostrt_numa_node_mask": (c_int, [c_void_p, c_int, c_void_p]),
        "hostrt_numa_distance": (c_int, [c_void_p, c_int, c_int]), "hostrt_numa_cpus_per_node": (c_int, [c_void_p]),
        "hostrt_numa_cpus_on_node": (c_int, [c_void_p, c_int]), "hostrt_numa_total_cpus": (c_int, [c_void_p]),
        "hostrt_numa_mem_kb": (c_long, [c_void_p, c_int, c_int]), "hostrt_numa_debug": (c_int, [c_void_p, c_char_p, c_int]),
        "hostrt_parse_cpulist": (c_int, [c_char_p, POINTER(c_int), c_int]),
        "hostrt_parse_meminfo": (c_long, [c_char_p, c_char_p]),
        "hostrt_current_cpu_node": (None, [POINTER(c_int), POINTER(c_int)]),
        "hostrt_current_cpu_node_rseq": (None, [POINTER(c_int), POINTER(c_int)]),
        "hostrt_cpumask_bytes": (c_int, []), "hostrt_cpumask_set": (None, [c_void_p, c_long]),
        "hostrt_cpumask_clear": (None, [c_void_p, c_long]), "hostrt_cpumask_test": (c_int, [c_void_p, c_long]),
        "hostrt_cpumask_clear_all": (None, [c_void_p]), "hostrt_cpumask_set_all": (None, [c_void_p]),
        "hostrt_cpumask_count": (c_long, [c_void_p]),
        "hostrt_set_thread_affinity": (c_long, [c_void_p, c_ulong]), "hostrt_get_thread_affinity": (c_long, [c_void_p, c_ulong]),
        "hostrt_arena_create": (c_void_p, [c_int, c_ulong, c_ulong, c_long]), "hostrt_arena_destroy": (None, [c_void_p]),
        "hostrt_arena_valid": (c_int, [c_void_p]), "hostrt_arena_alloc": (c_void_p, [c_void_p, c_ulong]),
        "hostrt_arena_mark": (c_ulong, [c_void_p]), "hostrt_arena_reset_to": (None, [c_void_p, c_ulong]),
        "hostrt_arena_reset": (None, [c_void_p]), "hostrt_arena_remaining": (c_ulong, [c_void_p]),
        "hostrt_arena_mapped_bytes": (c_ulong, [c_void_p]), "hostrt_arena_unmap_status": (c_long, [c_void_p]),
        "hostrt_arena_used": (c_ulong, [c_void_p]), "hostrt_arena_base": (c_void_p, [c_void_p]),
        "hostrt_arena_verify_placement": (c_int, [c_void_p]),
        "hostrt_pool_create": (c_void_p, [c_int, c_void_p, c_ulong, c_int, c_ulong]), "hostrt_pool_destroy": (None, [c_void_p]),
        "hostrt_pool_valid": (c_int, [c_void_p]), "hostrt_pool_capacity": (c_int, [c_void_p]),
        "hostrt_pool_futex_flags": (c_uint, [c_void_p]), "hostrt_pool_running": (c_int, [c_void_p]),
        "hostrt_pool_launch": (c_int, [c_void_p, c_void_p] + [c_ulonglong] * 6),
        "hostrt_pool_wait_all": (c_long, [c_void_p, c_long]), "hostrt_pool_wait_any": (c_int, [c_void_p, c_long]),
        "hostrt_gate_wait": (c_long, [c_void_p, c_long]), "hostrt_gate_release": (None, [c_void_p]),
        "hostrt_gate_reset": (None, [c_void_p]),
        "hostrt_chain_reduce": (c_long, [c_void_p, c_int, c_long, POINTER(c_longlong)]),
        "hostrt_butterfly_allreduce": (c_long, [c_void_p, c_int, POINTER(c_longlong), c_long]),
        "hostrt_fabric_allreduce": (c_long, [c_void_p, c_int, POINTER(c_double), POINTER(c_double), c_int, c_long, c_int]),
        "hostrt_range_check": (c_int, [c_ulonglong, c_ulonglong, c_ulonglong, c_void_p]),
        "hostrt_team_create": (c_void_p, [c_void_p, c_int]), "hostrt_team_destroy": (None, [c_void_p]),
        "hostrt_team_size": (c_int, [c_void_p]), "hostrt_team_jobs_run": (c_ulonglong, [c_void_p]),
        "hostrt_team_valid": (c_int, [c_void_p]), "hostrt_team_stragglers": (c_int, [c_void_p]),
        "hostrt_team_node_of": (c_int, [c_void_p, c_int]), "hostrt_team_run_sleep": (c_long, [c_void_p, c_long, c_long]),
        "hostrt_w8a8_linear_team": (c_long, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
                                             c_void_p, c_void_p, c_void_p, POINTER(c_long)]),
        "hostrt_weights_create": (c_void_p, [c_void_p, c_void_p, c_int, c_int]), "hostrt_weights_destroy": (None, [c_void_p]),
        "hostrt_weights_misplaced": (c_int, [c_void_p]),
        "hostrt_w8a8_linear_sharded": (c_long, [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
                                                c_void_p, c_void_p, POINTER(c_long)]),
        "hostrt_fabric_token_exchange": (c_long, [c_void_p, c_int, c_int, c_int, c_int, c_long, c_uint, c_int, c_int, POINTER(c_int)]),
        "hostrt_fill_reduce": (c_long, [c_void_p, c_ulonglong, c_ulonglong, c_int, POINTER(c_double), POINTER(c_long),
                                        POINTER(c_int), POINTER(c_int)]),
        "hostrt_fill_reduce_serial": (c_double, [c_ulonglong, c_ulonglong]),
        "hostrt_w8a8_linear": (c_long, [c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                                        c_void_p, c_void_p, c_void_p, POINTER(c_long)]),
        "hostrt_philox_uniform": (c_float, [c_ulonglong, c_ulonglong]),
        "hostrt_philox_block": (None, [c_ulonglong, c_ulonglong, POINTER(c_uint)]),
        "hostrt_scenario_count": (c_int, []), "hostrt_scenario_name": (c_char_p, [c_int]),
        "hostrt_scenario_run": (c_int, [c_int, c_char_p, c_int]), "hostrt_run_all_scenarios": (c_int, [c_int]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    return L


def worker_address(name: str) -> int:
    """Address of one of the library's built-in native workers (``hostrt_worker_*``)."""
    return ctypes.cast(getattr(lib(), name), c_void_p).value


class CpuMask:
    """1,024-bit CPU set with the kernel's cpu_set_t layout (reference: numa/cpumask.mojo:4-61)."""

    BYTES = 128

    def __init__(self, cpus=()):
        self._buf = (ctypes.c_ubyte * self.BYTES)()
        for c in cpus:
            self.set(c)

    @classmethod
    def from_cpu_list(cls, cpus):
        return cls(cpus)

    def set(self, cpu): lib().hostrt_cpumask_set(self._buf, cpu)
    def clear(self, cpu): lib().hostrt_cpumask_clear(self._buf, cpu)
    def test(self, cpu) -> bool: return bool(lib().hostrt_cpumask_test(self._buf, cpu))
    def clear_all(self): lib().hostrt_cpumask_clear_all(self._buf)
    def set_all(self): lib().hostrt_cpumask_set_all(self._buf)
    def count(self) -> int: return lib().hostrt_cpumask_count(self._buf)
    def byte_size(self) -> int: return self.BYTES
    def ptr(self): return self._buf
    def to_bytes(self) -> bytes: return bytes(self._buf)
    def cpus(self): return [i for i in range(self.BYTES * 8) if self.test(i)]


def parse_cpulist(text: str):
    out = (c_int * 4096)()
    n = lib().hostrt_parse_cpulist(text.encode(), out, 4096)
    return list(out[:n])


def parse_meminfo(text: str, field: str) -> int:
    return lib().hostrt_parse_meminfo(text.encode(), field.encode())


class NumaInfo:
    """NUMA topology read from sysfs (reference: numa/numa.mojo:84-176).  ``root`` can point at a fixture tree."""

    def __init__(self, root: str | None = None):
        self._h = lib().hostrt_numa_create((root or "").encode())

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().hostrt_numa_destroy(self._h)
            except TypeError:          # interpreter shutdown: module globals are already gone
                pass
            self._h = None

    @property
    def ok(self) -> bool: return bool(lib().hostrt_numa_ok(self._h))
    @property
    def num_nodes(self) -> int: return lib().hostrt_numa_num_nodes(self._h)
    @property
    def node_ids(self): return [lib().hostrt_numa_node_id(self._h, i) for i in range(self.num_nodes)]

    def get_node_cpus(self, node: int):
        out = (c_int * 4096)()
        n = lib().hostrt_numa_node_cpus(self._h, node, out, 4096)
        return list(out[:n])

    def get_node_mask(self, node: int) -> CpuMask:
        m = CpuMask()
        lib().hostrt_numa_node_mask(self._h, node, m.ptr())
        return m

    def distance(self, a: int, b: int) -> int: return lib().hostrt_numa_distance(self._h, a, b)
    def cpus_per_node(self) -> int: return lib().hostrt_numa_cpus_per_node(self._h)
    def cpus_on_node(self, node: int) -> int: return lib().hostrt_numa_cpus_on_node(self._h, node)
    def total_cpus(self) -> int: return lib().hostrt_numa_total_cpus(self._h)
    def mem_total_kb(self, node: int) -> int: return lib().hostrt_numa_mem_kb(self._h, node, 0)
    def mem_free_kb(self, node: int) -> int: return lib().hostrt_numa_mem_kb(self._h, node, 1)

    def debug_string(self) -> str:
        buf = create_string_buffer(8192)
        lib().hostrt_numa_debug(self._h, buf, 8192)
        return buf.value.decode()

    def print_debug(self): print(self.debug_string(), end="")


def get_current_cpu_and_node():
    c, n = c_int(), c_int()
    lib().hostrt_current_cpu_node(byref(c), byref(n))
    return c.value, n.value


def get_cpu_and_node_rseq():
    c, n = c_int(), c_int()
    lib().hostrt_current_cpu_node_rseq(byref(c), byref(n))
    return c.value, n.value


def set_thread_affinity(mask: CpuMask) -> int:
    return lib().hostrt_set_thread_affinity(mask.ptr(), mask.BYTES)


def get_thread_affinity() -> CpuMask:
    m = CpuMask()
    lib().hostrt_get_thread_affinity(m.ptr(), m.BYTES)
    return m


class NumaArena:
    """NUMA-bound bump allocator (reference: threading/numa_arena.mojo:6-140).  ``alloc`` returns an address or None."""

    def __init__(self, node: int, size: int, alignment: int = 8, page_size: int = PAGE_THP_2MB):
        self._h = lib().hostrt_arena_create(node, size, alignment, page_size)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().hostrt_arena_destroy(self._h)
            self._h = None

    def __bool__(self): return bool(lib().hostrt_arena_valid(self._h))
    def alloc(self, nbytes: int): return lib().hostrt_arena_alloc(self._h, nbytes)
    def mark(self) -> int: return lib().hostrt_arena_mark(self._h)
    def reset_to(self, watermark: int): lib().hostrt_arena_reset_to(self._h, watermark)
    def reset(self): lib().hostrt_arena_reset(self._h)
    def remaining(self) -> int: return lib().hostrt_arena_remaining(self._h)
    def used(self) -> int: return lib().hostrt_arena_used(self._h)
    def mapped_bytes(self) -> int: return lib().hostrt_arena_mapped_bytes(self._h)

    def unmap(self) -> int:
        """Destroy the arena now and return what munmap answered (0 or -errno)."""
        h, self._h = self._h, None
        return lib().hostrt_arena_unmap_status(h) if h else 0

    def base(self): return lib().hostrt_arena_base(self._h)
    def verify_placement(self) -> bool: return bool(lib().hostrt_arena_verify_placement(self._h))


class ThreadPool:
    """Fixed-capacity pool of one-shot clone3 threads (reference: threading/linux_threading.mojo:43-158)."""

    def __init__(self, capacity: int, cpu_mask: CpuMask | None = None, numa_node: int | None = None,
                 stack_size: int = 64 * 1024):
        self._mask = cpu_mask
        self._h = lib().hostrt_pool_create(capacity, cpu_mask.ptr() if cpu_mask else None,
                                           CpuMask.BYTES if cpu_mask else 0,
                                           -1 if numa_node is None else numa_node, stack_size)

    @classmethod
    def for_numa_node(cls, info: NumaInfo, node: int, **kw):
        return cls(info.cpus_on_node(node), info.get_node_mask(node), node, **kw)

    @classmethod
    def for_numa_node_excluding(cls, info: NumaInfo, node: int, exclude_cpu: int, **kw):
        m = info.get_node_mask(node)
        n = info.cpus_on_node(node)
        if m.test(exclude_cpu):
            m.clear(exclude_cpu)
            n -= 1
        return cls(n, m, node, **kw)

    def close(self):
        if getattr(self, "_h", None):
            lib().hostrt_pool_destroy(self._h)
            self._h = None

    __del__ = close

    def __bool__(self): return bool(lib().hostrt_pool_valid(self._h))
    def __len__(self): return lib().hostrt_pool_capacity(self._h)
    def __iter__(self): return iter(range(len(self)))
    @property
    def futex_flags(self) -> int: return lib().hostrt_pool_futex_flags(self._h)
    def running(self) -> int: return lib().hostrt_pool_running(self._h)

    def launch(self, fn_addr: int, *args: int) -> bool:
        assert len(args) <= 6, "at most six 8-byte arguments"
        a = list(args) + [0] * (6 - len(args))
        return lib().hostrt_pool_launch(self._h, fn_addr, *a) >= 0

    def wait_all(self, timeout_ns: int = WAIT_FOREVER) -> int: return lib().hostrt_pool_wait_all(self._h, timeout_ns)
    def wait_any(self, timeout_ns: int = WAIT_FOREVER) -> int: return lib().hostrt_pool_wait_any(self._h, timeout_ns)


class MutexGate:
    """Single-use binary latch on a 32-bit word at ``addr`` (reference: threading/linux_threading.mojo:172-198)."""

    def __init__(self, addr: int): self.addr = addr
    @classmethod
    def from_addr(cls, addr: int): return cls(addr)
    def wait(self, timeout_ns: int = WAIT_FOREVER) -> int: return lib().hostrt_gate_wait(self.addr, timeout_ns)
    def release(self): lib().hostrt_gate_release(self.addr)
    def reset(self): lib().hostrt_gate_reset(self.addr)


def chain_reduce(info: NumaInfo, world: int, timeout_ns: int = 10_000_000_000):
    v = c_longlong()
    st = lib().hostrt_chain_reduce(info._h, world, timeout_ns, byref(v))
    return st, v.value


def butterfly_allreduce(info: NumaInfo, world: int, timeout_ns: int = 10_000_000_000):
    out = (c_longlong * max(world, 1))()
    st = lib().hostrt_butterfly_allreduce(info._h, world, out, timeout_ns)
    return st, list(out)


def fabric_allreduce(info: NumaInfo, values, rounds: int = 1, timeout_ns: int = 2_000_000_000, drop_rank: int = -1):
    w = len(values)
    inp = (c_double * w)(*values)
    out = (c_double * w)()
    st = lib().hostrt_fabric_allreduce(info._h, w, inp, out, rounds, timeout_ns, drop_rank)
    return st, list(out)


def fabric_token_exchange(info: NumaInfo, world: int, rows_per_rank: int = 64, blocks: int = 4, iters: int = 50,
                          timeout_ns: int = 2_000_000_000, skew_seed: int = 1, mode: int = 3, fault: int = 0):
    """Threads-as-ranks run of the token-sharded all-gather / reduce-scatter protocol; returns (status, mismatches).
    mode 1 all-gather only, 2 reduce-scatter only, 3 both; fault 1 drops the wait for the done acknowledgements, fault 2
    uses a single buffer instead of two (a hole the run must report as mismatches)."""
    mis = c_int()
    st = lib().hostrt_fabric_token_exchange(info._h, world, rows_per_rank, blocks, iters, timeout_ns, skew_seed, mode, fault,
                                            byref(mis))
    return st, mis.value


def fill_reduce(info: NumaInfo, n_elems: int = 16 * 1024 * 1024, seed: int = 0, max_workers_per_node: int = 0):
    s, ns, w, mis = c_double(), c_long(), c_int(), c_int()
    st = lib().hostrt_fill_reduce(info._h, n_elems, seed, max_workers_per_node, byref(s), byref(ns), byref(w), byref(mis))
    return {"status": st, "sum": s.value, "elapsed_ns": ns.value, "workers": w.value, "misplaced": mis.value}


class WorkerTeam:
    """Parked, pinned workers (one per core of every NUMA node) that are woken for each job instead of being created
    for it (``csrc/hostrt/team.hpp``).  Pass it to ``w8a8_linear(..., team=...)``."""

    def __init__(self, info: NumaInfo, max_workers_per_node: int = 0):
        self._h = lib().hostrt_team_create(info._h, max_workers_per_node)
        if not self._h:
            raise RuntimeError("could not create the worker team")

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().hostrt_team_destroy(self._h)
            except TypeError:          # interpreter shutdown
                pass
            self._h = None

    close = __del__

    @property
    def size(self) -> int: return lib().hostrt_team_size(self._h)
    @property
    def jobs_run(self) -> int: return lib().hostrt_team_jobs_run(self._h)
    @property
    def valid(self) -> bool: return bool(lib().hostrt_team_valid(self._h))
    @property
    def stragglers(self) -> bool: return bool(lib().hostrt_team_stragglers(self._h))

    def node_of(self, worker: int) -> int: return lib().hostrt_team_node_of(self._h, worker)

    def run_sleep(self, sleep_ms: int, timeout_ms: int) -> int:
        """Every worker sleeps ``sleep_ms`` inside one job while the caller waits ``timeout_ms`` at most; returns the
        status of ``WorkerTeam::run`` (0, or -ETIMEDOUT = -110).  A timed-out team is invalid from then on."""
        return lib().hostrt_team_run_sleep(self._h, sleep_ms, timeout_ms)


class HostWeights:
    """int8 weights [N, K] copied into NUMA arenas so that each team worker's output-channel range is local to the node
    the worker is pinned to (``NodeShardedWeights`` in ``csrc/hostrt/w8a8_host.hpp``)."""

    def __init__(self, team: WorkerTeam, wq, sw):
        import torch
        assert wq.dtype == torch.int8 and wq.is_contiguous() and not wq.is_cuda and sw.dtype == torch.float32
        self.team, self.N, self.K = team, wq.shape[0], wq.shape[1]
        self.sw = sw.contiguous()
        self._h = lib().hostrt_weights_create(team._h, wq.data_ptr(), self.N, self.K)
        if not self._h:
            raise MemoryError("could not place the weights in the node arenas")

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                lib().hostrt_weights_destroy(self._h)
            except TypeError:
                pass
            self._h = None

    @property
    def misplaced(self) -> int:
        """Shards whose first page is not on its reader's node (-1 when the kernel does not tell)."""
        return lib().hostrt_weights_misplaced(self._h)


def w8a8_linear(info: NumaInfo, x, wq, sw, max_workers_per_node: int = 0, force_scalar: bool = False, isa: str = "best",
                team: "WorkerTeam | None" = None, weights: "HostWeights | None" = None):
    """W8A8 Hadamard linear on the host CPUs over the pinned worker pools (``csrc/hostrt/w8a8_host.cpp``).

    x: torch bf16 [M, K] (CPU), wq: int8 [N, K], sw: fp32 [N].  Returns a dict with ``y`` (bf16 [M, N]), the quantised
    activations ``q`` / ``sx``, the exact int32 accumulators ``acc`` and timing / dispatch info.  ``isa``: "best"
    (AMX int8, else AVX-512 VNNI, else scalar), "vnni" (no AMX), "scalar"."""
    import torch
    if weights is not None:
        team, sw = weights.team, weights.sw
        N = weights.N
        assert x.shape[1] == weights.K
    else:
        assert wq.dtype == torch.int8 and sw.dtype == torch.float32 and wq.is_contiguous() and sw.is_contiguous()
        N = wq.shape[0]
    assert x.dtype == torch.bfloat16 and not x.is_cuda and x.is_contiguous()
    M, K = x.shape
    y = torch.empty((M, N), dtype=torch.bfloat16)
    q = torch.empty((M, K), dtype=torch.int8)
    sx = torch.empty((M,), dtype=torch.float32)
    acc = torch.empty((M, N), dtype=torch.int32)
    info5 = (c_long * 5)()
    mode = 1 if (force_scalar or isa == "scalar") else (2 if isa == "vnni" else 0)
    if weights is not None:
        st = lib().hostrt_w8a8_linear_sharded(team._h, weights._h, x.data_ptr(), M, sw.data_ptr(), y.data_ptr(), mode,
                                              q.data_ptr(), sx.data_ptr(), acc.data_ptr(), info5)
    elif team is not None:
        st = lib().hostrt_w8a8_linear_team(team._h, x.data_ptr(), M, K, wq.data_ptr(), sw.data_ptr(), N, y.data_ptr(), mode,
                                           q.data_ptr(), sx.data_ptr(), acc.data_ptr(), info5)
    else:
        st = lib().hostrt_w8a8_linear(info._h, x.data_ptr(), M, K, wq.data_ptr(), sw.data_ptr(), N, y.data_ptr(),
                                      max_workers_per_node, mode, q.data_ptr(), sx.data_ptr(), acc.data_ptr(), info5)
    return {"status": st, "y": y, "q": q, "sx": sx, "acc": acc, "quant_ns": info5[0], "gemm_ns": info5[1],
            "workers": info5[2], "used_vnni": bool(info5[3]), "isa": ("scalar", "avx512-vnni", "amx-int8")[info5[3]]}


def philox_uniform(i: int, seed: int) -> float:
    return lib().hostrt_philox_uniform(i, seed)


def run_scenarios():
    """Runs the twelve integration scenarios; returns [(name, result, detail)]."""
    out = []
    for i in range(lib().hostrt_scenario_count()):
        buf = create_string_buffer(256)
        r = lib().hostrt_scenario_run(i, buf, 256)
        out.append((lib().hostrt_scenario_name(i).decode(), r, buf.value.decode()))
    return out
