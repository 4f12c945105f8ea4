"""Per-rank runtime services under the engine: where the rank runs and where its memory lives.

The reference parks its orchestrator on a chosen CPU (test_linux_threading.mojo:112-115), pins every worker to the
CPUs of its NUMA node (threading/linux_threading.mojo:160-162, 316-318) and gives every node its own arena from which
the node-local buffers are carved (test_linux_threading.mojo:237-250, threading/numa_arena.mojo:6-87).  A rank of this
runtime is one process driving one B200, so the same three steps are:

  * ``GpuTopology`` tells which NUMA node the rank's GPU hangs off (PCI bus id -> sysfs);
  * the rank's host thread is pinned to that node's CPUs with the raw ``sched_setaffinity`` of the host runtime, so the
    launch path, the pinned staging buffers and the NIC / PCIe root of the GPU share a socket;
  * one ``HbmArena`` (a CUDA virtual-memory reservation) backs the rank's long-lived device buffers: the paged KV
    cache, its page table and lengths, the kernels' scratch, counters and status words.  ``used() / remaining() /
    high_water()`` are the reference arena's own counters (threading/numa_arena.mojo:72-78) and go into the metrics.

Everything degrades to "not pinned" / "torch allocator" with a recorded reason when a piece is missing (no sysfs
node for the GPU, no permission to set affinity, driver without virtual memory management): serving must not depend on it.
"""
from __future__ import annotations

import os

import torch


class RankRuntime:
    def __init__(self, device: torch.device, pin: bool | None = None):
        self.device = device
        self.index = device.index if device.index is not None else torch.cuda.current_device()
        self.gpu: dict = {}
        self.numa_node = -1
        self.pinned_cpus: list[int] = []
        self.notes: list[str] = []
        self.arena = None             # the KV arena of the running batch (replaced when the batch geometry changes)
        self.scratch_arena = None     # kernels' scratch, counters, status words: lives as long as the rank
        if pin is None:
            pin = os.environ.get("B200RT_PIN", "1") not in ("0", "false")
        self._discover()
        if pin:
            self._pin()

    # ---- topology -------------------------------------------------------------------------------------------
    def _discover(self) -> None:
        try:
            from .. import devrt
            topo = devrt.GpuTopology()
            if topo.status < 0 or self.index >= topo.num_devices:
                self.notes.append(f"GPU topology unavailable (status {topo.status})")
                return
            self.gpu = topo.gpu(self.index)
            self.numa_node = int(self.gpu.get("numa_node", -1))
            self.peers = topo.peers_of(self.index).devices()
        except Exception as e:      # the engine works without it
            self.notes.append(f"GPU topology unavailable: {type(e).__name__}: {e}")

    def _pin(self) -> None:
        """Pin the calling (rank) thread to the CPUs of the GPU's NUMA node."""
        try:
            from .. import hostrt
            info = hostrt.NumaInfo()
            node = self.numa_node
            if node < 0 or node not in info.node_ids:
                self.notes.append("the GPU reports no NUMA node: host thread left unpinned")
                return
            cpus = info.get_node_cpus(node)
            if not cpus:
                self.notes.append(f"NUMA node {node} has no CPUs: host thread left unpinned")
                return
            allowed = set(os.sched_getaffinity(0))
            usable = [c for c in cpus if c in allowed]
            if not usable:
                self.notes.append(f"none of node {node}'s CPUs is in this process's cpuset: host thread left unpinned")
                return
            mask = hostrt.CpuMask()
            for c in usable:
                mask.set(c)
            rc = hostrt.set_thread_affinity(mask)
            if rc not in (0, None, True):
                self.notes.append(f"sched_setaffinity failed ({rc}): host thread left unpinned")
                return
            self.pinned_cpus = usable
        except Exception as e:
            self.notes.append(f"pinning failed: {type(e).__name__}: {e}")

    def where_am_i(self) -> tuple[int, int]:
        """(cpu, numa node) the calling thread runs on right now (getcpu)."""
        from .. import hostrt
        return hostrt.get_current_cpu_and_node()

    # ---- memory ---------------------------------------------------------------------------------------------
    def _new_arena(self, nbytes: int):
        if os.environ.get("B200RT_ARENA", "1") in ("0", "false"):
            return None
        try:
            from .. import devrt
            a = devrt.HbmArena(self.index, int(nbytes), alignment=1024)
            if not a:
                self.notes.append(f"HBM arena of {nbytes} bytes refused (status {a.status}): torch allocator used instead")
                return None
            return a
        except Exception as e:
            self.notes.append(f"HBM arena unavailable: {type(e).__name__}: {e}")
            return None

    def make_arena(self, nbytes: int) -> bool:
        """(Re)create the KV arena with room for ``nbytes``.  The previous one is released as soon as the last tensor
        carved from it is gone (tensors keep their arena alive).  False (with a note) when it cannot be made."""
        self.arena = None
        self.arena = self._new_arena(nbytes)
        return self.arena is not None

    def make_scratch_arena(self, nbytes: int) -> bool:
        if self.scratch_arena is None:
            self.scratch_arena = self._new_arena(nbytes)
        return self.scratch_arena is not None

    @staticmethod
    def _zeros_from(arena, shape, dtype):
        t = arena.tensor(tuple(shape), dtype) if arena is not None else None
        return None if t is None else t.zero_()

    def zeros(self, shape, dtype) -> torch.Tensor:
        """Zero-filled tensor from the KV arena (torch allocator when there is no arena or it is full)."""
        t = self._zeros_from(self.arena, shape, dtype)
        if t is None:
            if self.arena is not None:
                self.notes.append(f"arena full at {tuple(shape)} {dtype}: torch allocator used for this tensor")
            t = torch.zeros(tuple(shape), dtype=dtype, device=self.device)
        return t

    def scratch_zeros(self, shape, dtype) -> torch.Tensor:
        t = self._zeros_from(self.scratch_arena, shape, dtype)
        return t if t is not None else torch.zeros(tuple(shape), dtype=dtype, device=self.device)

    def owns(self, t: torch.Tensor) -> bool:
        for a in (self.arena, self.scratch_arena):
            if a is not None and a.base() <= t.data_ptr() < a.base() + a.size():
                return True
        return False

    def report(self) -> dict:
        r = {"gpu": self.gpu.get("name"), "sm_count": self.gpu.get("sm_count"), "gpu_numa_node": self.numa_node,
             "pinned_cpus": len(self.pinned_cpus), "notes": self.notes[-6:]}
        try:
            cpu, node = self.where_am_i()
            r["host_thread"] = {"cpu": cpu, "numa_node": node}
        except Exception:
            pass
        for key, a in (("kv_arena", self.arena), ("scratch_arena", self.scratch_arena)):
            if a is not None:
                r[key] = {"size": a.size(), "used": a.used(), "remaining": a.remaining(), "high_water": a.high_water(),
                          "placement_ok": a.verify_placement()}
        return r
