"""Symmetric (peer-mapped) HBM for one rank group: the GPU form of the reference's shared arena that every worker
can address (test_linux_threading.mojo:426-435) and of its futex gates (threading/linux_threading.mojo:174-198).

Every rank allocates the same number of bytes; after the rendezvous each rank holds a pointer to every other rank's
block (NVLink / NVSwitch peer mapping) and, where the fabric supports it, one NVLS multicast pointer that addresses all
copies at once.  The first ``FLAG_BYTES`` of the block are the rank's flag words (epochs written by peers); the rest is
a bump-allocated data heap whose offsets are identical on every rank.  The kernels that read and write peers are this
package's own.  Allocation and mapping have two backends, chosen by ``B200RT_SYMM``:

* ``torch`` (default): ``torch.distributed._symmetric_memory`` - peer pointers and, where the fabric has it, the NVLS
  multicast pointer the ``multimem`` kernels use.
* ``native``: this package's device runtime (``devrt.SymmSegment``: a virtual-memory block per rank, exported as a
  POSIX descriptor, handed to the peers over unix sockets and mapped by each of them).  Peer pointers only by
  default, so the kernels take their peer-store paths and a rank that dies leaves no multicast binding behind;
  ``B200RT_SYMM_MC=1`` also creates a multicast object over the blocks (``cuMulticastCreate`` on rank 0, every rank
  adds its device and binds its block) and maps it, which gives the ``multimem`` kernels their pointer.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import _lib

FLAG_BYTES = 4096
CANARY_BYTES = 64                      # debug mode: guard words before and after every allocation
CANARY_WORD = 0x5AFEC0DE
AR_ONE_SHOT_P2P, AR_ONE_SHOT_NVLS, AR_TWO_SHOT_NVLS, AR_CHAIN, AR_BUTTERFLY, AR_LOW_LATENCY = 0, 1, 2, 3, 4, 5
_DTYPES = {torch.bfloat16: 0, torch.float32: 1, torch.float64: 2}


class SymmetricHeap:
    def __init__(self, nbytes: int, group=None, device=None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (nbytes + 4095) // 4096 * 4096
        total = FLAG_BYTES + self.nbytes
        self.backend = os.environ.get("B200RT_SYMM", "torch").lower()
        self.segment = None
        if self.backend == "native":
            ptrs, mc = self._native_rendezvous(total)
        else:
            self.block = symm_mem.empty(total, dtype=torch.uint8, device=self.device)
            self.block.zero_()
            self.handle = symm_mem.rendezvous(self.block, group=self.group.group_name)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
            mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.flag_ptrs = ptrs
        self.data_ptrs = [p + FLAG_BYTES for p in ptrs]
        self.mc_data_ptr = mc + FLAG_BYTES if mc else 0
        self._c_data = (ctypes.c_void_p * self.world)(*self.data_ptrs)
        self._c_flags = (ctypes.c_void_p * self.world)(*self.flag_ptrs)
        self.offset = 0
        # Debug mode (B200RT_DEBUG=1 / the range-checked kernel library): every allocation is fenced by canary words
        # that check_status() verifies - the reference's guard pages (threading/linux_threading.mojo:148,419-420)
        # for a heap that cannot have any - and the kernels are told the heap's extent so they can refuse offsets
        # beyond it.
        self.debug = bool(_lib.lib().b200_debug_compiled()) if torch.cuda.is_available() else False
        self._canaries: list[int] = []
        if self.debug:
            _lib.lib().b200_debug_set_heap_extent(self.nbytes)
        # device-resident epoch words of this rank: [epoch, exit counter, stage counters...]
        self.epoch_words = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def _native_rendezvous(self, total: int):
        """Own block through the device runtime, peers' blocks mapped from the descriptors they hand over."""
        from .. import devrt
        dev = self.device.index if self.device.index is not None else torch.cuda.current_device()
        torch.cuda.init()
        torch.zeros(1, device=self.device)                       # the primary context exists before the driver calls
        self.segment = devrt.SymmSegment(dev, total, self.world, self.rank)

        def gather(name):
            names = [None] * self.world
            dist.all_gather_object(names, name, group=self.group)
            return names

        fds = devrt.exchange_fds(self.segment.export_fd(), self.rank, self.world, gather)
        try:
            for r, fd in fds.items():
                rc = self.segment.map_peer(r, fd)
                if rc != 0:
                    raise RuntimeError(f"mapping rank {r}'s block failed with status {rc}")
        finally:
            for fd in fds.values():
                os.close(fd)
            os.close(self.segment.export_fd())
        self.block = self.segment.local_tensor()[:total]
        self.block.zero_()
        self.handle = None
        mc = 0
        if os.environ.get("B200RT_SYMM_MC", "0") not in ("0", "") and self.world > 1:
            mc = self._native_multicast(gather)
        return [self.segment.peer_ptr(r) for r in range(self.world)], mc

    def _native_multicast(self, gather) -> int:
        """Bind every rank's block to one multicast object and map it; every rank learns of a failure on any rank."""
        from .. import devrt
        seg = self.segment

        def agree(rc: int, what: str):
            codes = [None] * self.world
            dist.all_gather_object(codes, rc, group=self.group)
            if any(c < 0 for c in codes):
                raise RuntimeError(f"multicast object: {what} failed with status {codes} (one entry per rank)")

        own = seg.mc_create() if self.rank == 0 else os.open(os.devnull, os.O_RDONLY)
        agree(min(own, 0), "cuMulticastCreate / export on rank 0")
        fds = devrt.exchange_fds(own, self.rank, self.world, gather)
        try:
            rc = seg.mc_import(fds[0]) if self.rank != 0 else 0
        finally:
            for fd in fds.values():
                os.close(fd)
            os.close(own)
        agree(rc, "import of the multicast handle")
        agree(seg.mc_add_device(), "cuMulticastAddDevice")          # also the barrier: every device is in before any bind
        agree(seg.mc_bind(), "cuMulticastBindMem / map")
        return seg.mc_ptr

    @property
    def has_multicast(self) -> bool:
        return self.mc_data_ptr != 0

    # -- bump allocation: same offsets on every rank as long as every rank makes the same calls ----------------
    def alloc(self, nbytes: int, align: int = 256) -> int:
        if self.debug:
            # [canary][allocation][canary]; every rank makes the same calls, so the offsets still agree
            lead = (self.offset + CANARY_BYTES + align - 1) // align * align
            end = lead + nbytes + CANARY_BYTES
            if end > self.nbytes:
                raise MemoryError(f"symmetric heap exhausted ({end} > {self.nbytes})")
            for off in (lead - CANARY_BYTES, lead + nbytes):
                self.tensor(off, (CANARY_BYTES // 4,), torch.int32).fill_(CANARY_WORD)
                self._canaries.append(off)
            self.offset = end
            return lead
        start = (self.offset + align - 1) // align * align
        if start + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted ({start + nbytes} > {self.nbytes})")
        self.offset = start + nbytes
        return start

    def check_canaries(self) -> list[int]:
        """Offsets of the guard blocks that no longer hold the canary pattern (debug mode; synchronises)."""
        bad = []
        for off in self._canaries:
            if off + CANARY_BYTES <= self.offset and not bool((self.tensor(off, (CANARY_BYTES // 4,), torch.int32) == CANARY_WORD).all().item()):
                bad.append(off)
        return bad

    def mark(self) -> int: return self.offset
    def reset_to(self, w: int):
        if w <= self.offset:
            self.offset = w
            self._canaries = [c for c in self._canaries if c + CANARY_BYTES <= w]
    def remaining(self) -> int: return self.nbytes - self.offset
    def used(self) -> int: return self.offset

    def tensor(self, offset: int, shape, dtype) -> torch.Tensor:
        """Local view of this rank's bytes at ``offset``."""
        n = 1
        for s in shape:
            n *= s
        nb = n * torch.empty((), dtype=dtype).element_size()
        return self.block[FLAG_BYTES + offset: FLAG_BYTES + offset + nb].view(dtype).view(*shape)

    def alloc_tensor(self, shape, dtype, align: int = 256):
        n = 1
        for s in shape:
            n *= s
        off = self.alloc(n * torch.empty((), dtype=dtype).element_size(), align)
        return off, self.tensor(off, shape, dtype)

    def check_status(self):
        st = self.status.tolist()
        if st[1] != 0:
            self.status.zero_()
            raise RuntimeError(f"range-checked kernel refused heap offset {(st[3] & 0xffffffff) << 32 | (st[2] & 0xffffffff)} "
                               f"(heap of {self.nbytes} bytes): the access was skipped")
        if st[0] != 0:
            self.status.zero_()
            raise RuntimeError(f"peer kernel status {st[0]} (5 = a flag from a peer never arrived)")
        if self.debug:
            bad = self.check_canaries()
            if bad:
                raise RuntimeError(f"symmetric heap canaries overwritten at offsets {bad[:8]}: a kernel wrote outside its allocation")

    # -- collectives --------------------------------------------------------------------------------------------
    def all_reduce(self, offset: int, n: int, dtype: torch.dtype, out: torch.Tensor | None, *, algo: int | None = None,
                   residual: torch.Tensor | None = None, scratch_offset: int = 0, trailing_barrier: bool = True,
                   limit_ms: int = 2000, max_ctas: int = 64) -> torch.Tensor | None:
        """Sum the ``n`` elements every rank holds at ``offset`` of its heap.  The result goes to ``out`` (any local
        tensor), or stays in place in every heap for the two-shot NVLS algorithm when ``out`` is None."""
        if algo is None:
            nbytes = n * torch.empty((), dtype=dtype).element_size()
            if self.has_multicast and dtype != torch.float64 and nbytes % 16 == 0:
                algo = AR_ONE_SHOT_NVLS if nbytes <= (512 << 10) else AR_TWO_SHOT_NVLS
            else:
                algo = AR_ONE_SHOT_P2P
        rc = _lib.lib().b200_peer_allreduce(
            self._c_data, self._c_flags, self.mc_data_ptr or None, self.world, self.rank, offset, scratch_offset,
            out.data_ptr() if out is not None else None, _lib.ptr(residual), n, _DTYPES[dtype], algo,
            self.epoch_words.data_ptr(), self.status.data_ptr(), limit_ms, 1 if trailing_barrier else 0, max_ctas,
            _lib.stream())
        _lib.check(rc, "peer_allreduce")
        return out
