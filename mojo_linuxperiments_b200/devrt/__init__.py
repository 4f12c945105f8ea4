"""Device runtime: GPU / NVLink topology, device masks and per-GPU HBM arenas (C++ core in ``csrc/devrt``).

These are the GPU-side counterparts of the reference's ``NumaInfo`` (numa/numa.mojo:84-176), ``CpuMask``
(numa/cpumask.mojo:4-61) and ``NumaArena`` (threading/numa_arena.mojo:6-140).  Memory handed out by an ``HbmArena``
can be viewed as a torch tensor (``HbmArena.tensor``) without copying.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, byref, c_char_p, c_int, c_ulonglong, c_void_p, create_string_buffer
from functools import lru_cache
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent.parent / "_lib" / "libb200_devrt.so"
NO_DRIVER = -1000


@lru_cache(maxsize=None)
def lib() -> ctypes.CDLL:
    if not _LIB_PATH.exists():
        from .. import _build
        _build.build_devrt()
    L = ctypes.CDLL(str(_LIB_PATH))
    U = c_ulonglong
    sig = {
        "devrt_reload_driver": (None, []),
        "devrt_topology_create": (c_void_p, []), "devrt_topology_destroy": (None, [c_void_p]),
        "devrt_topology_status": (c_int, [c_void_p]), "devrt_topology_num_devices": (c_int, [c_void_p]),
        "devrt_topology_peer_access": (c_int, [c_void_p, c_int, c_int]),
        "devrt_topology_distance": (c_int, [c_void_p, c_int, c_int]),
        "devrt_topology_peers_of": (U, [c_void_p, c_int]), "devrt_topology_fully_connected": (c_int, [c_void_p]),
        "devrt_topology_gpu": (c_int, [c_void_p, c_int, c_char_p, c_int, POINTER(c_int), POINTER(c_int), POINTER(U),
                                       POINTER(U), POINTER(c_int), POINTER(c_int), c_char_p, c_int]),
        "devrt_topology_debug": (c_int, [c_void_p, c_char_p, c_int]),
        "devrt_arena_create": (c_void_p, [c_int, U, U]), "devrt_arena_destroy": (None, [c_void_p]),
        "devrt_arena_valid": (c_int, [c_void_p]), "devrt_arena_status": (c_int, [c_void_p]),
        "devrt_arena_alloc": (U, [c_void_p, U]), "devrt_arena_mark": (U, [c_void_p]),
        "devrt_arena_reset_to": (None, [c_void_p, U]), "devrt_arena_reset": (None, [c_void_p]),
        "devrt_arena_remaining": (U, [c_void_p]), "devrt_arena_used": (U, [c_void_p]),
        "devrt_arena_size": (U, [c_void_p]), "devrt_arena_high_water": (U, [c_void_p]),
        "devrt_arena_base": (U, [c_void_p]), "devrt_arena_verify_placement": (c_int, [c_void_p]),
        "devrt_symm_create": (c_void_p, [c_int, U, c_int, c_int]), "devrt_symm_destroy": (None, [c_void_p]),
        "devrt_symm_export_fd": (c_int, [c_void_p]), "devrt_symm_map_peer": (c_int, [c_void_p, c_int, c_int]),
        "devrt_symm_base": (U, [c_void_p]), "devrt_symm_stride": (U, [c_void_p]),
        "devrt_symm_peer_ptr": (U, [c_void_p, c_int]), "devrt_symm_mapped": (c_int, [c_void_p, c_int]),
        "devrt_symm_mc_create": (c_int, [c_void_p]), "devrt_symm_mc_import": (c_int, [c_void_p, c_int]),
        "devrt_symm_mc_add_device": (c_int, [c_void_p]), "devrt_symm_mc_bind": (c_int, [c_void_p]),
        "devrt_symm_mc_ptr": (U, [c_void_p]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    return L


class DeviceMask:
    """Bitset over at most 64 GPUs (peer sets, rank groups)."""

    def __init__(self, devices=(), raw: int = 0):
        self.raw = raw
        for d in devices:
            self.set(d)

    def set(self, d: int):
        if 0 <= d < 64:
            self.raw |= 1 << d

    def clear(self, d: int):
        if 0 <= d < 64:
            self.raw &= ~(1 << d)

    def test(self, d: int) -> bool: return 0 <= d < 64 and bool((self.raw >> d) & 1)
    def clear_all(self): self.raw = 0
    def count(self) -> int: return bin(self.raw).count("1")
    def devices(self): return [d for d in range(64) if self.test(d)]


class GpuTopology:
    def __init__(self):
        self._h = lib().devrt_topology_create()

    def __del__(self):
        if getattr(self, "_h", None):
            lib().devrt_topology_destroy(self._h)
            self._h = None

    @property
    def status(self) -> int: return lib().devrt_topology_status(self._h)
    @property
    def num_devices(self) -> int: return lib().devrt_topology_num_devices(self._h)
    def peer_access(self, a: int, b: int) -> int: return lib().devrt_topology_peer_access(self._h, a, b)
    def distance(self, a: int, b: int) -> int: return lib().devrt_topology_distance(self._h, a, b)
    def peers_of(self, d: int) -> DeviceMask: return DeviceMask(raw=lib().devrt_topology_peers_of(self._h, d))
    def fully_connected(self) -> bool: return bool(lib().devrt_topology_fully_connected(self._h))

    def gpu(self, d: int) -> dict:
        name, pci = create_string_buffer(256), create_string_buffer(64)
        sm, cc, mc, numa = c_int(), c_int(), c_int(), c_int()
        tot, fr = c_ulonglong(), c_ulonglong()
        rc = lib().devrt_topology_gpu(self._h, d, name, 256, byref(sm), byref(cc), byref(tot), byref(fr), byref(mc),
                                      byref(numa), pci, 64)
        if rc != 0:
            raise IndexError(d)
        return {"name": name.value.decode(), "sm_count": sm.value, "cc": cc.value, "mem_total": tot.value,
                "mem_free": fr.value, "multicast": bool(mc.value), "numa_node": numa.value, "pci_bus_id": pci.value.decode()}

    def debug_string(self) -> str:
        buf = create_string_buffer(16384)
        lib().devrt_topology_debug(self._h, buf, 16384)
        return buf.value.decode()

    def print_debug(self): print(self.debug_string(), end="")


class _ArenaView:
    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
        self._owner = owner


class HbmArena:
    """Bump allocator over one virtual-memory reservation on a GPU; same contract as the host ``NumaArena``."""

    def __init__(self, device: int, size: int, alignment: int = 256):
        self.device = device
        self._h = lib().devrt_arena_create(device, size, alignment)

    def __del__(self):
        if getattr(self, "_h", None):
            lib().devrt_arena_destroy(self._h)
            self._h = None

    def __bool__(self): return bool(lib().devrt_arena_valid(self._h))
    @property
    def status(self) -> int: return lib().devrt_arena_status(self._h)
    def alloc(self, nbytes: int):
        p = lib().devrt_arena_alloc(self._h, nbytes)
        return p or None
    def mark(self) -> int: return lib().devrt_arena_mark(self._h)
    def reset_to(self, w: int): lib().devrt_arena_reset_to(self._h, w)
    def reset(self): lib().devrt_arena_reset(self._h)
    def remaining(self) -> int: return lib().devrt_arena_remaining(self._h)
    def used(self) -> int: return lib().devrt_arena_used(self._h)
    def size(self) -> int: return lib().devrt_arena_size(self._h)
    def high_water(self) -> int: return lib().devrt_arena_high_water(self._h)
    def base(self) -> int: return lib().devrt_arena_base(self._h)
    def verify_placement(self) -> bool: return bool(lib().devrt_arena_verify_placement(self._h))

    def tensor(self, shape, dtype):
        """Allocate from the arena and view the bytes as a torch tensor on this arena's GPU (no copy)."""
        import math
        import torch
        n = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        p = self.alloc(n)
        if p is None:
            return None
        raw = torch.as_tensor(_ArenaView(p, n, self), device=torch.device("cuda", self.device))
        return raw.view(dtype).view(*shape)


class SymmSegment:
    """This rank's block of a symmetric heap and the mappings of its peers' blocks (``csrc/devrt`` ``SymmSegment``).

    ``export_fd()`` is a POSIX descriptor of the local block; once a peer's descriptor has reached this process
    (``exchange_fds``), ``map_peer`` maps that peer's block at ``peer_ptr(peer)``.  The reference's workers share one
    mmap'd arena by address (test_linux_threading.mojo:426-435); processes that own one GPU each share HBM this way.
    """

    def __init__(self, device: int, nbytes: int, world: int, rank: int):
        self.device, self.world, self.rank = device, world, rank
        self._h = lib().devrt_symm_create(device, nbytes, world, rank)
        if not self._h:
            raise RuntimeError(f"symmetric segment of {nbytes} bytes on device {device}: the driver refused it "
                               "(no driver, no virtual-memory support, or no shareable handles)")

    def close(self):
        if getattr(self, "_h", None):
            lib().devrt_symm_destroy(self._h)
            self._h = None

    __del__ = close

    def export_fd(self) -> int: return lib().devrt_symm_export_fd(self._h)
    def map_peer(self, peer: int, fd: int) -> int: return lib().devrt_symm_map_peer(self._h, peer, fd)
    def mapped(self, r: int) -> bool: return bool(lib().devrt_symm_mapped(self._h, r))
    @property
    def base(self) -> int: return lib().devrt_symm_base(self._h)
    @property
    def stride(self) -> int: return lib().devrt_symm_stride(self._h)
    def peer_ptr(self, r: int) -> int: return lib().devrt_symm_peer_ptr(self._h, r)

    # Multicast object over all ranks' blocks.  Order across ranks: rank 0 ``mc_create()`` (returns a descriptor for the
    # others) / the others ``mc_import(fd)``; all ``mc_add_device()``; barrier; all ``mc_bind()``; barrier; ``mc_ptr``.
    def mc_create(self) -> int: return lib().devrt_symm_mc_create(self._h)
    def mc_import(self, fd: int) -> int: return lib().devrt_symm_mc_import(self._h, fd)
    def mc_add_device(self) -> int: return lib().devrt_symm_mc_add_device(self._h)
    def mc_bind(self) -> int: return lib().devrt_symm_mc_bind(self._h)
    @property
    def mc_ptr(self) -> int: return lib().devrt_symm_mc_ptr(self._h)

    def local_tensor(self):
        """The local block as a uint8 torch tensor (no copy; the segment must outlive it)."""
        import torch
        view = _ArenaView(self.peer_ptr(self.rank), self.stride, self)
        return torch.as_tensor(view, device=torch.device("cuda", self.device))


def exchange_fds(fd: int, rank: int, world: int, all_gather_names, timeout_s: float = 60.0) -> dict[int, int]:
    """Hand ``fd`` to every other rank process of this host and collect theirs: {peer rank: descriptor}.

    Descriptors cross processes as SCM_RIGHTS ancillary data on unix sockets in the abstract namespace (nothing is
    left in the file system).  ``all_gather_names(name) -> list[str]`` publishes this rank's socket name and returns
    everybody's (``torch.distributed.all_gather_object`` in practice; any out-of-band channel works).  The caller
    owns the returned descriptors and closes them after mapping.
    """
    import os
    import socket
    import threading
    name = f"\0b200rt-symm-{os.getpid()}-{rank}-{os.urandom(6).hex()}"
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.bind(name)
    srv.listen(world)
    srv.settimeout(timeout_s)
    errors: list[BaseException] = []

    def serve():
        try:
            for _ in range(world - 1):
                c, _addr = srv.accept()
                with c:
                    c.settimeout(timeout_s)
                    c.recv(8)                                    # the requester's rank (kept for the log of a failure)
                    socket.send_fds(c, [rank.to_bytes(4, "little")], [fd])
        except BaseException as e:                               # noqa: BLE001 - reported to the caller's thread
            errors.append(e)

    th = threading.Thread(target=serve, daemon=True)
    th.start()
    names = all_gather_names(name)
    got: dict[int, int] = {}
    try:
        for r in range(world):
            if r == rank:
                continue
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
                c.settimeout(timeout_s)
                c.connect(names[r])
                c.sendall(rank.to_bytes(8, "little"))
                msg, fds, _flags, _addr = socket.recv_fds(c, 4, 1)
                if len(fds) != 1 or int.from_bytes(msg, "little") != r:
                    raise RuntimeError(f"rank {r} answered the descriptor request with {len(fds)} descriptors")
                got[r] = fds[0]
        th.join(timeout_s)
        if th.is_alive() or errors:
            raise RuntimeError(f"descriptor exchange: serving side failed ({errors[:1] or 'timed out'})")
    except BaseException:
        for f in got.values():
            os.close(f)
        raise
    finally:
        srv.close()
    return got
