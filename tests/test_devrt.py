"""Device runtime against a host-memory stand-in for the CUDA driver (CPU), and against the real driver (GPU)."""
import os
import subprocess
from pathlib import Path

import pytest

from mojo_linuxperiments_b200 import devrt as D

FAKE_SRC = Path(__file__).parent / "fake_cuda" / "fake_cuda.c"


@pytest.fixture()
def fake_driver(tmp_path, monkeypatch):
    so = tmp_path / "libfakecuda.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(so), str(FAKE_SRC)], check=True)
    monkeypatch.setenv("B200RT_LIBCUDA", str(so))
    D.lib().devrt_reload_driver()
    yield monkeypatch
    monkeypatch.delenv("B200RT_LIBCUDA", raising=False)
    D.lib().devrt_reload_driver()


def test_device_mask():
    m = D.DeviceMask([0, 3, 63, 64, -1])
    assert m.count() == 3 and m.test(3) and not m.test(64) and m.devices() == [0, 3, 63]
    m.clear(3)
    assert not m.test(3)
    m.clear_all()
    assert m.count() == 0


def test_no_driver_is_reported_not_raised(monkeypatch):
    monkeypatch.setenv("B200RT_LIBCUDA", "/nonexistent/libcuda.so")
    D.lib().devrt_reload_driver()
    t = D.GpuTopology()
    assert t.status == D.NO_DRIVER and t.num_devices == 0 and not t.fully_connected()
    a = D.HbmArena(0, 1 << 20)
    assert not a and a.status == D.NO_DRIVER and a.alloc(16) is None
    monkeypatch.delenv("B200RT_LIBCUDA")
    D.lib().devrt_reload_driver()


def test_topology_on_fake_driver(fake_driver, tmp_path):
    pci = tmp_path / "pci"
    for i, node in enumerate([0, 1, 1, 0]):
        d = pci / f"0000:{0x10 + i:02x}:00.0"
        d.mkdir(parents=True)
        (d / "numa_node").write_text(f"{node}\n")
    fake_driver.setenv("B200RT_PCI_SYSFS", str(pci))
    fake_driver.setenv("FAKE_CUDA_DEVICES", "4")
    t = D.GpuTopology()
    assert t.status == 0 and t.num_devices == 4 and t.fully_connected()
    g = t.gpu(2)
    assert g["sm_count"] == 148 and g["cc"] == 100 and g["multicast"] and g["numa_node"] == 1
    assert g["mem_total"] == 180 << 30 and g["mem_free"] == (170 - 2) << 30
    assert t.distance(1, 1) == 0 and t.distance(0, 3) == 1 and t.distance(0, 9) == -1
    assert t.peers_of(1).devices() == [0, 2, 3]
    assert "Fake B200 #3" in t.debug_string()
    fake_driver.setenv("FAKE_CUDA_NO_PEER", "1")
    t2 = D.GpuTopology()
    assert not t2.fully_connected() and t2.distance(0, 1) == -1 and t2.peers_of(0).count() == 0


def test_hbm_arena_contract_on_fake_driver(fake_driver):
    a = D.HbmArena(1, 3 << 20, alignment=256)
    assert a and a.size() == 4 << 20                     # rounded to the 2 MiB granularity
    assert a.used() == 0 and a.verify_placement()
    p1, p2 = a.alloc(100), a.alloc(100)
    assert p1 == a.base() and p2 == a.base() + 256
    m = a.mark()
    assert a.alloc(1 << 20) is not None
    assert a.alloc(4 << 20) is None                      # refused, state unchanged
    used = a.used()
    a.reset_to(used + 1)
    assert a.used() == used
    a.reset_to(m)
    assert a.used() == m and a.high_water() == used
    a.reset()
    assert a.used() == 0 and a.remaining() == a.size()
    fake_driver.setenv("FAKE_CUDA_FAIL_CREATE", "1")
    b = D.HbmArena(0, 1 << 20)
    assert not b and b.alloc(8) is None


@pytest.mark.gpu
def test_real_topology_and_arena_tensor():
    import torch
    D.lib().devrt_reload_driver()
    t = D.GpuTopology()
    assert t.status == 0 and t.num_devices == torch.cuda.device_count()
    g = t.gpu(0)
    assert g["sm_count"] == torch.cuda.get_device_properties(0).multi_processor_count and g["cc"] == 100
    a = D.HbmArena(0, 8 << 20)
    assert a and a.verify_placement()
    x = a.tensor((1024, 256), torch.float32)
    x.fill_(3.0)
    assert float(x.sum()) == 3.0 * 1024 * 256 and x.data_ptr() == a.base()
    y = a.tensor((16,), torch.int64)
    assert y.data_ptr() >= a.base() + 1024 * 256 * 4 and a.used() >= 1024 * 256 * 4 + 128
    del x, y
    if t.num_devices > 1:
        assert t.fully_connected() and t.distance(0, 1) == 1


def test_symmetric_segments_on_fake_driver(fake_driver):
    """Two ranks' segments: each exports a descriptor, maps the other's block at rank * stride, refuses repeats."""
    import threading
    fake_driver.setenv("FAKE_CUDA_DEVICES", "2")
    world = 2
    segs = [D.SymmSegment(r, (3 << 20) + 5, world, r) for r in range(world)]
    assert all(s.stride == 4 << 20 for s in segs)                       # rounded up to the 2 MiB granularity
    for r, s in enumerate(segs):
        assert s.mapped(r) and not s.mapped(1 - r) and s.peer_ptr(1) - s.peer_ptr(0) == s.stride and s.export_fd() >= 0
    names, got, bar = [None] * world, [None] * world, threading.Barrier(world)

    def gather_for(r):
        def gather(name):
            names[r] = name
            bar.wait(10)
            return list(names)
        return gather

    def run(r):
        got[r] = D.exchange_fds(segs[r].export_fd(), r, world, gather_for(r), timeout_s=10)

    ths = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    [t.start() for t in ths]
    [t.join(20) for t in ths]
    assert got[0] is not None and set(got[0]) == {1} and set(got[1]) == {0}
    for r, s in enumerate(segs):
        fd = got[r][1 - r]
        assert fd != segs[1 - r].export_fd()                              # a descriptor of its own, not the sender's
        assert s.map_peer(1 - r, fd) == 0 and s.mapped(1 - r)
        assert s.map_peer(1 - r, fd) != 0                                 # already mapped
        assert s.map_peer(r, fd) != 0 and s.map_peer(7, fd) != 0          # own slot, out of range
        os.close(fd)
    [s.close() for s in segs]


def test_symmetric_segment_refusals(fake_driver):
    fake_driver.setenv("FAKE_CUDA_FAIL_EXPORT", "1")
    with pytest.raises(RuntimeError):
        D.SymmSegment(0, 1 << 20, 2, 0)
    fake_driver.delenv("FAKE_CUDA_FAIL_EXPORT")
    for args in [(0, 0, 2, 0), (0, 1 << 20, 2, 2), (0, 1 << 20, 0, 0), (0, 1 << 20, 65, 0)]:
        with pytest.raises(RuntimeError):
            D.SymmSegment(*args)


def test_symmetric_segment_multicast_object_on_fake_driver(fake_driver):
    """Order of the multicast calls: create on rank 0, import elsewhere, every device added before any block is bound."""
    fake_driver.setenv("FAKE_CUDA_DEVICES", "2")
    segs = [D.SymmSegment(r, 1 << 20, 2, r) for r in range(2)]
    assert all(s.stride == 4 << 20 for s in segs)            # rounded to the multicast granularity of the fake (4 MiB)
    assert segs[1].mc_bind() != 0 and segs[1].mc_add_device() != 0      # nothing to bind / add to yet
    fd = segs[0].mc_create()
    assert fd >= 0 and segs[0].mc_create() < 0                           # one object per segment
    assert segs[1].mc_import(fd) == 0
    os.close(fd)
    assert segs[0].mc_add_device() == 0
    assert segs[0].mc_bind() != 0                                        # the other device has not been added
    assert segs[1].mc_add_device() == 0
    assert segs[0].mc_bind() == 0 and segs[1].mc_bind() == 0
    assert segs[0].mc_ptr != 0 and segs[0].mc_ptr != segs[0].base and segs[0].mc_bind() != 0
    [s.close() for s in segs]
    fake_driver.setenv("FAKE_CUDA_NO_MULTICAST", "1")
    s = D.SymmSegment(0, 1 << 20, 2, 0)
    assert s.mc_create() < 0 and s.mc_ptr == 0
    s.close()


def _fd_exchange_worker(rank, world, q_names, q_out):
    """One process of the descriptor exchange: owns an anonymous file, hands it to the peers, reads theirs."""
    import os as _os
    from mojo_linuxperiments_b200 import devrt as _D
    mine = _os.memfd_create(f"rank{rank}")
    _os.write(mine, f"from-{rank}".encode())

    def gather(name):
        q_names.put((rank, name))
        names = {}
        while len(names) < world:            # every process reads the full set (each entry is put back for the others)
            k, v = q_names.get()
            names[k] = v
            q_names.put((k, v))
        return [names[i] for i in range(world)]

    got = _D.exchange_fds(mine, rank, world, gather, timeout_s=20)
    seen = {}
    for peer, fd in got.items():
        seen[peer] = _os.pread(fd, 64, 0).decode()
        _os.close(fd)
    q_out.put((rank, seen))


def test_descriptors_cross_real_processes():
    """SCM_RIGHTS over abstract unix sockets between separate processes: each receives working descriptors of the
    others' anonymous files (what carries the exported HBM handles between rank processes)."""
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    world = 3
    q_names, q_out = ctx.Queue(), ctx.Queue()
    ps = [ctx.Process(target=_fd_exchange_worker, args=(r, world, q_names, q_out)) for r in range(world)]
    [p.start() for p in ps]
    results = [q_out.get(timeout=60) for _ in range(world)]
    [p.join(30) for p in ps]
    assert all(p.exitcode == 0 for p in ps)
    reads = {r: v for r, v in results if isinstance(v, dict)}
    for r in range(world):
        assert reads[r] == {p: f"from-{p}" for p in range(world) if p != r}
