"""Device-runtime behaviours on a real GPU: stream pool (launch / wait_all / wait_any) and the bounded-wait status path."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bounded_wait_launcher():
    """Returns work(slot, limit_ms): one kernel of this library that waits for a flag nobody sets and gives up after
    ``limit_ms`` (status 5) - device work of a known duration that needs no allocation and a single launch."""
    from mojo_linuxperiments_b200.ops import _lib
    lib = _lib.lib()
    keep = []

    def make():
        heap = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
        flags = torch.zeros(1024, dtype=torch.int32, device="cuda")
        words = torch.zeros(8, dtype=torch.int32, device="cuda")
        status = torch.zeros(4, dtype=torch.int32, device="cuda")
        out = torch.zeros(64, dtype=torch.float32, device="cuda")
        data = (ctypes.c_void_p * 2)(heap.data_ptr(), heap.data_ptr())
        fl = (ctypes.c_void_p * 2)(flags.data_ptr(), flags.data_ptr())
        keep.append((heap, flags, words, status, out, data, fl))
        return keep[-1]

    slots = [make() for _ in range(3)]

    def work(i, limit_ms):
        heap, flags, words, status, out, data, fl = slots[i]
        rc = lib.b200_peer_allreduce(data, fl, None, 2, 0, 0, 4096, out.data_ptr(), None, 64, 1, 0, words.data_ptr(),
                                     status.data_ptr(), limit_ms, 0, 1, torch.cuda.current_stream().cuda_stream)
        assert rc == 0
    return work, slots


def test_stream_pool_launch_wait_any_order_and_reuse():
    from mojo_linuxperiments_b200.devrt.streams import StreamPool
    pool = StreamPool(3)
    assert pool.wait_any(0.1) == -1
    work, slots = _bounded_wait_launcher()
    work(0, 1)                                        # first use loads the kernel's module, which can synchronise
    torch.cuda.synchronize()
    for i, limit_ms in enumerate((600, 300, 20)):     # slot 0 is busy longest
        assert pool.launch(work, i, limit_ms) == i, [pool._busy(j) for j in range(3)]
    assert pool.launch(work, 0, 1) == -1              # every slot busy
    order = [pool.wait_any(10.0) for _ in range(3)]
    assert order == [2, 1, 0]
    assert pool.wait_any(0.1) == -1 and pool.wait_all(10.0) == 0
    assert all(int(s[3][0].item()) == 5 for s in slots)              # each wait ran out and said so
    assert pool.launch(work, 1, 1) == 0 and pool.wait_all() == 0     # slots are reusable


def test_peer_wait_that_nothing_satisfies_times_out_cleanly():
    """A flag that no rank ever sets: the kernel gives up after its limit, records status 5 and the context stays usable."""
    from mojo_linuxperiments_b200.ops import _lib
    lib = _lib.lib()
    heap = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    flags = torch.zeros(1024, dtype=torch.int32, device="cuda")
    words = torch.zeros(8, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    out = torch.zeros(64, dtype=torch.float32, device="cuda")
    # "world" of two whose second member is only a pointer to the same memory: its flag is never written
    data = (ctypes.c_void_p * 2)(heap.data_ptr(), heap.data_ptr())
    fl = (ctypes.c_void_p * 2)(flags.data_ptr(), flags.data_ptr())
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    rc = lib.b200_peer_allreduce(data, fl, None, 2, 0, 0, 4096, out.data_ptr(), None, 64, 1, 0, words.data_ptr(),
                                 status.data_ptr(), 50, 1, 4, torch.cuda.current_stream().cuda_stream)
    t1.record()
    torch.cuda.synchronize()
    assert rc == 0
    assert int(status[0].item()) == 5                  # ST_TIMEOUT_PEER_FLAG
    assert 40.0 <= t0.elapsed_time(t1) < 2000.0         # one or two 50 ms limits, not forever
    y = torch.ones(4, device="cuda") * 2                # the context is alive
    assert float(y.sum()) == 8.0
