"""Device-runtime behaviours on a real GPU: stream pool (launch / wait_all / wait_any) and the bounded-wait status path."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_stream_pool_launch_wait_any_order_and_reuse():
    from mojo_linuxperiments_b200.devrt.streams import StreamPool
    pool = StreamPool(3)
    assert pool.wait_any(0.1) == -1
    out = torch.zeros(3, device="cuda")
    a = torch.randn((8192, 8192), device="cuda", dtype=torch.bfloat16)

    def work(i, reps):
        x = a
        for _ in range(reps):                         # reps x ~0.8 ms of device work, queued asynchronously
            x = (x @ a) * 1e-2
        out[i] = i + 1

    work(0, 1)                                        # first use of a kernel may load its module, which can
    torch.cuda.synchronize()                          # synchronise the device: do that before anything is timed
    out.zero_()
    import time
    for i, reps in enumerate((80, 20, 1)):
        t0 = time.monotonic()
        got = pool.launch(work, i, reps)
        dt = time.monotonic() - t0
        assert got == i, (got, i, dt, [pool._busy(j) for j in range(3)])
    assert pool.launch(work, 0, 1) == -1              # every slot busy
    order = [pool.wait_any(10.0) for _ in range(3)]
    assert order == [2, 1, 0]
    assert pool.wait_any(0.1) == -1 and pool.wait_all(10.0) == 0
    assert out.tolist() == [1.0, 2.0, 3.0]
    assert pool.launch(work, 1, 1) == 0 and pool.wait_all() == 0      # slots are reusable


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
