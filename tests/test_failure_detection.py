"""Failure detection without any GPU fault: gloo ranks on the CPU, the failure is a rank that exits between steps."""
import os
import subprocess
import sys

import pytest

from mojo_linuxperiments_b200.utils.health import Heartbeat, RankFailure

HERE = os.path.dirname(os.path.abspath(__file__))


class _DictStore:
    def __init__(self): self.d = {}
    def set(self, k, v): self.d[k] = v
    def get(self, k): return self.d[k].encode()
    def check(self, keys): return all(k in self.d for k in keys)


def test_heartbeat_declares_a_silent_rank_dead_and_keeps_live_ones():
    store = _DictStore()
    a = Heartbeat(store, 0, 3, interval_s=0.02, timeout_s=0.2).start()
    b = Heartbeat(store, 1, 3, interval_s=0.02, timeout_s=0.2).start()      # rank 2 never starts
    try:
        assert a.wait_for_failure(2.0) == [2]
        with pytest.raises(RankFailure) as ei:
            a.check()
        assert ei.value.ranks == [2]
        b.stop()                                                            # now rank 1 goes quiet as well
        import time
        t0 = time.monotonic()
        while 1 not in a.dead_ranks() and time.monotonic() - t0 < 3.0:
            time.sleep(0.02)
        assert a.dead_ranks() == [1, 2]
    finally:
        a.stop()
        b.stop()


def test_rank_that_leaves_between_steps_is_noticed_by_the_others():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=3", "--master-addr", "127.0.0.1",
           "--master-port", "29611", os.path.join(HERE, "mp_heartbeat.py"), "1"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=120)
    # two survivors report; their lines may interleave on the shared pipe, so count occurrences
    assert p.stdout.count("RESULT") == 2, p.stdout[-2000:] + p.stderr[-2000:]
    assert p.stdout.count("dead=[1] raised=True") == 2, p.stdout[-2000:]
