"""Worker for tests/test_failure_detection.py: gloo ranks on the CPU, one of which leaves between steps."""
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from mojo_linuxperiments_b200.utils.health import Heartbeat, RankFailure  # noqa: E402


def main():
    victim = int(sys.argv[1])
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=0.5).start()
    x = torch.ones(4) * (rank + 1)
    for step in range(3):                       # healthy steps: a collective, then a health check
        hb.check()
        dist.all_reduce(x)
    if rank == victim:
        hb.stop()                               # leaves between steps, nothing in flight
        print(f"rank {rank} leaving", flush=True)
        os._exit(0)
    t0 = time.monotonic()
    dead = hb.wait_for_failure(5.0)
    dt = time.monotonic() - t0
    try:
        hb.check()
        raised = False
    except RankFailure as e:
        raised = e.ranks == [victim]
    print(f"RESULT rank={rank} dead={dead} raised={raised} after={dt:.2f}", flush=True)
    hb.stop()
    os._exit(0 if (dead == [victim] and raised and dt < 4.0) else 1)


if __name__ == "__main__":
    main()
