"""Config-1 workload on GPUs: Philox fill of a float32 buffer split by global element index, local sum, and (with
more than one rank) a peer-memory all-reduce of the per-GPU sums - the GPU side of the reference's
per-node fill + tree reduce (test_linux_threading.mojo:217-302, 400-553)."""
from __future__ import annotations

import torch

from . import _lib


class FillReduce:
    def __init__(self, n_elems: int, world: int = 1, rank: int = 0, device=None, max_ctas: int = 148 * 8):
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.n, self.world, self.rank = n_elems, world, rank
        self.begin = (n_elems * rank // world) & ~3
        self.end = n_elems if rank == world - 1 else ((n_elems * (rank + 1) // world) & ~3)
        self.buf = torch.empty(self.end - self.begin, dtype=torch.float32, device=self.device)
        self.partials = torch.zeros(max_ctas, dtype=torch.float64, device=self.device)
        self.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.result = torch.zeros(1, dtype=torch.float64, device=self.device)
        self.max_ctas = max_ctas

    def run(self, seed: int = 0) -> torch.Tensor:
        """Fill this rank's slice and leave its sum in ``self.result`` (device double)."""
        rc = _lib.lib().b200_fill_uniform_reduce(self.buf.data_ptr(), self.begin, self.end, seed, self.partials.data_ptr(),
                                                 self.max_ctas, self.counter.data_ptr(), self.result.data_ptr(), _lib.stream())
        _lib.check(rc, "fill_uniform_reduce")
        return self.result


def where_am_i(ctas: int = 296, rank_tag: int = 0, device=None):
    """Locality tags written by ``ctas`` CTAs: int32 [ctas, 4] = (SM id, number of SM ids, rank tag, CTA index) - the
    in-kernel counterpart of the host runtime's ``get_current_cpu_and_node`` (reference: numa/numa.mojo:6-24)."""
    import torch
    from . import _lib
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    out = torch.full((ctas, 4), -1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().b200_where_am_i(out.data_ptr(), ctas, rank_tag, _lib.stream()), "where_am_i")
    return out
