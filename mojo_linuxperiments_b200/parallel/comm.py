"""Rank group of one model replica: NCCL for bootstrap and as the unfused baseline, peer memory for the product.

A ``Comm`` with world 1 is a no-op object, so single-GPU code paths need no special casing.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class Comm:
    def __init__(self, group=None):
        self.group = group
        if group is None and not (dist.is_available() and dist.is_initialized()):
            self.world, self.rank = 1, 0
        else:
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)

    @staticmethod
    def single() -> "Comm":
        c = Comm.__new__(Comm)
        c.group, c.world, c.rank = None, 1, 0
        return c

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(x, group=self.group)
        return x

    def all_gather(self, x: torch.Tensor) -> torch.Tensor:
        """[...] -> [world, ...]"""
        if self.world == 1:
            return x.unsqueeze(0)
        out = torch.empty((self.world,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.group)
        return out

    def barrier(self):
        if self.world > 1:
            dist.barrier(group=self.group)
