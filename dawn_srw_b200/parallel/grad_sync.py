"""Gradient synchronisation across ranks (library path: NCCL / gloo).

Which replicas hold a parameter decides its reduction (the reference leaves
this to XLA SPMD, scripts/train_jax.py:724-732):

The objective is the mean of the per-rank losses and every collective in the
forward pass back-propagates with its true transpose, so a rank's gradients are
partial sums:

* non-pool parameters are replicated on every rank -> sum over the world,
  divided by the world size;
* pool tensors are split over the shard group and replicated over the
  data-parallel group -> sum over the data-parallel group, divided by the
  world size (a rank's pool gradient already contains the contributions of
  every rank of its shard group: they arrive through the all-reduced /
  all-gathered output gradient).

Small tensors are packed into one flat bucket per reduction; pool tensors are
reduced in place.  The squared global norm counts each parameter once: pool
slices are summed over the shard group, replicated parameters are taken from
the local copy.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

from ..train.optimizer import wd_group_of


class GradSync:
    def __init__(self, topo):
        self.topo = topo

    def _is_pool(self, name: str) -> bool:
        return wd_group_of(name) == "pool"

    def reduce(self, named, grads: List[torch.Tensor]) -> List[torch.Tensor]:
        t = self.topo
        if t.world == 1:
            return grads
        small = [g for (n, _), g in zip(named, grads) if not self._is_pool(n)]
        if small:
            flat = torch.cat([g.reshape(-1).float() for g in small])
            dist.all_reduce(flat, group=t.world_group)
            flat /= t.world
            off = 0
            for g in small:
                g.copy_(flat[off: off + g.numel()].view_as(g))
                off += g.numel()
        pool_div = float(t.world)
        for (n, _), g in zip(named, grads):
            if self._is_pool(n):
                if t.pool_shards == 1:
                    dist.all_reduce(g, group=t.world_group)
                elif t.dp > 1:
                    dist.all_reduce(g, group=t.dp_group)
                g /= pool_div
        return grads

    def global_sq_norm(self, named, grads: List[torch.Tensor]) -> torch.Tensor:
        t = self.topo
        rep = [g.float().square().sum() for (n, _), g in zip(named, grads) if not self._is_pool(n)]
        pool = [g.float().square().sum() for (n, _), g in zip(named, grads) if self._is_pool(n)]
        dev = grads[0].device
        rep_s = torch.stack(rep).sum() if rep else torch.zeros((), device=dev)
        pool_s = torch.stack(pool).sum() if pool else torch.zeros((), device=dev)
        if t.pool_shards > 1:
            pool_s = pool_s.clone()
            dist.all_reduce(pool_s, group=t.shard_group)
        return rep_s + pool_s
