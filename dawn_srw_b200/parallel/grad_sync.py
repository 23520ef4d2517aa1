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

* pool tensors that stay whole on every rank while other pools are sharded
  (``training.shard_pools``) behave like replicated parameters: sum over the world;
* weights sharded by rows over the data-parallel ranks (parallel/fsdp.py, dense
  baseline) arrive already summed by their reduce-scatter -> only divided by
  the world size; their squared norm is summed over that group.

Small tensors are packed into one flat bucket per reduction; pool tensors are
reduced in place.  The squared global norm counts each parameter once: pool
slices are summed over the shard group, replicated parameters are taken from
the local copy.

Overlap with backward (``attach``): the gradients of replicated parameters are
final at different times during backward (per-layer tensors early, the shared
router and the embeddings at the very end).  A post-accumulate hook appends
each finished gradient to the current bucket and launches an asynchronous
all-reduce as soon as the bucket holds ``bucket_bytes``; ``reduce`` then only
flushes the last bucket, waits and copies back.  The hook order is a property
of the graph, so all ranks build identical buckets.  Pool gradients complete
only when the whole backward is done (every layer adds into them) and are
reduced afterwards as before.
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

from ..train.optimizer import wd_group_of


class GradSync:
    def __init__(self, topo):
        self.topo = topo
        self._overlap = False
        self._bucket_bytes = 0
        self._open: List[torch.nn.Parameter] = []     # finished gradients not yet launched
        self._open_bytes = 0
        self._inflight = []                            # (flat, work, params)
        self._hooks = []

    # ---- overlap with backward ---------------------------------------------
    def attach(self, named_params, bucket_bytes: int = 32 << 20) -> None:
        """Start reducing replicated-parameter gradients while backward still runs.
        Only valid when every backward is followed by ``reduce`` on the ``.grad``
        tensors themselves (no gradient accumulation over micro-steps)."""
        if self.topo.world == 1 or self._overlap:
            return
        self._overlap, self._bucket_bytes = True, int(bucket_bytes)
        for n, p in named_params:
            if p.requires_grad and not self._is_pool(n) and not self._is_rowsharded(p):
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad_ready))

    def detach(self) -> None:
        for h in self._hooks:
            h.remove()
        self._hooks, self._overlap = [], False
        self.discard()

    def discard(self) -> None:
        """Forget the gradients of a backward whose result is not used (every
        rank must call it at the same point)."""
        for _flat, work, _ps in self._inflight:
            work.wait()
        self._inflight, self._open, self._open_bytes = [], [], 0

    def _on_grad_ready(self, p: torch.nn.Parameter) -> None:
        self._open.append(p)
        self._open_bytes += p.grad.numel() * 4
        if self._open_bytes >= self._bucket_bytes:
            self._launch()

    def _launch(self) -> None:
        if not self._open:
            return
        ps = self._open
        flat = torch.cat([p.grad.reshape(-1).float() for p in ps])
        work = dist.all_reduce(flat, group=self.topo.world_group, async_op=True)
        self._inflight.append((flat, work, ps))
        self._open, self._open_bytes = [], 0

    def _finish_overlapped(self, named, grads) -> set:
        """Wait for the buckets launched during backward; returns the ids of the
        gradient tensors they covered."""
        self._launch()
        by_param = {id(p): g for (_, p), g in zip(named, grads)}
        done = set()
        for flat, work, ps in self._inflight:
            work.wait()
            flat /= self.topo.world
            off = 0
            for p in ps:
                g = by_param.get(id(p))
                n = p.numel()
                if g is not None:
                    g.copy_(flat[off: off + n].view_as(g))
                    done.add(id(g))
                off += n
        self._inflight = []
        return done

    def _is_pool(self, name: str) -> bool:
        return wd_group_of(name) == "pool"

    @staticmethod
    def _is_replicated_pool(p) -> bool:
        """A pool tensor kept whole on every rank although other pools are sharded."""
        return getattr(p, "_pool_replicated", False)

    @staticmethod
    def _is_rowsharded(p) -> bool:
        return getattr(p, "_fsdp_rows", None) is not None

    def reduce(self, named, grads: List[torch.Tensor]) -> List[torch.Tensor]:
        t = self.topo
        if t.world == 1:
            return grads
        done = self._finish_overlapped(named, grads) if self._overlap else set()
        small = [g for (n, p), g in zip(named, grads)
                 if not self._is_pool(n) and not self._is_rowsharded(p) and id(g) not in done]
        if small:
            flat = torch.cat([g.reshape(-1).float() for g in small])
            dist.all_reduce(flat, group=t.world_group)
            flat /= t.world
            off = 0
            for g in small:
                g.copy_(flat[off: off + g.numel()].view_as(g))
                off += g.numel()
        pool_div = float(t.world)
        for (n, p), g in zip(named, grads):
            if self._is_rowsharded(p):
                g /= pool_div
            elif self._is_pool(n):
                if t.pool_shards == 1 or self._is_replicated_pool(p):
                    dist.all_reduce(g, group=t.world_group)
                elif t.dp > 1:
                    dist.all_reduce(g, group=t.dp_group)
                g /= pool_div
        return grads

    def global_sq_norm(self, named, grads: List[torch.Tensor]) -> torch.Tensor:
        t = self.topo
        sq = lambda g: g.float().square().sum()
        rep = [sq(g) for (n, p), g in zip(named, grads) if not self._is_pool(n) and not self._is_rowsharded(p)]
        # replicated pools count once (the local copy), like any replicated parameter
        rep += [sq(g) for (n, p), g in zip(named, grads) if self._is_pool(n) and self._is_replicated_pool(p)]
        pool = [sq(g) for (n, p), g in zip(named, grads)
                if self._is_pool(n) and not self._is_replicated_pool(p)]
        rows = [(sq(g), p._fsdp_group) for (_, p), g in zip(named, grads) if self._is_rowsharded(p)]
        dev = grads[0].device
        rep_s = torch.stack(rep).sum() if rep else torch.zeros((), device=dev)
        pool_s = torch.stack(pool).sum() if pool else torch.zeros((), device=dev)
        if t.pool_shards > 1:
            pool_s = pool_s.clone()
            dist.all_reduce(pool_s, group=t.shard_group)
        total = rep_s + pool_s
        if rows:
            rows_s = torch.stack([v for v, _ in rows]).sum()
            dist.all_reduce(rows_s, group=rows[0][1])
            total = total + rows_s
        return total
