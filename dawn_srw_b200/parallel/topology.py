"""Process topology: data-parallel replicas x pool-shard groups.

The reference lays devices out as a 2-D mesh ``('data', 'model')``: the batch is
split over ``data`` and the unit axis of every pool over ``model``
(reference: scripts/train_jax.py:929-975).  Here one process drives one GPU and
the same two axes are ``torch.distributed`` process groups:

* ``shard_group`` (size ``pool_shards``): ranks that together hold one copy of
  every pool, ``U / pool_shards`` units each.  With ``seq_shard`` the
  activations between pool ops are also split over this group by whole
  sequences, so attention stays local to a rank.
* ``dp_group`` (size ``dp``): ranks holding the same pool slice on different
  batch shards; pool gradients are reduced over it.

Ranks are laid out shard-major: ``rank = dp_index * pool_shards + shard_index``,
so a shard group is a contiguous block of GPUs on one NVSwitch domain.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class PoolShard:
    """Which slice of every pool's unit axis this rank stores."""
    index: int = 0
    count: int = 1
    align: int = 8          # local row count is padded to a multiple of this

    def per_rank(self, n_units: int) -> int:
        per = -(-n_units // self.count)
        return -(-per // self.align) * self.align if self.count > 1 else n_units

    def slice_of(self, n_units: int) -> Tuple[int, int, int]:
        """(lo, hi, padded_rows): this rank holds global units [lo, hi) in a
        buffer of ``padded_rows`` rows; rows beyond ``hi - lo`` are padding that
        must contribute nothing to any statistic."""
        per = self.per_rank(n_units)
        lo = min(self.index * per, n_units)
        hi = min(lo + per, n_units)
        return lo, hi, per


@dataclass
class Topology:
    rank: int = 0
    world: int = 1
    local_rank: int = 0
    pool_shards: int = 1
    dp: int = 1
    seq_shard: bool = False
    shard_group: Optional[object] = None
    dp_group: Optional[object] = None
    world_group: Optional[object] = None
    cpu_group: Optional[object] = None      # gloo group for host-side consensus

    @property
    def shard_index(self) -> int:
        return self.rank % self.pool_shards

    @property
    def dp_index(self) -> int:
        return self.rank // self.pool_shards

    @property
    def pool_shard(self) -> PoolShard:
        return PoolShard(self.shard_index, self.pool_shards)

    @property
    def is_main(self) -> bool:
        return self.rank == 0

    @property
    def batch_replicas(self) -> int:
        """How many distinct batch shards exist: every rank gets its own
        sequences when activations are sequence-sharded, otherwise one shard
        per data-parallel replica."""
        return self.world if (self.seq_shard or self.pool_shards == 1) else self.dp

    @property
    def batch_index(self) -> int:
        return self.rank if (self.seq_shard or self.pool_shards == 1) else self.dp_index


def env_rank_world() -> Tuple[int, int, int]:
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def init_topology(pool_shards: int = 1, dp: int = 0, seq_shard: bool = False,
                  backend: Optional[str] = None, timeout_s: float = 600.0) -> Topology:
    """Join the job (env:// rendezvous) and build the groups.  With world 1 no
    process group is created."""
    import datetime
    rank, world, local_rank = env_rank_world()
    if world == 1:
        return Topology()
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(local_rank)
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local_rank)
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    pool_shards = max(1, int(pool_shards))
    if world % pool_shards != 0:
        raise ValueError(f"world size {world} is not a multiple of pool_shards {pool_shards}")
    dp_expected = world // pool_shards
    if dp and dp != dp_expected:
        raise ValueError(f"dp={dp} x pool_shards={pool_shards} != world size {world}")
    dp = dp_expected
    shard_group = dp_group = None
    for d in range(dp):
        ranks = list(range(d * pool_shards, (d + 1) * pool_shards))
        g = dist.new_group(ranks) if pool_shards > 1 else None
        if rank in ranks:
            shard_group = g
    for s in range(pool_shards):
        ranks = list(range(s, world, pool_shards))
        g = dist.new_group(ranks) if dp > 1 else None
        if rank in ranks:
            dp_group = g
    cpu_group = dist.new_group(list(range(world)), backend="gloo") if backend != "gloo" else dist.group.WORLD
    return Topology(rank=rank, world=world, local_rank=local_rank, pool_shards=pool_shards, dp=dp,
                    seq_shard=bool(seq_shard and pool_shards > 1), shard_group=shard_group,
                    dp_group=dp_group, world_group=dist.group.WORLD, cpu_group=cpu_group)
