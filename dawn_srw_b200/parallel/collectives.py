"""Autograd-aware collectives over ``torch.distributed`` (NCCL on GPUs, gloo on
CPU ranks).  These are the *library* data plane: the control plane, the
baseline every fused kernel is compared with, and the path CPU-rank tests use.

Every rank's loss is treated as one term of the objective ``mean_r L_r`` and
each collective back-propagates with its true transpose (forward / backward):

* ``sum_over_shards``     all-reduce / all-reduce
* ``gather_tokens``       all-gather(dim 0) / reduce-scatter(dim 0)
* ``scatter_tokens_sum``  reduce-scatter(dim 0) / all-gather(dim 0)
* ``mean_over_group``     mean / mean

``copy_to_shards`` / ``reduce_from_shards`` (identity <-> all-reduce) are the
Megatron-style pair for groups that compute one loss redundantly; the model
code does not use them, they are kept for experiments.

The reference expresses the same algebra as ``lax.psum`` inside ``shard_map``
(reference: models/dawn_spatial_v41_exp.py:455-458, 579-586).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def group_size(group) -> int:
    if group is None or not dist.is_available() or not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None or not dist.is_available() or not dist.is_initialized():
        return 0
    return dist.get_rank(group)


# Optional kernel path for small fp32 sums: (callable, max elements) per group,
# installed by the owner of a symmetric-memory workspace for that group.
_SMALL_ALLREDUCE = {}


def register_small_allreduce(group, fn, max_elems: int) -> None:
    _SMALL_ALLREDUCE[id(group)] = (fn, int(max_elems))


def _all_reduce_sum_(y: torch.Tensor, group) -> None:
    """In-place sum over ``group``.  Shapes and dtypes agree on all ranks, so
    all ranks pick the same path."""
    hit = _SMALL_ALLREDUCE.get(id(group))
    if (hit is not None and y.is_cuda and y.dtype == torch.float32 and y.is_contiguous()
            and 0 < y.numel() <= hit[1]):
        hit[0](y)
    else:
        dist.all_reduce(y, group=group)


class _CopyToShards(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromShards(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        y = x.contiguous().clone()
        dist.all_reduce(y, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _SumOverShards(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        y = x.contiguous().clone()
        _all_reduce_sum_(y, group)
        return y

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        _all_reduce_sum_(g, ctx.group)
        return g, None


class _GatherTokens(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        x = x.contiguous()
        out = x.new_empty((n * x.shape[0],) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        n = dist.get_world_size(ctx.group)
        g = g.contiguous()
        out = g.new_empty((g.shape[0] // n,) + tuple(g.shape[1:]))
        _reduce_scatter(out, g, ctx.group)
        return out, None


class _ScatterTokensSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        x = x.contiguous()
        out = x.new_empty((x.shape[0] // n,) + tuple(x.shape[1:]))
        _reduce_scatter(out, x, group)
        return out

    @staticmethod
    def backward(ctx, g):
        n = dist.get_world_size(ctx.group)
        g = g.contiguous()
        out = g.new_empty((n * g.shape[0],) + tuple(g.shape[1:]))
        dist.all_gather_into_tensor(out, g, group=ctx.group)
        return out, None


def _reduce_scatter(out, inp, group):
    """reduce_scatter_tensor, with an all-reduce + slice fallback for gloo
    (which has no reduce-scatter)."""
    backend = dist.get_backend(group)
    if backend == "gloo":
        tmp = inp.clone()
        dist.all_reduce(tmp, group=group)
        r = dist.get_rank(group)
        out.copy_(tmp[r * out.shape[0]:(r + 1) * out.shape[0]])
    else:
        dist.reduce_scatter_tensor(out, inp, group=group)


def copy_to_shards(x, group):
    return x if group_size(group) == 1 else _CopyToShards.apply(x, group)


def reduce_from_shards(x, group):
    return x if group_size(group) == 1 else _ReduceFromShards.apply(x, group)


def sum_over_shards(x, group):
    return x if group_size(group) == 1 else _SumOverShards.apply(x, group)


def gather_tokens(x, group):
    return x if group_size(group) == 1 else _GatherTokens.apply(x, group)


def scatter_tokens_sum(x, group):
    return x if group_size(group) == 1 else _ScatterTokensSum.apply(x, group)


def all_reduce_nograd(x: torch.Tensor, group, op: str = "sum") -> torch.Tensor:
    """All-reduce of an observational (stop-gradient) quantity."""
    if group_size(group) == 1:
        return x
    y = x.detach().contiguous().clone()
    if op == "sum":
        _all_reduce_sum_(y, group)
        return y
    red = {"max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[op]
    dist.all_reduce(y, op=red, group=group)
    return y


def mean_over_group(x: torch.Tensor, group) -> torch.Tensor:
    """Differentiable mean over a data-parallel group.  The transpose of a
    mean-over-ranks is again a mean-over-ranks of the cotangents."""
    if group_size(group) == 1:
        return x
    return _PMean.apply(x, group)


class _PMean(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        n = dist.get_world_size(group)
        y = x.contiguous().clone()
        _all_reduce_sum_(y, group)
        return y / n

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        _all_reduce_sum_(g, ctx.group)
        return g / dist.get_world_size(ctx.group), None
