"""Parameter sharding of the dense baseline over the data-parallel ranks.

The reference shards every 2-D kernel of the baseline model along its first
axis over the data axis of the mesh and leaves the embeddings replicated
(scripts/train_jax.py:959-963); XLA inserts the gathers.  Here the same layout
is explicit:

* ``shard_dense_weights(model, group)`` replaces the weight of every
  ``nn.Linear`` inside ``model.layers`` by this rank's block of rows (the row
  count is padded to a multiple of the group size; the padding rows are zero
  and never used).  Biases, LayerNorm parameters and embeddings stay replicated.
* ``sharded_linear(be, x, lin)`` is the layer: the bf16 compute copies of the
  row blocks are all-gathered right before the GEMM (half the bytes of an fp32
  gather), nothing gathered is kept for backward; backward gathers again,
  computes ``dx`` and the full weight gradient, and reduce-scatters the latter so
  that every rank receives the summed gradient of its own rows only.  Master
  weights, gradients and Adam moments therefore exist once across the group.
* ``full_state_dict`` / ``load_full_state_dict`` convert between the sharded
  parameters and the ordinary (unsharded) checkpoint layout.

Gradient convention (as everywhere in this package): each rank's loss is one
term of the mean over ranks, so the reduce-scattered weight gradient is a sum
over ranks and ``GradSync`` only divides it by the world size; its squared norm
is summed over the group.  Parameters sharded here carry ``_fsdp_rows``.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.distributed as dist
import torch.nn as nn

from .collectives import _reduce_scatter, group_rank, group_size


def _rows_per_rank(rows: int, world: int) -> int:
    return (rows + world - 1) // world


def shard_dense_weights(model: nn.Module, group) -> int:
    """Shard the Linear weights of ``model.layers`` over ``group``; returns the
    number of weights sharded.  Every rank must hold identical full weights
    (same seed, or a checkpoint loaded before the call)."""
    world, rank = group_size(group), group_rank(group)
    if world <= 1:
        return 0
    n = 0
    for lin in model.layers.modules():
        if not isinstance(lin, nn.Linear) or hasattr(lin.weight, "_fsdp_rows"):
            continue
        full = lin.weight.data
        rows = full.shape[0]
        per = _rows_per_rank(rows, world)
        block = torch.zeros(per, full.shape[1], dtype=full.dtype, device=full.device)
        lo, hi = rank * per, min(rows, (rank + 1) * per)
        if hi > lo:
            block[: hi - lo] = full[lo:hi]
        p = nn.Parameter(block, requires_grad=lin.weight.requires_grad)
        p._fsdp_rows = rows
        p._fsdp_group = group
        lin.weight = p
        n += 1
    model._fsdp_group = group
    return n


def _gather_rows(block: torch.Tensor, rows: int, group) -> torch.Tensor:
    """[per, in] blocks of all ranks -> [rows, in]."""
    world = group_size(group)
    out = torch.empty(world * block.shape[0], block.shape[1], dtype=block.dtype, device=block.device)
    dist.all_gather_into_tensor(out, block.contiguous(), group=group)
    return out[:rows]


class _ShardedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_block, bias, rows, group, use_engine):
        cdt = torch.bfloat16 if use_engine else w_block.dtype
        w = _gather_rows(w_block.detach().to(cdt), rows, group)
        xc = x.detach().to(cdt)
        if use_engine:
            from ..ops import cuda_backend as CB
            y = CB.gemm(CB._bf16_2d(xc), False, w, False, out_dtype=torch.float32, bias=bias)
        else:
            y = (xc @ w.t()).float()
            if bias is not None:
                y = y + bias
        ctx.save_for_backward(xc, w_block)
        ctx.rows, ctx.group, ctx.use_engine, ctx.has_bias = rows, group, use_engine, bias is not None
        ctx.x_dtype = x.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, w_block = ctx.saved_tensors
        rows, group = ctx.rows, ctx.group
        world = group_size(group)
        per = w_block.shape[0]
        cdt = xc.dtype
        w = _gather_rows(w_block.detach().to(cdt), rows, group)
        dyc = dy.detach().to(cdt)
        full = torch.zeros(world * per, w_block.shape[1], dtype=torch.float32, device=dy.device)
        if ctx.use_engine:
            from ..ops import cuda_backend as CB
            dyb = CB._bf16_2d(dyc)
            dx = CB.gemm(dyb, False, w, True, out_dtype=torch.float32)
            CB.gemm(dyb, True, CB._bf16_2d(xc), True, out=full[:rows], accumulate=True)   # dy^T . x
        else:
            dx = (dyc @ w).float()
            full[:rows] = (dyc.t() @ xc).float()
        dw = torch.empty(per, w_block.shape[1], dtype=torch.float32, device=dy.device)
        _reduce_scatter(dw, full, group)
        db = dy.float().sum(0) if ctx.has_bias else None
        return dx.to(ctx.x_dtype), dw.to(w_block.dtype), db, None, None, None


def sharded_linear(be, x: torch.Tensor, lin: nn.Linear) -> torch.Tensor:
    """``lin(x)`` for a layer whose weight may have been sharded by
    ``shard_dense_weights`` (falls through to the backend's linear otherwise)."""
    w = lin.weight
    rows = getattr(w, "_fsdp_rows", None)
    if rows is None:
        return be.linear(x, w, lin.bias)
    use_engine = x.is_cuda and getattr(be, "name", "") == "sm100a"
    return _ShardedLinearFn.apply(x, w, lin.bias, rows, w._fsdp_group, use_engine)


@torch.no_grad()
def full_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    """State dict with the sharded weights gathered back to full size (a
    collective: every rank of the group calls it)."""
    sd = {}
    for name, t in model.state_dict().items():
        sd[name] = t
    for name, p in model.named_parameters():
        rows = getattr(p, "_fsdp_rows", None)
        if rows is not None:
            sd[name] = _gather_rows(p.data, rows, p._fsdp_group).clone()
    return sd


@torch.no_grad()
def load_full_state_dict(model: nn.Module, sd: Dict[str, torch.Tensor], strict: bool = True):
    """Load an unsharded state dict into a model whose weights are sharded."""
    own = dict(model.named_parameters())
    own.update(dict(model.named_buffers()))
    missing = [k for k in own if k not in sd]
    unexpected = [k for k in sd if k not in own]
    if strict and (missing or unexpected):
        raise KeyError(f"state dict mismatch: missing {missing}, unexpected {unexpected}")
    for name, dst in own.items():
        if name not in sd:
            continue
        src = sd[name]
        rows = getattr(dst, "_fsdp_rows", None)
        if rows is None:
            dst.data.copy_(src)
            continue
        group = dst._fsdp_group
        per, rank = dst.shape[0], group_rank(group)
        lo, hi = rank * per, min(rows, (rank + 1) * per)
        dst.data.zero_()
        if hi > lo:
            dst.data[: hi - lo].copy_(src[lo:hi])
    return missing, unexpected
