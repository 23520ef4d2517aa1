"""Partitioned optimizer: gradient reduce-scatter, AdamW on the owned slice and
parameter all-gather as one step, with the moments sharded over the replicas.

Parameters that are replicated over a group of ranks (everything over the
world under pure data parallelism; pool slices over the data-parallel group
when the pools are also sharded) are packed, per weight-decay group, into one
flat fp32 buffer; the gradients live in a second flat buffer of the same
layout (``p.grad`` is a view, so backward accumulates straight into it).  Rank
``k`` of the group owns slice ``k`` of both and keeps Adam moments for that
slice only, so optimizer state shrinks by the group size (the reference
replicates parameters and optimizer state and leaves the reduction to XLA
SPMD, scripts/train_jax.py:724-732, 2028-2120).

One optimizer step is

    barrier | own slice <- scale * sum over replicas of their gradients, |g|^2
            | global norm (one scalar all-reduce) -> clip factor
            | AdamW on the slice, new parameters stored to every replica | barrier

On CUDA with peer-mapped (symmetric) memory the two data movements are kernels
that load the replicas' gradients and store the new parameters over NVLink
(ops/csrc/comm_kernels.cu: ``zero_reduce_kernel``, ``zero_adam_scatter_kernel``);
no library collective touches the bulk data.  Without it (CPU ranks, or
``peer_kernels=False``) the same arithmetic runs on ``torch.distributed``
collectives, which is also what the tests compare against.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..train.optimizer import wd_group_of


class _Bucket:
    """One flat (parameters, gradients) pair replicated over ``group``."""

    def __init__(self, key, wd: float, group, gsize: int, grank: int):
        self.key, self.wd, self.group, self.gsize, self.grank = key, wd, group, gsize, grank
        self.names: List[str] = []
        self.params: List[torch.nn.Parameter] = []
        self.offsets: List[int] = []
        self.total = 0

    def add(self, name, p):
        self.names.append(name)
        self.params.append(p)
        self.offsets.append(self.total)
        self.total += p.numel()


class PartitionedAdamW:
    """Drop-in for ``train.optimizer.DawnAdamW`` (same update rule, schedule,
    clip, weight-decay groups and accumulation) with sharded optimizer state."""

    def __init__(self, named_params: Iterable[Tuple[str, torch.nn.Parameter]], topo, *, lr: float,
                 weight_decay: float = 0.1, pool_weight_decay: float = 0.02, betas=(0.9, 0.95),
                 eps: float = 1e-8, clip_norm: float = 1.0,
                 schedule: Optional[Callable[[int], float]] = None, accumulation_steps: int = 1,
                 peer_kernels: Optional[bool] = None):
        self.topo = topo
        self.named = [(n, p) for n, p in named_params if p.requires_grad]
        self.lr, self.betas, self.eps, self.clip_norm = lr, betas, eps, clip_norm
        self.wd = {"base": weight_decay, "pool": pool_weight_decay, "none": 0.0}
        self.schedule = schedule or (lambda step: lr)
        self.accumulation_steps = max(1, int(accumulation_steps))
        self.count, self.micro = 0, 0
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.last_lr = float(self.schedule(0))
        dev = self.named[0][1].device
        self.device = dev
        if peer_kernels is None:
            peer_kernels = dev.type == "cuda" and topo.world > 1
        self.peer = bool(peer_kernels)
        self._ws: Dict[str, object] = {}
        self._full_state = None

        buckets: Dict[Tuple[str, str], _Bucket] = {}
        for n, p in self.named:
            wdg = wd_group_of(n)
            if wdg == "pool" and topo.pool_shards > 1 and not getattr(p, "_pool_replicated", False):
                kind, group, gsize, grank = "dp", topo.dp_group, topo.dp, topo.dp_index
            else:
                kind, group, gsize, grank = "world", topo.world_group, topo.world, topo.rank
            b = buckets.get((kind, wdg))
            if b is None:
                b = buckets[(kind, wdg)] = _Bucket((kind, wdg), self.wd[wdg], group, gsize, grank)
            b.add(n, p)
        self.buckets = [buckets[k] for k in sorted(buckets)]
        for b in self.buckets:
            self._materialise(b)

    # ------------------------------------------------------------------
    def _workspace(self, b: _Bucket):
        from .symm import SymmWorkspace
        ws = self._ws.get(b.key[0])
        if ws is None:
            ws = self._ws[b.key[0]] = SymmWorkspace(b.group, self.device)
        return ws

    def _materialise(self, b: _Bucket):
        quantum = 4 * b.gsize
        b.slice = ((b.total + quantum - 1) // quantum) * 4
        b.padded = b.slice * b.gsize
        b.lo = b.slice * b.grank
        dev = self.device
        b.use_peer = self.peer and b.gsize > 1
        if b.use_peer:
            ws = self._workspace(b)
            name = "zero_%s_%s" % b.key
            pbuf = ws.alloc(name + "_p", (b.padded,), torch.float32)
            gbuf = ws.alloc(name + "_g", (b.padded,), torch.float32)
            b.pflat, b.gflat = pbuf.local, gbuf.local
            b.p_ptrs = torch.tensor(pbuf.ptrs, dtype=torch.int64, device=dev)
            b.g_ptrs = torch.tensor(gbuf.ptrs, dtype=torch.int64, device=dev)
            b.ws = ws
        else:
            b.pflat = torch.empty(b.padded, dtype=torch.float32, device=dev)
            b.gflat = torch.empty(b.padded, dtype=torch.float32, device=dev)
        b.pflat.zero_()
        b.gflat.zero_()
        for p, off in zip(b.params, b.offsets):
            n = p.numel()
            if p.dtype != torch.float32:
                raise TypeError("partitioned optimizer expects fp32 master parameters")
            b.pflat[off: off + n].copy_(p.data.reshape(-1))
            p.data = b.pflat[off: off + n].view(p.shape)
            p.grad = b.gflat[off: off + n].view(p.shape)
        b.m = torch.zeros(b.slice, dtype=torch.float32, device=dev)
        b.v = torch.zeros(b.slice, dtype=torch.float32, device=dev)
        b.g_own = torch.zeros(b.slice, dtype=torch.float32, device=dev)
        if b.use_peer:
            torch.cuda.synchronize(dev)
            dist.barrier(group=b.group)

    # ------------------------------------------------------------------
    def describe_groups(self) -> str:
        parts = [f"{b.key[0]}/{b.key[1]}: {len(b.params)} tensors, {b.total:,} elements, "
                 f"slice {b.slice:,} of {b.gsize}" for b in self.buckets]
        return "partitioned AdamW (" + ("peer kernels" if self.peer else "library collectives") + \
            "): " + "; ".join(parts)

    def state_bytes(self) -> int:
        """Bytes of Adam moments this rank holds."""
        return sum(2 * b.slice * 4 for b in self.buckets)

    def zero_grad(self):
        """Clears the flat gradient buffers once an accumulation window is
        complete (inside a window the gradients keep accumulating)."""
        if self.micro != 0:
            return
        for b in self.buckets:
            b.gflat.zero_()
            for p, off in zip(b.params, b.offsets):     # re-attach views a caller may have dropped
                if p.grad is None or p.grad.data_ptr() != b.gflat.data_ptr() + 4 * off:
                    p.grad = b.gflat[off: off + p.numel()].view(p.shape)

    def _reattach_foreign_grads(self):
        """A ``.grad`` that was replaced (set to None and re-created by
        autograd) is copied back into the flat buffer."""
        for b in self.buckets:
            for p, off in zip(b.params, b.offsets):
                g = p.grad
                view = b.gflat[off: off + p.numel()].view(p.shape)
                if g is None:
                    p.grad = view
                elif g.data_ptr() != view.data_ptr():
                    view.add_(g)
                    p.grad = view

    # ------------------------------------------------------------------
    @torch.no_grad()
    def step(self) -> bool:
        self._reattach_foreign_grads()
        k = self.accumulation_steps
        self.micro += 1
        if self.micro < k:
            return False
        self.micro = 0
        t = self.topo
        scale = 1.0 / (t.world * k)
        dev = self.device
        sq = torch.zeros(1, dtype=torch.float32, device=dev)
        if self.peer:
            from ..ops import cuda_backend as CB
            e = CB.ext()
        for b in self.buckets:
            if b.gsize == 1:
                b.g_own[: b.total].copy_(b.gflat[: b.total]).mul_(scale)
                sq += b.g_own.square().sum()
            elif b.use_peer:
                b.ws.barrier()           # every replica's backward has finished writing gradients
                e.zero_reduce(b.g_ptrs, b.gsize, b.lo, b.slice, scale, b.g_own, sq)
                CB.count_launches(2)
            else:
                dist.all_reduce(b.gflat, group=b.group)
                b.g_own.copy_(b.gflat[b.lo: b.lo + b.slice]).mul_(scale)
                sq += b.g_own.square().sum()
        if t.world > 1:
            dist.all_reduce(sq, group=t.world_group)
        norm = sq.sqrt().reshape(())
        self.last_grad_norm = norm
        clip_scale = (self.clip_norm / torch.clamp(norm, min=self.clip_norm)).reshape(1)
        self.count += 1
        step_no = self.count
        lr = float(self.schedule(step_no - 1))
        self.last_lr = lr
        b1, b2 = self.betas
        bc1, bc2 = 1.0 - b1 ** step_no, 1.0 - b2 ** step_no
        for b in self.buckets:
            if b.use_peer:
                e.zero_adam_scatter(b.p_ptrs, b.gsize, b.grank, b.lo, b.slice, b.g_own, b.m, b.v,
                                    clip_scale, lr, b1, b2, self.eps, b.wd, bc1, bc2)
                b.ws.barrier()           # all replicas' stores have landed; gradients may be cleared
                CB.count_launches(2)
            else:
                own = b.pflat[b.lo: b.lo + b.slice]
                g = b.g_own * clip_scale
                b.m.mul_(b1).add_(g, alpha=1.0 - b1)
                b.v.mul_(b2).addcmul_(g, g, value=1.0 - b2)
                upd = (b.m / bc1) / ((b.v / bc2).sqrt() + self.eps)
                if b.wd != 0.0:
                    upd = upd + b.wd * own
                own.add_(upd, alpha=-lr)
                if b.gsize > 1:
                    parts = [torch.empty_like(own) for _ in range(b.gsize)]
                    dist.all_gather(parts, own.contiguous(), group=b.group)
                    b.pflat.copy_(torch.cat(parts))
            torch._C._increment_version(list(b.params))
        self._full_state = None
        return True

    # ------------------------------------------------------------------
    def gather_state(self) -> None:
        """Collective over every bucket's group: assemble the full per-parameter
        moments so that ``state_dict()`` (called on the writing ranks only) has
        a layout-independent form."""
        full = {"exp_avg": {}, "exp_avg_sq": {}}
        for b in self.buckets:
            for key, own in (("exp_avg", b.m), ("exp_avg_sq", b.v)):
                if b.gsize > 1:
                    parts = [torch.empty_like(own) for _ in range(b.gsize)]
                    dist.all_gather(parts, own, group=b.group)
                    flat = torch.cat(parts)
                else:
                    flat = own
                for n, p, off in zip(b.names, b.params, b.offsets):
                    full[key][n] = flat[off: off + p.numel()].view(p.shape).cpu()
        self._full_state = full

    def state_dict(self) -> Dict:
        if self._full_state is None:
            if any(b.gsize > 1 for b in self.buckets):
                raise RuntimeError("call gather_state() on every rank before state_dict()")
            self.gather_state()
        acc = None
        if self.micro:
            acc = {n: p.grad.detach().clone() for n, p in self.named}
        return {"count": self.count, "micro": self.micro, "exp_avg": self._full_state["exp_avg"],
                "exp_avg_sq": self._full_state["exp_avg_sq"], "acc": acc}

    def load_state_dict(self, sd: Dict):
        self.count, self.micro = int(sd["count"]), int(sd.get("micro", 0))
        for b in self.buckets:
            for key, own in (("exp_avg", b.m), ("exp_avg_sq", b.v)):
                flat = torch.zeros(b.padded, dtype=torch.float32, device=self.device)
                for n, p, off in zip(b.names, b.params, b.offsets):
                    flat[off: off + p.numel()].copy_(sd[key][n].reshape(-1).to(self.device))
                own.copy_(flat[b.lo: b.lo + b.slice])
        acc = sd.get("acc")
        if acc is not None:
            for n, p in self.named:
                p.grad.copy_(acc[n].to(self.device))
        self.last_lr = float(self.schedule(max(self.count - 1, 0)))
        self._full_state = None
