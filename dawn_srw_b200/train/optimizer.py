"""Optimizer: global-norm clip -> Adam moments -> two decoupled weight-decay
groups -> learning-rate schedule, with optional gradient accumulation.

Update rule (reference: scripts/train_jax.py:2028-2120, an optax chain of
``clip_by_global_norm(1.0)``, ``scale_by_adam(b1=0.9, b2=0.95, eps=1e-8)``,
two masked ``add_decayed_weights`` and ``scale_by_learning_rate``):

    g   <- g * min(1, clip / ||g||_global)
    m   <- b1 m + (1-b1) g ;  v <- b2 v + (1-b2) g^2
    u   <- (m / (1-b1^t)) / (sqrt(v / (1-b2^t)) + eps) + wd_group * p
    p   <- p - lr(t-1) * u

Weight-decay groups by parameter name: the nine pool tensors get
``pool_weight_decay``; other matrices get ``weight_decay``; biases, LayerNorm
weights and the ``*_scale`` pool output scales get none.  The schedule is a
linear warm-up from ``0.1 lr`` to ``lr`` followed by a cosine decay back to
``0.1 lr``; it counts optimizer steps (after accumulation).

On CUDA the per-tensor math runs in one fused multi-tensor kernel per group
(``ops/cuda_backend.fused_adamw``); on CPU it is plain torch.  With a
data-parallel group the gradient all-reduce is issued per bucket before the
norm (see ``parallel/grad_sync.py``).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

POOL_PARAM_NAMES = ("qk_emb", "v_emb", "know_emb", "qk_read", "v_read", "know_read",
                    "qk_write", "v_write", "know_write")


def warmup_cosine(step: int, peak: float, warmup_steps: int, total_steps: int,
                  floor_ratio: float = 0.1) -> float:
    """optax.warmup_cosine_decay_schedule(init=0.1*peak, peak, warmup, decay_steps=total,
    end=0.1*peak) evaluated at ``step``."""
    lo = peak * floor_ratio
    if warmup_steps > 0 and step < warmup_steps:
        return lo + (peak - lo) * step / warmup_steps
    span = max(total_steps - warmup_steps, 1)
    frac = min(max(step - warmup_steps, 0) / span, 1.0)
    return lo + (peak - lo) * 0.5 * (1.0 + math.cos(math.pi * frac))


def wd_group_of(name: str) -> str:
    """'pool', 'base' or 'none' for a dotted parameter name."""
    leaf = name.split(".")[-1]
    if "bias" in leaf:
        return "none"
    if leaf.endswith("_scale"):
        return "none"
    if "norm" in name.lower() and leaf in ("weight", "scale"):
        return "none"
    if any(n in name for n in POOL_PARAM_NAMES):
        return "pool"
    return "base"


class DawnAdamW:
    def __init__(self, named_params: Iterable[Tuple[str, torch.nn.Parameter]], *, lr: float,
                 weight_decay: float = 0.1, pool_weight_decay: float = 0.02,
                 betas=(0.9, 0.95), eps: float = 1e-8, clip_norm: float = 1.0,
                 schedule: Optional[Callable[[int], float]] = None, accumulation_steps: int = 1,
                 grad_sync=None, fused: Optional[bool] = None):
        self.named = [(n, p) for n, p in named_params if p.requires_grad]
        self.lr, self.betas, self.eps, self.clip_norm = lr, betas, eps, clip_norm
        self.wd = {"base": weight_decay, "pool": pool_weight_decay, "none": 0.0}
        self.groups: Dict[str, List[int]] = {"base": [], "pool": [], "none": []}
        for i, (n, _) in enumerate(self.named):
            self.groups[wd_group_of(n)].append(i)
        self.schedule = schedule or (lambda step: lr)
        self.accumulation_steps = max(1, int(accumulation_steps))
        self.grad_sync = grad_sync
        self.count = 0            # optimizer steps taken
        self.micro = 0            # micro-steps inside the current accumulation window
        self.exp_avg = [torch.zeros_like(p, memory_format=torch.preserve_format) for _, p in self.named]
        self.exp_avg_sq = [torch.zeros_like(p, memory_format=torch.preserve_format) for _, p in self.named]
        self._acc: Optional[List[torch.Tensor]] = None
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.last_lr = float(self.schedule(0))
        dev = self.named[0][1].device if self.named else torch.device("cpu")
        self.fused = (dev.type == "cuda") if fused is None else fused
        self._fused_impl = None

    # ------------------------------------------------------------------
    def describe_groups(self) -> str:
        return (f"WD groups: base ({self.wd['base']}) = {len(self.groups['base'])} tensors, "
                f"pool ({self.wd['pool']}) = {len(self.groups['pool'])} tensors, "
                f"none = {len(self.groups['none'])} tensors")

    def zero_grad(self):
        for _, p in self.named:
            p.grad = None

    def _grads(self) -> List[torch.Tensor]:
        return [p.grad if p.grad is not None else torch.zeros_like(p) for _, p in self.named]

    @torch.no_grad()
    def step(self) -> bool:
        """Consume the current ``.grad``s.  Returns True when parameters were
        updated (the last micro-step of an accumulation window)."""
        k = self.accumulation_steps
        grads = self._grads()
        if k > 1:
            if self._acc is None:
                self._acc = [g.clone() for g in grads]
            else:
                torch._foreach_add_(self._acc, grads)
            self.micro += 1
            if self.micro < k:
                return False
            grads = self._acc
            torch._foreach_div_(grads, float(k))
            self._acc, self.micro = None, 0
        if self.grad_sync is not None:
            grads = self.grad_sync.reduce(self.named, grads)
        if self.grad_sync is not None:
            sq = self.grad_sync.global_sq_norm(self.named, grads)
        elif self.fused:
            from ..ops.cuda_backend import grad_sq_norm
            sq = grad_sq_norm(grads)
        else:
            sq = torch.stack([g.float().square().sum() for g in grads]).sum()
        norm = sq.sqrt()
        self.last_grad_norm = norm
        clip_scale = self.clip_norm / torch.clamp(norm, min=self.clip_norm)
        self.count += 1
        t = self.count
        lr = float(self.schedule(t - 1))
        self.last_lr = lr
        b1, b2 = self.betas
        bc1, bc2 = 1.0 - b1 ** t, 1.0 - b2 ** t
        if self.fused:
            from ..ops.cuda_backend import fused_adamw
            for gname, idx in self.groups.items():
                if idx:
                    fused_adamw([self.named[i][1] for i in idx], [grads[i] for i in idx],
                                [self.exp_avg[i] for i in idx], [self.exp_avg_sq[i] for i in idx],
                                clip_scale, lr, b1, b2, self.eps, self.wd[gname], bc1, bc2)
            return True
        for gname, idx in self.groups.items():
            wd = self.wd[gname]
            for i in idx:
                p = self.named[i][1]
                g = grads[i].float() * clip_scale
                m, v = self.exp_avg[i], self.exp_avg_sq[i]
                m.mul_(b1).add_(g, alpha=1.0 - b1)
                v.mul_(b2).addcmul_(g, g, value=1.0 - b2)
                upd = (m / bc1) / ((v / bc2).sqrt() + self.eps)
                if wd != 0.0:
                    upd = upd + wd * p
                p.add_(upd, alpha=-lr)
        return True

    # ------------------------------------------------------------------
    def state_dict(self) -> Dict:
        return {"count": self.count, "micro": self.micro,
                "exp_avg": {n: m for (n, _), m in zip(self.named, self.exp_avg)},
                "exp_avg_sq": {n: v for (n, _), v in zip(self.named, self.exp_avg_sq)},
                "acc": None if self._acc is None else {n: a for (n, _), a in zip(self.named, self._acc)}}

    def load_state_dict(self, sd: Dict):
        self.count, self.micro = int(sd["count"]), int(sd.get("micro", 0))
        for i, (n, p) in enumerate(self.named):
            self.exp_avg[i].copy_(sd["exp_avg"][n].to(p.device))
            self.exp_avg_sq[i].copy_(sd["exp_avg_sq"][n].to(p.device))
        acc = sd.get("acc")
        self._acc = None if acc is None else [acc[n].to(p.device) for n, p in self.named]
        self.last_lr = float(self.schedule(max(self.count - 1, 0)))
