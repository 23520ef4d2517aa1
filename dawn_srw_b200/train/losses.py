"""Loss assembly for training.

total = CE + lb_w * aux + tau_reg_w * tau_reg + div_w * diversity
        + dead_w * dead_penalty + explore_w * explore * [step >= warm-up]
for the SRW models; CE alone for the dense baseline
(reference: scripts/train_jax.py:679-702).

Exploration ("reward-prediction-error") loss, reference :566-677: with
``dev = stopgrad(CE_tok - global_mean_CE)`` and ``signal = dev if dev > 0 else
asym * dev``, sum ``signal * tau_offset`` over layers and routes for every valid
token, switching an element off when a further push would leave
``[lower, upper]``; divide by the number of valid tokens.  The global mean is
taken over all data-parallel ranks.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ..ops.reference import pool_diversity
from ..parallel import collectives as C


def global_mean_ce(per_token_ce, valid_mask, group=None):
    vm = valid_mask.float()
    tot = torch.stack([(per_token_ce.detach() * vm).sum(), vm.sum()])
    if C.group_size(group) > 1:
        tot = tot.clone()
        dist.all_reduce(tot, group=group)
    return tot[0] / (tot[1] + 1e-8)


def exploration_loss(result: Dict[str, Any], *, asymmetry: float, lower: float, upper: float,
                     eps: float, group=None, quantiles: bool = True):
    pce, vmask = result["per_token_ce"], result["valid_mask"]
    a_tau, k_tau = result["attn_tau_offset"], result["know_tau_offset"]       # [L,B,S,3], [L,B,S,1]
    vm = vmask.float()
    gmean = global_mean_ce(pce, vmask, group)
    dev = (pce - gmean).detach()
    signal = torch.where(dev > 0, dev, asymmetry * dev)
    a_t, k_t = a_tau[:, :, :-1, :], k_tau[:, :, :-1, :]
    sig = signal[None, :, :, None]
    vmb = vm[None, :, :, None]

    def off_mask(t):
        return ((sig > 0) & (t <= lower + eps)) | ((sig < 0) & (t >= upper - eps))
    a_off, k_off = off_mask(a_t), off_mask(k_t)
    vsum = vm.sum() + 1e-8
    ex_a = (sig * a_t * (~a_off).float() * vmb).sum() / vsum
    ex_k = (sig * k_t * (~k_off).float() * vmb).sum() / vsum
    stats: Dict[str, torch.Tensor] = {}
    with torch.no_grad():
        pos = (dev > 0).float() * vm
        neg = (dev < 0).float() * vm
        stats.update(
            global_mean_ce=gmean, explore_attn_raw=ex_a.detach(), explore_know_raw=ex_k.detach(),
            pos_frac=pos.sum() / vsum,
            pos_mean=(dev.clamp(min=0) * vm).sum() / (pos.sum() + 1e-8),
            neg_mean=((-dev).clamp(min=0) * vm).sum() / (neg.sum() + 1e-8),
            explore_block_frac_a=(a_off.float() * vmb).sum() / (vmb.sum() * a_t.shape[0] * a_t.shape[-1] + 1e-8),
            explore_block_frac_k=(k_off.float() * vmb).sum() / (vmb.sum() * k_t.shape[0] * k_t.shape[-1] + 1e-8),
            sig_pos_max=(signal * vm).max(), sig_neg_max=(-(signal * vm)).max())
        if quantiles:
            for nm, t in (("attn", a_tau), ("know", k_tau)):
                flat = t.detach().float().flatten()
                if flat.numel() > 1_000_000:          # quantile() has an input-size limit
                    flat = flat[:: flat.numel() // 1_000_000 + 1]
                stats[f"{nm}_tau_off_min"], stats[f"{nm}_tau_off_max"] = t.min(), t.max()
                stats[f"{nm}_tau_off_p99"] = torch.quantile(flat, 0.99)
                stats[f"{nm}_tau_off_p01"] = torch.quantile(flat, 0.01)
                stats[f"{nm}_tau_off_neg_frac"] = (t < 0).float().mean()
    return ex_a + ex_k, stats


def global_strided_sample(w_local: torch.Tensor, n_total: int, shard, group,
                          max_sample: int = 4096) -> torch.Tensor:
    """The rows ``w[::stride][:max_sample]`` of the *global* pool tensor, on
    every rank of ``group``, when each rank stores a contiguous slice of the
    unit axis (``shard.slice_of``).  Every rank picks the sampled rows that fall
    into its slice, the picks are all-gathered (autograd: reduce-scatter of the
    cotangents) and put back into global order.  Which rows each rank holds
    follows from the slice arithmetic, so no sizes are exchanged.  Pools of at
    most ``max_sample`` rows are gathered whole (reference sampling rule:
    scripts/train_jax.py:440-485)."""
    world = C.group_size(group)
    stride = max(1, n_total // max_sample) if n_total > max_sample else 1
    PoolShard = type(shard)
    picks = []
    for k in range(world):
        lo, hi, _ = PoolShard(k, world, shard.align).slice_of(n_total)
        first = lo + ((-lo) % stride)
        picks.append(list(range(first, hi, stride)))
    cmax = max(1, max(len(pk) for pk in picks))
    mine = picks[shard.index]
    lo = shard.slice_of(n_total)[0]
    buf = w_local.new_zeros((cmax,) + tuple(w_local.shape[1:]))
    if mine:
        idx = torch.tensor([g - lo for g in mine], device=w_local.device)
        buf = torch.cat([w_local.index_select(0, idx), buf[len(mine):]], dim=0)
    gathered = C.gather_tokens(buf, group)                       # [world * cmax, ...]
    keep = [k * cmax + i for k in range(world) for i in range(len(picks[k]))][:max_sample]
    return gathered.index_select(0, torch.tensor(keep, device=w_local.device))


def total_loss(result: Dict[str, Any], model, tcfg, step: int, *, is_baseline: bool,
               dp_group=None, backend=None, want_stats: bool = True):
    """Returns (total, parts) where parts holds the unweighted components."""
    ce = result["loss"]
    z = ce.new_zeros(())
    parts: Dict[str, torch.Tensor] = {"ce_loss": ce}
    if is_baseline:
        parts.update(aux_loss=z, tau_reg=z, div_loss=z, dead_penalty=z, explore_loss_raw=z,
                     orth_loss=z)
        return ce, parts
    aux = result["aux_loss"]
    tau_reg = result.get("tau_reg", z)
    dead = result.get("dead_penalty", z)
    pool = model.neuron_pool
    tensors = []
    shard_group = getattr(model, "shard_group", None)
    sharded = C.group_size(shard_group) > 1
    if tcfg.diversity_weight != 0.0:
        for name in ("qk", "v", "know"):
            n = pool.n_valid(name)
            for k in ("emb", "read", "write"):
                w = getattr(pool, f"{name}_{k}")[:n]
                if sharded and name in pool.sharded_names:
                    # the statistic is defined on a sample of the whole pool, not of a shard
                    w = global_strided_sample(w, pool.sizes[name], pool.shard, shard_group)
                tensors.append(w)
    if tcfg.diversity_weight != 0.0:
        div = backend.diversity(tensors) if backend is not None else pool_diversity(tensors)
    else:
        div = z
    explore, ex_stats = z, {}
    if tcfg.exploration_weight != 0.0 and "per_token_ce" in result:
        explore, ex_stats = exploration_loss(
            result, asymmetry=tcfg.exploration_asymmetry, lower=tcfg.exploration_lower_bound,
            upper=tcfg.exploration_upper_bound, eps=tcfg.exploration_bound_eps, group=dp_group,
            quantiles=want_stats)
    active = 1.0 if step >= tcfg.exploration_warmup_steps else 0.0
    total = (ce + tcfg.load_balance_weight * aux + tcfg.tau_reg_weight * tau_reg
             + tcfg.diversity_weight * div + tcfg.dead_penalty_weight * dead
             + tcfg.exploration_weight * explore * active)
    parts.update(aux_loss=aux, tau_reg=tau_reg, div_loss=div, dead_penalty=dead, orth_loss=z,
                 explore_loss_raw=explore, explore_loss_weighted=tcfg.exploration_weight * explore * active,
                 **ex_stats)
    return total, parts
