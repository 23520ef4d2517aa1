"""Plain-PyTorch statement of the SRW pool op.

This is (a) the fp32 CPU oracle every CUDA kernel is tested against, (b) the
path CPU ranks (gloo) use to test sharding logic and (c) on a GPU, with
``compute_dtype=torch.bfloat16``, the *library baseline*: the same math through
``torch.matmul`` + NCCL, against which the fused sm_100a kernels are measured.

Math (reference: models/dawn_spatial_v41_exp.py:352-637 single route,
:640-909 paired routes; v4.0.1 models/legacy/dawn_spatial_v401_exp.py:230-363;
v3.9.4 models/dawn_spatial_v394_exp.py:180-260):

    s      = h . emb^T                                  [T, R, U]
    mu, sd = mean_U(s), sqrt(mean_U(s^2) - mu^2) + 1e-8  (over the GLOBAL pool)
    tau    = mu + tau_off * sd
    g, dt  = gate(s, tau, sd)                            (see ops/gates.py)
    xr     = x . read^T                                  [T, U]   (shared by routes)
    out    = ((g * xr) . write) / max(sum_U dt, 1)       [T, R, D]

Units may be sharded over ``shard_group`` (each rank holds ``U_local`` rows of
emb/read/write); per-token sums are all-reduced.  ``n_valid`` marks how many
local rows are real: trailing rows are padding and contribute nothing.

Gradient convention for multi-rank runs: every rank's loss is one term of the
objective ``mean_r L_r`` and every collective back-propagates with its true
transpose (all-reduce <-> all-reduce, all-gather <-> reduce-scatter), exactly
like ``psum`` inside the reference's ``shard_map``.  A rank's parameter
gradients are therefore partial sums; ``parallel/grad_sync.py`` adds them over
the ranks that hold a copy and divides by the world size.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Optional

import torch
import torch.utils.checkpoint as ckpt

from .gates import (GATE_GELU_Z, GATE_RELU_CLIP, GATE_TWO_STAGE, GateSpec,
                    gate_forward)
from ..parallel import collectives as C


@dataclass
class SRWResult:
    out: torch.Tensor                       # [T, R, D] fp32, before the pool scale
    lb: torch.Tensor                        # load-balance statistic (scalar)
    dead_penalty: torch.Tensor              # scalar (0 unless the gate has one)
    diag: Dict[str, torch.Tensor] = field(default_factory=dict)
    gates: Optional[torch.Tensor] = None    # [T, R, U_local] raw gate (analysis)
    den: Optional[torch.Tensor] = None      # [T, R] denominator
    outs: Optional[list] = None             # per-route [T, D] tensors when `out` was not stacked

    def route(self, i: int) -> torch.Tensor:
        """Output of route ``i`` ([T, D]) whichever way the backend stored it."""
        return self.outs[i] if self.outs is not None else self.out[:, i]

    def stacked(self) -> torch.Tensor:
        return self.out if self.out is not None else torch.stack(self.outs, dim=1)


def normalize_rows(w: torch.Tensor) -> torch.Tensor:
    return w / (torch.linalg.vector_norm(w, dim=-1, keepdim=True) + 1e-8)


def prepare_pool_ref(emb, read, write, spec: GateSpec, dtype):
    """Forward-time pool preparation: optional row unit-norm, then cast."""
    if spec.normalize_pool:
        emb, read, write = normalize_rows(emb), normalize_rows(read), normalize_rows(write)
    return emb.to(dtype), read.to(dtype), write.to(dtype)


def _mm(a, b_t, dtype):
    """a[..., K] @ b_t[N, K]^T in ``dtype`` with fp32 result."""
    return (a.to(dtype) @ b_t.to(dtype).t()).float()


def finalize_diag(spec: GateSpec, acc: Dict[str, torch.Tensor], gmax, s3, s4, gsum, den_sum, mu, sd,
                  tau, U_tot: int, dead_cnt, int_max, int_cap, shard_group) -> Dict[str, torch.Tensor]:
    """Routing diagnostics of one pool-op call from per-token accumulators over this rank's
    units (reference: models/dawn_spatial_v41_exp.py:519-534, 588-635).  ``acc`` holds
    [T, R, 1] sums "active", "strong", "band", "zsum", "b075", "b030", "glogg"; ``gmax`` the
    per-token gate maximum; ``s3`` / ``s4`` the raw third / fourth score moments' sums; ``gsum``
    and ``den_sum`` are already summed over the shard group, the accumulators are summed here."""
    T, R = mu.shape[0], mu.shape[1]
    red = lambda t: C.all_reduce_nograd(t, shard_group, "sum")
    active = red(acc["active"])
    gmax_g = C.all_reduce_nograd(gmax, shard_group, "max")
    s3g, s4g = red(s3), red(s4)
    cube = s3g / U_tot
    third = cube - 3.0 * mu * sd ** 2 - mu ** 3
    quad = s4g / U_tot
    fourth = quad - 4.0 * mu * cube + 6.0 * mu ** 2 * sd ** 2 + 3.0 * mu ** 4
    glogg = red(acc["glogg"])
    if spec.kind == GATE_TWO_STAGE:
        adenom = active.clamp(min=1.0)
        z_mean_active = gsum / (active + 1e-8)
        gs_eps = gsum.clamp(min=1e-6)
        ent = -torch.where(gsum > 1e-6, glogg, torch.zeros_like(glogg)) / gs_eps + torch.log(gs_eps)
        ent = torch.where(torch.isfinite(ent), ent, torch.zeros_like(ent))
        z_sum_out = den_sum.mean()
    else:
        adenom = active + 1e-8
        z_mean_active = red(acc["zsum"]) / (active + 1e-8)
        gs_eps = gsum + 1e-8
        ent = -glogg / gs_eps + torch.log(gs_eps)
        z_sum_out = red(acc["zsum"]).mean()
    return {
        "active_frac": (active / U_tot).mean(dim=1).squeeze(-1),     # [T]
        "gate_max": gmax_g.mean(dim=1).squeeze(-1),                  # [T]
        "score_std": sd.mean(),
        "gate_sum": gsum.mean(),
        "active_n_mean": active.mean(),
        "strong": (red(acc["strong"]) / U_tot).mean(),
        "phi_binary": (red(acc["band"]) / U_tot).mean(),
        "z_mean_active": z_mean_active.mean(),
        "tau_abs_mean": tau.mean(),
        "z_lt_075": (red(acc["b075"]) / adenom).mean(),
        "z_lt_030": (red(acc["b030"]) / adenom).mean(),
        "score_skew": (third / (sd ** 3 + 1e-8)).mean(),
        "active_per_token_std": active.std(unbiased=False),
        "gate_entropy": ent.mean(),
        "z_sum": z_sum_out,
        "score_kurt": (fourth / (sd ** 4 + 1e-8)).mean(),
        "dead_count": red(dead_cnt),
        "int_max": C.all_reduce_nograd(int_max, shard_group, "max"),
        "int_cap_frac": red(int_cap) / float(T * R * U_tot),
    }


def srw_pool_ref(x, h, tau_off, emb, read, write, spec: GateSpec, *,
                 compute_dtype=torch.float32, chunk_size: Optional[int] = None,
                 n_valid: Optional[int] = None, n_total: Optional[int] = None,
                 shard_group=None, dp_group=None, unit_mask=None,
                 want_diag: bool = True, return_gates: bool = False,
                 use_checkpoint: bool = False, seq_sharded: bool = False) -> SRWResult:
    """x [T,D]; h [T,R,r]; tau_off [T,R]; emb [U,r]; read/write [U,D] (already
    prepared by ``prepare_pool_ref``).  Inputs x/h/tau_off are replicated over
    ``shard_group``; ``dp_group`` is only used by the load-balance and
    dead-unit statistics, which the reference reduces over data shards."""
    T, R, r = h.shape
    U_loc = emb.shape[0] if n_valid is None else n_valid
    emb, read, write = emb[:U_loc], read[:U_loc], write[:U_loc]
    if unit_mask is not None:
        unit_mask = unit_mask[:U_loc].to(torch.float32)
    nsh = C.group_size(shard_group)
    seq_sharded = bool(seq_sharded and nsh > 1)
    U_tot = n_total if n_total is not None else U_loc * nsh
    if seq_sharded and nsh > 1:
        # each rank holds T/nsh tokens: gather them so every rank scores all
        # tokens against its units (backward: reduce-scatter of dx/dh/dtau)
        x = C.gather_tokens(x, shard_group)
        h = C.gather_tokens(h, shard_group)
        tau_off = C.gather_tokens(tau_off, shard_group)
        T = h.shape[0]
    # without sequence sharding every rank of the group holds its own (equal)
    # copy of x/h/tau_off and uses it as is
    cs = U_loc if not chunk_size else min(chunk_size, U_loc)
    bounds = [(a, min(a + cs, U_loc)) for a in range(0, U_loc, cs)]
    f32 = torch.float32
    hq = h.to(compute_dtype)
    xq = x.to(compute_dtype)

    # ---- pass 1: per-token score moments over the global pool -------------
    s1 = torch.zeros(T, R, 1, dtype=f32, device=x.device)
    s2, s3, s4 = s1.clone(), s1.clone(), s1.clone()
    ns_sum = torch.zeros((), dtype=f32, device=x.device)
    ns_sq = torch.zeros((), dtype=f32, device=x.device)
    for a, b in bounds:
        def _stats(hq_, ec):
            s = _mm(hq_, ec, compute_dtype)                     # [T,R,cs]
            m = s.mean(dim=(0, 1))
            return (s.sum(-1, keepdim=True), (s * s).sum(-1, keepdim=True),
                    (s ** 3).sum(-1, keepdim=True), (s ** 4).sum(-1, keepdim=True),
                    m.sum(), (m * m).sum())
        o = (ckpt.checkpoint(_stats, hq, emb[a:b], use_reentrant=False)
             if use_checkpoint else _stats(hq, emb[a:b]))
        s1, s2, s3, s4 = s1 + o[0], s2 + o[1], s3 + o[2].detach(), s4 + o[3].detach()
        ns_sum, ns_sq = ns_sum + o[4], ns_sq + o[5]
    # the statistics feed each rank's own gates, so their cotangents differ per
    # rank and are summed in backward
    s1 = C.sum_over_shards(s1, shard_group)
    s2 = C.sum_over_shards(s2, shard_group)
    mu = s1 / U_tot
    sd = torch.sqrt(s2 / U_tot - mu * mu) + 1e-8
    tau = mu + tau_off.unsqueeze(-1) * sd
    # load balance: statistic of the per-unit mean score, computed per data
    # shard and then averaged over data shards (reference :476-483).
    ns_sum = C.mean_over_group(ns_sum, dp_group)
    ns_sq = C.mean_over_group(ns_sq, dp_group)
    ns_sum = C.sum_over_shards(ns_sum, shard_group)
    ns_sq = C.sum_over_shards(ns_sq, shard_group)
    mean_score = ns_sum / U_tot
    var_score = ns_sq / U_tot - mean_score ** 2
    lb = var_score / (mean_score ** 2 + var_score + 1e-2)

    # ---- pass 2: gate + read + write --------------------------------------
    D = x.shape[-1]
    raw_out = torch.zeros(T, R, D, dtype=f32, device=x.device)
    zero = lambda: torch.zeros(T, R, 1, dtype=f32, device=x.device)
    acc = {k: zero() for k in ("gsum", "den", "active", "strong", "band", "zsum",
                               "b075", "b030", "glogg")}
    gmax = torch.full((T, R, 1), -1e9, dtype=f32, device=x.device)
    dead_pen = torch.zeros((), dtype=f32, device=x.device)
    dead_cnt = torch.zeros((), dtype=f32, device=x.device)
    int_max = torch.zeros((), dtype=f32, device=x.device)
    int_cap = torch.zeros((), dtype=f32, device=x.device)
    gates_out = [] if return_gates else None
    cap_thr = spec.epsilon + spec.max_intensity - 1e-3

    for a, b in bounds:
        um = None if unit_mask is None else unit_mask[a:b]

        def _core(hq_, xq_, tau_, sd_, ec, rc, wc):
            s = _mm(hq_, ec, compute_dtype)
            g, dterm, aux = gate_forward(spec, s, tau_, sd_)
            if um is not None:
                g, dterm = g * um, dterm * um
            xr = _mm(xq_, rc, compute_dtype)                     # [T,cs]
            p = (g.to(compute_dtype) * xr.to(compute_dtype).unsqueeze(1))
            c_out = (p.to(compute_dtype) @ wc.to(compute_dtype)).float()
            return c_out, g, dterm, s, aux
        if use_checkpoint:
            c_out, g, dterm, s, aux = ckpt.checkpoint(
                _core, hq, xq, tau, sd, emb[a:b], read[a:b], write[a:b], use_reentrant=False)
        else:
            c_out, g, dterm, s, aux = _core(hq, xq, tau, sd, emb[a:b], read[a:b], write[a:b])
        raw_out = raw_out + c_out
        acc["gsum"] = acc["gsum"] + g.sum(-1, keepdim=True)
        acc["den"] = acc["den"] + dterm.sum(-1, keepdim=True)
        if return_gates:
            gates_out.append(g.detach())
        gd = g.detach()
        gmax = torch.maximum(gmax, gd.max(-1, keepdim=True).values)
        if spec.has_dead_penalty:
            mg = gd.amax(dim=(0, 1))
            ms = s.mean(dim=(0, 1))
            mg = C.all_reduce_nograd(mg, dp_group, "max")
            ms = C.mean_over_group(ms, dp_group)
            dead = (mg < spec.dead_threshold).float()
            dead_pen = dead_pen + (torch.relu(-ms) * dead).sum()
            dead_cnt = dead_cnt + dead.sum()
        if want_diag:
            with torch.no_grad():
                if spec.kind == GATE_TWO_STAGE:
                    act, inten = aux["activation"], aux["intensity"]
                    acc["active"] += (act > 0.5).float().sum(-1, keepdim=True)
                    acc["strong"] += (act > 0.9).float().sum(-1, keepdim=True)
                    acc["band"] += ((act > 0.1) & (act < 0.9)).float().sum(-1, keepdim=True)
                    acc["zsum"] += inten.sum(-1, keepdim=True)
                    acc["b075"] += ((act > 0.05) & (act < 0.95)).float().sum(-1, keepdim=True)
                    acc["b030"] += ((act > 0.2) & (act < 0.8)).float().sum(-1, keepdim=True)
                    int_max = torch.maximum(int_max, inten.max())
                    int_cap = int_cap + (inten >= cap_thr).float().sum()
                elif spec.kind == GATE_GELU_Z:
                    z, phi = aux["z"], aux["phi"]
                    acc["active"] += (gd > 0).float().sum(-1, keepdim=True)
                    acc["strong"] += (gd > 0.5).float().sum(-1, keepdim=True)
                    acc["band"] += ((phi > 0.95) | (phi < 0.05)).float().sum(-1, keepdim=True)
                    acc["zsum"] += torch.where(z > 0, z, torch.zeros_like(z)).sum(-1, keepdim=True)
                    acc["b075"] += ((z > 0) & (z < 0.75)).float().sum(-1, keepdim=True)
                    acc["b030"] += ((z > 0) & (z < 0.30)).float().sum(-1, keepdim=True)
                else:
                    acc["active"] += (aux["raw"] > 0).float().sum(-1, keepdim=True)
                acc["glogg"] += (gd * torch.log(gd + 1e-8)).sum(-1, keepdim=True)

    gsum = C.sum_over_shards(acc["gsum"], shard_group)
    den_sum = C.sum_over_shards(acc["den"], shard_group)   # divides each rank's own partial output
    den = den_sum.clamp(min=1.0)
    out = raw_out / den
    if seq_sharded:
        out = C.scatter_tokens_sum(out.to(compute_dtype), shard_group).float()
        r_, n_ = C.group_rank(shard_group), out.shape[0]
        den = den[r_ * n_:(r_ + 1) * n_]
    elif nsh > 1:
        # the cross-shard sum carries bf16 partials when computing in bf16
        out = C.sum_over_shards(out.to(compute_dtype), shard_group).float()
    dead_pen = C.sum_over_shards(dead_pen, shard_group)

    diag: Dict[str, torch.Tensor] = {}
    if want_diag:
        with torch.no_grad():
            diag = finalize_diag(spec, acc, gmax, s3, s4, gsum.detach(), den_sum.detach(), mu.detach(),
                                 sd.detach(), tau.detach(), U_tot, dead_cnt, int_max, int_cap,
                                 shard_group)
    gates = torch.cat(gates_out, dim=-1) if return_gates else None
    return SRWResult(out=out, lb=lb, dead_penalty=dead_pen, diag=diag, gates=gates,
                     den=den.squeeze(-1))
