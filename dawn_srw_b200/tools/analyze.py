#!/usr/bin/env python
"""Analysis suite for a trained DAWN-SRW checkpoint.

    python -m dawn_srw_b200.tools.analyze --checkpoint run/best_model.pt [--config cfg.yaml]
        [--bin-val val.bin | --synthetic] [--only info,health,...] [--skip weights]
        [--batch-size 8] [--n-batches 4] [--output out_dir]

Analyses (``--only`` / ``--skip`` keys), each a function returning a JSON-able
dict; the selection mirrors the SRW part of the reference's analysis CLI
(scripts/analysis/standalone/spatial_analysis.py:6933-7287):

  info         parameter counts, configuration, forward FLOPs per token
  val          validation loss / perplexity / accuracy
  health       pool norm statistics, dead rows, scales, tau biases
  weights      pairwise |cos| summary and effective rank per pool tensor
  generate     sampled continuations (temperature / top-k, KV cache)
  routing      per layer and route: active units per token, gate entropy, top-1 mass
  gate_dist    quantiles of the raw gate values per route
  utilization  fraction of units ever selected, per pool and per layer
  sel_gini     Gini coefficient of per-unit selection frequency
  layer_role   attention vs knowledge output norm per layer
  intervene    loss change when the most-used knowledge units are suppressed
  pool_geom    spectrum of the pool embeddings (variance explained by top directions)
  rw_align     cos(read_u, write_u) per unit and its correlation with selection frequency
  tau_dist     threshold offsets produced by the tau heads on the sample (per route: mean,
               spread, quantiles, fraction below zero)
  drift        movement of the pool tensors against a second checkpoint (--compare-checkpoint)
  cross_ref    Q vs K specialisation of the shared QK pool (share of units used by one route only,
               Jaccard overlap of the per-token selections)
  layer_sim    cosine similarity of the per-unit selection profile between layers
  sel_trans    how much of a token's selected set survives from one layer to the next
  gate_ci      bootstrap confidence interval of the active fraction per route
  read_cov / write_cov   participation ratio of the selection-weighted read / write vectors
  samples      for the most-used knowledge units: the token ids that open them most strongly
  resid_dyn    residual-stream dynamics: norm per layer, rotation between consecutive layers and
               from the embedding to the last layer, top-1 agreement of each layer's read-out
  z_dist       distribution of the standardised score z = (s - mean) / std of the first layer's
               knowledge route (quantiles, fraction above the threshold)
  addit        additivity of suppressions: loss change of two unit sets together vs separately
  cross_suppress  effect of suppressing the most-used units of one pool on the loss and on the
               activity of the other pools

  r1           Q / K specialisation of the shared pool (q_ratio thresholds 0.7 / 0.3)
  r2           token-class selectivity of the knowledge units, specialists per class
  r3           knowledge units by contrastive score (target text vs the rest)
  r4           layer balance: attention vs knowledge output norm, averaged over the sample
  r5           suppression sweep of the top contrastive units (1 / 3 / 5 / 10 %) vs random
  rw_proj      read / write vectors against the token embeddings (what a unit reads / writes)
  act_context  contexts in which the most-used knowledge units open most strongly
  gate_mech    denominator statistics, floor activity, top-1 share of the gate mass
  comp_expr    effective rank of the write vectors spanned by a token's active set
  neuron_cluster  k-means clusters in emb / read / write space and their co-activation lift
  deep         corrective (cos(r,w) < -0.5) vs neutral vs amplifying units: selection and gate share
  op_space     diversity of the router projections, uniqueness of active sets, emb geometry
  compose      knowledge output split into corrective / neutral / amplifying contributions
  phase        phase boundary and baseline crossover from training logs (--dawn-log, --baseline-log)
  combo        distinct active sets, reuse entropy
  dom_supp     class-targeted vs random suppression with a selectivity index
  rw_func      cos(read, write) bins against selection frequency and gate mass
  tau_grad     gradient reaching the tau heads from the task loss vs from the auxiliary loss
  rw_cov       alias for read_cov,write_cov

All analyses run on one device through the model's public inference API
(models/inference.py); the second half of the list lives in tools/analyze_ext.py.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
from typing import Callable, Dict, List

import torch

from ..data.loaders import BinDataLoader, BinDataset, SyntheticDataset
from ..models import inference as I
from .common import load_model, tokenizer_or_none

ROUTES = ("Q", "K", "V", "Know")
POOL_OF = {"Q": "qk", "K": "qk", "V": "v", "Know": "know"}


class Context:
    def __init__(self, model, cfg, info, args):
        self.model, self.cfg, self.info, self.args = model, cfg, info, args
        self.device = next(model.parameters()).device
        self._batches = None
        self._gates = None

    def batches(self) -> List[torch.Tensor]:
        if self._batches is None:
            a, S = self.args, self.cfg.model.max_seq_len
            if a.synthetic or not a.bin_val:
                ds = SyntheticDataset(a.batch_size * a.n_batches, S, self.cfg.model.vocab_size, seed=1)
            else:
                ds = BinDataset(a.bin_val, S, self.cfg.data.max_val_tokens)
            loader = BinDataLoader(ds, a.batch_size, pin=False)
            self._batches = [loader.batch(i)[0].to(self.device).long()
                             for i in range(min(a.n_batches, len(loader)))]
        return self._batches

    def gates(self) -> Dict[str, torch.Tensor]:
        """analysis_forward(mode='full') of the first batch (cached)."""
        if self._gates is None:
            self._gates = I.analysis_forward(self.model, self.batches()[0], mode="full")
        return self._gates


# ---------------------------------------------------------------------------
def analyze_info(c: Context) -> Dict:
    m = c.model
    n_params = sum(p.numel() for p in m.parameters())
    pool = sum(p.numel() for n, p in m.named_parameters() if "neuron_pool" in n)
    out = {"parameters": n_params, "pool_parameters": pool, "config": m.get_config(),
           "checkpoint": c.info}
    if hasattr(m, "n_know"):
        out["flops_per_token"] = I.estimate_flops_per_token(m)
    return out


def analyze_val(c: Context) -> Dict:
    loss, ppl, acc, n = I.vectorized_eval(c.model, iter(c.batches()))
    return {"val_loss": loss, "ppl": ppl, "accuracy_pct": acc, "valid_tokens": n}


def analyze_health(c: Context) -> Dict:
    return I.neuron_health(c.model)


def analyze_weights(c: Context) -> Dict:
    return I.weight_analysis(c.model, max_rows=c.args.max_rows)


def analyze_generate(c: Context) -> Dict:
    a = c.args
    tok = tokenizer_or_none()
    prompts = a.prompt or ["the"]
    outs = []
    for ptxt in prompts:
        if tok is not None:
            ids = torch.tensor([tok.encode(ptxt, add_special_tokens=False)], device=c.device)
        else:
            ids = c.batches()[0][:1, :8]
        gen, stats = I.generate(c.model, ids, max_new_tokens=a.max_new_tokens,
                                temperature=a.temperature, top_k=a.top_k)
        rec = {"prompt": ptxt, "token_ids": gen[0].tolist(),
               "tokens_per_sec": stats["tokens_per_sec"]}
        if tok is not None:
            rec["text"] = tok.decode(gen[0].tolist())
        outs.append(rec)
    return {"samples": outs, "tokenizer": "bert-base-uncased" if tok is not None else None}


def analyze_routing(c: Context) -> Dict:
    g = c.gates()
    out = {}
    for r in ROUTES:
        raw, nrm = g[f"gate_{r}_raw"], g[f"gate_{r}"]                # [L,B,S,N]
        active = (raw > 0).float().sum(-1)                           # units per token
        ent = -(nrm * torch.log(nrm.clamp(min=1e-12))).sum(-1)
        out[r] = {"active_per_token_mean": active.mean(dim=(1, 2)).tolist(),
                  "active_per_token_std": active.std(dim=(1, 2), unbiased=False).tolist(),
                  "gate_entropy": ent.mean(dim=(1, 2)).tolist(),
                  "top1_mass": nrm.max(-1).values.mean(dim=(1, 2)).tolist(),
                  "n_units": int(raw.shape[-1])}
    return out


def analyze_gate_dist(c: Context) -> Dict:
    g = c.gates()
    qs = torch.tensor([0.5, 0.9, 0.99, 0.999], device=c.device)
    out = {}
    for r in ROUTES:
        raw = g[f"gate_{r}_raw"].float()
        pos = raw[raw > 0]
        rec = {"zero_frac": float((raw <= 0).float().mean()), "max": float(raw.max())}
        if pos.numel():
            sample = pos[torch.randint(0, pos.numel(), (min(pos.numel(), 1_000_000),), device=pos.device)]
            for q, v in zip(qs.tolist(), torch.quantile(sample, qs).tolist()):
                rec[f"p{q * 100:g}"] = v
            rec["mean_active"] = float(pos.mean())
        out[r] = rec
    return out


def _selection_counts(c: Context) -> Dict[str, torch.Tensor]:
    """Per route: [L, N] number of tokens that selected each unit."""
    g = c.gates()
    return {r: (g[f"gate_{r}_raw"] > 0).float().sum(dim=(1, 2)) for r in ROUTES}


def analyze_utilization(c: Context) -> Dict:
    cnt = _selection_counts(c)
    out = {}
    for r in ROUTES:
        k = cnt[r]
        out[r] = {"used_frac_per_layer": (k > 0).float().mean(-1).tolist(),
                  "used_frac_any_layer": float((k.sum(0) > 0).float().mean()),
                  "never_used": int((k.sum(0) == 0).sum())}
    return out


def _gini(x: torch.Tensor) -> float:
    x = torch.sort(x.flatten().double()).values
    n = x.numel()
    if n == 0 or float(x.sum()) == 0.0:
        return 0.0
    idx = torch.arange(1, n + 1, dtype=torch.double, device=x.device)
    return float(((2 * idx - n - 1) * x).sum() / (n * x.sum()))


def analyze_sel_gini(c: Context) -> Dict:
    cnt = _selection_counts(c)
    return {r: {"gini_all_layers": _gini(cnt[r].sum(0)),
                "gini_per_layer": [_gini(row) for row in cnt[r]]} for r in ROUTES}


def analyze_layer_role(c: Context) -> Dict:
    g = c.gates()
    a, k = g["attn_out_norm"], g["know_out_norm"]
    return {"attn_out_norm": a.tolist(), "know_out_norm": k.tolist(),
            "know_share": (k / (a + k).clamp(min=1e-12)).tolist()}


def _mean_loss(logits: torch.Tensor, ids: torch.Tensor) -> float:
    lp = torch.log_softmax(logits[:, :-1].float(), -1)
    return float(-lp.gather(-1, ids[:, 1:].unsqueeze(-1)).mean())


def analyze_intervene(c: Context) -> Dict:
    m, ids = c.model, c.batches()[0]
    cnt = _selection_counts(c)["Know"].sum(0)
    base = _mean_loss(c.gates()["logits"], ids)
    out = {"baseline_loss": base, "suppressed": []}
    for k in c.args.suppress_top:
        k = min(int(k), cnt.numel())
        mask = torch.zeros(m.neuron_pool.know_emb.shape[0], dtype=torch.bool, device=c.device)
        mask[torch.topk(cnt, k).indices] = True
        logits = I.build_suppressed_forward(m, {"know": mask})(ids)
        rnd = torch.zeros_like(mask)
        rnd[torch.randperm(cnt.numel(), device=c.device)[:k]] = True
        logits_r = I.build_suppressed_forward(m, {"know": rnd})(ids)
        out["suppressed"].append({"k": k, "loss_top_used": _mean_loss(logits, ids),
                                  "loss_random": _mean_loss(logits_r, ids)})
    return out


def analyze_pool_geom(c: Context) -> Dict:
    out = {}
    p = c.model.neuron_pool
    for name in ("qk", "v", "know"):
        e = getattr(p, f"{name}_emb")[: p.n_valid(name)].float()
        e = e - e.mean(0, keepdim=True)
        sv = torch.linalg.svdvals(e.cpu())
        var = sv.square() / sv.square().sum()
        out[name] = {"top8_variance": var[:8].tolist(),
                     "dims_for_90pct": int((var.cumsum(0) < 0.9).sum()) + 1,
                     "participation_ratio": float(1.0 / var.square().sum())}
    return out


def analyze_rw_align(c: Context) -> Dict:
    p = c.model.neuron_pool
    cnt = _selection_counts(c)
    freq = {"qk": (cnt["Q"] + cnt["K"]).sum(0), "v": cnt["V"].sum(0), "know": cnt["Know"].sum(0)}
    out = {}
    for name in ("qk", "v", "know"):
        n = p.n_valid(name)
        rd = getattr(p, f"{name}_read")[:n].float()
        wr = getattr(p, f"{name}_write")[:n].float()
        cos = torch.nn.functional.cosine_similarity(rd, wr, dim=-1)
        f = freq[name][:n].float()
        rec = {"cos_mean": float(cos.mean()), "cos_std": float(cos.std(unbiased=False)),
               "cos_min": float(cos.min()), "cos_max": float(cos.max()),
               "frac_negative": float((cos < 0).float().mean())}
        if float(f.std(unbiased=False)) > 0 and float(cos.std(unbiased=False)) > 0:
            rec["corr_with_selection_freq"] = float(torch.corrcoef(torch.stack([cos, f]))[0, 1])
        out[name] = rec
    return out


def analyze_tau_dist(c: Context) -> Dict:
    m, ids = c.model, c.batches()[0]
    be = I._be(m, c.device)
    B, S = ids.shape
    x = be.embed(ids, m.token_emb.weight, m.pos_emb.weight).float()
    blk = m.layers[0]
    n1 = be.layer_norm(x, blk.norm1.weight, blk.norm1.bias).reshape(B * S, m.d_model)
    rt = m.router
    taus = {"attn": be.linear(n1, rt.tau_attn.weight, rt.tau_attn.bias).float(),
            "know": be.linear(n1, rt.tau_know.weight, rt.tau_know.bias).float()}
    names = {"attn": ("Q", "K", "V"), "know": ("Know",)}
    qs = torch.tensor([0.01, 0.5, 0.99], device=c.device)
    out = {"layer": 0}
    for key, t in taus.items():
        for i, nm in enumerate(names[key]):
            col = t[:, i]
            q = torch.quantile(col, qs).tolist()
            out[nm] = {"mean": float(col.mean()), "std": float(col.std(unbiased=False)),
                       "p01": q[0], "p50": q[1], "p99": q[2],
                       "neg_frac": float((col < 0).float().mean())}
    return out


def analyze_drift(c: Context) -> Dict:
    other = c.args.compare_checkpoint
    if not other:
        return {"skipped": "pass --compare-checkpoint to measure drift against another checkpoint"}
    ref, _, info = load_model(other, c.args.config, device=str(c.device))
    out = {"against": info}
    p, q = c.model.neuron_pool, ref.neuron_pool
    for name in ("qk", "v", "know"):
        n = p.n_valid(name)
        for kind in ("emb", "read", "write"):
            a = getattr(p, f"{name}_{kind}")[:n].float()
            b = getattr(q, f"{name}_{kind}")[:n].float()
            cos = torch.nn.functional.cosine_similarity(a, b, dim=-1)
            out[f"{name}_{kind}"] = {"rel_l2": float((a - b).norm() / b.norm().clamp(min=1e-12)),
                                     "row_cos_mean": float(cos.mean()), "row_cos_min": float(cos.min())}
    return out


def analyze_cross_ref(c: Context) -> Dict:
    g = c.gates()
    q, k = g["gate_Q_raw"] > 0, g["gate_K_raw"] > 0                     # [L,B,S,N]
    fq, fk = q.float().sum(dim=(0, 1, 2)), k.float().sum(dim=(0, 1, 2))
    used = (fq + fk) > 0
    share_q = fq / (fq + fk).clamp(min=1.0)
    special = ((share_q > 0.9) | (share_q < 0.1)) & used
    inter = (q & k).float().sum(-1)
    union = (q | k).float().sum(-1).clamp(min=1.0)
    return {"units_used": int(used.sum()), "specialised_frac": float(special.float().sum() / used.float().sum().clamp(min=1.0)),
            "q_only_frac": float(((share_q > 0.9) & used).float().sum() / used.float().sum().clamp(min=1.0)),
            "token_jaccard_mean": float((inter / union).mean())}


def analyze_layer_sim(c: Context) -> Dict:
    cnt = _selection_counts(c)
    out = {}
    for r in ROUTES:
        prof = torch.nn.functional.normalize(cnt[r].float(), dim=-1)      # [L,N]
        sim = prof @ prof.t()
        L = sim.shape[0]
        off = sim[~torch.eye(L, dtype=torch.bool, device=sim.device)]
        out[r] = {"adjacent": [float(sim[i, i + 1]) for i in range(L - 1)],
                  "mean_off_diagonal": float(off.mean()) if off.numel() else 1.0}
    return out


def analyze_sel_trans(c: Context) -> Dict:
    g = c.gates()
    out = {}
    for r in ROUTES:
        sel = g[f"gate_{r}_raw"] > 0                                        # [L,B,S,N]
        keep = []
        for l in range(sel.shape[0] - 1):
            a, b = sel[l], sel[l + 1]
            keep.append(float(((a & b).float().sum(-1) / a.float().sum(-1).clamp(min=1.0)).mean()))
        out[r] = {"survival_to_next_layer": keep}
    return out


def analyze_gate_ci(c: Context) -> Dict:
    g = c.gates()
    gen = torch.Generator(device="cpu").manual_seed(0)
    out = {}
    for r in ROUTES:
        frac = (g[f"gate_{r}_raw"] > 0).float().mean(-1).flatten().cpu()      # per (layer, token)
        n = frac.numel()
        boots = torch.stack([frac[torch.randint(0, n, (n,), generator=gen)].mean() for _ in range(200)])
        lo, hi = torch.quantile(boots, torch.tensor([0.025, 0.975])).tolist()
        out[r] = {"active_frac": float(frac.mean()), "ci95": [lo, hi], "tokens": n}
    return out


def _coverage(c: Context, kind: str) -> Dict:
    p = c.model.neuron_pool
    cnt = _selection_counts(c)
    freq = {"qk": (cnt["Q"] + cnt["K"]).sum(0), "v": cnt["V"].sum(0), "know": cnt["Know"].sum(0)}
    out = {}
    for name in ("qk", "v", "know"):
        n = p.n_valid(name)
        w = getattr(p, f"{name}_{kind}")[:n].float()
        f = freq[name][:n].float()
        f = f / f.sum().clamp(min=1e-12)
        cov = (w * f[:, None]).t() @ w                                       # [D,D], selection-weighted
        ev = torch.linalg.eigvalsh(cov.cpu().double()).clamp(min=0)
        out[name] = {"participation_ratio": float(ev.sum() ** 2 / ev.square().sum().clamp(min=1e-30)),
                     "dims": int(w.shape[1])}
    return out


def analyze_read_cov(c: Context) -> Dict:
    return _coverage(c, "read")


def analyze_write_cov(c: Context) -> Dict:
    return _coverage(c, "write")


def analyze_samples(c: Context) -> Dict:
    g, ids = c.gates(), c.batches()[0]
    raw = g["gate_Know_raw"]                                                 # [L,B,S,N]
    cnt = (raw > 0).float().sum(dim=(0, 1, 2))
    top_units = torch.topk(cnt, min(5, cnt.numel())).indices.tolist()
    tok = tokenizer_or_none()
    out = []
    for u in top_units:
        strength = raw[..., u].max(0).values                                  # [B,S] strongest layer
        k = min(8, strength.numel())
        flat = torch.topk(strength.flatten(), k).indices
        tids = ids.flatten()[flat].tolist()
        rec = {"unit": u, "selected_by_tokens": int(cnt[u]), "top_token_ids": tids}
        if tok is not None:
            rec["top_tokens"] = tok.convert_ids_to_tokens(tids)
        out.append(rec)
    return {"know_units": out}


def analyze_resid_dyn(c: Context) -> Dict:
    m, ids = c.model, c.batches()[0]
    be = I._be(m, c.device)
    pools = I._pools(m, be)
    B, S = ids.shape
    D, H = m.d_model, m.n_heads
    heads = lambda t: t.reshape(B, S, H, D // H).transpose(1, 2)
    x = be.embed(ids, m.token_emb.weight, m.pos_emb.weight).float()
    states = [x]
    for blk in m.layers:
        n = be.layer_norm(x, blk.norm1.weight, blk.norm1.bias).reshape(B * S, D)
        q, k, v, _, _ = I._layer_qkv(m, be, n, pools)
        o = be.attention(heads(q), heads(k), heads(v), 0.0, False).transpose(1, 2).reshape(B * S, D)
        x = x + be.linear(o, blk.attn.expand_O.weight, None).float().reshape(B, S, D)
        n = be.layer_norm(x, blk.norm2.weight, blk.norm2.bias).reshape(B * S, D)
        ko, _ = I._know(m, be, n, pools)
        x = x + ko.float().reshape(B, S, D)
        states.append(x)
    cos = torch.nn.functional.cosine_similarity
    deg = lambda a, b: float(torch.rad2deg(torch.acos(cos(a, b, dim=-1).clamp(-1, 1))).mean())
    final_top1 = be.logits(be.layer_norm(states[-1], m.norm.weight, m.norm.bias), m.token_emb.weight).argmax(-1)
    agree = []
    for st in states[1:]:
        top1 = be.logits(be.layer_norm(st, m.norm.weight, m.norm.bias), m.token_emb.weight).argmax(-1)
        agree.append(float((top1 == final_top1).float().mean()))
    return {"norm_per_layer": [float(torch.linalg.vector_norm(s_, dim=-1).mean()) for s_ in states],
            "rotation_deg_per_layer": [deg(states[i], states[i + 1]) for i in range(len(states) - 1)],
            "rotation_deg_total": deg(states[0], states[-1]),
            "cumulative_rotation_deg": sum(deg(states[i], states[i + 1]) for i in range(len(states) - 1)),
            "top1_agreement_with_final": agree}


def analyze_z_dist(c: Context) -> Dict:
    m, ids = c.model, c.batches()[0]
    be = I._be(m, c.device)
    B, S = ids.shape
    x = be.embed(ids, m.token_emb.weight, m.pos_emb.weight).float()
    blk = m.layers[0]
    # knowledge route of the first layer, scores against the (optionally normalised) embeddings
    n1 = be.layer_norm(x, blk.norm1.weight, blk.norm1.bias).reshape(B * S, m.d_model)
    h = be.linear(n1, m.router.proj_know.weight, m.router.proj_know.bias).float()
    p = m.neuron_pool
    emb = p.know_emb[: p.n_valid("know")].float()
    if m.gate.normalize_pool:
        emb = emb / (torch.linalg.vector_norm(emb, dim=-1, keepdim=True) + 1e-8)
    s = h @ emb.t()
    z = (s - s.mean(-1, keepdim=True)) / (s.std(-1, unbiased=False, keepdim=True) + 1e-8)
    off = be.linear(n1, m.router.tau_know.weight, m.router.tau_know.bias).float()      # [T,1]
    flat = z.flatten()
    sample = flat[torch.randint(0, flat.numel(), (min(flat.numel(), 1_000_000),), device=flat.device)]
    qs = torch.tensor([0.01, 0.25, 0.5, 0.75, 0.99, 0.999], device=c.device)
    qv = torch.quantile(sample, qs).tolist()
    return {"quantiles": dict(zip(["p1", "p25", "p50", "p75", "p99", "p99.9"], qv)),
            "skew": float((z ** 3).mean()), "excess_kurtosis": float((z ** 4).mean() - 3.0),
            "frac_above_threshold": float((z > off).float().mean()),
            "threshold_offset_mean": float(off.mean())}


def _loss_with(c: Context, masks: Dict[str, torch.Tensor]) -> float:
    ids = c.batches()[0]
    return _mean_loss(I.build_suppressed_forward(c.model, masks)(ids), ids)


def _top_mask(c: Context, pool: str, counts: torch.Tensor, k: int, skip: int = 0) -> torch.Tensor:
    n_rows = getattr(c.model.neuron_pool, f"{pool}_emb").shape[0]
    mask = torch.zeros(n_rows, dtype=torch.bool, device=c.device)
    idx = torch.topk(counts, min(k + skip, counts.numel())).indices[skip:]
    mask[idx] = True
    return mask


def analyze_addit(c: Context) -> Dict:
    cnt = _selection_counts(c)["Know"].sum(0)
    k = max(1, min(int(c.args.suppress_top[0]) if c.args.suppress_top else 16, cnt.numel() // 2))
    a, b = _top_mask(c, "know", cnt, k), _top_mask(c, "know", cnt, k, skip=k)
    base = _mean_loss(c.gates()["logits"], c.batches()[0])
    la, lb, lab = _loss_with(c, {"know": a}), _loss_with(c, {"know": b}), _loss_with(c, {"know": a | b})
    return {"k": k, "baseline": base, "delta_a": la - base, "delta_b": lb - base, "delta_ab": lab - base,
            "interaction": (lab - base) - (la - base) - (lb - base)}


def analyze_cross_suppress(c: Context) -> Dict:
    cnt = _selection_counts(c)
    freq = {"qk": (cnt["Q"] + cnt["K"]).sum(0), "v": cnt["V"].sum(0), "know": cnt["Know"].sum(0)}
    base = _mean_loss(c.gates()["logits"], c.batches()[0])
    k = int(c.args.suppress_top[0]) if c.args.suppress_top else 16
    out = {"baseline": base, "k": k}
    for pool in ("qk", "v", "know"):
        kk = max(1, min(k, freq[pool].numel() // 2))
        out[pool] = {"loss_delta": _loss_with(c, {pool: _top_mask(c, pool, freq[pool], kk)}) - base}
    return out


ANALYSES: Dict[str, Callable[[Context], Dict]] = {
    "info": analyze_info, "val": analyze_val, "health": analyze_health, "weights": analyze_weights,
    "generate": analyze_generate, "routing": analyze_routing, "gate_dist": analyze_gate_dist,
    "utilization": analyze_utilization, "sel_gini": analyze_sel_gini,
    "layer_role": analyze_layer_role, "intervene": analyze_intervene, "pool_geom": analyze_pool_geom,
    "rw_align": analyze_rw_align, "tau_dist": analyze_tau_dist, "drift": analyze_drift,
    "cross_ref": analyze_cross_ref, "layer_sim": analyze_layer_sim, "sel_trans": analyze_sel_trans,
    "gate_ci": analyze_gate_ci, "read_cov": analyze_read_cov, "write_cov": analyze_write_cov,
    "samples": analyze_samples, "resid_dyn": analyze_resid_dyn, "z_dist": analyze_z_dist,
    "addit": analyze_addit, "cross_suppress": analyze_cross_suppress,
}
SPATIAL_ONLY = {"health", "weights", "routing", "gate_dist", "utilization", "sel_gini", "layer_role",
                "intervene", "pool_geom", "rw_align", "tau_dist", "drift", "cross_ref", "layer_sim",
                "sel_trans", "gate_ci", "read_cov", "write_cov", "samples", "resid_dyn", "z_dist",
                "addit", "cross_suppress"}

from .analyze_ext import EXTRA_ANALYSES, NEEDS_GRAD  # noqa: E402  (second half of the suite)
ANALYSES.update(EXTRA_ANALYSES)
SPATIAL_ONLY |= set(EXTRA_ANALYSES) - {"phase"}
# meta keys of the reference's CLI: rw_cov = read_cov + write_cov
ALIASES = {"rw_cov": ["read_cov", "write_cov"]}


def run(model, cfg, info, args) -> Dict:
    keys = [k for k in (args.only.split(",") if args.only else ANALYSES) if k]
    keys = [kk for k in keys for kk in ALIASES.get(k, [k])]
    skip = {kk for k in (args.skip.split(",") if args.skip else []) for kk in ALIASES.get(k, [k])}
    unknown = [k for k in keys if k not in ANALYSES]
    if unknown:
        raise SystemExit(f"unknown analysis key(s) {unknown}; choose from {sorted(ANALYSES)}")
    ctx = Context(model, cfg, info, args)
    results = {}
    for k in keys:
        if k in skip or (k in SPATIAL_ONLY and not cfg.model.is_spatial):
            continue
        if k in NEEDS_GRAD:
            results[k] = ANALYSES[k](ctx)
        else:
            with torch.no_grad():
                results[k] = ANALYSES[k](ctx)
    return results


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawTextHelpFormatter)
    ap.add_argument("--checkpoint")
    ap.add_argument("--config")
    ap.add_argument("--bin-val")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--only", default="")
    ap.add_argument("--skip", default="")
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--n-batches", type=int, default=4)
    ap.add_argument("--max-rows", type=int, default=2048)
    ap.add_argument("--prompt", action="append")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--suppress-top", type=int, nargs="*", default=[16, 128])
    ap.add_argument("--compare-checkpoint")
    ap.add_argument("--target-prompt", action="append",
                    help="target text of the contrastive analyses r3 / r5 (needs the tokenizer)")
    ap.add_argument("--p6-samples", type=int, default=32, help="token samples of comp_expr")
    ap.add_argument("--dom-supp-levels", default="0.01,0.05",
                    help="comma-separated suppression fractions of dom_supp")
    ap.add_argument("--dawn-log", help="training metrics (JSONL or CSV) for the phase analysis")
    ap.add_argument("--baseline-log", help="a baseline run's metrics for the crossover step")
    ap.add_argument("--output")
    ap.add_argument("--library", action="store_true")
    ap.add_argument("--device")
    args = ap.parse_args(argv)
    model, cfg, info = load_model(args.checkpoint, args.config, device=args.device,
                                  library=args.library)
    results = run(model, cfg, info, args)
    text = json.dumps(results, indent=2, default=lambda o: o if not isinstance(o, float) or math.isfinite(o) else None)
    if args.output:
        os.makedirs(args.output, exist_ok=True)
        with open(os.path.join(args.output, "analysis.json"), "w") as f:
            f.write(text)
    print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
