"""Second half of the analysis suite: the reference's rebuttal analyses (R.1-R.5),
the read / write interpretation analyses (P1, P2, P5-P10, P12), the selection
combinatorics, the domain suppression sweep, the read-write angle vs function
study, the tau gradient split and the training-log phase analysis
(reference: scripts/analysis/standalone/spatial_analysis.py, functions at
:860 r1, :1116 r2, :1409 r3, :983 r4, :1546 r5, :2010 rw_proj, :2104 act_context,
:2474 gate_mech, :2643 comp_expr, :2781 neuron_cluster, :3419 deep, :3643 op_space,
:4194 compose, :4830 phase, :5710 combo, :5988 dom_supp, :6184 rw_func, :6445 tau_grad).

Every function takes the ``Context`` of tools/analyze.py and returns a JSON-able
dict.  They run on one device through the model's public inference API and on
the gate tensors of ``analysis_forward``; where the reference needs a part-of-
speech tagger or curated fact prompts (not available offline) the token classes
come from the tokenizer's surface forms (or token-id buckets without one) and
the "target" texts from ``--target-prompt`` (default: the first sequence of the
sample against the rest), which keeps the statistics the same.
"""
from __future__ import annotations

import json
import math
import os
from collections import Counter
from typing import Dict, List

import torch

from ..models import inference as I
from .common import tokenizer_or_none

ROUTES = ("Q", "K", "V", "Know")


def _sel_counts(c):
    g = c.gates()
    return {r: (g[f"gate_{r}_raw"] > 0).float().sum(dim=(1, 2)) for r in ROUTES}


def _mid(c) -> int:
    return c.model.n_layers // 2


def _unit(w: torch.Tensor) -> torch.Tensor:
    return w / (torch.linalg.vector_norm(w, dim=-1, keepdim=True) + 1e-8)


def _pool(c, name: str, kind: str) -> torch.Tensor:
    p = c.model.neuron_pool
    return getattr(p, f"{name}_{kind}")[: p.n_valid(name)].float()


def _mean_loss(logits, ids) -> float:
    lp = torch.log_softmax(logits[:, :-1].float(), -1)
    return float(-lp.gather(-1, ids[:, 1:].unsqueeze(-1)).mean())


def _token_prob(logits, ids) -> torch.Tensor:
    """probability the model gives to each next token, [B, S-1]"""
    lp = torch.log_softmax(logits[:, :-1].float(), -1)
    return lp.gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1).exp()


# --------------------------------------------------------------------------- R.1
def analyze_r1(c) -> Dict:
    """Q/K specialisation of the shared pool: q_ratio = q_count / (q_count + k_count) per unit,
    Q-specialised above 0.7, K-specialised below 0.3."""
    cnt = _sel_counts(c)
    q, k = cnt["Q"].sum(0), cnt["K"].sum(0)
    used = (q + k) > 0
    ratio = q / (q + k).clamp(min=1.0)
    n_used = float(used.float().sum().clamp(min=1.0))
    q_spec, k_spec = (ratio > 0.7) & used, (ratio < 0.3) & used
    per_layer = []
    for l in range(cnt["Q"].shape[0]):
        ql, kl = cnt["Q"][l], cnt["K"][l]
        ul = (ql + kl) > 0
        rl = ql / (ql + kl).clamp(min=1.0)
        per_layer.append(float((((rl > 0.7) | (rl < 0.3)) & ul).float().sum() / ul.float().sum().clamp(min=1.0)))
    return {"units_used": int(used.sum()), "q_specialised_frac": float(q_spec.float().sum() / n_used),
            "k_specialised_frac": float(k_spec.float().sum() / n_used),
            "shared_frac": float((used & ~q_spec & ~k_spec).float().sum() / n_used),
            "specialised_frac_per_layer": per_layer,
            "q_ratio_histogram": torch.histc(ratio[used], bins=10, min=0.0, max=1.0).tolist()}


# --------------------------------------------------------------------------- token classes
def _token_classes(c, ids: torch.Tensor):
    """-> (class index per token [B,S], class names).  With a tokenizer: punctuation, number,
    word-piece continuation, short word, long word; without: five token-id buckets."""
    tok = tokenizer_or_none()
    V = c.cfg.model.vocab_size
    if tok is None or tok.vocab_size != V:
        names = [f"id_bucket_{i}" for i in range(5)]
        return (ids * 5 // max(V, 1)).clamp(max=4), names
    names = ["punct", "number", "continuation", "short_word", "long_word"]
    table = torch.zeros(V, dtype=torch.long)
    for t, i in tok.get_vocab().items():
        if i >= V:
            continue
        if t.startswith("##"):
            k = 2
        elif t.isdigit():
            k = 1
        elif not any(ch.isalnum() for ch in t):
            k = 0
        else:
            k = 3 if len(t) <= 3 else 4
        table[i] = k
    return table.to(ids.device)[ids], names


def analyze_r2(c) -> Dict:
    """Class selectivity of the knowledge units (the reference uses part-of-speech tags):
    selectivity[u, cls] = P(u active | cls) / P(u active); a specialist has selectivity > 2 and a
    mean gate weight > 0.1 on that class."""
    g, ids = c.gates(), c.batches()[0]
    cls, names = _token_classes(c, ids)
    nrm = g["gate_Know"][_mid(c)].float()                                 # [B,S,N] normalised gate
    act = (g["gate_Know_raw"][_mid(c)] > 0).float()
    p_act = act.mean(dim=(0, 1)).clamp(min=1e-9)
    out = {"layer": _mid(c), "classes": {}}
    n_spec_total = torch.zeros_like(p_act, dtype=torch.bool)
    for k, nm in enumerate(names):
        m = (cls == k)
        n_tok = int(m.sum())
        if n_tok == 0:
            out["classes"][nm] = {"tokens": 0}
            continue
        p_c = act[m].mean(0)
        sel = p_c / p_act
        w = nrm[m].mean(0) * nrm.shape[-1]                               # weight relative to uniform
        spec = (sel > 2.0) & (w > 0.1) & (p_act > 1e-6)
        n_spec_total |= spec
        top = torch.topk(sel * (p_act > 1e-6), min(5, sel.numel()))
        out["classes"][nm] = {"tokens": n_tok, "specialists": int(spec.sum()),
                              "max_selectivity": float(top.values[0]),
                              "top_units": top.indices.tolist()}
    out["specialist_units"] = int(n_spec_total.sum())
    return out


# --------------------------------------------------------------------------- R.3 / R.5
def _target_and_baseline(c):
    """Target token ids [1, S'] (from --target-prompt when a tokenizer is there, else the first
    sequence of the sample) and baseline ids (the other sequences)."""
    ids = c.batches()[0]
    tok = tokenizer_or_none()
    prompts = getattr(c.args, "target_prompt", None)
    if tok is not None and prompts:
        enc = tok.encode(" ".join(prompts), add_special_tokens=False)[: c.cfg.model.max_seq_len]
        if len(enc) >= 2:
            return torch.tensor([enc], device=c.device), ids
    return ids[:1], ids[1:] if ids.shape[0] > 1 else ids


def _contrastive(c):
    tgt, base = _target_and_baseline(c)
    mid = _mid(c)
    ft = (I.analysis_forward(c.model, tgt, mode="full")["gate_Know_raw"][mid] > 0).float().mean(dim=(0, 1))
    fb = (I.analysis_forward(c.model, base, mode="full")["gate_Know_raw"][mid] > 0).float().mean(dim=(0, 1))
    return ft - fb, ft, fb, tgt


def analyze_r3(c) -> Dict:
    """Knowledge units by contrastive score: activation frequency on the target text minus the
    frequency on the baseline text (middle layer)."""
    score, ft, fb, tgt = _contrastive(c)
    top = torch.topk(score, min(20, score.numel()))
    return {"layer": _mid(c), "target_tokens": int(tgt.numel()),
            "top_units": top.indices.tolist(), "top_scores": top.values.tolist(),
            "target_freq_of_top": ft[top.indices].tolist(), "baseline_freq_of_top": fb[top.indices].tolist(),
            "units_with_positive_score": int((score > 0).sum())}


def analyze_r5(c) -> Dict:
    """Suppression sweep: switch off the top N % of knowledge units by contrastive score and
    measure the drop of the probability of the target text's tokens (against a random set)."""
    score, _, _, tgt = _contrastive(c)
    m = c.model
    n_rows = m.neuron_pool.know_emb.shape[0]
    base_p = float(_token_prob(I.analysis_forward(m, tgt, mode="light")["logits"], tgt).mean())
    out = {"baseline_target_prob": base_p, "levels": []}
    gen = torch.Generator(device="cpu").manual_seed(0)
    for frac in (0.01, 0.03, 0.05, 0.10):
        k = max(1, int(frac * score.numel()))
        mask = torch.zeros(n_rows, dtype=torch.bool, device=c.device)
        mask[torch.topk(score, k).indices] = True
        rnd = torch.zeros_like(mask)
        rnd[torch.randperm(score.numel(), generator=gen)[:k].to(c.device)] = True
        p_t = float(_token_prob(I.build_suppressed_forward(m, {"know": mask})(tgt), tgt).mean())
        p_r = float(_token_prob(I.build_suppressed_forward(m, {"know": rnd})(tgt), tgt).mean())
        out["levels"].append({"frac": frac, "k": k, "target_prob": p_t, "random_prob": p_r,
                              "drop_targeted": base_p - p_t, "drop_random": base_p - p_r})
    return out


# --------------------------------------------------------------------------- R.4
def analyze_r4(c) -> Dict:
    """Layer balance: attention vs knowledge output norm per layer, averaged over the sample."""
    a_sum, k_sum, n = None, None, 0
    for ids in c.batches():
        g = I.analysis_forward(c.model, ids, mode="light")
        a, k = g["attn_out_norm"].float(), g["know_out_norm"].float()
        a_sum = a if a_sum is None else a_sum + a
        k_sum = k if k_sum is None else k_sum + k
        n += 1
    a, k = a_sum / n, k_sum / n
    ratio = a / (a + k).clamp(min=1e-12)
    return {"attn_out_norm": a.tolist(), "know_out_norm": k.tolist(), "attn_share": ratio.tolist(),
            "attn_share_mean": float(ratio.mean()), "batches": n}


# --------------------------------------------------------------------------- P1
def analyze_rw_proj(c) -> Dict:
    """Read / write vectors against the token embeddings: which tokens a unit reads from and
    writes towards (cosine with the unit-normed embedding table)."""
    emb = _unit(c.model.token_emb.weight.float())
    cnt = _sel_counts(c)
    freq = {"qk": (cnt["Q"] + cnt["K"]).sum(0), "v": cnt["V"].sum(0), "know": cnt["Know"].sum(0)}
    tok = tokenizer_or_none()
    out = {}
    for name in ("qk", "v", "know"):
        rd, wr = _unit(_pool(c, name, "read")), _unit(_pool(c, name, "write"))
        n = rd.shape[0]
        units = torch.topk(freq[name][:n], min(8, n)).indices
        recs, best_r, best_w = [], [], []
        for chunk in torch.split(torch.arange(n, device=c.device), 4096):
            best_r.append((rd[chunk] @ emb.t()).max(-1).values)
            best_w.append((wr[chunk] @ emb.t()).max(-1).values)
        for u in units.tolist():
            tr = torch.topk(rd[u] @ emb.t(), 5)
            tw = torch.topk(wr[u] @ emb.t(), 5)
            rec = {"unit": u, "read_tokens": tr.indices.tolist(), "read_cos": tr.values.tolist(),
                   "write_tokens": tw.indices.tolist(), "write_cos": tw.values.tolist()}
            if tok is not None and tok.vocab_size == emb.shape[0]:
                rec["read_text"] = tok.convert_ids_to_tokens(tr.indices.tolist())
                rec["write_text"] = tok.convert_ids_to_tokens(tw.indices.tolist())
            recs.append(rec)
        out[name] = {"most_used_units": recs, "mean_best_read_cos": float(torch.cat(best_r).mean()),
                     "mean_best_write_cos": float(torch.cat(best_w).mean())}
    return out


# --------------------------------------------------------------------------- P2
def analyze_act_context(c) -> Dict:
    """Contexts in which the most-used knowledge units open most strongly (middle layer): the
    token and its neighbours on both sides."""
    g, ids = c.gates(), c.batches()[0]
    raw = g["gate_Know_raw"][_mid(c)].float()                              # [B,S,N]
    cnt = (raw > 0).float().sum(dim=(0, 1))
    tok = tokenizer_or_none()
    B, S = ids.shape
    out = []
    for u in torch.topk(cnt, min(5, cnt.numel())).indices.tolist():
        flat = torch.topk(raw[..., u].flatten(), min(5, B * S)).indices
        ctxs = []
        for f in flat.tolist():
            b, s = divmod(f, S)
            win = ids[b, max(0, s - 4): s + 3].tolist()
            rec = {"gate": float(raw[b, s, u]), "position": s, "window_ids": win}
            if tok is not None and tok.vocab_size == c.cfg.model.vocab_size:
                rec["window_text"] = tok.decode(win)
            ctxs.append(rec)
        out.append({"unit": u, "selected_by_tokens": int(cnt[u]), "contexts": ctxs})
    return {"layer": _mid(c), "units": out}


# --------------------------------------------------------------------------- P5
def analyze_gate_mech(c) -> Dict:
    """Gate mechanics per route and layer: the denominator (sum of gate values) and how often
    its floor of 1 is active, the share of the gate mass held by the strongest unit, and the
    mean positive gate value."""
    g = c.gates()
    out = {}
    for r in ROUTES:
        raw = g[f"gate_{r}_raw"].float()                                   # [L,B,S,N]
        den = raw.sum(-1)
        pos = raw > 0
        out[r] = {"den_mean": den.mean(dim=(1, 2)).tolist(), "den_min": den.amin(dim=(1, 2)).tolist(),
                  "den_floor_active_frac": (den < 1.0).float().mean(dim=(1, 2)).tolist(),
                  "top1_share": (raw.max(-1).values / den.clamp(min=1e-9)).mean(dim=(1, 2)).tolist(),
                  "mean_positive_gate": (raw.sum(dim=(1, 2, 3)) / pos.float().sum(dim=(1, 2, 3)).clamp(min=1.0)).tolist(),
                  "tokens_with_no_active_unit": (pos.sum(-1) == 0).float().mean(dim=(1, 2)).tolist()}
    return out


# --------------------------------------------------------------------------- P6
def _effective_rank(mat: torch.Tensor) -> float:
    sv = torch.linalg.svdvals(mat.double().cpu())
    p = sv / sv.sum().clamp(min=1e-30)
    return float(torch.exp(-(p * torch.log(p.clamp(min=1e-30))).sum()))


def analyze_comp_expr(c) -> Dict:
    """Compositional expressiveness: effective rank of the write vectors a token's active set
    spans (middle layer, sampled tokens) against the size of the set."""
    g = c.gates()
    raw = g["gate_Know_raw"][_mid(c)].float()
    B, S, N = raw.shape
    wr = _unit(_pool(c, "know", "write"))
    gen = torch.Generator(device="cpu").manual_seed(0)
    n_samples = min(getattr(c.args, "p6_samples", 32), B * S)
    idx = torch.randperm(B * S, generator=gen)[:n_samples].tolist()
    sizes, ranks, wranks = [], [], []
    for f in idx:
        b, s = divmod(f, S)
        gt = raw[b, s, : wr.shape[0]]
        act = torch.nonzero(gt > 0).flatten()
        if act.numel() < 2:
            continue
        act = act[torch.topk(gt[act], min(512, act.numel())).indices]
        sizes.append(int((gt > 0).sum()))
        ranks.append(_effective_rank(wr[act]))
        wranks.append(_effective_rank(wr[act] * gt[act, None]))
    if not sizes:
        return {"samples": 0}
    mean = lambda v: float(sum(v) / len(v))
    return {"layer": _mid(c), "samples": len(sizes), "active_set_size_mean": mean(sizes),
            "effective_rank_mean": mean(ranks), "gate_weighted_effective_rank_mean": mean(wranks),
            "rank_over_dim": mean(ranks) / wr.shape[1]}


# --------------------------------------------------------------------------- P7
def _kmeans(x: torch.Tensor, k: int, iters: int = 20, seed: int = 0):
    gen = torch.Generator(device="cpu").manual_seed(seed)
    cent = x[torch.randperm(x.shape[0], generator=gen)[:k].to(x.device)].clone()
    for _ in range(iters):
        lab = (x @ cent.t()).argmax(-1)
        for j in range(k):
            m = lab == j
            if m.any():
                cent[j] = _unit(x[m].mean(0, keepdim=True))[0]
    return (x @ cent.t()).argmax(-1), cent


def analyze_neuron_cluster(c) -> Dict:
    """Clusters of the knowledge units in embedding / read / write space (spherical k-means on
    a sample) and whether units of one cluster fire together (co-activation within vs across)."""
    g = c.gates()
    act = (g["gate_Know_raw"][_mid(c)] > 0).float().flatten(0, 1)          # [T,N]
    n = _pool(c, "know", "emb").shape[0]
    gen = torch.Generator(device="cpu").manual_seed(0)
    sample = torch.randperm(n, generator=gen)[: min(n, 4096)].to(c.device)
    k = max(2, min(16, sample.numel() // 8))
    a = act[:, sample]
    freq = a.mean(0)
    co = (a.t() @ a) / a.shape[0]                                          # P(i and j)
    lift = co / (freq[:, None] * freq[None, :]).clamp(min=1e-9)
    out = {"layer": _mid(c), "units_sampled": int(sample.numel()), "k": k}
    eye = torch.eye(sample.numel(), dtype=torch.bool, device=c.device)
    for kind in ("emb", "read", "write"):
        x = _unit(_pool(c, "know", kind)[sample])
        lab, cent = _kmeans(x, k)
        same = (lab[:, None] == lab[None, :]) & ~eye
        valid = (freq[:, None] > 0) & (freq[None, :] > 0) & ~eye
        out[kind] = {"cluster_sizes": torch.bincount(lab, minlength=k).tolist(),
                     "mean_cos_to_centroid": float((x * cent[lab]).sum(-1).mean()),
                     "coactivation_lift_within": float(lift[same & valid].mean()) if (same & valid).any() else None,
                     "coactivation_lift_across": float(lift[~same & valid].mean()) if (~same & valid).any() else None}
    return out


# --------------------------------------------------------------------------- P8 + P9
def analyze_deep(c) -> Dict:
    """Corrective units (cos(read, write) < -0.5, which subtract what they read) against the
    rest: how much of the selection and of the gate mass they take per layer."""
    g = c.gates()
    rd, wr = _pool(c, "know", "read"), _pool(c, "know", "write")
    cos = torch.nn.functional.cosine_similarity(rd, wr, dim=-1)
    n = cos.numel()
    groups = {"corrective": cos < -0.5, "neutral": (cos >= -0.5) & (cos <= 0.5), "amplifying": cos > 0.5}
    raw = g["gate_Know_raw"][..., :n].float()                              # [L,B,S,n]
    sel = (raw > 0).float()
    out = {"units": {k: int(v.sum()) for k, v in groups.items()}, "per_layer": {}}
    tot_sel = sel.sum(dim=(1, 2, 3)).clamp(min=1.0)
    tot_mass = raw.sum(dim=(1, 2, 3)).clamp(min=1e-9)
    for k, m in groups.items():
        out["per_layer"][k] = {
            "selection_share": (sel[..., m].sum(dim=(1, 2, 3)) / tot_sel).tolist(),
            "gate_mass_share": (raw[..., m].sum(dim=(1, 2, 3)) / tot_mass).tolist()}
    out["cos_mean"] = float(cos.mean())
    return out


# --------------------------------------------------------------------------- P10
def _know_router_h(c, ids):
    m = c.model
    be = I._be(m, c.device)
    B, S = ids.shape
    x = be.embed(ids, m.token_emb.weight, m.pos_emb.weight).float()
    blk = m.layers[0]
    n1 = be.layer_norm(x, blk.norm1.weight, blk.norm1.bias).reshape(B * S, m.d_model)
    return be.linear(n1, m.router.proj_know.weight, m.router.proj_know.bias).float()


def analyze_op_space(c) -> Dict:
    """Operation space: diversity of the router projections h (participation ratio), uniqueness
    of the tokens' active sets, geometry of the unit embeddings and superposition (units per
    dimension of the routing space)."""
    g, ids = c.gates(), c.batches()[0]
    h = _know_router_h(c, ids)
    hc = h - h.mean(0, keepdim=True)
    ev = torch.linalg.eigvalsh((hc.t() @ hc / hc.shape[0]).double().cpu()).clamp(min=0)
    act = g["gate_Know_raw"][_mid(c)] > 0
    sets = Counter(hash(row.nonzero().flatten().cpu().numpy().tobytes()) for row in act.flatten(0, 1))
    emb = _unit(_pool(c, "know", "emb"))
    gen = torch.Generator(device="cpu").manual_seed(0)
    idx = torch.randperm(emb.shape[0], generator=gen)[: min(emb.shape[0], 2048)].to(c.device)
    sim = emb[idx] @ emb[idx].t()
    off = sim[~torch.eye(idx.numel(), dtype=torch.bool, device=c.device)]
    return {"h_participation_ratio": float(ev.sum() ** 2 / ev.square().sum().clamp(min=1e-30)),
            "d_route": int(h.shape[1]),
            "unique_active_sets_frac": len(sets) / max(1, sum(sets.values())),
            "emb_abs_cos_mean": float(off.abs().mean()), "emb_abs_cos_p99": float(torch.quantile(off.abs().float(), 0.99)),
            "units_per_route_dim": emb.shape[0] / emb.shape[1]}


# --------------------------------------------------------------------------- P12
def analyze_compose(c) -> Dict:
    """Composition of the knowledge output (first layer): contributions of corrective
    (cos(r, w) < -0.5), neutral and amplifying units to the un-normalised output, as norms and
    as cosine with the full output."""
    m, ids = c.model, c.batches()[0]
    be = I._be(m, c.device)
    B, S = ids.shape
    x = be.embed(ids, m.token_emb.weight, m.pos_emb.weight).float()
    n2 = be.layer_norm(x, m.layers[0].norm2.weight, m.layers[0].norm2.bias).reshape(B * S, m.d_model).float()
    rd, wr = _pool(c, "know", "read"), _pool(c, "know", "write")
    if m.gate.normalize_pool:
        rd, wr = _unit(rd), _unit(wr)
    n = rd.shape[0]
    gate = c.gates()["gate_Know_raw"][0].flatten(0, 1)[:, :n].float()       # first layer, [T,n]
    p = gate * (n2 @ rd.t())
    cos_rw = torch.nn.functional.cosine_similarity(_pool(c, "know", "read"), _pool(c, "know", "write"), dim=-1)
    full = p @ wr
    groups = {"corrective": cos_rw < -0.5, "neutral": (cos_rw >= -0.5) & (cos_rw <= 0.5),
              "amplifying": cos_rw > 0.5}
    out = {"full_norm": float(torch.linalg.vector_norm(full, dim=-1).mean())}
    for k, msk in groups.items():
        part = p[:, msk] @ wr[msk]
        out[k] = {"units": int(msk.sum()), "norm": float(torch.linalg.vector_norm(part, dim=-1).mean()),
                  "cos_with_full": float(torch.nn.functional.cosine_similarity(part, full, dim=-1).nan_to_num().mean()),
                  "cos_with_input": float(torch.nn.functional.cosine_similarity(part, n2, dim=-1).nan_to_num().mean())}
    return out


# --------------------------------------------------------------------------- phase
def _load_log(path: str) -> List[Dict]:
    rows = []
    with open(path) as f:
        first = f.readline()
        f.seek(0)
        if first.lstrip().startswith("{"):
            for line in f:
                line = line.strip()
                if line:
                    rec = json.loads(line)
                    if rec.get("type", "train") in ("train", "train_analysis"):
                        rows.append(rec)
        else:
            import csv
            for rec in csv.DictReader(f):
                rows.append({k: float(v) if v not in ("", None) else None for k, v in rec.items()})
    return sorted(rows, key=lambda r_: r_.get("step", 0))


def analyze_phase(c) -> Dict:
    """Phase dynamics from training logs (metrics JSONL of this framework or CSV): loss, active
    fraction and tau series, the step where the loss curve crosses a baseline run's, and the
    steepest change of the knowledge-pool active fraction as the phase boundary."""
    path = getattr(c.args, "dawn_log", None)
    if not path or not os.path.exists(path):
        return {"skipped": "pass --dawn-log (and optionally --baseline-log) with training metrics"}
    rows = _load_log(path)
    if not rows:
        return {"skipped": f"no training records in {path}"}
    series = lambda key: [(r_["step"], r_[key]) for r_ in rows if r_.get(key) is not None and "step" in r_]
    loss = series("ce_loss") or series("loss") or series("total_loss")
    act = series("know_active")
    tau = series("know_tau_mean")
    out = {"records": len(rows), "first_step": rows[0].get("step"), "last_step": rows[-1].get("step"),
           "final_loss": loss[-1][1] if loss else None}
    if len(act) >= 3:
        d = [(act[i + 1][1] - act[i][1]) / max(act[i + 1][0] - act[i][0], 1) for i in range(len(act) - 1)]
        j = max(range(len(d)), key=lambda i: abs(d[i]))
        out["phase_boundary_step"] = act[j + 1][0]
        out["know_active_start_end"] = [act[0][1], act[-1][1]]
    if tau:
        out["know_tau_start_end"] = [tau[0][1], tau[-1][1]]
    base = getattr(c.args, "baseline_log", None)
    if base and os.path.exists(base) and loss:
        brow = _load_log(base)
        bl = [(r_["step"], r_.get("ce_loss", r_.get("loss", r_.get("total_loss")))) for r_ in brow if "step" in r_]
        bl = [(s, v) for s, v in bl if v is not None]
        cross = None
        for s, v in loss:
            prev = [bv for bs, bv in bl if bs <= s]
            if prev and v < prev[-1]:
                cross = s
                break
        out["crossover_step"] = cross
        if cross is not None and out["last_step"]:
            out["crossover_frac_of_run"] = cross / out["last_step"]
    return out


# --------------------------------------------------------------------------- combo
def analyze_combo(c) -> Dict:
    """Combinatorial coverage: number of distinct active sets over the sample (per route, middle
    layer), how often sets repeat and the entropy of the reuse distribution."""
    g = c.gates()
    out = {"layer": _mid(c)}
    for r in ROUTES:
        act = (g[f"gate_{r}_raw"][_mid(c)] > 0).flatten(0, 1)
        cnt = Counter(hash(row.nonzero().flatten().cpu().numpy().tobytes()) for row in act)
        n = sum(cnt.values())
        probs = torch.tensor([v / n for v in cnt.values()], dtype=torch.float64)
        out[r] = {"tokens": n, "unique_sets": len(cnt), "unique_frac": len(cnt) / max(n, 1),
                  "most_common_share": max(cnt.values()) / max(n, 1),
                  "reuse_entropy_bits": float(-(probs * torch.log2(probs)).sum()),
                  "max_entropy_bits": math.log2(max(n, 1))}
    return out


# --------------------------------------------------------------------------- dom_supp
def analyze_dom_supp(c) -> Dict:
    """Domain suppression: for every token class (the reference uses text domains) suppress the
    knowledge units most selective for it at several levels and compare the loss increase on
    that class with the increase on the other classes and with random suppression; the
    selectivity index is (delta_in - delta_out) / (delta_in + delta_out)."""
    g, ids = c.gates(), c.batches()[0]
    m = c.model
    cls, names = _token_classes(c, ids)
    act = (g["gate_Know_raw"][_mid(c)] > 0).float()
    p_act = act.mean(dim=(0, 1)).clamp(min=1e-9)
    n_rows = m.neuron_pool.know_emb.shape[0]
    levels = [float(x) for x in str(getattr(c.args, "dom_supp_levels", "0.01,0.05")).split(",")]

    def class_losses(logits):
        lp = torch.log_softmax(logits[:, :-1].float(), -1)
        nll = -lp.gather(-1, ids[:, 1:].unsqueeze(-1)).squeeze(-1)
        tgt_cls = cls[:, 1:]
        return [float(nll[tgt_cls == k].mean()) if (tgt_cls == k).any() else float("nan") for k in range(len(names))]
    base = class_losses(g["logits"])
    gen = torch.Generator(device="cpu").manual_seed(0)
    out = {"classes": names, "baseline_loss": base, "results": []}
    for k, nm in enumerate(names):
        msk = cls == k
        if not msk.any():
            continue
        sel = act[msk].mean(0) / p_act
        for frac in levels:
            kk = max(1, int(frac * sel.numel()))
            mask = torch.zeros(n_rows, dtype=torch.bool, device=c.device)
            mask[torch.topk(sel, kk).indices] = True
            rnd = torch.zeros_like(mask)
            rnd[torch.randperm(sel.numel(), generator=gen)[:kk].to(c.device)] = True
            lt = class_losses(I.build_suppressed_forward(m, {"know": mask})(ids))
            lr = class_losses(I.build_suppressed_forward(m, {"know": rnd})(ids))
            d_in = lt[k] - base[k]
            others = [lt[j] - base[j] for j in range(len(names)) if j != k and not math.isnan(lt[j])]
            d_out = sum(others) / max(len(others), 1)
            den = abs(d_in) + abs(d_out)
            out["results"].append({"class": nm, "frac": frac, "k": kk, "delta_in": d_in, "delta_out": d_out,
                                   "delta_in_random": lr[k] - base[k],
                                   "selectivity_index": (d_in - d_out) / den if den > 0 else 0.0})
    return out


# --------------------------------------------------------------------------- rw_func
def analyze_rw_func(c) -> Dict:
    """cos(read, write) of the knowledge units in ten bins against what the units do: selection
    frequency, mean gate value when selected and share of the gate mass."""
    g = c.gates()
    cos = torch.nn.functional.cosine_similarity(_pool(c, "know", "read"), _pool(c, "know", "write"), dim=-1)
    n = cos.numel()
    raw = g["gate_Know_raw"][..., :n].float()
    sel = (raw > 0).float().sum(dim=(0, 1, 2))
    mass = raw.sum(dim=(0, 1, 2))
    edges = torch.linspace(float(cos.min()) - 1e-3, float(cos.max()) + 1e-3, 11, device=cos.device)
    which = torch.bucketize(cos, edges[1:-1])
    bins = []
    for b in range(10):
        m = which == b
        if not m.any():
            bins.append({"lo": float(edges[b]), "hi": float(edges[b + 1]), "units": 0})
            continue
        bins.append({"lo": float(edges[b]), "hi": float(edges[b + 1]), "units": int(m.sum()),
                     "selection_freq_mean": float(sel[m].mean()),
                     "mean_gate_when_selected": float(mass[m].sum() / sel[m].sum().clamp(min=1.0)),
                     "gate_mass_share": float(mass[m].sum() / mass.sum().clamp(min=1e-9))})
    rec = {"bins": bins}
    if float(sel.std(unbiased=False)) > 0 and float(cos.std(unbiased=False)) > 0:
        rec["corr_cos_vs_selection_freq"] = float(torch.corrcoef(torch.stack([cos, sel]))[0, 1])
    return rec


# --------------------------------------------------------------------------- tau_grad
def analyze_tau_grad(c) -> Dict:
    """Gradient that reaches the tau heads from the task loss against the one from the
    auxiliary (load-balance / tau regulariser) loss: Frobenius norms per batch and their ratio."""
    m = c.model
    heads = [m.router.tau_attn.weight, m.router.tau_attn.bias, m.router.tau_know.weight, m.router.tau_know.bias]
    was_training = m.training
    m.eval()
    task, aux = [], []
    with torch.enable_grad():
        for ids in c.batches()[: max(1, min(2, len(c.batches())))]:
            for which, store in (("loss", task), ("aux_loss", aux)):
                res = m(ids, labels=ids, want_diag=False, deterministic=True)
                val = res[which]
                grads = torch.autograd.grad(val, heads, allow_unused=True) if val.requires_grad else [None] * 4
                sq = sum(float(g_.float().square().sum()) for g_ in grads if g_ is not None)
                store.append(math.sqrt(sq))
    m.train(was_training)
    tn, an = sum(task) / len(task), sum(aux) / len(aux)
    return {"task_tau_grad_norm": tn, "aux_tau_grad_norm": an, "ratio_task_over_aux": tn / (an + 1e-12),
            "per_batch": {"task": task, "aux": aux}}


EXTRA_ANALYSES = {
    "r1": analyze_r1, "r2": analyze_r2, "r3": analyze_r3, "r4": analyze_r4, "r5": analyze_r5,
    "rw_proj": analyze_rw_proj, "act_context": analyze_act_context, "gate_mech": analyze_gate_mech,
    "comp_expr": analyze_comp_expr, "neuron_cluster": analyze_neuron_cluster, "deep": analyze_deep,
    "op_space": analyze_op_space, "compose": analyze_compose, "phase": analyze_phase,
    "combo": analyze_combo, "dom_supp": analyze_dom_supp, "rw_func": analyze_rw_func,
    "tau_grad": analyze_tau_grad,
}
NEEDS_GRAD = {"tau_grad"}
