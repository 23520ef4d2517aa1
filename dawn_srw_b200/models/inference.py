"""Inference and analysis API of the SRW models.

Functions (reference: models/dawn_spatial_v41_exp.py — prefill/decode_step
:1772-1957, vectorized_eval :1964-2070, vectorized_neuron_health and
vectorized_weight_analysis :2073-2133, analysis_forward :2136-2243,
build_suppressed_forward :2246-2338):

* ``prefill(model, ids)`` -> ``(logits [B,S,V], cache_K, cache_V, S)`` with
  caches ``[L, B, H, max_seq, d_head]``;
* ``decode_step(model, tok, cache_K, cache_V, length)`` -> ``(logits [B,V],
  cache_K, cache_V, length + 1)``;
* ``generate(model, ids, ...)``: KV-cache sampler with temperature / top-k;
* ``vectorized_eval(model, batches)`` -> ``(avg_loss, ppl, acc %, n_valid)``;
  note its valid mask is ``label > 0`` (pad id 0), unlike training's
  ``label != -100`` — kept as in the reference and documented;
* ``analysis_forward(model, ids, mode)``: per-layer gates ``[L,B,S,N]``
  (normalised; ``mode='full'`` adds raw) and per-layer output norms;
* ``build_suppressed_forward(model, masks)`` -> ``forward_fn(ids) -> logits``
  with per-pool boolean unit masks zeroing gates.  The reference's version of
  this function still evaluates an older gate (z*Phi(z) with sum of z+ as
  denominator) inside its newest model file; here the model's own gate is used;
* ``neuron_health`` / ``weight_analysis``: pool norm statistics, dead counts,
  cosine-similarity and effective-rank summaries.

No dropout, no load-balance terms.  Everything runs through the model's
backend (sm_100a kernels on a GPU, plain torch on CPU).
"""
from __future__ import annotations

import math
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

from ..ops import reference as R
from ..ops.backend import ParallelCtx


def _be(model, device):
    return model._backend(device)


def _pools(model, be):
    """Prepared pools (compute copies, Gram statistics) for inference.  They
    depend only on the pool parameters, so they are kept until a parameter
    changes (its autograd version or storage moves) instead of being rebuilt
    for every decoded token."""
    ps = model.neuron_pool
    key = tuple((p.data_ptr(), p._version, p.device) for p in ps.parameters()) + (id(be),)
    hit = getattr(model, "_inference_pools", None)
    if hit is not None and hit[0] == key:
        return hit[1]
    with torch.no_grad():
        pools = model.prepare_pools(be)
    model._inference_pools = (key, pools)
    return pools


def _srw(model, be, x, h, tau, pools, name, *, return_gates=False, unit_mask=None):
    return be.srw(x, h, tau, pools[name], model.gate, pctx=model.pctx(name), want_diag=False,
                  return_gates=return_gates, unit_mask=unit_mask)


def _layer_qkv(model, be, normed, pools, masks=None, return_gates=False):
    """normed [T,D] -> Q,K,V [T,D] (+ gates)."""
    rt, r = model.router, model.d_route
    T = normed.shape[0]
    h_all = be.linear(normed, rt.proj_attn.weight, rt.proj_attn.bias)
    tau_all = be.linear(normed, rt.tau_attn.weight, rt.tau_attn.bias).float()
    m = masks or {}
    rq = _srw(model, be, normed, h_all[:, :2 * r].reshape(T, 2, r), tau_all[:, 0:2], pools, "qk",
              return_gates=return_gates, unit_mask=m.get("qk"))
    rv = _srw(model, be, normed, h_all[:, 2 * r:].reshape(T, 1, r), tau_all[:, 2:3], pools, "v",
              return_gates=return_gates, unit_mask=m.get("v"))
    qs, vs = model.pool_scale("qk"), model.pool_scale("v")
    return rq.route(0) * qs, rq.route(1) * qs, rv.route(0) * vs, rq, rv


def _know(model, be, normed, pools, masks=None, return_gates=False):
    rt = model.router
    T = normed.shape[0]
    h = be.linear(normed, rt.proj_know.weight, rt.proj_know.bias)
    tau = be.linear(normed, rt.tau_know.weight, rt.tau_know.bias).float()
    res = _srw(model, be, normed, h.reshape(T, 1, model.d_route), tau, pools, "know",
               return_gates=return_gates, unit_mask=(masks or {}).get("know"))
    return res.route(0) * model.pool_scale("know"), res


def _is_dense(model) -> bool:
    return getattr(model, "version", "") == "baseline"


def _dense_layer_cached(model, be, x, lyr, li, cache_k, cache_v, pos0: int, decode: bool):
    """One layer of the dense baseline on x [B,S,D] whose first position is
    ``pos0``; K / V of the new positions are written into the caches
    (reference: vanilla_cached_forward, models/baseline_transformer_jax.py)."""
    import torch.nn.functional as F
    B, S, D = x.shape
    H = model.n_heads
    dh = D // H
    a = lyr.attn
    n = be.layer_norm(x, lyr.norm1.weight, lyr.norm1.bias).reshape(B * S, D)
    heads = lambda t: t.float().reshape(B, S, H, dh).transpose(1, 2)
    q = heads(be.linear(n, a.q_proj.weight, a.q_proj.bias))
    k = heads(be.linear(n, a.k_proj.weight, a.k_proj.bias))
    v = heads(be.linear(n, a.v_proj.weight, a.v_proj.bias))
    cache_k[li, :, :, pos0: pos0 + S] = k
    cache_v[li, :, :, pos0: pos0 + S] = v
    if decode:
        o = R.cached_attention(q, cache_k[li], cache_v[li], pos0 + 1)
    else:
        o = be.attention(q, k, v, 0.0, False)
    o = o.transpose(1, 2).reshape(B * S, D)
    x = x + be.linear(o, a.o_proj.weight, None).reshape(B, S, D)
    n = be.layer_norm(x, lyr.norm2.weight, lyr.norm2.bias).reshape(B * S, D)
    hdn = F.gelu(be.linear(n, lyr.ffn.w_up.weight, lyr.ffn.w_up.bias), approximate="tanh")
    return x + be.linear(hdn, lyr.ffn.w_down.weight, lyr.ffn.w_down.bias).reshape(B, S, D)


def _dense_prefill(model, input_ids):
    B, S = input_ids.shape
    dev = input_ids.device
    be = _be(model, dev)
    L, H, D = model.n_layers, model.n_heads, model.d_model
    cache_k = torch.zeros(L, B, H, model.max_seq_len, D // H, device=dev)
    cache_v = torch.zeros_like(cache_k)
    x = be.embed(input_ids, model.token_emb.weight, model.pos_emb.weight).float()
    for li, lyr in enumerate(model.layers):
        x = _dense_layer_cached(model, be, x, lyr, li, cache_k, cache_v, 0, False)
    x = be.layer_norm(x, model.norm.weight, model.norm.bias)
    return be.logits(x, model.token_emb.weight), cache_k, cache_v, S


def _dense_decode(model, token, cache_k, cache_v, length):
    B = token.shape[0]
    be = _be(model, token.device)
    D = model.d_model
    x = (model.token_emb.weight[token] + model.pos_emb.weight[length]).float().reshape(B, 1, D)
    for li, lyr in enumerate(model.layers):
        x = _dense_layer_cached(model, be, x, lyr, li, cache_k, cache_v, length, True)
    x = be.layer_norm(x, model.norm.weight, model.norm.bias)
    return be.logits(x, model.token_emb.weight)[:, 0], cache_k, cache_v, length + 1


@torch.no_grad()
def prefill(model, input_ids: torch.Tensor):
    B, S = input_ids.shape
    if S > model.max_seq_len:
        raise ValueError(f"Sequence length {S} exceeds max_seq_len")
    if _is_dense(model):
        return _dense_prefill(model, input_ids)
    dev = input_ids.device
    be = _be(model, dev)
    pools = _pools(model, be)
    L, H, D = model.n_layers, model.n_heads, model.d_model
    dh = D // H
    cache_k = torch.zeros(L, B, H, model.max_seq_len, dh, device=dev)
    cache_v = torch.zeros_like(cache_k)
    x = be.embed(input_ids, model.token_emb.weight, model.pos_emb.weight).float()
    heads = lambda t: t.reshape(B, S, H, dh).transpose(1, 2)
    for li, blk in enumerate(model.layers):
        n = be.layer_norm(x, blk.norm1.weight, blk.norm1.bias).reshape(B * S, D)
        q, k, v, _, _ = _layer_qkv(model, be, n, pools)
        qh, kh, vh = heads(q), heads(k), heads(v)
        cache_k[li, :, :, :S] = kh
        cache_v[li, :, :, :S] = vh
        o = be.attention(qh, kh, vh, 0.0, False).transpose(1, 2).reshape(B * S, D)
        x = x + be.linear(o, blk.attn.expand_O.weight, None).reshape(B, S, D)
        n = be.layer_norm(x, blk.norm2.weight, blk.norm2.bias).reshape(B * S, D)
        ko, _ = _know(model, be, n, pools)
        x = x + ko.reshape(B, S, D)
    x = be.layer_norm(x, model.norm.weight, model.norm.bias)
    return be.logits(x, model.token_emb.weight), cache_k, cache_v, S


@torch.no_grad()
def decode_step(model, token: torch.Tensor, cache_k, cache_v, length: int):
    """token [B] (ids of the newest position) -> logits [B,V] for the next one."""
    B = token.shape[0]
    if length >= model.max_seq_len:
        raise ValueError("KV cache is full")
    if _is_dense(model):
        return _dense_decode(model, token, cache_k, cache_v, length)
    dev = token.device
    be = _be(model, dev)
    pools = _pools(model, be)
    H, D = model.n_heads, model.d_model
    dh = D // H
    x = (model.token_emb.weight[token] + model.pos_emb.weight[length]).float().reshape(B, 1, D)
    for li, blk in enumerate(model.layers):
        n = be.layer_norm(x, blk.norm1.weight, blk.norm1.bias).reshape(B, D)
        q, k, v, _, _ = _layer_qkv(model, be, n, pools)
        cache_k[li, :, :, length] = k.reshape(B, H, dh)
        cache_v[li, :, :, length] = v.reshape(B, H, dh)
        o = R.cached_attention(q.reshape(B, H, 1, dh), cache_k[li], cache_v[li], length + 1)
        o = o.reshape(B, D)
        x = x + be.linear(o, blk.attn.expand_O.weight, None).reshape(B, 1, D)
        n = be.layer_norm(x, blk.norm2.weight, blk.norm2.bias).reshape(B, D)
        ko, _ = _know(model, be, n, pools)
        x = x + ko.reshape(B, 1, D)
    x = be.layer_norm(x, model.norm.weight, model.norm.bias)
    return be.logits(x, model.token_emb.weight)[:, 0], cache_k, cache_v, length + 1


def sample_token(logits: torch.Tensor, temperature: float = 1.0, top_k: int = 0,
                 top_p: float = 0.0, generator=None) -> torch.Tensor:
    if temperature <= 0:
        return logits.argmax(-1)
    lg = logits.float() / temperature
    if top_k and top_k < lg.shape[-1]:
        kth = lg.topk(top_k, dim=-1).values[..., -1:]
        lg = lg.masked_fill(lg < kth, float("-inf"))
    if top_p and 0.0 < top_p < 1.0:
        srt, idx = lg.sort(dim=-1, descending=True)
        cum = srt.softmax(-1).cumsum(-1)
        drop = cum - srt.softmax(-1) > top_p
        srt = srt.masked_fill(drop, float("-inf"))
        lg = torch.full_like(lg, float("-inf")).scatter(-1, idx, srt)
    return torch.multinomial(lg.softmax(-1), 1, generator=generator).squeeze(-1)


@torch.no_grad()
def generate(model, input_ids: torch.Tensor, max_new_tokens: int = 32, temperature: float = 1.0,
             top_k: int = 0, top_p: float = 0.0, stop_ids: Iterable[int] = (), generator=None
             ) -> Tuple[torch.Tensor, Dict[str, float]]:
    """KV-cache sampling (reference sampler: scripts/analysis/standalone/
    spatial_analysis.py:444-546).  Returns the full sequences and tokens/s."""
    import time
    model.eval()
    logits, ck, cv, length = prefill(model, input_ids)
    out = [input_ids]
    nxt = sample_token(logits[:, -1], temperature, top_k, top_p, generator)
    stop = set(int(s) for s in stop_ids)
    t0, n = time.perf_counter(), 0
    for _ in range(max_new_tokens):
        out.append(nxt[:, None])
        n += 1
        if length >= model.max_seq_len or (stop and all(int(t) in stop for t in nxt)):
            break
        lg, ck, cv, length = decode_step(model, nxt, ck, cv, length)
        nxt = sample_token(lg, temperature, top_k, top_p, generator)
    if input_ids.is_cuda:
        torch.cuda.synchronize()
    dt = max(time.perf_counter() - t0, 1e-9)
    return torch.cat(out, dim=1), {"new_tokens": n, "tokens_per_sec": n * input_ids.shape[0] / dt}


@torch.no_grad()
def vectorized_eval(model, batches: Iterable[torch.Tensor]):
    """(avg_loss, ppl, accuracy %, n_valid) over ``batches`` of token ids; sums
    stay on the device until the end.  Valid positions are ``label > 0``."""
    model.eval()
    tot = None
    for ids in batches:
        ids = ids.long()
        labels = torch.where(ids > 0, ids, torch.full_like(ids, -100))
        r = model(ids, labels=labels, want_diag=False)
        cur = torch.stack([r["loss"].double() * r["valid_count"], r["correct"].double(),
                           r["valid_count"].double()])
        tot = cur if tot is None else tot + cur
    if tot is None:
        return 0.0, 1.0, 0.0, 0
    loss_sum, correct, valid = tot.tolist()
    avg = loss_sum / max(valid, 1.0)
    return avg, math.exp(min(avg, 50.0)), 100.0 * correct / max(valid, 1.0), int(valid)


@torch.no_grad()
def analysis_forward(model, input_ids: torch.Tensor, mode: str = "light") -> Dict[str, torch.Tensor]:
    """Forward that also returns the gates of every layer.

    ``gate_{Q,K,V,Know}``: [L, B, S, N] gate / sum(gate); with ``mode='full'``
    also ``gate_*_raw``.  ``attn_out_norm`` / ``know_out_norm``: [L]."""
    model.eval()
    B, S = input_ids.shape
    dev = input_ids.device
    be = _be(model, dev)
    pools = _pools(model, be)
    H, D = model.n_heads, model.d_model
    dh = D // H
    x = be.embed(input_ids, model.token_emb.weight, model.pos_emb.weight).float()
    heads = lambda t: t.reshape(B, S, H, dh).transpose(1, 2)
    names = ("Q", "K", "V", "Know")
    norm_g: Dict[str, List] = {n: [] for n in names}
    raw_g: Dict[str, List] = {n: [] for n in names}
    a_norms, k_norms = [], []

    def keep(name, g):                       # g [T, U]
        g = g.reshape(B, S, -1).float()
        norm_g[name].append(g / g.sum(-1, keepdim=True).clamp(min=1e-8))
        if mode == "full":
            raw_g[name].append(g)
    for blk in model.layers:
        n = be.layer_norm(x, blk.norm1.weight, blk.norm1.bias).reshape(B * S, D)
        q, k, v, rq, rv = _layer_qkv(model, be, n, pools, return_gates=True)
        keep("Q", rq.gates[:, 0]); keep("K", rq.gates[:, 1]); keep("V", rv.gates[:, 0])
        o = be.attention(heads(q), heads(k), heads(v), 0.0, False).transpose(1, 2).reshape(B * S, D)
        ao = be.linear(o, blk.attn.expand_O.weight, None)
        a_norms.append(torch.linalg.vector_norm(ao.float(), dim=-1).mean())
        x = x + ao.reshape(B, S, D)
        n = be.layer_norm(x, blk.norm2.weight, blk.norm2.bias).reshape(B * S, D)
        ko, rk = _know(model, be, n, pools, return_gates=True)
        keep("Know", rk.gates[:, 0])
        k_norms.append(torch.linalg.vector_norm(ko.float(), dim=-1).mean())
        x = x + ko.reshape(B, S, D)
    x = be.layer_norm(x, model.norm.weight, model.norm.bias)
    out = {"logits": be.logits(x, model.token_emb.weight),
           "attn_out_norm": torch.stack(a_norms), "know_out_norm": torch.stack(k_norms)}
    for nme in names:
        out[f"gate_{nme}"] = torch.stack(norm_g[nme])
        if mode == "full":
            out[f"gate_{nme}_raw"] = torch.stack(raw_g[nme])
    return out


def build_suppressed_forward(model, masks: Dict[str, torch.Tensor]) -> Callable[[torch.Tensor], torch.Tensor]:
    """``masks``: {'qk' | 'v' | 'know': bool [N]} with True = unit is suppressed.
    Returns ``forward_fn(ids) -> logits`` with those units' gates forced to zero."""
    keep = {k: (~v.bool()).float() for k, v in masks.items()}

    @torch.no_grad()
    def forward_fn(input_ids: torch.Tensor) -> torch.Tensor:
        model.eval()
        B, S = input_ids.shape
        dev = input_ids.device
        be = _be(model, dev)
        pools = _pools(model, be)
        km = {k: v.to(dev) for k, v in keep.items()}
        H, D = model.n_heads, model.d_model
        dh = D // H
        heads = lambda t: t.reshape(B, S, H, dh).transpose(1, 2)
        x = be.embed(input_ids, model.token_emb.weight, model.pos_emb.weight).float()
        for blk in model.layers:
            n = be.layer_norm(x, blk.norm1.weight, blk.norm1.bias).reshape(B * S, D)
            q, k, v, _, _ = _layer_qkv(model, be, n, pools, masks=km)
            o = be.attention(heads(q), heads(k), heads(v), 0.0, False).transpose(1, 2).reshape(B * S, D)
            x = x + be.linear(o, blk.attn.expand_O.weight, None).reshape(B, S, D)
            n = be.layer_norm(x, blk.norm2.weight, blk.norm2.bias).reshape(B * S, D)
            ko, _ = _know(model, be, n, pools, masks=km)
            x = x + ko.reshape(B, S, D)
        x = be.layer_norm(x, model.norm.weight, model.norm.bias)
        return be.logits(x, model.token_emb.weight)
    return forward_fn


@torch.no_grad()
def neuron_health(model, dead_norm: float = 1e-6) -> Dict[str, float]:
    """Norm statistics and dead counts per pool tensor, tau biases."""
    out: Dict[str, float] = {}
    p = model.neuron_pool
    for name in ("qk", "v", "know"):
        n = p.n_valid(name)
        for kind in ("emb", "read", "write"):
            norms = torch.linalg.vector_norm(getattr(p, f"{name}_{kind}")[:n].float(), dim=-1)
            key = f"{name}_{kind}"
            out[f"{key}_norm_mean"] = float(norms.mean())
            out[f"{key}_norm_min"] = float(norms.min())
            out[f"{key}_norm_max"] = float(norms.max())
            out[f"{key}_norm_std"] = float(norms.std(unbiased=False))
            out[f"{key}_dead"] = int((norms < dead_norm).sum())
        if model.gate.learnable_scale:
            out[f"{name}_scale"] = float(getattr(p, f"{name}_scale")[0])
    rt = model.router
    out["tau_know_bias"] = float(rt.tau_know.bias[0])
    for i, nm in enumerate("qkv"):
        out[f"tau_attn_bias_{nm}"] = float(rt.tau_attn.bias[i])
    return out


@torch.no_grad()
def weight_analysis(model, max_rows: int = 2048) -> Dict[str, float]:
    """Cosine-similarity summary (at most ``max_rows`` stride-sampled rows) and
    SVD effective rank (exp of the singular-value entropy) per pool tensor."""
    out: Dict[str, float] = {}
    p = model.neuron_pool
    for name in ("qk", "v", "know"):
        n = p.n_valid(name)
        for kind in ("emb", "read", "write"):
            w = getattr(p, f"{name}_{kind}")[:n].float()
            if w.shape[0] > max_rows:
                w = w[:: w.shape[0] // max_rows][:max_rows]
            u = w / (torch.linalg.vector_norm(w, dim=-1, keepdim=True) + 1e-8)
            sim = u @ u.t()
            m = sim.shape[0]
            off = sim - torch.diag(torch.diagonal(sim))
            key = f"{name}_{kind}"
            out[f"{key}_cos_abs_mean"] = float(off.abs().sum() / (m * m - m))
            out[f"{key}_cos_max"] = float(off.max())
            sv = torch.linalg.svdvals(w.cpu())
            ps = sv / sv.sum()
            out[f"{key}_effective_rank"] = float(torch.exp(-(ps * torch.log(ps + 1e-12)).sum()))
    return out


def estimate_flops_per_token(model, seq_len: Optional[int] = None) -> Dict[str, float]:
    """Forward FLOPs per token (reference estimator: spatial_analysis.py:247-256);
    scores are counted once here (the Gram-matrix statistics need no second pass)."""
    D, r, L, H = model.d_model, model.d_route, model.n_layers, model.n_heads
    S = seq_len or model.max_seq_len
    nq, nv, nk = model.n_qk, model.n_v, model.n_know
    scores = 2 * r * (2 * nq + nv + nk)
    read = 2 * D * (nq + nv + nk)
    write = 2 * D * (2 * nq + nv + nk)
    attn = 4 * S * D / 2 + 2 * D * D
    router = 2 * D * (4 * r + 4)
    per_layer = scores + read + write + attn + router
    head = 2 * D * model.vocab_size
    return {"per_layer": per_layer, "lm_head": head, "total": L * per_layer + head}
