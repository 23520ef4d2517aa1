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


def _fast_infer(model, be) -> bool:
    """Forward-only kernels path: unsharded pools on a backend that has it."""
    return hasattr(be, "srw_infer") and model.shard_group is None


def _layer_qkv(model, be, normed, pools, masks=None, return_gates=False):
    """normed [T,D] -> Q,K,V [T,D] (+ gates)."""
    rt, r = model.router, model.d_route
    T = normed.shape[0]
    m = masks or {}
    if hasattr(be, "linear_cat") and not torch.is_grad_enabled():
        h_all, tau_all = be.linear_cat(normed, (rt.proj_attn, rt.tau_attn))
    else:
        h_all = be.linear(normed, rt.proj_attn.weight, rt.proj_attn.bias)
        tau_all = be.linear(normed, rt.tau_attn.weight, rt.tau_attn.bias).float()
    if not m and not return_gates and _fast_infer(model, be):
        q, k = be.srw_infer(normed, h_all[:, :2 * r].reshape(T, 2, r), tau_all[:, 0:2], pools["qk"],
                            model.gate, n_total=model.n_qk, out_scale=model.pool_scale("qk"))
        (v,) = be.srw_infer(normed, h_all[:, 2 * r:].reshape(T, 1, r), tau_all[:, 2:3], pools["v"],
                            model.gate, n_total=model.n_v, out_scale=model.pool_scale("v"))
        return q, k, v, None, None
    rq = _srw(model, be, normed, h_all[:, :2 * r].reshape(T, 2, r), tau_all[:, 0:2], pools, "qk",
              return_gates=return_gates, unit_mask=m.get("qk"))
    rv = _srw(model, be, normed, h_all[:, 2 * r:].reshape(T, 1, r), tau_all[:, 2:3], pools, "v",
              return_gates=return_gates, unit_mask=m.get("v"))
    qs, vs = model.pool_scale("qk"), model.pool_scale("v")
    return rq.route(0) * qs, rq.route(1) * qs, rv.route(0) * vs, rq, rv


def _know(model, be, normed, pools, masks=None, return_gates=False):
    rt = model.router
    T = normed.shape[0]
    if hasattr(be, "linear_cat") and not torch.is_grad_enabled():
        h, tau = be.linear_cat(normed, (rt.proj_know, rt.tau_know))
    else:
        h = be.linear(normed, rt.proj_know.weight, rt.proj_know.bias)
        tau = be.linear(normed, rt.tau_know.weight, rt.tau_know.bias).float()
    if not masks and not return_gates and _fast_infer(model, be):
        (out,) = be.srw_infer(normed, h.reshape(T, 1, model.d_route), tau, pools["know"], model.gate,
                              n_total=model.n_know, out_scale=model.pool_scale("know"))
        return out, None
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


class DecodeSession:
    """KV-cache decoding with the whole per-token step captured in a CUDA graph.

    One decoded token is about forty small launches per layer (LayerNorm, router
    GEMMs, statistics, three gate kernels, three split-K write GEMMs, cache
    attention, O projection, ...).  At batch 1 the kernels of the 400M model stream
    about 12 GB of pool weights per token, i.e. a couple of milliseconds of HBM
    time, which is less than the time the host needs to issue those launches one
    by one; a graph replays them in one submission.  For that the step must have
    static shapes and addresses: the position is a device scalar (position
    embedding by ``index_select``, cache write by ``index_copy_``, attention over
    the whole cache under a position mask), the token ids arrive in a fixed buffer.

    ``session = DecodeSession(model, cache_k, cache_v, length)`` after ``prefill``;
    ``logits = session.step(tokens)`` per new token.  On CPU, for the dense baseline
    or with ``use_graph=False`` it runs the same step eagerly."""

    def __init__(self, model, cache_k, cache_v, length: int, use_graph: Optional[bool] = None):
        self.model, self.cache_k, self.cache_v = model, cache_k, cache_v
        dev = cache_k.device
        self.B = cache_k.shape[1]
        self.length = int(length)
        self.tok = torch.zeros(self.B, dtype=torch.long, device=dev)
        self.pos = torch.full((1,), self.length, dtype=torch.long, device=dev)
        self.be = _be(model, dev)
        self.pools = None if _is_dense(model) else _pools(model, self.be)
        if use_graph is None:
            use_graph = dev.type == "cuda" and not _is_dense(model) and _fast_infer(model, self.be)
        self.graph, self.out = None, None
        self.use_graph = bool(use_graph)

    @torch.no_grad()
    def _step_static(self):
        m, be, pools = self.model, self.be, self.pools
        B, H, D = self.B, m.n_heads, m.d_model
        dh = D // H
        x = (m.token_emb.weight.index_select(0, self.tok)
             + m.pos_emb.weight.index_select(0, self.pos)).float().reshape(B, 1, D)
        n_valid = self.pos + 1                                   # cache positions in use
        fused_attn = (hasattr(be, "decode_attention") and self.cache_k.is_cuda
                      and self.cache_k.dtype == torch.float32 and self.cache_k[0].is_contiguous()
                      and dh <= 128)
        for li, blk in enumerate(m.layers):
            n = be.layer_norm(x, blk.norm1.weight, blk.norm1.bias).reshape(B, D)
            q, k, v, _, _ = _layer_qkv(m, be, n, pools)
            if fused_attn:
                o = be.decode_attention(q, k, v, self.cache_k[li], self.cache_v[li], self.pos, H)
            else:
                self.cache_k[li].index_copy_(2, self.pos, k.reshape(B, H, 1, dh).to(self.cache_k.dtype))
                self.cache_v[li].index_copy_(2, self.pos, v.reshape(B, H, 1, dh).to(self.cache_v.dtype))
                o = R.cached_attention(q.reshape(B, H, 1, dh), self.cache_k[li], self.cache_v[li], n_valid)
            x = x + be.linear(o.reshape(B, D), blk.attn.expand_O.weight, None).reshape(B, 1, D)
            n = be.layer_norm(x, blk.norm2.weight, blk.norm2.bias).reshape(B, D)
            ko, _ = _know(m, be, n, pools)
            x = x + ko.reshape(B, 1, D)
        x = be.layer_norm(x, m.norm.weight, m.norm.bias)
        return be.logits(x, m.token_emb.weight)[:, 0]

    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B] -> logits [B, V] of the next position."""
        if self.length >= self.model.max_seq_len:
            raise ValueError("KV cache is full")
        if not self.use_graph:
            lg, self.cache_k, self.cache_v, self.length = decode_step(
                self.model, tokens, self.cache_k, self.cache_v, self.length)
            return lg
        self.tok.copy_(tokens)
        self.pos.fill_(self.length)
        if self.graph is None:
            # warm up on a side stream (lazy initialisation must not happen during capture),
            # then capture; the warm-up writes the same cache slot the replay writes again
            side = torch.cuda.Stream(device=self.tok.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._step_static()
            torch.cuda.current_stream().wait_stream(side)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self.out = self._step_static()
        self.graph.replay()
        self.length += 1
        return self.out.clone()


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
             top_k: int = 0, top_p: float = 0.0, stop_ids: Iterable[int] = (), generator=None,
             use_graph: Optional[bool] = None) -> Tuple[torch.Tensor, Dict[str, float]]:
    """KV-cache sampling (reference sampler: scripts/analysis/standalone/
    spatial_analysis.py:444-546).  Returns the full sequences and tokens/s."""
    import time
    model.eval()
    logits, ck, cv, length = prefill(model, input_ids)
    session = DecodeSession(model, ck, cv, length, use_graph=use_graph)
    out = [input_ids]
    nxt = sample_token(logits[:, -1], temperature, top_k, top_p, generator)
    stop = set(int(s) for s in stop_ids)
    sync = torch.cuda.synchronize if input_ids.is_cuda else (lambda: None)
    t0, n, t1 = time.perf_counter(), 0, None
    for _ in range(max_new_tokens):
        out.append(nxt[:, None])
        n += 1
        if session.length >= model.max_seq_len or (stop and all(int(t) in stop for t in nxt)):
            break
        lg = session.step(nxt)
        nxt = sample_token(lg, temperature, top_k, top_p, generator)
        if t1 is None:                 # the first step carries the graph capture
            sync()
            t1 = time.perf_counter()
    sync()
    t2 = time.perf_counter()
    B = input_ids.shape[0]
    stats = {"new_tokens": n, "tokens_per_sec": n * B / max(t2 - t0, 1e-9),
             "first_step_s": (t1 - t0) if t1 is not None else 0.0, "graph": session.use_graph}
    if t1 is not None and n > 2:
        stats["steady_tokens_per_sec"] = (n - 2) * B / max(t2 - t1, 1e-9)
    return torch.cat(out, dim=1), stats


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
