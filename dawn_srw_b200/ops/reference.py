"""Plain-PyTorch reference implementations of every op other than the SRW pool
op (which lives in ``srw_ref.py``).  They define the numerics the CUDA kernels
are tested against and run the model on CPU.

Reference math: LayerNorm eps 1e-6 with population variance
(models/dawn_spatial_v41_exp.py:321-324); causal softmax attention scaled by
sqrt(d_head) (:1055-1071); tied-embedding cross entropy on shifted labels with
``-100`` ignored (:1642-1668); pool diversity loss (scripts/train_jax.py:440-485).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def layer_norm(x, weight, bias, eps: float = 1e-6):
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = (xf - mean).square().mean(-1, keepdim=True)
    return ((xf - mean) / torch.sqrt(var + eps) * weight.float() + bias.float()).to(x.dtype)


def linear(x, weight, bias=None, compute_dtype=None):
    """y = x @ weight^T + bias; weight is [out, in] (torch convention)."""
    if compute_dtype is None or compute_dtype == x.dtype == weight.dtype:
        return F.linear(x, weight, bias)
    y = F.linear(x.to(compute_dtype), weight.to(compute_dtype)).float()
    return y if bias is None else y + bias.float()


def dropout(x, p: float, training: bool):
    """Keep-mask dropout scaled by 1/keep; identity at eval (the reference fixed
    an eval-time 1/keep scaling bug, models/dawn_spatial_v41_exp.py:308-318)."""
    if not training or p == 0.0:
        return x
    return F.dropout(x, p, True)


def embed(ids, tok_emb, pos_emb):
    S = ids.shape[1]
    return tok_emb[ids] + pos_emb[:S].unsqueeze(0)


def causal_attention(q, k, v, dropout_p: float = 0.0, training: bool = False):
    """q,k,v [B,H,S,dh] -> [B,H,S,dh]; full S x S softmax with causal mask."""
    dh = q.shape[-1]
    S = q.shape[-2]
    s = (q.float() @ k.float().transpose(-1, -2)) / math.sqrt(dh)
    causal = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
    s = s.masked_fill(~causal, torch.finfo(torch.float32).min)
    w = torch.softmax(s, dim=-1)
    w = dropout(w, dropout_p, training)
    return (w @ v.float()).to(q.dtype)


def cached_attention(q, cache_k, cache_v, length):
    """Decode-time attention of q [B,H,1,dh] over cache[:, :, :length]."""
    dh = q.shape[-1]
    s = (q.float() @ cache_k.float().transpose(-1, -2)) / math.sqrt(dh)   # [B,H,1,maxS]
    pos = torch.arange(cache_k.shape[2], device=q.device)
    s = s.masked_fill(pos.view(1, 1, 1, -1) >= length, torch.finfo(torch.float32).min)
    return (torch.softmax(s, -1) @ cache_v.float()).to(q.dtype)


def lm_head_ce(x, tok_emb, labels, compute_dtype=None):
    """Tied-logit cross entropy.

    x [B,S,D] (final-normed), labels [B,S] with -100 = ignore.  Positions
    0..S-2 predict labels 1..S-1.  Returns (loss, per_token_ce [B,S-1],
    correct, valid_count, valid_mask)."""
    sx = x[:, :-1, :]
    sl = labels[:, 1:].long()
    valid = sl != -100
    logits = linear(sx, tok_emb, None, compute_dtype).float()
    logp = torch.log_softmax(logits, dim=-1)
    safe = torch.where(valid, sl, torch.zeros_like(sl))
    tl = -logp.gather(-1, safe.unsqueeze(-1)).squeeze(-1)
    per_tok = tl * valid
    loss = per_tok.sum() / (valid.sum() + 1e-8)
    pred = logits.argmax(-1)
    correct = ((pred == sl) & valid).sum()
    return loss, per_tok, correct, valid.sum(), valid


def logits_from_hidden(x, tok_emb, compute_dtype=None):
    return linear(x, tok_emb, None, compute_dtype).float()


def pool_diversity(tensors, max_sample: int = 4096):
    """Mean |cos| between distinct rows, per pool tensor, averaged over tensors.
    Pools larger than ``max_sample`` rows are stride-subsampled."""
    total = 0.0
    for w in tensors:
        n_rows = w.shape[0]
        if n_rows > max_sample:
            stride = n_rows // max_sample
            w = w[::stride][:max_sample]
        n = w.float() / (torch.linalg.vector_norm(w.float(), dim=-1, keepdim=True) + 1e-8)
        sim = n @ n.t()
        m = sim.shape[0]
        off = sim.abs().sum() - sim.diagonal().abs().sum()
        total = total + off / float(m * m - m)
    return total / len(tensors)
