"""Dense pre-LayerNorm Transformer baseline with the same result-dict interface
as DAWN (``aux_loss`` = 0).

Reference: models/baseline_transformer_jax.py:19-184 — Q/K/V projections with
bias, O projection without, FFN Dense -> GELU -> dropout -> Dense, tied
embedding cross entropy.  Flax layer names ``layer_<i>`` map to
``layers.<i>``; ``ffn/Dense_0|1`` map to ``ffn.w_up|w_down``.
"""
from __future__ import annotations

import math
from typing import Any, Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint as ckpt

from ..ops.backend import default_backend
from ..parallel.fsdp import sharded_linear
from .dawn import _LN


class StandardAttention(nn.Module):
    def __init__(self, d_model, n_heads):
        super().__init__()
        self.n_heads = n_heads
        self.q_proj = nn.Linear(d_model, d_model)
        self.k_proj = nn.Linear(d_model, d_model)
        self.v_proj = nn.Linear(d_model, d_model)
        self.o_proj = nn.Linear(d_model, d_model, bias=False)


class StandardFFN(nn.Module):
    def __init__(self, d_model, d_ff):
        super().__init__()
        self.w_up = nn.Linear(d_model, d_ff)
        self.w_down = nn.Linear(d_ff, d_model)


class TransformerLayer(nn.Module):
    def __init__(self, d_model, n_heads, d_ff):
        super().__init__()
        self.attn = StandardAttention(d_model, n_heads)
        self.ffn = StandardFFN(d_model, d_ff)
        self.norm1 = _LN(d_model)
        self.norm2 = _LN(d_model)


class VanillaTransformer(nn.Module):
    version = "baseline"

    def __init__(self, vocab_size=30522, d_model=384, d_ff=1536, n_layers=12, n_heads=6,
                 max_seq_len=512, dropout_rate=0.1, gradient_checkpointing=False, seed=0,
                 backend=None):
        super().__init__()
        self.vocab_size, self.d_model, self.d_ff = vocab_size, d_model, d_ff
        self.n_layers, self.n_heads, self.max_seq_len = n_layers, n_heads, max_seq_len
        self.dropout_rate = dropout_rate
        self.gradient_checkpointing = gradient_checkpointing
        self.token_emb = nn.Embedding(vocab_size, d_model)
        self.pos_emb = nn.Embedding(max_seq_len, d_model)
        self.layers = nn.ModuleList([TransformerLayer(d_model, n_heads, d_ff) for _ in range(n_layers)])
        self.norm = _LN(d_model)
        self.backend = backend
        gen = torch.Generator().manual_seed(seed)
        nn.init.normal_(self.token_emb.weight, std=0.02, generator=gen)
        nn.init.normal_(self.pos_emb.weight, std=0.02, generator=gen)
        for m in self.modules():
            if isinstance(m, nn.Linear):
                nn.init.normal_(m.weight, std=1.0 / math.sqrt(m.in_features), generator=gen)
                if m.bias is not None:
                    nn.init.zeros_(m.bias)

    def get_config(self):
        return {"model_version": "baseline", "vocab_size": self.vocab_size, "d_model": self.d_model,
                "d_ff": self.d_ff, "n_layers": self.n_layers, "n_heads": self.n_heads,
                "max_seq_len": self.max_seq_len}

    def get_model_info(self):
        return [f"VanillaTransformer: d_model={self.d_model}, d_ff={self.d_ff}, "
                f"n_layers={self.n_layers}, n_heads={self.n_heads}"]

    def set_parallel(self, **kw):
        pass

    def _backend(self, device):
        if self.backend is None:
            self.backend = default_backend(device)
        return self.backend

    def _layer(self, be, x, lyr, training):
        B, S, D = x.shape
        H = self.n_heads
        n = be.layer_norm(x, lyr.norm1.weight, lyr.norm1.bias).reshape(B * S, D)
        heads = lambda t: t.reshape(B, S, H, D // H).transpose(1, 2)
        a = lyr.attn
        lin = lambda t, layer: sharded_linear(be, t, layer)     # gathers row-sharded weights
        q = heads(lin(n, a.q_proj))
        k = heads(lin(n, a.k_proj))
        v = heads(lin(n, a.v_proj))
        o = be.attention(q, k, v, self.dropout_rate, training).transpose(1, 2).reshape(B * S, D)
        x = x + lin(o, a.o_proj).reshape(B, S, D)
        n = be.layer_norm(x, lyr.norm2.weight, lyr.norm2.bias).reshape(B * S, D)
        hdn = F.gelu(lin(n, lyr.ffn.w_up), approximate="tanh")
        hdn = be.dropout(hdn, self.dropout_rate, training)
        return x + lin(hdn, lyr.ffn.w_down).reshape(B, S, D)

    def forward(self, input_ids, labels=None, attention_mask=None, *, want_diag=False,
                deterministic: Optional[bool] = None) -> Dict[str, Any]:
        training = self.training if deterministic is None else (not deterministic)
        if self.backend is None:
            self.backend = default_backend(input_ids.device)
        be = self.backend
        x = be.embed(input_ids, self.token_emb.weight, self.pos_emb.weight)
        x = be.dropout(x, self.dropout_rate, training)
        for lyr in self.layers:
            if self.gradient_checkpointing and training and torch.is_grad_enabled():
                x = ckpt.checkpoint(self._layer, be, x, lyr, training, use_reentrant=False)
            else:
                x = self._layer(be, x, lyr, training)
        x = be.layer_norm(x, self.norm.weight, self.norm.bias)
        res: Dict[str, Any] = {"aux_loss": x.new_zeros(())}
        if labels is not None:
            loss, per_tok, correct, nvalid, vmask = be.lm_head_ce(x, self.token_emb.weight, labels)
            res.update(loss=loss, correct=correct, valid_count=nvalid)
        else:
            res["logits"] = be.logits(x, self.token_emb.weight)
        return res
