"""DAWN-SRW language model (PyTorch module).

A decoder-only LM whose Q, K, V and feed-forward ("Know") projections are
composed per token from three pools of rank-1 Select-Read-Write units shared
by all layers.  One class covers the three registered gate variants
(``spatial-r1-v3.9.4``, ``-v4.0.1``, ``-v4.1``); the variant is a ``GateSpec``.

Parameter names mirror the reference's Flax tree in dotted form so checkpoints
convert 1:1 (reference: models/dawn_spatial_v41_exp.py:916-976, 1212-1283):

    token_emb.weight [V,D]            pos_emb.weight [max_seq,D]
    neuron_pool.{qk,v,know}_{emb [U,r], read [U,D], write [U,D]}
    neuron_pool.{qk,v,know}_scale [1]                       (absent in v3.9.4)
    router.proj_attn.{weight [3r,D], bias [3r]}  router.proj_know.{weight [r,D], bias}
    router.tau_attn.{weight [3,D], bias [3]}     router.tau_know.{weight [1,D], bias [1]}
    layers.{i}.norm1.{weight,bias}  layers.{i}.norm2.{weight,bias}
    layers.{i}.attn.expand_O.weight [D,D]
    norm.{weight,bias}

Dense weights are stored torch-style ``[out, in]`` (the Flax kernels are
``[in, out]``; the converter transposes).  ``proj_attn`` output is ordered
``[h_Q | h_K | h_V]`` and ``tau_attn`` rows are ``[Q, K, V]``.

Forward (reference: DAWN.__call__ :1285-1692, _attn_forward :983-1139,
_know_forward :1142-1205): embedding -> per layer {LN, router, paired SRW for
Q/K, SRW for V, causal attention, O-proj, residual, LN, SRW on the Know pool,
residual} -> final LN -> tied-embedding CE.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.utils.checkpoint as ckpt

from ..utils.tracing import trace
from ..ops.backend import ParallelCtx, ReferenceBackend, default_backend
from ..ops.gates import GateSpec, gate_spec_for
from ..parallel.topology import PoolShard

POOLS = ("qk", "v", "know")


def _unit_rows(n, d, gen):
    w = torch.randn(n, d, generator=gen, dtype=torch.float32)
    return w / (torch.linalg.vector_norm(w, dim=-1, keepdim=True) + 1e-8)


class NeuronPool(nn.Module):
    """The nine pool tensors + three learnable output scales.  With a
    ``PoolShard`` each rank stores only its (padded) slice of unit rows."""

    def __init__(self, n_qk, n_v, n_know, d_model, d_route, spec: GateSpec,
                 shard: Optional[PoolShard] = None, gen=None, sharded_names=None):
        super().__init__()
        self.sizes = {"qk": n_qk, "v": n_v, "know": n_know}
        self.shard = shard or PoolShard(0, 1)
        # Pools named here are split over the shard group; the others are kept whole on every
        # rank (small pools: no per-layer traffic, one gradient all-reduce per step instead).
        self.sharded_names = set(POOLS if sharded_names is None else sharded_names)
        unknown = self.sharded_names - set(POOLS)
        if unknown:
            raise ValueError(f"unknown pool names {sorted(unknown)}; pools are {POOLS}")
        for name, n in self.sizes.items():
            lo, hi, padded = self.shard_of(name).slice_of(n)
            replicated = self.shard.count > 1 and name not in self.sharded_names
            for kind, dim in (("emb", d_route), ("read", d_model), ("write", d_model)):
                full = _unit_rows(n, dim, gen)
                local = torch.zeros(padded, dim)
                local[: hi - lo] = full[lo:hi]
                prm = nn.Parameter(local)
                if replicated:
                    prm._pool_replicated = True      # gradient: all-reduced over every rank
                self.register_parameter(f"{name}_{kind}", prm)
        if spec.learnable_scale:
            for name in POOLS:
                self.register_parameter(
                    f"{name}_scale", nn.Parameter(torch.full((1,), math.sqrt(d_model))))

    def shard_of(self, name: str) -> PoolShard:
        return self.shard if name in self.sharded_names else PoolShard(0, 1)

    def n_valid(self, name: str) -> int:
        lo, hi, _ = self.shard_of(name).slice_of(self.sizes[name])
        return hi - lo

    def tensors(self, name: str):
        return (getattr(self, f"{name}_emb"), getattr(self, f"{name}_read"),
                getattr(self, f"{name}_write"))


class Router(nn.Module):
    def __init__(self, d_model, d_route, gen=None):
        super().__init__()
        self.proj_attn = nn.Linear(d_model, 3 * d_route)
        self.proj_know = nn.Linear(d_model, d_route)
        self.tau_attn = nn.Linear(d_model, 3)
        self.tau_know = nn.Linear(d_model, 1)
        # Flax Dense default: lecun-normal kernel, zero bias; tau heads start at
        # zero kernel and bias -0.5 (reference :969-976).
        for lin in (self.proj_attn, self.proj_know):
            nn.init.normal_(lin.weight, std=1.0 / math.sqrt(d_model), generator=gen)
            nn.init.zeros_(lin.bias)
        for lin in (self.tau_attn, self.tau_know):
            nn.init.zeros_(lin.weight)
            nn.init.constant_(lin.bias, -0.5)


class _LN(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d))
        self.bias = nn.Parameter(torch.zeros(d))


class AttentionCircuit(nn.Module):
    def __init__(self, d_model, gen=None):
        super().__init__()
        self.expand_O = nn.Linear(d_model, d_model, bias=False)
        nn.init.normal_(self.expand_O.weight, std=0.02, generator=gen)


class DAWNBlock(nn.Module):
    def __init__(self, d_model, gen=None):
        super().__init__()
        self.norm1 = _LN(d_model)
        self.norm2 = _LN(d_model)
        self.attn = AttentionCircuit(d_model, gen)


# how each per-layer metric is folded over layers (default: mean)
_FOLD_MAX = {"qk_emb_norm_max", "v_emb_norm_max", "know_emb_norm_max", "attn_int_max", "know_int_max"}
_FOLD_MIN = {"qk_emb_norm_min", "v_emb_norm_min", "know_emb_norm_min"}


class DAWN(nn.Module):
    def __init__(self, vocab_size=30522, d_model=384, n_layers=12, n_heads=6, max_seq_len=512,
                 d_route=128, n_qk=1580, n_v=2600, n_know=25200, dropout_rate=0.1,
                 router_dropout=0.1, gradient_checkpointing=False,
                 model_version="spatial-r1-v4.1", gate: Optional[GateSpec] = None,
                 pool_shard: Optional[PoolShard] = None, seed: int = 0, backend=None,
                 sharded_pools=None):
        super().__init__()
        if d_model % n_heads != 0:
            raise ValueError(f"d_model ({d_model}) must be divisible by n_heads ({n_heads})")
        self.version = model_version
        self.gate = gate or gate_spec_for(model_version)
        self.vocab_size, self.d_model, self.n_layers, self.n_heads = vocab_size, d_model, n_layers, n_heads
        self.max_seq_len, self.d_route = max_seq_len, d_route
        self.n_qk, self.n_v, self.n_know = n_qk, n_v, n_know
        self.dropout_rate, self.router_dropout = dropout_rate, router_dropout
        self.gradient_checkpointing = gradient_checkpointing
        gen = torch.Generator().manual_seed(seed)
        self.token_emb = nn.Embedding(vocab_size, d_model)
        self.pos_emb = nn.Embedding(max_seq_len, d_model)
        nn.init.normal_(self.token_emb.weight, std=0.02, generator=gen)
        nn.init.normal_(self.pos_emb.weight, std=0.02, generator=gen)
        self.neuron_pool = NeuronPool(n_qk, n_v, n_know, d_model, d_route, self.gate, pool_shard, gen,
                                      sharded_names=sharded_pools)
        self.router = Router(d_model, d_route, gen)
        self.layers = nn.ModuleList([DAWNBlock(d_model, gen) for _ in range(n_layers)])
        self.norm = _LN(d_model)
        self.backend = backend
        self.shard_group = None       # process group over which pool units are split
        self.dp_group = None          # data-parallel group (LB / dead statistics)
        self.world_group = None       # every rank of the job (replicated pools under sharding)
        self.seq_sharded = False

    # ------------------------------------------------------------------
    def set_parallel(self, shard_group=None, dp_group=None, seq_sharded=False, world_group=None):
        self.shard_group, self.dp_group, self.seq_sharded = shard_group, dp_group, seq_sharded
        self.world_group = world_group

    def _backend(self, device):
        if self.backend is None:
            self.backend = default_backend(device)
        return self.backend

    def get_config(self) -> Dict[str, Any]:
        return {"model_version": self.version, "vocab_size": self.vocab_size,
                "d_model": self.d_model, "n_layers": self.n_layers, "n_heads": self.n_heads,
                "max_seq_len": self.max_seq_len, "d_route": self.d_route,
                "n_qk": self.n_qk, "n_v": self.n_v, "n_know": self.n_know}

    def get_model_info(self) -> List[str]:
        return [f"DAWN v{self.version}: Sense-Read-Write",
                f"  d_model={self.d_model}, d_route={self.d_route}, "
                f"n_layers={self.n_layers}, n_heads={self.n_heads}",
                f"  QK: {self.n_qk}, V: {self.n_v}, Know: {self.n_know}",
                f"  Per neuron: emb[{self.d_route}] + read[{self.d_model}] + write[{self.d_model}]"]

    def pool_scale(self, name: str):
        if self.gate.learnable_scale:
            return getattr(self.neuron_pool, f"{name}_scale")
        return math.sqrt(float(self.d_model))

    def pctx(self, name: str) -> ParallelCtx:
        if self.shard_group is not None and name not in self.neuron_pool.sharded_names:
            # a pool kept whole on every rank: the op runs on this rank's own tokens; its
            # per-unit statistics are averaged over all ranks that see different tokens
            n = self.neuron_pool.sizes[name]
            peers = self.world_group if self.seq_sharded else self.dp_group
            if self.seq_sharded and self.world_group is not None:
                import torch.distributed as dist
                if dist.get_world_size(self.shard_group) == dist.get_world_size(self.world_group):
                    peers = self.shard_group     # same ranks; this group has the peer-memory all-reduce
            return ParallelCtx(shard_group=None, dp_group=peers, n_total=n, n_valid=n,
                               seq_sharded=False)
        return ParallelCtx(shard_group=self.shard_group, dp_group=self.dp_group,
                           n_total=self.neuron_pool.sizes[name],
                           n_valid=self.neuron_pool.n_valid(name), seq_sharded=self.seq_sharded)

    def prepare_pools(self, be):
        return {n: be.prepare_pool(*self.neuron_pool.tensors(n), self.gate, self.pctx(n))
                for n in POOLS}

    # ------------------------------------------------------------------
    def _attn(self, be, x, pools, blk, training, want_diag, m):
        B, S, D = x.shape
        r, H = self.d_route, self.n_heads
        T = B * S
        rt = self.router
        xf = x.reshape(T, D)
        with trace("attn/router"):
            h_all = be.linear(xf, rt.proj_attn.weight, rt.proj_attn.bias)
            h_all = be.dropout(h_all, self.router_dropout, training)
            tau_all = be.linear(xf, rt.tau_attn.weight, rt.tau_attn.bias).float()    # [T,3]
        h_qk = h_all[:, : 2 * r].reshape(T, 2, r)
        h_v = h_all[:, 2 * r:].reshape(T, 1, r)
        qk_scale, v_scale = self.pool_scale("qk"), self.pool_scale("v")
        with trace("attn/srw_qkv"):
            # the paired Q/K call and the V call read the same activations: one group
            res_qk, res_v = be.srw_group(xf, [
                dict(h=h_qk, tau_off=tau_all[:, 0:2], pool=pools["qk"], pctx=self.pctx("qk"),
                     out_scale=qk_scale),
                dict(h=h_v, tau_off=tau_all[:, 2:3], pool=pools["v"], pctx=self.pctx("v"),
                     out_scale=v_scale)], self.gate, want_diag=want_diag)
        Q, K, V = res_qk.route(0), res_qk.route(1), res_v.route(0)
        dh = D // H
        to_heads = lambda t: t.reshape(B, S, H, dh).transpose(1, 2)
        with trace("attn/self_attention"):
            o = be.attention(to_heads(Q), to_heads(K), to_heads(V), self.dropout_rate, training)
            o = o.transpose(1, 2).reshape(T, D)
        with trace("attn/expand_O"):
            out = be.linear(o, blk.attn.expand_O.weight, None)
        out_d = out.reshape(B, S, D)       # dropout is applied with the residual add (_layer)
        tau_relu = torch.relu(tau_all).mean()
        lb = (res_qk.lb + res_v.lb) / 3.0
        if self.gate.tau_reg_in_aux:
            aux, tau_reg = lb + 0.01 * tau_relu, None
        else:
            aux, tau_reg = lb, tau_relu
        if want_diag:
            with torch.no_grad():
                self._attn_diag(m, res_qk, res_v, Q, K, V, o, out, tau_all, dh, qk_scale, v_scale)
        zero = tau_relu.new_zeros(())
        return out_d, (aux, res_qk.dead_penalty + res_v.dead_penalty,
                       tau_all.reshape(B, S, 3), tau_reg if tau_reg is not None else zero)

    def _know(self, be, x, pools, training, want_diag, m):
        B, S, D = x.shape
        T = B * S
        rt = self.router
        xf = x.reshape(T, D)
        with trace("know/router"):
            h = be.linear(xf, rt.proj_know.weight, rt.proj_know.bias)
            h = be.dropout(h, self.router_dropout, training)
            tau = be.linear(xf, rt.tau_know.weight, rt.tau_know.bias).float()         # [T,1]
        k_scale = self.pool_scale("know")
        with trace("know/srw"):
            (res,) = be.srw_group(xf, [dict(h=h.reshape(T, 1, self.d_route), tau_off=tau,
                                            pool=pools["know"], pctx=self.pctx("know"),
                                            out_scale=k_scale)], self.gate, want_diag=want_diag)
        out = res.route(0)
        raw = (out.detach() / k_scale) if want_diag else None     # pre-scale output, diagnostics only
        out_d = out.reshape(B, S, D)       # dropout is applied with the residual add (_layer)
        tau_relu = torch.relu(tau).mean()
        if self.gate.tau_reg_in_aux:
            aux, tau_reg = res.lb + 0.01 * tau_relu, None
        else:
            aux, tau_reg = res.lb, tau_relu
        if want_diag:
            with torch.no_grad():
                self._know_diag(m, res, raw, out, tau)
        zero = tau_relu.new_zeros(())
        return out_d, (aux, res.dead_penalty, tau.reshape(B, S, 1),
                       tau_reg if tau_reg is not None else zero)

    # ---- diagnostics (observational, no grad) ---------------------------
    @staticmethod
    def _rownorm_mean(t):
        return torch.linalg.vector_norm(t.float(), dim=-1).mean()

    def _attn_diag(self, m, rq, rv, Q, K, V, o, out, tau_all, dh, qk_scale, v_scale):
        dq, dv = rq.diag, rv.diag
        if not dq:
            return
        a = m.setdefault
        avg2 = lambda k: (dq[k] + dv[k]) / 2
        m["attn_qk_active"].append(dq["active_frac"].mean())
        m["attn_v_active"].append(dv["active_frac"].mean())
        m["attn_raw_gate_max"].append(torch.maximum(dq["gate_max"].mean(), dv["gate_max"].mean()))
        for src, dst in (("score_std", "attn_score_std"), ("gate_sum", "attn_gate_sum"),
                         ("active_n_mean", "attn_active_n_mean"), ("strong", "attn_strong"),
                         ("tau_abs_mean", "attn_tau_abs_mean"), ("z_lt_075", "attn_z_lt_075"),
                         ("z_lt_030", "attn_z_lt_030"), ("score_skew", "attn_score_skew"),
                         ("active_per_token_std", "attn_active_per_token_std"),
                         ("gate_entropy", "attn_gate_entropy"), ("z_sum", "attn_z_sum"),
                         ("score_kurt", "attn_score_kurt"), ("int_cap_frac", "attn_int_cap_frac")):
            m[dst].append(avg2(src))
        m["attn_qk_phi_binary"].append(dq["phi_binary"])
        m["attn_v_phi_binary"].append(dv["phi_binary"])
        m["attn_qk_z_mean_active"].append(dq["z_mean_active"])
        m["attn_v_z_mean_active"].append(dv["z_mean_active"])
        m["attn_dead_count"].append(dq["dead_count"] + dv["dead_count"])
        m["attn_int_max"].append(torch.maximum(dq["int_max"], dv["int_max"]))
        m["attn_out_norm"].append(self._rownorm_mean(out))
        m["attn_tau_mean"].append(tau_all.mean())
        m["attn_tau_std"].append(tau_all.std(dim=0, unbiased=False))
        m["attn_tau_kernel_norm"].append(torch.sqrt(self.router.tau_attn.weight.float().square().sum() + 1e-12))
        m["attn_qk_raw_norm"].append(self._rownorm_mean(rq.stacked()) / qk_scale)
        m["attn_v_raw_norm"].append(self._rownorm_mean(rv.stacked()) / v_scale)
        qn, kn = self._rownorm_mean(Q.reshape(-1, dh)), self._rownorm_mean(K.reshape(-1, dh))
        m["debug_q_norm"].append(qn)
        m["debug_k_norm"].append(kn)
        m["debug_v_norm"].append(self._rownorm_mean(V.reshape(-1, dh)))
        m["debug_logit_max"].append(qn * kn / math.sqrt(dh))
        m["debug_o_input_norm"].append(self._rownorm_mean(o.reshape(-1, dh)))

    def _know_diag(self, m, res, raw, out, tau):
        d = res.diag
        if not d:
            return
        m["know_active"].append(d["active_frac"].mean())
        m["know_raw_gate_max"].append(d["gate_max"].mean())
        for src, dst in (("score_std", "know_score_std"), ("gate_sum", "know_gate_sum"),
                         ("active_n_mean", "know_active_n_mean"), ("strong", "know_strong"),
                         ("phi_binary", "know_phi_binary"), ("z_mean_active", "know_z_mean_active"),
                         ("tau_abs_mean", "know_tau_abs_mean"), ("z_lt_075", "know_z_lt_075"),
                         ("z_lt_030", "know_z_lt_030"), ("score_skew", "know_score_skew"),
                         ("active_per_token_std", "know_active_per_token_std"),
                         ("gate_entropy", "know_gate_entropy"), ("z_sum", "know_z_sum"),
                         ("score_kurt", "know_score_kurt"), ("dead_count", "know_dead_count"),
                         ("int_max", "know_int_max"), ("int_cap_frac", "know_int_cap_frac")):
            m[dst].append(d[src])
        m["know_raw_out_norm"].append(self._rownorm_mean(raw))
        m["know_out_norm"].append(self._rownorm_mean(out))
        m["know_tau_mean"].append(tau.mean())
        m["know_tau_std"].append(tau.std(unbiased=False))
        m["know_tau_kernel_norm"].append(torch.sqrt(self.router.tau_know.weight.float().square().sum() + 1e-12))

    def _pool_norm_diag(self, res):
        p = self.neuron_pool
        with torch.no_grad():
            for name in POOLS:
                n = p.n_valid(name)
                norms = torch.linalg.vector_norm(getattr(p, f"{name}_emb")[:n].float(), dim=-1)
                key = "know_emb_norm" if name == "know" else f"{name}_emb_norm_mean"
                res[key] = norms.mean()
                res[f"{name}_emb_norm_max"] = norms.max()
                res[f"{name}_emb_norm_min"] = norms.min()
                res[f"{name}_emb_norm_std"] = norms.std(unbiased=False)
            nk = p.n_valid("know")
            res["know_read_norm"] = torch.linalg.vector_norm(p.know_read[:nk].float(), dim=-1).mean()
            res["know_write_norm"] = torch.linalg.vector_norm(p.know_write[:nk].float(), dim=-1).mean()

    # ------------------------------------------------------------------
    def _layer(self, be, x, pools, blk, training, want_diag, m):
        """One block.  Returns the new residual stream and the differentiable
        side outputs (aux, dead penalty, tau offsets, tau_reg) of both halves."""
        normed = be.layer_norm(x, blk.norm1.weight, blk.norm1.bias)
        a_out, a_ex = self._attn(be, normed, pools, blk, training, want_diag, m)
        x = be.dropout_add(x, a_out, self.dropout_rate, training)
        normed = be.layer_norm(x, blk.norm2.weight, blk.norm2.bias)
        k_out, k_ex = self._know(be, normed, pools, training, want_diag, m)
        x = be.dropout_add(x, k_out, self.dropout_rate, training)
        return (x,) + tuple(a_ex) + tuple(k_ex)

    def forward(self, input_ids, labels=None, attention_mask=None, *, want_diag: bool = True,
                deterministic: Optional[bool] = None) -> Dict[str, Any]:
        B, S = input_ids.shape
        if S > self.max_seq_len:
            raise ValueError(f"Sequence length {S} exceeds max_seq_len")
        training = self.training if deterministic is None else (not deterministic)
        be = self._backend(input_ids.device)
        with trace("embed"):
            x = be.embed(input_ids, self.token_emb.weight, self.pos_emb.weight)
            x = be.dropout(x, self.dropout_rate, training)
        with trace("prepare_pools"):
            pools = self.prepare_pools(be)
        from collections import defaultdict
        m: Dict[str, list] = defaultdict(list)
        names = ("attn_aux", "attn_dead_penalty", "attn_tau_offset", "attn_tau_reg",
                 "know_aux", "know_dead_penalty", "know_tau_offset", "know_tau_reg")
        for blk in self.layers:
            if self.gradient_checkpointing and training and torch.is_grad_enabled():
                # diagnostics are appended on the first pass; whatever the
                # recomputation appends later is ignored ([:L] below)
                outs = ckpt.checkpoint(self._layer, be, x, pools, blk, training, want_diag, m,
                                       use_reentrant=False, preserve_rng_state=True)
            else:
                outs = self._layer(be, x, pools, blk, training, want_diag, m)
            x = outs[0]
            for nm, val in zip(names, outs[1:]):
                m[nm].append(val)
        if self.gate.tau_reg_in_aux:
            m.pop("attn_tau_reg"), m.pop("know_tau_reg")
        res: Dict[str, Any] = {}
        L = self.n_layers
        attn_aux = torch.stack(m["attn_aux"][:L])
        know_aux = torch.stack(m["know_aux"][:L])
        res["aux_loss"] = (attn_aux + know_aux).mean()
        res["attn_aux"], res["know_aux"] = attn_aux.mean(), know_aux.mean()
        adp = torch.stack(m["attn_dead_penalty"][:L]).mean()
        kdp = torch.stack(m["know_dead_penalty"][:L]).mean()
        res["attn_dead_penalty"], res["know_dead_penalty"], res["dead_penalty"] = adp, kdp, adp + kdp
        if m["attn_tau_reg"]:
            atr, ktr = torch.stack(m["attn_tau_reg"][:L]), torch.stack(m["know_tau_reg"][:L])
            res["tau_reg"] = (atr + ktr).mean()
            res["attn_tau_reg"], res["know_tau_reg"] = atr.mean(), ktr.mean()
        res["attn_tau_offset"] = torch.stack(m["attn_tau_offset"][:L])     # [L,B,S,3]
        res["know_tau_offset"] = torch.stack(m["know_tau_offset"][:L])     # [L,B,S,1]
        skip = {"attn_aux", "know_aux", "attn_dead_penalty", "know_dead_penalty",
                "attn_tau_reg", "know_tau_reg", "attn_tau_offset", "know_tau_offset"}
        if want_diag:
            with torch.no_grad():
                for k, vals in m.items():
                    if k in skip or not vals:
                        continue
                    st = torch.stack([v.float() for v in vals[:L]])
                    if k in _FOLD_MAX:
                        res[k] = st.max()
                    elif k in _FOLD_MIN:
                        res[k] = st.min()
                    elif k == "attn_tau_std":
                        res[k] = st.mean(dim=0)
                    else:
                        res[k] = st.mean()
                    if k in ("attn_out_norm", "know_out_norm"):
                        res[f"per_layer_{k}"] = st
                self._pool_norm_diag(res)
                res["debug_residual_norm"] = self._rownorm_mean(x)
                res["debug_emb_norm"] = self._rownorm_mean(self.token_emb.weight)
                res["debug_o_proj_norm"] = torch.stack(
                    [torch.linalg.matrix_norm(b.attn.expand_O.weight.float()) for b in self.layers]).mean()
        x = be.layer_norm(x, self.norm.weight, self.norm.bias)
        if labels is not None:
            with trace("lm_head_ce"):
                loss, per_tok, correct, nvalid, vmask = be.lm_head_ce(x, self.token_emb.weight, labels)
            res.update(loss=loss, correct=correct, valid_count=nvalid, per_token_ce=per_tok,
                       valid_mask=vmask)
        else:
            res["logits"] = be.logits(x, self.token_emb.weight)
        return res
