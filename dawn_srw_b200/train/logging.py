"""Run logging: a text log and a JSONL metrics stream, rank 0 only.

Two cadences (reference: scripts/train_jax.py:1303-1623, 2983-3079): REGULAR
records every ``log_interval`` steps (plus steps 1, 5, 10, 20, 50) and ANALYSIS
records every ``log_interval * log_analysis_multiplier`` steps.  JSONL record
types: ``train``, ``train_analysis``, ``val``, ``val_epoch``; key names are the
reference's so downstream log analysis keeps working.
"""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, Iterable, Optional

import torch

EARLY_STEPS = (1, 5, 10, 20, 50)

TRAIN_KEYS = [
    "total_loss", "ce_loss", "aux_loss", "tau_reg", "orth_loss", "div_loss", "aux_weighted",
    "tau_reg_weighted", "orth_weighted", "div_weighted", "dead_penalty", "attn_dead_penalty",
    "know_dead_penalty", "dead_penalty_weighted", "explore_loss_raw", "explore_loss_weighted",
    "accuracy", "grad_norm", "lr", "drift_qk_emb", "drift_v_emb", "drift_know_emb",
    "attn_qk_active", "attn_v_active", "know_active", "attn_strong", "know_strong",
    "attn_raw_gate_max", "know_raw_gate_max", "attn_int_max", "know_int_max", "attn_dead_count",
    "know_dead_count", "attn_tau_mean", "know_tau_mean", "attn_out_norm", "know_out_norm",
    "tau_know_bias", "tau_attn_bias_0", "tau_attn_bias_1", "tau_attn_bias_2", "attn_tau_abs_mean",
    "know_tau_abs_mean", "attn_tau_off_min", "attn_tau_off_max", "attn_tau_off_p99",
    "attn_tau_off_p01", "attn_tau_off_neg_frac", "know_tau_off_min", "know_tau_off_max",
    "know_tau_off_p99", "know_tau_off_p01", "know_tau_off_neg_frac", "attn_score_std",
    "know_score_std", "know_emb_norm", "know_emb_norm_min", "know_emb_norm_std",
    "qk_emb_norm_mean", "qk_emb_norm_min", "qk_emb_norm_std", "v_emb_norm_mean", "v_emb_norm_min",
    "v_emb_norm_std", "global_mean_ce", "pos_frac", "pos_mean", "neg_mean", "explore_attn_raw",
    "explore_know_raw", "explore_block_frac_a", "explore_block_frac_k", "sig_pos_max", "sig_neg_max",
]
ANALYSIS_KEYS = [
    "attn_score_skew", "know_score_skew", "attn_score_kurt", "know_score_kurt",
    "attn_active_per_token_std", "know_active_per_token_std", "attn_gate_entropy",
    "know_gate_entropy", "attn_qk_phi_binary", "attn_v_phi_binary", "know_phi_binary",
    "attn_z_lt_075", "know_z_lt_075", "attn_z_lt_030", "know_z_lt_030", "attn_int_cap_frac",
    "know_int_cap_frac", "qk_emb_norm_max", "v_emb_norm_max", "know_emb_norm_max",
    "attn_tau_std_q", "attn_tau_std_k", "attn_tau_std_v", "know_tau_std", "attn_tau_kernel_norm",
    "know_tau_kernel_norm", "attn_qk_raw_norm", "attn_v_raw_norm", "know_raw_out_norm",
    "attn_z_sum", "know_z_sum", "debug_residual_norm", "debug_emb_norm", "debug_o_proj_norm",
    "debug_q_norm", "debug_k_norm", "debug_v_norm", "debug_logit_max", "debug_o_input_norm",
]


def is_log_step(step: int, interval: int) -> bool:
    return step in EARLY_STEPS or (interval > 0 and step % interval == 0)


def is_analysis_step(step: int, interval: int, mult: int) -> bool:
    return interval > 0 and mult > 0 and step % (interval * mult) == 0


def _f(v) -> Any:
    if isinstance(v, torch.Tensor):
        return v.item() if v.numel() == 1 else [float(x) for x in v.flatten().tolist()]
    return v


class RunLogger:
    def __init__(self, run_dir: Optional[str], enabled: bool = True, stamp: Optional[str] = None):
        self.enabled = enabled and run_dir is not None
        self.txt = self.jsonl = None
        if self.enabled:
            os.makedirs(run_dir, exist_ok=True)
            stamp = stamp or time.strftime("%Y%m%d_%H%M%S")
            existing_t = sorted(f for f in os.listdir(run_dir) if f.startswith("training_log_"))
            existing_j = sorted(f for f in os.listdir(run_dir) if f.startswith("metrics_"))
            # resumed runs keep appending to the files they already have
            self.txt = os.path.join(run_dir, existing_t[-1] if existing_t else f"training_log_{stamp}.txt")
            self.jsonl = os.path.join(run_dir, existing_j[-1] if existing_j else f"metrics_{stamp}.jsonl")

    def message(self, msg: str, echo: bool = True):
        if echo and self.enabled:
            print(msg, flush=True)
        if self.enabled:
            with open(self.txt, "a") as f:
                f.write(msg + "\n")

    def record(self, rec: Dict[str, Any]):
        if self.enabled:
            rec = dict(rec)
            rec.setdefault("timestamp", time.time())
            with open(self.jsonl, "a") as f:
                f.write(json.dumps(rec) + "\n")


class Heartbeat:
    """Per-rank liveness file for an external supervisor: every rank rewrites
    ``heartbeat_rank{r}.json`` (step, wall time, pid) at most every
    ``min_interval`` seconds.  A rank stuck in a collective or a crashed
    process stops refreshing its file; ``stale_ranks`` lists the ranks whose
    file is older than a limit (tools/watchdog.py wraps it).  The reference has
    no heartbeat (its only liveness signal is the SIGTERM flag exchange)."""

    def __init__(self, run_dir: Optional[str], rank: int, world: int, min_interval: float = 10.0):
        self.path = None if run_dir is None else os.path.join(run_dir, f"heartbeat_rank{rank}.json")
        self.rank, self.world, self.min_interval = rank, world, float(min_interval)
        self._last = 0.0

    def beat(self, step: int, force: bool = False) -> None:
        now = time.time()
        if self.path is None or (not force and now - self._last < self.min_interval):
            return
        self._last = now
        os.makedirs(os.path.dirname(self.path), exist_ok=True)
        tmp = self.path + ".tmp"
        with open(tmp, "w") as f:
            json.dump({"rank": self.rank, "world": self.world, "step": int(step), "time": now,
                       "pid": os.getpid()}, f)
        os.replace(tmp, self.path)


def stale_ranks(run_dir: str, max_age_s: float, now: Optional[float] = None) -> Dict[str, Any]:
    """{'world', 'missing': [...], 'stale': {rank: age_s}, 'steps': {rank: step}} from the
    heartbeat files of ``run_dir``."""
    now = time.time() if now is None else now
    beats = {}
    for fn in os.listdir(run_dir):
        if fn.startswith("heartbeat_rank") and fn.endswith(".json"):
            try:
                with open(os.path.join(run_dir, fn)) as f:
                    b = json.load(f)
                beats[int(b["rank"])] = b
            except (ValueError, KeyError, OSError):
                continue
    world = max([b.get("world", 1) for b in beats.values()], default=0)
    return {"world": world, "missing": [r for r in range(world) if r not in beats],
            "stale": {r: now - b["time"] for r, b in beats.items() if now - b["time"] > max_age_s},
            "steps": {r: b["step"] for r, b in beats.items()}}


def build_train_record(step, epoch, metrics: Dict[str, Any], *, steps_per_sec, elapsed,
                       analysis: bool = False) -> Dict[str, Any]:
    rec = {"type": "train_analysis" if analysis else "train", "step": step, "epoch": epoch,
           "steps_per_sec": steps_per_sec, "elapsed": elapsed}
    keys = TRAIN_KEYS + (ANALYSIS_KEYS if analysis else [])
    for k in keys:
        if k in metrics:
            rec[k] = _f(metrics[k])
    for k in ("per_layer_attn_out_norm", "per_layer_know_out_norm"):
        if k in metrics:
            rec[k] = _f(metrics[k])
    if analysis and torch.cuda.is_available():
        free, total = torch.cuda.mem_get_info()
        rec["hbm_used_gb"] = (total - free) / 2 ** 30
        rec["hbm_peak_gb"] = torch.cuda.max_memory_allocated() / 2 ** 30
        rec["hbm_limit_gb"] = total / 2 ** 30
    return rec


def format_regular(rec: Dict[str, Any]) -> str:
    g = lambda k, d=0.0: d if rec.get(k) is None or isinstance(rec.get(k), list) else rec.get(k)
    lines = [
        f"[step {rec['step']:>7d} | ep {rec['epoch']}] loss {g('total_loss'):.4f} (ce {g('ce_loss'):.4f} "
        f"aux {g('aux_loss'):.4f} div {g('div_loss'):.4f} dead {g('dead_penalty'):.4f} "
        f"explore {g('explore_loss_raw'):.5f}) acc {g('accuracy'):.4f}",
        f"    lr {g('lr'):.3e}  grad_norm {g('grad_norm'):.3f}  {g('steps_per_sec'):.3f} it/s  "
        f"elapsed {g('elapsed'):.0f}s",
        f"    active: qk {g('attn_qk_active'):.4f} v {g('attn_v_active'):.4f} know {g('know_active'):.4f}  "
        f"strong: attn {g('attn_strong'):.4f} know {g('know_strong'):.4f}",
        f"    gate_max: attn {g('attn_raw_gate_max'):.3f} know {g('know_raw_gate_max'):.3f}  "
        f"int_max: attn {g('attn_int_max'):.3f} know {g('know_int_max'):.3f}  "
        f"dead: attn {g('attn_dead_count'):.0f} know {g('know_dead_count'):.0f}",
        f"    tau: attn {g('attn_tau_mean'):.4f} know {g('know_tau_mean'):.4f}  bias know {g('tau_know_bias'):.4f} "
        f"attn [{g('tau_attn_bias_0'):.3f} {g('tau_attn_bias_1'):.3f} {g('tau_attn_bias_2'):.3f}]",
        f"    out_norm: attn {g('attn_out_norm'):.3f} know {g('know_out_norm'):.3f}  "
        f"score_std: attn {g('attn_score_std'):.4f} know {g('know_score_std'):.4f}",
        f"    emb_norm: qk {g('qk_emb_norm_mean'):.3f} v {g('v_emb_norm_mean'):.3f} know {g('know_emb_norm'):.3f}  "
        f"drift: qk {g('drift_qk_emb'):.2e} v {g('drift_v_emb'):.2e} know {g('drift_know_emb'):.2e}",
        f"    explore: gmean_ce {g('global_mean_ce'):.4f} pos_frac {g('pos_frac'):.3f} "
        f"block a {g('explore_block_frac_a'):.3f} k {g('explore_block_frac_k'):.3f}",
    ]
    return "\n".join(lines)


def format_analysis(rec: Dict[str, Any]) -> str:
    g = lambda k, d=0.0: d if rec.get(k) is None or isinstance(rec.get(k), list) else rec.get(k)
    lines = [
        f"  [analysis] skew a/k {g('attn_score_skew'):.3f}/{g('know_score_skew'):.3f}  "
        f"kurt a/k {g('attn_score_kurt'):.3f}/{g('know_score_kurt'):.3f}",
        f"    entropy a/k {g('attn_gate_entropy'):.3f}/{g('know_gate_entropy'):.3f}  "
        f"active/token std a/k {g('attn_active_per_token_std'):.2f}/{g('know_active_per_token_std'):.2f}",
        f"    boundary: qk {g('attn_qk_phi_binary'):.4f} v {g('attn_v_phi_binary'):.4f} know {g('know_phi_binary'):.4f}  "
        f"int_cap a/k {g('attn_int_cap_frac'):.2e}/{g('know_int_cap_frac'):.2e}",
        f"    tau std q/k/v {g('attn_tau_std_q'):.4f}/{g('attn_tau_std_k'):.4f}/{g('attn_tau_std_v'):.4f} "
        f"know {g('know_tau_std'):.4f}  kernel norm a/k {g('attn_tau_kernel_norm'):.4f}/{g('know_tau_kernel_norm'):.4f}",
        f"    raw norms qk {g('attn_qk_raw_norm'):.3f} v {g('attn_v_raw_norm'):.3f} know {g('know_raw_out_norm'):.3f}  "
        f"z_sum a/k {g('attn_z_sum'):.2f}/{g('know_z_sum'):.2f}",
        f"    debug: resid {g('debug_residual_norm'):.2f} emb {g('debug_emb_norm'):.3f} o_proj {g('debug_o_proj_norm'):.3f} "
        f"q {g('debug_q_norm'):.3f} k {g('debug_k_norm'):.3f} v {g('debug_v_norm'):.3f} logit_max {g('debug_logit_max'):.3f}",
        f"    hbm used/peak/limit {g('hbm_used_gb'):.1f}/{g('hbm_peak_gb'):.1f}/{g('hbm_limit_gb'):.1f} GB",
    ]
    return "\n".join(lines)
