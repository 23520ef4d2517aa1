import json
import math
import os

import pytest
import torch

from dawn_srw_b200.train import checkpoint as ck
from dawn_srw_b200.train.logging import ANALYSIS_KEYS, TRAIN_KEYS
from dawn_srw_b200.train.trainer import NonFiniteLoss, Trainer

from helpers import tiny_config


def _params(tr):
    return {n: p.detach().clone() for n, p in tr.model.named_parameters()}


def test_resume_is_deterministic(tmp_path):
    """8 steps in one go == 4 steps, checkpoint, new process state, 4 more."""
    cfg = tiny_config(max_steps=8, checkpoint_interval=4, dead_penalty_weight=0.05)
    a = Trainer(cfg, run_dir=str(tmp_path / "a"), total_steps=8)
    os.makedirs(a.run_dir, exist_ok=True)
    a.fit()
    cfg_b = tiny_config(max_steps=4, checkpoint_interval=4, dead_penalty_weight=0.05)
    b = Trainer(cfg_b, run_dir=str(tmp_path / "b"), total_steps=8)
    os.makedirs(b.run_dir, exist_ok=True)
    b.fit()
    cfg_c = tiny_config(max_steps=8, checkpoint_interval=4, dead_penalty_weight=0.05)
    c = Trainer(cfg_c, run_dir=str(tmp_path / "b"), total_steps=8)
    c.resume(os.path.join(str(tmp_path / "b"), "checkpoint_step4.pt"))
    assert c.global_step == 4 and c.step_in_epoch == 4 and c.optimizer.count == 4
    c.fit()
    pa, pc = _params(a), _params(c)
    for n in pa:
        assert torch.allclose(pa[n], pc[n], atol=1e-7), n


def test_jsonl_schema(tmp_path):
    cfg = tiny_config(max_steps=4, log_interval=2, log_analysis_multiplier=2, val_interval=4,
                      dead_penalty_weight=0.05, exploration_weight=1e-3, exploration_warmup_steps=0)
    run = str(tmp_path / "r")
    os.makedirs(run)
    Trainer(cfg, run_dir=run).fit()
    recs = [json.loads(l) for f in os.listdir(run) if f.startswith("metrics_")
            for l in open(os.path.join(run, f))]
    types = {r["type"] for r in recs}
    assert {"train", "train_analysis", "val"} <= types
    tr = next(r for r in recs if r["type"] == "train")
    missing = [k for k in TRAIN_KEYS + ["step", "epoch", "steps_per_sec", "elapsed", "timestamp",
                                        "per_layer_attn_out_norm", "per_layer_know_out_norm"]
               if k not in tr]
    assert not missing, missing
    an = next(r for r in recs if r["type"] == "train_analysis")
    missing = [k for k in ANALYSIS_KEYS if k not in an]
    assert not missing, missing
    v = next(r for r in recs if r["type"] == "val")
    assert {"step", "epoch", "val_loss", "val_acc", "timestamp"} <= set(v)
    assert os.path.exists(os.path.join(run, "config.json"))
    cfgj = json.load(open(os.path.join(run, "config.json")))
    assert set(cfgj) == {"model", "training"}


def test_non_finite_loss_stops_training(tmp_path):
    cfg = tiny_config(max_steps=3)
    tr = Trainer(cfg, run_dir=None)
    with torch.no_grad():
        tr.model.token_emb.weight.fill_(float("nan"))
    with pytest.raises(NonFiniteLoss):
        tr.fit()


def test_max_steps_counts_micro_steps_and_the_schedule_runs_on_optimizer_steps():
    """With gradient accumulation k, max_steps micro-steps are max_steps / k
    optimizer steps: the cosine schedule must end there (at 0.1 * lr), not
    stretch over k times as many."""
    cfg = tiny_config(max_steps=8, gradient_accumulation_steps=2, lr=1e-2, warmup_ratio=0.25)
    tr = Trainer(cfg)
    assert tr.total_steps == 4
    tr.fit()
    assert tr.global_step == 8 and tr.optimizer.count == 4
    assert tr.schedule(0) == pytest.approx(1e-3)              # warm-up starts at 0.1 * lr
    assert tr.schedule(tr.total_steps) == pytest.approx(1e-3)  # cosine has reached 0.1 * lr
    assert tr.schedule(1) == pytest.approx(1e-2)              # one warm-up step of four


def test_loss_decreases_on_a_fixed_batch():
    cfg = tiny_config(lr=3e-3, diversity_weight=0.0)
    tr = Trainer(cfg, total_steps=1000)
    ids, mask = tr.train_loader.batch(0)
    first = float(tr.train_step(ids, mask)["ce_loss"])
    for _ in range(30):
        last = float(tr.train_step(ids, mask)["ce_loss"])
    assert last < first - 0.3


def test_sigterm_flag_writes_emergency_checkpoint(tmp_path):
    cfg = tiny_config(max_steps=50)
    run = str(tmp_path / "r")
    os.makedirs(run)
    tr = Trainer(cfg, run_dir=run)
    orig = tr.train_step

    def step_then_flag(*a, **k):
        out = orig(*a, **k)
        if tr.global_step == 3:
            tr.preempt_requested = True       # what the SIGTERM handler does
        return out
    tr.train_step = step_then_flag
    tr.fit()
    assert tr.global_step == 10               # the flag is polled every 10 steps
    assert os.path.exists(os.path.join(run, "emergency_step10.pt"))


def test_baseline_model_trains(tmp_path):
    cfg = tiny_config(version="baseline", max_steps=2)
    out = Trainer(cfg).fit()
    assert math.isfinite(out["total_loss"])


def test_gradient_accumulation_in_the_trainer():
    """Two micro-steps on the same batch with accumulation 2 give the update of
    one plain step on that batch (the mean of two equal gradients)."""
    torch.manual_seed(0)
    a = Trainer(tiny_config(gradient_accumulation_steps=2), total_steps=100)
    b = Trainer(tiny_config(), total_steps=100)
    b.model.load_state_dict(a.model.state_dict())
    ids, mask = a.train_loader.batch(0)
    before = _params(a)
    a.train_step(ids, mask)
    assert a.optimizer.count == 0
    for n, p in _params(a).items():
        assert torch.equal(p, before[n]), n          # nothing moves inside the window
    a.train_step(ids, mask)
    b.train_step(ids, mask)
    assert a.optimizer.count == 1 and b.optimizer.count == 1
    pa, pb = _params(a), _params(b)
    for n in pa:
        assert torch.allclose(pa[n], pb[n], atol=2e-6), n


def test_startup_report_leaves_training_state_untouched():
    from dawn_srw_b200.train.startup import startup_report
    tr = Trainer(tiny_config(version="spatial-r1-v4.0.1"), total_steps=50)
    before = _params(tr)
    lines = []
    rep = startup_report(tr, n_runs=1, print_fn=lines.append)
    assert rep["fwd_bwd_ms"] > 0 and rep["eta_hours"] > 0
    assert set(rep["ops_forward_ms"]) >= {"layer_norm", "srw_know", "self_attention"}
    assert any("forward+backward" in l for l in lines)
    for n, p in _params(tr).items():
        assert torch.equal(p, before[n]), n
    assert tr.optimizer.count == 0 and all(p.grad is None for p in tr.model.parameters())


def test_trace_ranges_cover_a_training_step():
    from dawn_srw_b200.utils import tracing
    tr = Trainer(tiny_config(version="spatial-r1-v4.0.1"), total_steps=50)
    ids, mask = tr.train_loader.batch(0)
    tracing.enable(timers=True)
    try:
        tr.train_step(ids, mask)
        rep = tracing.report()
    finally:
        tracing.enable(timers=False)
    L = tr.cfg.model.n_layers
    assert rep["forward"][0] == 1 and rep["backward"][0] == 1 and rep["optimizer"][0] == 1
    assert rep["attn/srw_qkv"][0] == L and rep["know/srw"][0] == L and rep["lm_head_ce"][0] == 1
    assert rep["forward"][1] >= rep["know/srw"][1] > 0
    assert "know/srw" in tracing.format_report(rep)
    tr.train_step(ids, mask)
    assert tracing.report() == {}                 # off again: nothing is recorded


def test_heartbeat_files_and_watchdog(tmp_path, capsys):
    import time
    from dawn_srw_b200.tools import watchdog as W
    from dawn_srw_b200.train.logging import Heartbeat, stale_ranks
    run = str(tmp_path / "run")
    tr = Trainer(tiny_config(max_steps=2), run_dir=run, total_steps=2)
    tr.fit()
    rep = stale_ranks(run, max_age_s=60)
    assert rep["world"] == 1 and not rep["stale"] and not rep["missing"] and rep["steps"][0] >= 1
    assert W.main([run, "--max-age", "60"]) == 0
    capsys.readouterr()
    # a second rank that stopped refreshing long ago, and a third that never wrote one
    hb = Heartbeat(run, rank=1, world=3)
    hb.beat(5, force=True)
    old = stale_ranks(run, max_age_s=60, now=time.time() + 3600)
    assert set(old["stale"]) == {0, 1} and old["missing"] == [2] and old["world"] == 3
    assert W.main([run, "--max-age", "60"]) == 3          # rank 2 is missing
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["missing"] == [2]
