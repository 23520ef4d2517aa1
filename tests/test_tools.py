"""Command-line tools on CPU: pretokenize -> train -> analyze / eval / generate."""
import json
import os

import numpy as np
import pytest
import torch

from helpers import tiny_config


def test_pretokenize_packs_rows_and_resumes(tmp_path):
    from dawn_srw_b200.data.loaders import ShardedBinDataset
    from dawn_srw_b200.tools import pretokenize as P
    txt = tmp_path / "docs.txt"
    txt.write_text("\n".join(f"document number {i} " + "x" * (i % 17) for i in range(200)))
    out = str(tmp_path / "tok" / "train")
    assert P.main(["--input", str(txt), "--output", out, "--seq-len", "16", "--shard-tokens", "640",
                   "--tokenizer", "bytes"]) == 0
    meta = json.load(open(out + "_meta.json"))
    assert meta["complete"] and meta["seq_len"] == 16 and len(meta["shards"]) > 1
    ds = ShardedBinDataset(out + "_meta.json", 16)
    rows = ds.rows(0, len(ds))
    stream = rows.reshape(-1)
    want = []
    for i in range(200):
        want += list((f"document number {i} " + "x" * (i % 17)).strip().encode()) + [256]
    assert np.array_equal(stream, np.asarray(want[: len(stream)], dtype=np.uint16))   # packed, no padding
    # resume: drop the last shard and its meta entry, run again, same shard count
    last = meta["shards"][-1]
    os.remove(os.path.join(os.path.dirname(out), last["path"]))
    assert P.main(["--input", str(txt), "--output", out, "--seq-len", "16", "--shard-tokens", "640",
                   "--tokenizer", "bytes", "--resume"]) == 0
    meta2 = json.load(open(out + "_meta.json"))
    assert meta2["complete"] and len(meta2["shards"]) >= len(meta["shards"]) - 1


def test_analysis_cli_runs_every_key(tmp_path):
    from dawn_srw_b200.tools import analyze as A
    from dawn_srw_b200.train.trainer import Trainer
    cfg = tiny_config(version="spatial-r1-v4.0.1", max_steps=2)
    tr = Trainer(cfg, run_dir=str(tmp_path / "run"), total_steps=2)
    os.makedirs(tr.run_dir, exist_ok=True)
    ids, mask = tr.train_loader.batch(0)
    tr.train_step(ids, mask)
    path = tr.save("checkpoint_step1.pt")
    out_dir = str(tmp_path / "ana")
    assert A.main(["--checkpoint", path, "--synthetic", "--batch-size", "2", "--n-batches", "2",
                   "--suppress-top", "4", "--max-new-tokens", "4", "--output", out_dir,
                   "--compare-checkpoint", path, "--device", "cpu"]) == 0
    res = json.load(open(os.path.join(out_dir, "analysis.json")))
    assert set(res) == set(A.ANALYSES)
    assert res["info"]["parameters"] > 0 and res["val"]["val_loss"] > 0
    L = cfg.model.n_layers
    assert len(res["routing"]["Know"]["gate_entropy"]) == L
    assert 0.0 <= res["utilization"]["Know"]["used_frac_any_layer"] <= 1.0
    assert 0.0 <= res["sel_gini"]["Q"]["gini_all_layers"] <= 1.0
    assert len(res["intervene"]["suppressed"]) == 1
    assert -1.0 <= res["rw_align"]["know"]["cos_mean"] <= 1.0
    assert res["tau_dist"]["Know"]["std"] >= 0.0
    # the rebuttal / interpretation / combinatorics half of the suite
    assert abs(res["r1"]["q_specialised_frac"] + res["r1"]["k_specialised_frac"] + res["r1"]["shared_frac"] - 1.0) < 1e-5
    assert len(res["r4"]["attn_share"]) == L and len(res["r5"]["levels"]) == 4
    assert res["r3"]["top_units"] and res["combo"]["Know"]["unique_sets"] >= 1
    assert 0.0 <= res["op_space"]["unique_active_sets_frac"] <= 1.0
    assert len(res["rw_func"]["bins"]) == 10 and sum(b["units"] for b in res["rw_func"]["bins"]) == cfg.model.n_know
    assert res["tau_grad"]["task_tau_grad_norm"] >= 0.0 and "skipped" in res["phase"]
    assert set(res["deep"]["units"]) == {"corrective", "neutral", "amplifying"}
    # every --only key of the reference's CLI is accepted (rw_cov expands to its two members)
    ref_keys = ("info,val,health,generate,weights,routing,samples,gate_dist,utilization,r1,r2,r3,r4,r5,"
                "rw_proj,act_context,layer_role,cross_suppress,gate_mech,comp_expr,neuron_cluster,cross_ref,"
                "deep,op_space,intervene,compose,rw_align,resid_dyn,phase,drift,gate_ci,write_cov,read_cov,"
                "rw_cov,sel_gini,sel_trans,combo,addit,dom_supp,rw_func,z_dist,tau_grad,pool_geom").split(",")
    assert all(k in A.ANALYSES or k in A.ALIASES for k in ref_keys)
    # phase dynamics from this framework's own metrics file
    log = tmp_path / "m.jsonl"
    log.write_text("\n".join(json.dumps({"type": "train", "step": s_, "ce_loss": 5.0 - 0.01 * s_,
                                          "know_active": 0.7 if s_ < 50 else 0.1, "know_tau_mean": 0.01 * s_})
                             for s_ in range(0, 100, 10)))
    base = tmp_path / "b.jsonl"
    base.write_text("\n".join(json.dumps({"type": "train", "step": s_, "ce_loss": 4.8 - 0.004 * s_})
                              for s_ in range(0, 100, 10)))
    assert A.main(["--checkpoint", path, "--synthetic", "--batch-size", "2", "--n-batches", "1",
                   "--only", "phase,rw_cov", "--dawn-log", str(log), "--baseline-log", str(base),
                   "--output", out_dir, "--device", "cpu"]) == 0
    res2 = json.load(open(os.path.join(out_dir, "analysis.json")))
    assert set(res2) == {"phase", "read_cov", "write_cov"}
    assert res2["phase"]["phase_boundary_step"] == 50 and res2["phase"]["crossover_step"] == 40
    assert res["drift"]["know_emb"]["rel_l2"] == 0.0          # compared with itself
    assert 0.0 <= res["cross_ref"]["token_jaccard_mean"] <= 1.0
    assert len(res["layer_sim"]["Know"]["adjacent"]) == L - 1
    assert len(res["sel_trans"]["Q"]["survival_to_next_layer"]) == L - 1
    lo, hi = res["gate_ci"]["V"]["ci95"]
    assert lo <= res["gate_ci"]["V"]["active_frac"] <= hi or abs(hi - lo) < 1e-6
    assert 1.0 <= res["write_cov"]["know"]["participation_ratio"] <= res["write_cov"]["know"]["dims"] + 1e-6
    assert res["samples"]["know_units"] and len(res["samples"]["know_units"][0]["top_token_ids"]) > 0
    assert len(res["resid_dyn"]["norm_per_layer"]) == L + 1
    assert res["resid_dyn"]["top1_agreement_with_final"][-1] == 1.0
    assert res["z_dist"]["quantiles"]["p1"] < res["z_dist"]["quantiles"]["p99"]
    ad = res["addit"]
    assert abs(ad["interaction"] - (ad["delta_ab"] - ad["delta_a"] - ad["delta_b"])) < 1e-9
    assert set(res["cross_suppress"]) >= {"qk", "v", "know", "baseline"}
    assert len(res["generate"]["samples"][0]["token_ids"]) >= 4
    # key selection
    assert A.main(["--checkpoint", path, "--synthetic", "--only", "info,health", "--device", "cpu"]) == 0
    with pytest.raises(SystemExit):
        A.main(["--checkpoint", path, "--only", "nope", "--device", "cpu"])


def test_train_eval_generate_clis_and_resume(tmp_path, capsys):
    """configs/smoke_tiny_synthetic.yaml through the train CLI (start-up report,
    checkpoints, resume from the newest run), then eval and generate on the result."""
    import glob
    from dawn_srw_b200.tools import eval as E, generate as G, train as T
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = os.path.join(root, "configs", "smoke_tiny_synthetic.yaml")
    ck = str(tmp_path / "ck")
    assert T.main(["--config", cfg, "--from-scratch", "--max-steps", "6", "--checkpoint-dir", ck]) == 0
    out = capsys.readouterr().out
    assert "[startup] forward+backward" in out and '"final"' in out
    runs = glob.glob(os.path.join(ck, "run_*"))
    assert len(runs) == 1
    ckpts = sorted(glob.glob(os.path.join(runs[0], "*.pt")))
    assert ckpts, os.listdir(runs[0])
    # a second invocation without --from-scratch resumes the same run folder
    assert T.main(["--config", cfg, "--max-steps", "8", "--checkpoint-dir", ck, "--no-startup-check"]) == 0
    out = capsys.readouterr().out
    assert "Resumed from" in out and len(glob.glob(os.path.join(ck, "run_*"))) == 1
    newest = max(glob.glob(os.path.join(runs[0], "*.pt")), key=os.path.getmtime)
    assert E.main(["--checkpoint", newest, "--synthetic", "--batch-size", "4", "--max-batches", "2"]) == 0
    rec = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rec["val_loss"] > 0 and rec["valid_tokens"] > 0
    assert G.main(["--checkpoint", newest, "--ids", "5,6,7", "--max-new-tokens", "5"]) == 0
    assert capsys.readouterr().out.strip()


def test_every_shipped_config_loads_without_unknown_keys():
    import glob
    import warnings
    from dawn_srw_b200.config import load_config
    from dawn_srw_b200.models.registry import MODEL_REGISTRY
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = sorted(glob.glob(os.path.join(root, "configs", "*.yaml")))
    assert len(files) >= 15
    for f in files:
        with warnings.catch_warnings():
            warnings.simplefilter("error")
            cfg = load_config(f)
        assert cfg.model.model_version in MODEL_REGISTRY, f
        t = cfg.training
        assert t.pool_shards >= 1 and (t.dp == 0 or t.dp * t.pool_shards in (1, 8)), f


def test_bench_reference_arm_reports_unavailable():
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0
    rec = json.loads(r.stdout.strip().splitlines()[-1])
    assert rec["impl"] == "reference" and "unavailable" in rec


def test_pretokenized_files_feed_the_trainer(tmp_path, capsys):
    """text -> pretokenize (byte tokenizer, sharded) -> YAML with bin_train / bin_val ->
    train CLI: the vocabulary size comes from the shard metadata and validation runs."""
    import yaml
    from dawn_srw_b200.tools import pretokenize as P, train as T
    rng = np.random.default_rng(0)
    words = ["alpha", "beta", "gamma", "delta", "epsilon", "zeta"]
    txt = tmp_path / "corpus.txt"
    txt.write_text("\n".join(" ".join(rng.choice(words, size=12)) for _ in range(400)))
    train_prefix, val_prefix = str(tmp_path / "data" / "train"), str(tmp_path / "data" / "val")
    for prefix in (train_prefix, val_prefix):
        assert P.main(["--input", str(txt), "--output", prefix, "--seq-len", "32",
                       "--shard-tokens", "8192", "--tokenizer", "bytes"]) == 0
    capsys.readouterr()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = yaml.safe_load(open(os.path.join(root, "configs", "smoke_tiny_synthetic.yaml")))
    cfg["data"].update(synthetic=False, bin_train=train_prefix, bin_val=val_prefix,
                       max_train_tokens=32 * 8 * 12)
    cfg["training"].update(val_interval=4, checkpoint_interval=0, log_interval=2)
    cfg_path = tmp_path / "cfg.yaml"
    cfg_path.write_text(yaml.safe_dump(cfg))
    assert T.main(["--config", str(cfg_path), "--from-scratch", "--max-steps", "8",
                   "--checkpoint-dir", str(tmp_path / "ck"), "--no-startup-check"]) == 0
    out = capsys.readouterr().out
    assert "[val @ 4]" in out and "[val @ 8]" in out
    import glob
    run = glob.glob(str(tmp_path / "ck" / "run_*"))[0]
    saved = json.load(open(os.path.join(run, "config.json")))
    assert saved["model"]["vocab_size"] == 257                  # byte tokenizer + separator
    recs = [json.loads(l) for l in open(glob.glob(os.path.join(run, "metrics_*.jsonl"))[0])]
    assert any(r.get("type") == "val" for r in recs) and any(r.get("type") == "train" for r in recs)


def test_inference_speed_harness(capsys):
    from dawn_srw_b200.tools import bench_inference as B
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = os.path.join(root, "configs", "smoke_tiny_synthetic.yaml")
    assert B.main(["--config", cfg, "--batch-sizes", "1,3", "--seq-len", "16", "--warmup", "1",
                   "--iters", "3", "--new-tokens", "4", "--device", "cpu"]) == 0
    recs = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert [r["batch"] for r in recs] == [1, 3]
    assert all(r["forward_tokens_per_sec"] > 0 and r["decode_new_tokens"] == 4 for r in recs)
    assert recs[0]["forward_ms_p50"] <= recs[0]["forward_ms_p95"] + 1e-9


def test_bench_clock_csv_parsing():
    import importlib.util
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(root, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    text = "\n".join([
        "0, 1965, 1965, 410.2, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active",
        "0, 1710, 1965, 995.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
        "0, 1650, 1965, 998.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
        "garbage line",
        "0, [N/A], 1965, 1.0, x, Not Active, Not Active, Not Active, Not Active",
    ])
    rec = bench.parse_clock_csv(text)
    assert rec == {"sm_mhz": 1710.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    hot = bench.parse_clock_csv("0, 900, 1965, 300, x, Active, Active, Not Active, Not Active")
    assert hot["reasons"] == ["hw_slowdown", "hw_thermal_slowdown"]
    assert bench.parse_clock_csv("") is None
    assert bench.ClockSampler(0).stop()["sm_mhz"] is None         # never started: neutral record


def test_launcher_builds_the_command_and_runs_a_detached_job(tmp_path):
    """tools/launch.py: dry run prints the torch.distributed.run line; a detached
    one-rank CPU job trains the smoke config, writes its log and PID file, and a
    second launch from the same place is refused while it is alive."""
    import subprocess
    import sys
    import time
    from dawn_srw_b200.tools import launch as Lh
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = os.path.join(root, "configs", "smoke_tiny_synthetic.yaml")
    cmd = Lh.build_command(cfg, 8, 29511, True, ["--max-steps", "3"])
    assert cmd[1:4] == ["-m", "torch.distributed.run", "--nnodes=1"]
    assert "--nproc-per-node=8" in cmd and "127.0.0.1" in cmd and cmd[-3:] == ["--from-scratch", "--max-steps", "3"]
    log = str(tmp_path / "train.log")
    env = dict(os.environ, PYTHONPATH=root, CUDA_VISIBLE_DEVICES="")
    base = [sys.executable, "-m", "dawn_srw_b200.tools.launch", "--log", log]
    from helpers import free_port
    r = subprocess.run(base + ["--config", cfg, "--gpus", "1", "--detach", "--from-scratch",
                               "--master-port", str(free_port()), "--", "--max-steps", "3",
                               "--no-startup-check", "--checkpoint-dir", str(tmp_path / "ck")],
                       env=env, capture_output=True, text=True, cwd=root)
    assert r.returncode == 0, r.stderr
    assert os.path.exists(log + ".pid")
    st = json.loads(subprocess.run(base + ["--status"], env=env, capture_output=True, text=True,
                                   cwd=root).stdout)
    assert st["pid"] > 0
    deadline = time.time() + 240
    while time.time() < deadline:
        st = json.loads(subprocess.run(base + ["--status"], env=env, capture_output=True, text=True,
                                       cwd=root).stdout)
        if not st["alive"]:
            break
        time.sleep(1.0)
    assert not st["alive"], open(log).read()[-2000:]
    text = open(log).read()
    assert '"final"' in text and "run_dir" in text, text[-2000:]
    # nothing alive any more: --stop reports that it had nothing to do
    out = subprocess.run(base + ["--stop"], env=env, capture_output=True, text=True, cwd=root).stdout
    assert json.loads(out) == {"stopped": False}
