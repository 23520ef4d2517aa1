"""Multi-rank logic on CPU ranks (gloo): sharded results equal the single-rank
result, host-side consensus protocols behave."""
import os

import pytest
import torch

from helpers import run_ranks, tiny_config

KW = dict(vocab_size=120, d_model=32, n_layers=2, n_heads=4, max_seq_len=16, d_route=8, n_qk=21,
          n_v=30, n_know=50, dropout_rate=0.0, router_dropout=0.0)


def _single(version, ids):
    from dawn_srw_b200.models.dawn import DAWN
    m = DAWN(**KW, model_version=version, seed=5)
    r = m(ids, labels=ids, want_diag=True)
    (r["loss"] + 0.1 * r["aux_loss"] + 0.05 * r["dead_penalty"]).backward()
    return m, r


def _sharded_worker(rank, world, version, seq_sharded):
    import torch.distributed as dist
    from dawn_srw_b200.models.dawn import DAWN
    from dawn_srw_b200.parallel.topology import init_topology
    topo = init_topology(pool_shards=world, seq_shard=seq_sharded, backend="gloo")
    torch.manual_seed(0)
    ids = torch.randint(0, 120, (4, 16))
    m = DAWN(**KW, model_version=version, seed=5, pool_shard=topo.pool_shard)
    m.set_parallel(shard_group=topo.shard_group, dp_group=None, seq_sharded=topo.seq_shard)
    local = ids[rank * 2:(rank + 1) * 2] if seq_sharded else ids
    r = m(local, labels=local, want_diag=True)
    (r["loss"] + 0.1 * r["aux_loss"] + 0.05 * r["dead_penalty"]).backward()
    g = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
    return {"loss": float(r["loss"]), "aux": float(r["aux_loss"]), "dead": float(r["dead_penalty"]),
            "active": float(r["know_active"]), "grads": g, "n_valid": m.neuron_pool.n_valid("qk")}


@pytest.mark.parametrize("version", ["spatial-r1-v4.0.1", "spatial-r1-v4.1"])
def test_pool_sharding_matches_single_rank(version):
    torch.manual_seed(0)
    ids = torch.randint(0, 120, (4, 16))
    m, r = _single(version, ids)
    outs = run_ranks(_sharded_worker, 2, version, False)
    assert sum(o["n_valid"] for o in outs) == 21            # 21 units over 2 ranks: 16 + 5 (padded)
    for o in outs:
        assert abs(o["loss"] - float(r["loss"])) < 1e-5
        assert abs(o["aux"] - float(r["aux_loss"])) < 1e-5
        assert abs(o["dead"] - float(r["dead_penalty"])) < 1e-5
        assert abs(o["active"] - float(r["know_active"])) < 1e-6
    full = {n: p.grad for n, p in m.named_parameters()}
    # objective = mean of the (here identical) per-rank losses; collectives use
    # true transposes, so replicated-parameter gradients are summed / world ...
    for n in ("router.proj_know.weight", "layers.0.attn.expand_O.weight", "token_emb.weight",
              "router.tau_attn.bias", "layers.1.norm2.weight"):
        got = (outs[0]["grads"][n] + outs[1]["grads"][n]) / 2
        assert torch.allclose(got, full[n], atol=2e-5), n
    # ... and rank k's pool rows hold world x the gradient of its units
    from dawn_srw_b200.parallel.topology import PoolShard
    for name, n_units in (("qk", 21), ("know", 50)):
        for kind in ("emb", "read", "write"):
            for k in range(2):
                lo, hi, _ = PoolShard(k, 2).slice_of(n_units)
                got = outs[k]["grads"][f"neuron_pool.{name}_{kind}"][: hi - lo] / 2
                assert torch.allclose(got, full[f"neuron_pool.{name}_{kind}"][lo:hi], atol=2e-5), (name, kind, k)


def test_sequence_sharding_matches_single_rank():
    version = "spatial-r1-v4.0.1"
    torch.manual_seed(0)
    ids = torch.randint(0, 120, (4, 16))
    m, r = _single(version, ids)
    outs = run_ranks(_sharded_worker, 2, version, True)
    # each rank's loss is the mean over its own sequences; equal token counts -> mean of means
    assert abs(sum(o["loss"] for o in outs) / 2 - float(r["loss"])) < 1e-5
    full = {n: p.grad for n, p in m.named_parameters()}
    from dawn_srw_b200.parallel.topology import PoolShard
    # objective = mean of per-rank losses: replicated grads sum over ranks / world,
    # pool grads are already summed over the shard group -> / world
    for n in ("router.proj_know.weight", "router.proj_attn.bias", "token_emb.weight",
              "layers.0.attn.expand_O.weight"):
        assert torch.allclose((outs[0]["grads"][n] + outs[1]["grads"][n]) / 2, full[n], atol=2e-5), n
    for kind in ("emb", "read", "write"):
        for k in range(2):
            lo, hi, _ = PoolShard(k, 2).slice_of(50)
            got = outs[k]["grads"][f"neuron_pool.know_{kind}"][: hi - lo] / 2
            assert torch.allclose(got, full[f"neuron_pool.know_{kind}"][lo:hi], atol=2e-5), (kind, k)


def _dp_trainer_worker(rank, world, pool_shards, seq_shard, zero=False, accum=1, ckpt_dir=None,
                       overlap=True):
    from dawn_srw_b200.parallel.topology import init_topology
    from dawn_srw_b200.train.trainer import Trainer
    topo = init_topology(pool_shards=pool_shards, seq_shard=seq_shard, backend="gloo")
    cfg = tiny_config(version="spatial-r1-v4.0.1", max_steps=3, diversity_weight=0.0,
                      zero_pool_state=zero, gradient_accumulation_steps=accum,
                      overlap_grad_reduce=overlap)
    tr = Trainer(cfg, topo=topo, device=torch.device("cpu"), total_steps=10, run_dir=ckpt_dir)
    for i in range(3 * accum):
        ids, mask = tr.train_loader.batch(i)
        m = tr.train_step(ids, mask)
    out = {"gn": float(m["grad_norm"]), "opt": type(tr.optimizer).__name__}
    if ckpt_dir is not None:
        # save, perturb, resume: parameters and sharded moments come back
        import os
        os.makedirs(ckpt_dir, exist_ok=True)
        tr.save("checkpoint_step3.pt")
        torch.distributed.barrier()
        tr2 = Trainer(cfg, topo=topo, device=torch.device("cpu"), total_steps=10, run_dir=ckpt_dir)
        tr2.resume(os.path.join(ckpt_dir, "checkpoint_step3.pt"))
        for t_ in (tr, tr2):
            ids, mask = t_.train_loader.batch(7)
            t_.train_step(ids, mask)
        out["resume_diff"] = max(float((a - b).abs().max()) for (_, a), (_, b) in zip(
            tr.model.named_parameters(), tr2.model.named_parameters()))
        out["state_bytes"] = tr.optimizer.state_bytes() if zero else 0
    out["sd"] = {n: p.detach().clone() for n, p in tr.model.named_parameters()}
    return out


def _dp_grad_worker(rank, world):
    """One forward/backward on this rank's half of the batch, then GradSync."""
    from dawn_srw_b200.parallel.grad_sync import GradSync
    from dawn_srw_b200.parallel.topology import init_topology
    from dawn_srw_b200.train.trainer import Trainer
    topo = init_topology(backend="gloo")
    cfg = tiny_config(version="spatial-r1-v4.0.1", diversity_weight=0.0, load_balance_weight=0.0)
    tr = Trainer(cfg, topo=topo, device=torch.device("cpu"), total_steps=10)
    ids, mask = tr.train_loader.batch(0)
    r = tr.model(ids.long(), labels=ids.long(), want_diag=False)
    r["loss"].backward()
    named = list(tr.model.named_parameters())
    sync = tr.optimizer.grad_sync          # hooks launched bucketed all-reduces during backward
    assert sync._overlap and (sync._inflight or sync._open)
    grads = sync.reduce(named, [p.grad for _, p in named])
    assert not sync._inflight and not sync._open
    return {n: g for (n, _), g in zip(named, grads)}


def test_data_parallel_gradients_match_single_process():
    from dawn_srw_b200.train.trainer import Trainer
    cfg = tiny_config(version="spatial-r1-v4.0.1", diversity_weight=0.0, load_balance_weight=0.0)
    ref = Trainer(cfg, device=torch.device("cpu"), total_steps=10)
    ids, mask = ref.train_loader.batch(0)
    ref.model(ids.long(), labels=ids.long(), want_diag=False)["loss"].backward()
    outs = run_ranks(_dp_grad_worker, 2)
    for n, p in ref.model.named_parameters():
        assert torch.allclose(outs[0][n], p.grad, atol=1e-6), n
        assert torch.equal(outs[0][n], outs[1][n]), n


def test_data_parallel_training_keeps_replicas_identical():
    outs = run_ranks(_dp_trainer_worker, 2, 1, False)
    for n in outs[0]["sd"]:
        assert torch.equal(outs[0]["sd"][n], outs[1]["sd"][n]), n
    assert outs[0]["gn"] == outs[1]["gn"]


def test_pool_and_sequence_sharded_training_runs_and_agrees_across_ranks():
    outs = run_ranks(_dp_trainer_worker, 2, 2, True)
    for n in ("router.proj_know.weight", "token_emb.weight", "layers.1.norm2.weight"):
        assert torch.allclose(outs[0]["sd"][n], outs[1]["sd"][n], atol=1e-6), n
    assert abs(outs[0]["gn"] - outs[1]["gn"]) < 1e-5


@pytest.mark.parametrize("layout", [(2, 1, False), (2, 2, True), (4, 2, True)])
def test_partitioned_optimizer_matches_replicated_adamw(layout):
    """Reduce-scatter + AdamW on the owned slice + all-gather gives the same
    parameters as all-reduce + full AdamW, for pure data parallelism, for
    sharded pools (pool slices private to a rank) and for dp 2 x pool shards 2
    (pool slices replicated over the data-parallel pair only)."""
    world, shards, seq = layout
    a = run_ranks(_dp_trainer_worker, world, shards, seq, False, 2)
    b = run_ranks(_dp_trainer_worker, world, shards, seq, True, 2)
    assert a[0]["opt"] == "DawnAdamW" and b[0]["opt"] == "PartitionedAdamW"
    for r in range(world):
        assert abs(a[r]["gn"] - b[r]["gn"]) < 1e-5
        for n in a[r]["sd"]:
            assert torch.allclose(a[r]["sd"][n], b[r]["sd"][n], atol=2e-6), (r, n)


def test_partitioned_optimizer_checkpoint_roundtrip(tmp_path):
    outs = run_ranks(_dp_trainer_worker, 2, 1, False, True, 1, str(tmp_path / "run"))
    assert outs[0]["resume_diff"] == 0.0 and outs[1]["resume_diff"] == 0.0
    n_params = sum(v.numel() for v in outs[0]["sd"].values())
    # two moments, fp32, half of the parameters each (plus padding)
    assert outs[0]["state_bytes"] <= 2 * 4 * (n_params // 2 + 64)


@pytest.mark.parametrize("layout", [(2, 1, False), (2, 2, True)])
def test_overlapped_gradient_reduction_changes_nothing(layout):
    world, shards, seq = layout
    a = run_ranks(_dp_trainer_worker, world, shards, seq, False, 1, None, True)
    b = run_ranks(_dp_trainer_worker, world, shards, seq, False, 1, None, False)
    for r in range(world):
        assert a[r]["gn"] == b[r]["gn"]
        for n in a[r]["sd"]:
            assert torch.equal(a[r]["sd"][n], b[r]["sd"][n]), (r, n)


def _consensus_worker(rank, world):
    from dawn_srw_b200.parallel.topology import init_topology
    from dawn_srw_b200.train.trainer import Trainer
    topo = init_topology(backend="gloo")
    tr = Trainer(tiny_config(), topo=topo, device=torch.device("cpu"), build_data=True)
    if rank == 1:
        tr.preempt_requested = True        # only one rank got the signal
    agreed = tr.preemption_consensus()
    tr.global_step = 7 if rank == 0 else 8
    try:
        tr.check_step_consistency()
        mismatch = False
    except RuntimeError:
        mismatch = True
    return agreed, mismatch


def test_preemption_consensus_and_step_check():
    outs = run_ranks(_consensus_worker, 2)
    assert all(a for a, _ in outs)          # every rank leaves the loop together
    assert all(m for _, m in outs)          # a split resume is detected on every rank


def _diversity_worker(rank, world):
    from dawn_srw_b200.ops.reference import pool_diversity
    from dawn_srw_b200.parallel.topology import PoolShard, init_topology
    from dawn_srw_b200.train.losses import global_strided_sample
    topo = init_topology(pool_shards=world, backend="gloo")
    out = {}
    for n_total, max_sample in ((50, 16), (21, 64)):           # strided sample / whole small pool
        full = torch.randn(n_total, 6, generator=torch.Generator().manual_seed(3))
        sh = PoolShard(rank, world)
        lo, hi, _ = sh.slice_of(n_total)
        local = full[lo:hi].clone().requires_grad_(True)
        sample = global_strided_sample(local, n_total, sh, topo.shard_group, max_sample)
        div = pool_diversity([sample], max_sample=max_sample)
        div.backward()
        out[n_total] = {"div": float(div), "grad": local.grad / world, "lo": lo, "hi": hi,
                        "rows": sample.detach().clone()}
    return out


def test_diversity_sample_of_a_sharded_pool_matches_the_global_sample():
    from dawn_srw_b200.ops.reference import pool_diversity
    outs = run_ranks(_diversity_worker, 2)
    for n_total, max_sample in ((50, 16), (21, 64)):
        full = torch.randn(n_total, 6, generator=torch.Generator().manual_seed(3)).requires_grad_(True)
        stride = max(1, n_total // max_sample) if n_total > max_sample else 1
        want_rows = full[::stride][:max_sample]
        ref = pool_diversity([full], max_sample=max_sample)
        ref.backward()
        for o in outs:
            r = o[n_total]
            assert torch.equal(r["rows"], want_rows.detach())
            assert abs(r["div"] - float(ref)) < 1e-6
            assert torch.allclose(r["grad"], full.grad[r["lo"]:r["hi"]], atol=1e-6)


def _dense_trainer_worker(rank, world, fsdp, ckpt_dir=None):
    import os
    from dawn_srw_b200.parallel.fsdp import full_state_dict
    from dawn_srw_b200.parallel.topology import init_topology
    from dawn_srw_b200.train.trainer import Trainer
    topo = init_topology(backend="gloo")
    cfg = tiny_config(version="baseline", max_steps=3, fsdp=fsdp)
    cfg.model.d_ff = 99                       # 99 rows over 2 ranks: blocks of 50 with one padding row
    tr = Trainer(cfg, topo=topo, device=torch.device("cpu"), total_steps=10, run_dir=ckpt_dir)
    for i in range(3):
        ids, mask = tr.train_loader.batch(i)
        m = tr.train_step(ids, mask)
    out = {"gn": float(m["grad_norm"]), "loss": float(m["total_loss"]), "fsdp": tr.fsdp,
           "local": sum(p.numel() for p in tr.model.parameters())}
    out["sd"] = {n: v.detach().clone() for n, v in full_state_dict(tr.model).items()}
    if ckpt_dir is not None:
        os.makedirs(ckpt_dir, exist_ok=True)
        tr.save("checkpoint_step3.pt")
        torch.distributed.barrier()
        tr2 = Trainer(cfg, topo=topo, device=torch.device("cpu"), total_steps=10, run_dir=ckpt_dir)
        tr2.resume(os.path.join(ckpt_dir, "checkpoint_step3.pt"))
        for t_ in (tr, tr2):
            ids, mask = t_.train_loader.batch(7)
            t_.train_step(ids, mask)
        out["resume_diff"] = max(float((a.detach() - b.detach()).abs().max()) for (_, a), (_, b) in zip(
            tr.model.named_parameters(), tr2.model.named_parameters()))
    return out


def test_row_sharded_dense_baseline_matches_replicated_training(tmp_path):
    """Linear weights of the dense baseline split by rows over the data-parallel ranks
    (gathered for each GEMM, gradients reduce-scattered): same losses, gradient norm and
    parameters as replicated data-parallel training; checkpoints are one file per rank
    and consolidate into the ordinary layout."""
    import glob
    from dawn_srw_b200.train import checkpoint as ck
    a = run_ranks(_dense_trainer_worker, 2, False)
    b = run_ranks(_dense_trainer_worker, 2, True, str(tmp_path / "run"))
    assert not a[0]["fsdp"] and b[0]["fsdp"]
    assert b[0]["local"] < 0.75 * a[0]["local"]              # a rank holds half of the layer weights
    for r in range(2):
        assert abs(a[r]["gn"] - b[r]["gn"]) < 1e-5 and abs(a[r]["loss"] - b[r]["loss"]) < 1e-5
        assert b[r]["resume_diff"] == 0.0
    for n in a[0]["sd"]:
        assert a[0]["sd"][n].shape == b[0]["sd"][n].shape, n
        assert torch.equal(b[0]["sd"][n], b[1]["sd"][n]), n
        if n.endswith("k_proj.bias"):
            continue      # softmax ignores a key bias: its gradient is rounding noise, which Adam normalises to +-lr
        assert torch.allclose(a[0]["sd"][n], b[0]["sd"][n], atol=2e-6), n
    files = sorted(glob.glob(str(tmp_path / "run" / "checkpoint_step3.shard*of2.pt")))
    assert len(files) == 2
    merged = torch.load(ck.consolidate(files, {}, str(tmp_path / "full.pt")), weights_only=False)
    for n, v in merged["params"].items():
        assert v.shape == a[0]["sd"][n].shape, n
    assert merged["opt_state"]["exp_avg"]["layers.0.ffn.w_up.weight"].shape == (99, 64)


def _hybrid_worker(rank, world, shard_pools, zero=False):
    from dawn_srw_b200.parallel.topology import init_topology
    from dawn_srw_b200.train.trainer import Trainer
    topo = init_topology(pool_shards=world, seq_shard=True, backend="gloo")
    cfg = tiny_config(version="spatial-r1-v4.1", max_steps=3, shard_pools=shard_pools, zero_pool_state=zero)
    tr = Trainer(cfg, topo=topo, device=torch.device("cpu"), total_steps=10)
    for i in range(3):
        ids, mask = tr.train_loader.batch(i)
        m = tr.train_step(ids, mask)
    return {"gn": float(m["grad_norm"]), "loss": float(m["total_loss"]), "opt": type(tr.optimizer).__name__,
            "sd": {n: p.detach().clone() for n, p in tr.model.named_parameters()}}


@pytest.mark.parametrize("zero", [False, True])
def test_small_pools_replicated_and_only_the_large_pool_sharded(zero):
    """training.shard_pools = [know]: the QK and V pools stay whole on every rank (their routes
    run on the rank's own tokens, their gradients are all-reduced), only the Know pool is
    split.  Same losses, gradient norm and parameters as with all pools sharded."""
    from dawn_srw_b200.parallel.topology import PoolShard
    a = run_ranks(_hybrid_worker, 2, None, zero)
    b = run_ranks(_hybrid_worker, 2, ["know"], zero)
    for r in range(2):
        assert abs(a[r]["gn"] - b[r]["gn"]) < 2e-5 and abs(a[r]["loss"] - b[r]["loss"]) < 2e-5

    def close(x, y, what):
        # the two layouts sum in different orders; Adam turns a rounding-level difference of a
        # near-zero gradient into a step of the size of the learning rate on single entries
        d = (x - y).abs()
        assert d.mean() < 2e-5 and d.max() < 5e-3, (what, float(d.mean()), float(d.max()))
    for n in a[0]["sd"]:
        if n.startswith("neuron_pool.qk_") or n.startswith("neuron_pool.v_"):
            if n.endswith("_scale"):
                continue
            full = b[0]["sd"][n]
            assert torch.equal(full, b[1]["sd"][n]), n                     # replicas stay identical
            n_units = full.shape[0]
            for k in range(2):
                lo, hi, _ = PoolShard(k, 2).slice_of(n_units)
                close(a[k]["sd"][n][: hi - lo], full[lo:hi], (n, k))
        else:
            close(a[0]["sd"][n], b[0]["sd"][n], n)
