import json
import os

import numpy as np
import pytest
import torch

from dawn_srw_b200.data.loaders import BinDataLoader, BinDataset, ShardedBinDataset, SyntheticDataset
from dawn_srw_b200.models.dawn import DAWN
from dawn_srw_b200.train import checkpoint as ck
from dawn_srw_b200.train.optimizer import DawnAdamW
from dawn_srw_b200.utils import flax_convert as fc


def test_bin_dataset_and_loader_slices(tmp_path):
    toks = np.arange(10 * 8 + 3, dtype=np.uint16)
    p = tmp_path / "t.bin"
    toks.tofile(p)
    ds = BinDataset(str(p), 8)
    assert len(ds) == 10
    a = BinDataLoader(ds, 4, batch_index=0, batch_replicas=2, pin=False)
    b = BinDataLoader(ds, 4, batch_index=1, batch_replicas=2, pin=False)
    assert len(a) == 2
    ia, _ = a.batch(1)
    ib, mb = b.batch(1)
    assert ia[0, 0] == 4 * 8 and ib[0, 0] == 6 * 8 and ia.shape == (2, 8) and int(mb.sum()) == 16
    a.reset(1)
    assert len(list(a)) == 1 and len(list(a)) == 2      # reset applies to the next pass only
    with pytest.raises(ValueError):
        BinDataLoader(ds, 5, batch_replicas=2)


def test_sharded_dataset_crosses_shard_boundaries(tmp_path):
    seq = 4
    shards = []
    start = 0
    for i, n in enumerate((3, 5, 2)):
        arr = np.arange(start, start + n * seq, dtype=np.uint16)
        path = tmp_path / f"d_{i:03d}.bin"
        arr.tofile(path)
        shards.append({"path": path.name, "sequences": n, "tokens": n * seq})
        start += n * seq
    (tmp_path / "_meta.json").write_text(json.dumps({"shards": shards, "vocab_size": 99, "num_shards": 3}))
    ds = ShardedBinDataset(str(tmp_path), seq)
    assert len(ds) == 10 and ds.vocab_size == 99
    rows = ds.rows(2, 9)
    assert np.array_equal(rows.flatten(), np.arange(2 * seq, 9 * seq))


def test_synthetic_rows_depend_only_on_index():
    ds = SyntheticDataset(32, 16, 1000, seed=3)
    assert np.array_equal(ds.rows(4, 6)[1], ds.rows(5, 6)[0])
    assert ds.rows(0, 4).max() < 1000


def _tiny():
    return DAWN(vocab_size=50, d_model=16, n_layers=1, n_heads=2, max_seq_len=8, d_route=4, n_qk=8,
                n_v=8, n_know=12)


def test_checkpoint_roundtrip_retention_and_latest(tmp_path):
    m = _tiny()
    opt = DawnAdamW(m.named_parameters(), lr=1e-3, fused=False)
    run = ck.new_run_dir(str(tmp_path), "spatial-r1-v4.1")
    kw = dict(epoch=0, step_in_epoch=0, steps_per_epoch=10, best_val_loss=1.0, config={}, training_config={})
    for s in (10, 20, 30, 40):
        ck.save_checkpoint(os.path.join(run, f"checkpoint_step{s}.pt"), m, opt, step=s, **kw)
    ck.save_checkpoint(os.path.join(run, "best_model.pt"), m, opt, step=20, **kw)
    ck.save_checkpoint(os.path.join(run, "checkpoint_epoch0.pt"), m, opt, step=25, **kw)
    ck.cleanup_old(run, keep_last=3)
    left = sorted(os.path.basename(f) for f in ck.list_checkpoints(run))
    assert left == ["best_model.pt", "checkpoint_epoch0.pt", "checkpoint_step20.pt",
                    "checkpoint_step30.pt", "checkpoint_step40.pt"]
    run_dir, latest = ck.find_latest(str(tmp_path))
    assert os.path.basename(latest) == "checkpoint_step40.pt"   # highest step, not best_model
    m2 = _tiny()
    with torch.no_grad():
        for p in m2.parameters():
            p.add_(1.0)
    blob = ck.load_checkpoint(latest, m2, None)
    assert blob["step"] == 40
    for a, b in zip(m.parameters(), m2.parameters()):
        assert torch.equal(a, b)


def test_corrupt_checkpoint_raises(tmp_path):
    m = _tiny()
    path = ck.save_checkpoint(str(tmp_path / "checkpoint_step1.pt"), m, None, epoch=0, step=1,
                              step_in_epoch=1, steps_per_epoch=1, best_val_loss=0.0, config={},
                              training_config={})
    data = bytearray(open(path, "rb").read())
    open(path, "wb").write(bytes(data[: len(data) // 2]))
    with pytest.raises(RuntimeError):
        ck.load_checkpoint(path, _tiny(), None)


def test_flax_msgpack_roundtrip_and_name_mapping(tmp_path):
    m = _tiny()
    sd = m.state_dict()
    path = str(tmp_path / "c.flax")
    fc.save_flax_checkpoint(path, sd, epoch=1, step=7, config={"d_model": 16})
    raw = fc.msgpack_restore(open(path, "rb").read())
    params = raw["params"]
    assert params["router"]["proj_attn"]["kernel"].shape == (16, 12)          # [in, out]
    assert params["block_0"]["attn"]["expand_O"]["kernel"].shape == (16, 16)
    assert params["block_0"]["norm1"]["scale"].shape == (16,)
    assert params["token_emb"]["embedding"].shape == (50, 16)
    assert params["neuron_pool"]["know_write"].shape == (12, 16)
    back = fc.load_flax_checkpoint(path)
    assert back["step"] == 7 and set(back["state_dict"]) == set(sd)
    for k in sd:
        assert torch.allclose(back["state_dict"][k], sd[k]), k
    # device-replicated checkpoints carry a leading singleton axis
    params["neuron_pool"]["qk_emb"] = params["neuron_pool"]["qk_emb"][None]
    sd2 = fc.flax_params_to_state_dict(params)
    assert sd2["neuron_pool.qk_emb"].shape == sd["neuron_pool.qk_emb"].shape


def test_optax_optimizer_state_converts_both_ways(tmp_path):
    """A hand-built tree in the layout flax.serialization gives an optax chain
    (tuple -> {"0",...}, NamedTuple -> field dict, EmptyState -> {}), with and
    without the MultiSteps wrapper, resumes DawnAdamW with its moments and
    step count; writing it back reproduces the tree."""
    import numpy as np
    m = _tiny()
    names = [n for n, _ in m.named_parameters()]
    rng = np.random.default_rng(0)
    sd = m.state_dict()
    mu = {n: torch.from_numpy(rng.standard_normal(tuple(sd[n].shape)).astype(np.float32)) for n in names}
    nu = {n: torch.from_numpy(rng.random(tuple(sd[n].shape)).astype(np.float32)) for n in names}
    acc = {n: torch.from_numpy(rng.standard_normal(tuple(sd[n].shape)).astype(np.float32)) for n in names}
    chain = {"0": {}, "1": {"count": np.asarray(7, np.int32), "mu": fc.state_dict_to_flax_params(mu),
                            "nu": fc.state_dict_to_flax_params(nu)},
             "2": {"inner_state": {}}, "3": {"inner_state": {}}, "4": {"count": np.asarray(7, np.int32)}}
    wrapped = {"mini_step": np.asarray(1, np.int32), "gradient_step": np.asarray(7, np.int32),
               "inner_opt_state": chain, "acc_grads": fc.state_dict_to_flax_params(acc), "skip_state": {}}
    # Dense kernels are stored [in, out] on the reference side
    assert chain["1"]["mu"]["router"]["proj_attn"]["kernel"].shape == (16, 12)
    for tree, k in ((chain, 1), (wrapped, 2)):
        path = str(tmp_path / f"c{k}.flax")
        open(path, "wb").write(fc.msgpack_serialize(
            {"params": fc.state_dict_to_flax_params(sd), "opt_state": tree, "epoch": 0, "step": 7 * k + (k - 1),
             "step_in_epoch": 3, "steps_per_epoch": 10, "best_val_loss": 2.5, "config": {}, "training_config": {}}))
        blob = fc.load_flax_checkpoint(path)
        st = blob["opt_state"]
        assert st["count"] == 7 and st["micro"] == (1 if k == 2 else 0)
        opt = DawnAdamW(m.named_parameters(), lr=1e-3, fused=False, accumulation_steps=k)
        opt.load_state_dict(st)
        assert opt.count == 7 and opt.micro == st["micro"]
        for (n, _), a, b in zip(opt.named, opt.exp_avg, opt.exp_avg_sq):
            assert torch.equal(a, mu[n]) and torch.equal(b, nu[n]), n
        if k == 2:      # the running mean of one micro-step is that micro-step's gradient sum
            for (n, _), a in zip(opt.named, opt._acc):
                assert torch.allclose(a, acc[n]), n
        back = fc.torch_opt_state_to_optax(opt.state_dict(), accumulation_steps=k)
        flat_a, flat_b = fc.flatten_tree(tree), fc.flatten_tree(back)
        assert set(flat_a) == set(flat_b)
        for key in flat_a:
            assert np.allclose(np.asarray(flat_a[key]), np.asarray(flat_b[key])), key
    # the command-line converter carries the optimizer state through
    from dawn_srw_b200.tools import convert_ckpt as cc
    pt = str(tmp_path / "c.pt")
    assert cc.main(["flax2pt", str(tmp_path / "c1.flax"), pt]) == 0
    assert torch.load(pt, weights_only=False)["opt_state"]["count"] == 7
    assert cc.main(["pt2flax", pt, str(tmp_path / "back.flax")]) == 0
    again = fc.load_flax_checkpoint(str(tmp_path / "back.flax"))
    assert again["opt_state"]["count"] == 7
    assert torch.equal(again["opt_state"]["exp_avg"]["router.proj_attn.weight"], mu["router.proj_attn.weight"])


def test_shard_consolidation(tmp_path):
    from dawn_srw_b200.parallel.topology import PoolShard
    full = _tiny()
    paths = []
    for i in range(2):
        m = DAWN(vocab_size=50, d_model=16, n_layers=1, n_heads=2, max_seq_len=8, d_route=4, n_qk=8,
                 n_v=8, n_know=12, pool_shard=PoolShard(i, 2))
        paths.append(ck.save_checkpoint(str(tmp_path / "checkpoint_step3.pt"), m, None, epoch=0, step=3,
                                        step_in_epoch=3, steps_per_epoch=9, best_val_loss=0.0, config={},
                                        training_config={}, shard_index=i, shard_count=2))
    out = ck.consolidate(paths, {"qk": 8, "v": 8, "know": 12}, str(tmp_path / "full.pt"))
    blob = torch.load(out, weights_only=False)
    for k, v in full.state_dict().items():
        assert torch.equal(blob["params"][k], v), k


def test_incomplete_shard_sets_are_not_resumed_from(tmp_path):
    """A job that died between two ranks' shard writes leaves shard 0 of the
    newest step without its siblings: auto-resume must fall back to the last
    complete step, and retention must not delete that step."""
    from dawn_srw_b200.parallel.topology import PoolShard
    run = ck.new_run_dir(str(tmp_path), "spatial-r1-v4.0.1")
    kw = dict(epoch=0, step_in_epoch=0, steps_per_epoch=10, best_val_loss=1.0, config={}, training_config={})
    models = [DAWN(vocab_size=50, d_model=16, n_layers=1, n_heads=2, max_seq_len=8, d_route=4, n_qk=8,
                   n_v=8, n_know=12, pool_shard=PoolShard(i, 2)) for i in range(2)]
    for s in (10, 20):
        for i, m in enumerate(models):
            ck.save_checkpoint(os.path.join(run, f"checkpoint_step{s}.pt"), m, None, step=s,
                               shard_index=i, shard_count=2, **kw)
    # step 30: only shard 0 made it to disk
    ck.save_checkpoint(os.path.join(run, "checkpoint_step30.pt"), models[0], None, step=30,
                       shard_index=0, shard_count=2, **kw)
    names = sorted(os.path.basename(f) for f in ck.list_checkpoints(run))
    assert names == ["checkpoint_step10.shard0of2.pt", "checkpoint_step20.shard0of2.pt"]
    _, latest = ck.find_latest(str(tmp_path))
    assert os.path.basename(latest) == "checkpoint_step20.shard0of2.pt"
    # rank 1 of the fallback step loads fine; the incomplete step would not
    assert ck.load_checkpoint(latest, models[1], None, shard_index=1, shard_count=2)["step"] == 20
    with pytest.raises(FileNotFoundError):
        ck.load_checkpoint(os.path.join(run, "checkpoint_step30.pt"), models[1], None,
                           shard_index=1, shard_count=2)
    # retention keeps the newest complete step and does not touch the newer, unfinished one
    removed = [os.path.basename(f) for f in ck.cleanup_old(run, keep_last=1)]
    assert sorted(removed) == ["checkpoint_step10.shard0of2.pt", "checkpoint_step10.shard1of2.pt"]
    assert os.path.exists(os.path.join(run, "checkpoint_step30.shard0of2.pt"))
    assert os.path.basename(ck.find_latest(str(tmp_path))[1]) == "checkpoint_step20.shard0of2.pt"


def test_fileio_local_and_url_paths(tmp_path):
    """The five file operations on local paths and on an fsspec URL (the
    in-process ``memory://`` filesystem stands in for a bucket)."""
    import numpy as np
    from dawn_srw_b200.config import load_config
    from dawn_srw_b200.data.loaders import load_data
    from dawn_srw_b200.utils import fileio as F
    p = str(tmp_path / "a" / "b.txt")
    with F.open_file(p, "w") as f:
        f.write("x")
    assert F.file_exists(p) and F.list_files(str(tmp_path / "a" / "*.txt")) == [p]
    F.delete_file(p)
    assert not F.file_exists(p)
    url = "memory://bucket/cfg.yaml"
    with F.open_file(url, "w") as f:
        f.write("seed: 7\nmodel:\n  d_model: 96\n")
    assert F.is_remote(url) and F.file_exists(url)
    cfg = load_config(url)
    assert cfg.seed == 7 and cfg.model.d_model == 96
    assert any(q.endswith("cfg.yaml") for q in F.list_files("memory://bucket/*.yaml"))
    # a remote token file is copied into the local cache and memory-mapped from there
    toks = (np.arange(16 * 8) % 100).astype(np.uint16)
    with F.open_file("memory://bucket/train.bin", "wb") as f:
        f.write(toks.tobytes())
    cfg.data.bin_train, cfg.data.bin_val = "memory://bucket/train.bin", None
    cfg.data.local_cache_dir = str(tmp_path / "cache")
    tl, vl, _ = load_data(cfg.data, 8, 4, 100)
    ids, mask = tl.batch(0)
    assert ids.shape == (4, 8) and int(ids[0, 1]) == 1 and vl is None
    F.delete_file(url)
    import pytest
    with pytest.raises(RuntimeError):
        F.file_exists("nosuchscheme://x/y")


def test_prefetching_loader_yields_the_same_batches_and_propagates_errors(tmp_path):
    import numpy as np
    import pytest
    from dawn_srw_b200.data.loaders import BinDataLoader, BinDataset, SyntheticDataset
    ds = SyntheticDataset(64, 8, 100, seed=3)
    plain = [b[0].clone() for b in BinDataLoader(ds, 8, prefetch=0)]
    ahead = [b[0].clone() for b in BinDataLoader(ds, 8, prefetch=3)]
    assert len(plain) == len(ahead) == 8 and all(torch.equal(a, b) for a, b in zip(plain, ahead))
    ld = BinDataLoader(ds, 8, prefetch=2)
    ld.reset(5)                                                   # resume position
    assert [int(b[0][0, 0]) for b in ld] == [int(p[0, 0]) for p in plain[5:]]
    it = iter(BinDataLoader(ds, 8, prefetch=2))                   # abandoning an iterator stops its thread
    next(it)
    it.close()

    class Broken(SyntheticDataset):
        def rows(self, lo, hi):
            if lo >= 16:
                raise OSError("disk went away")
            return super().rows(lo, hi)
    with pytest.raises(OSError):
        list(BinDataLoader(Broken(64, 8, 100), 8, prefetch=2))


def test_consolidate_keeps_replicated_pools_whole(tmp_path):
    """Shard files of a hybrid layout (only the Know pool split): the Know rows are
    concatenated with the padding dropped, the QK pool is taken as it is."""
    import torch
    from dawn_srw_b200.parallel.topology import PoolShard
    from dawn_srw_b200.train import checkpoint as ck
    n_know, n_qk = 21, 10
    know = torch.arange(n_know * 4, dtype=torch.float32).reshape(n_know, 4)
    qk = torch.randn(n_qk, 4)
    paths = []
    for k in range(2):
        lo, hi, padded = PoolShard(k, 2).slice_of(n_know)
        rows = torch.zeros(padded, 4)
        rows[: hi - lo] = know[lo:hi]
        blob = {"params": {"neuron_pool.know_emb": rows, "neuron_pool.qk_emb": qk.clone(),
                           "norm.weight": torch.ones(4)},
                "opt_state": None, "step": 3, "shard": {"index": k, "count": 2},
                "sharded_pools": ["know"]}
        path = str(tmp_path / f"checkpoint_step3.shard{k}of2.pt")
        torch.save(blob, path)
        paths.append(path)
    merged = torch.load(ck.consolidate(paths, {"know": n_know, "qk": n_qk, "v": 0}, str(tmp_path / "full.pt")),
                        weights_only=False)
    assert torch.equal(merged["params"]["neuron_pool.know_emb"], know)
    assert torch.equal(merged["params"]["neuron_pool.qk_emb"], qk)
    assert "sharded_pools" not in merged and merged["shard"] == {"index": 0, "count": 1}
