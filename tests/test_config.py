import warnings

import pytest
import yaml

from dawn_srw_b200.config import MODEL_PRESETS, config_from_dict, preset
from dawn_srw_b200.models.registry import MODEL_REGISTRY, build_model_from_config, count_parameters

REF_STYLE_YAML = """
seed: 1
data:
  bin_train: /data/c4_train
  bin_val: /data/c4_val.bin
  max_val_tokens: 10000000
model:
  model_version: "spatial-r1-v4.0.1"
  d_model: 1280
  n_layers: 18
  n_heads: 16
  d_route: 256
  n_know: 100000
  n_qk: 6400
  n_v: 10400
  max_seq_len: 512
  dropout: 0.1
  gradient_checkpointing: true
  router_dropout: 0.1
training:
  batch_size: 1024
  mesh_model: 2
  mesh_data: 8
  n_chunks_know: 4
  lr: 0.0003
  weight_decay: 0.1
  warmup_ratio: 0.08
  epsilon: 1.0e-4
  load_balance_weight: 0.1
use_amp: true
checkpoint_dir: /tmp/ckpt
"""


def test_reference_yaml_loads_with_aliases():
    cfg = config_from_dict(yaml.safe_load(REF_STYLE_YAML))
    assert cfg.seed == 1 and cfg.model.d_model == 1280 and cfg.model.n_know == 100000
    assert cfg.training.pool_shards == 2 and cfg.training.dp == 8      # mesh_model / mesh_data
    assert cfg.training.lr == 3e-4 and cfg.training.epsilon == pytest.approx(1e-4)
    assert cfg.model.d_head == 80 and cfg.model.is_spatial


def test_unknown_keys_warn():
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        config_from_dict({"model": {"d_modle": 3}, "trainin": {}})
    assert len(w) == 2


def test_d_bottleneck_and_learning_rate_aliases():
    cfg = config_from_dict({"model": {"d_bottleneck": 96}, "training": {"learning_rate": 1e-3}})
    assert cfg.model.d_route == 96 and cfg.training.lr == 1e-3


def _formula_params(m):
    D, L, r, V, S = m["d_model"], m["n_layers"], m["d_route"], 30522, 512
    pool = (m["n_qk"] + m["n_v"] + m["n_know"]) * (r + 2 * D)
    scales = 0 if m["model_version"].endswith("v3.9.4") else 3
    router = D * 3 * r + 3 * r + D * r + r + D * 3 + 3 + D + 1
    blocks = L * (4 * D + D * D)
    return V * D + S * D + pool + scales + router + blocks + 2 * D


def test_parameter_counts_match_published():
    # 40.2 M is the published count of the 40M model; the others follow from the shapes
    assert _formula_params(MODEL_PRESETS["40M"]) == 40_228_871
    assert abs(_formula_params(MODEL_PRESETS["400M"]) / 1e6 - 399.5) < 0.1
    assert abs(_formula_params(MODEL_PRESETS["1B"]) / 1e6 - 970.3) < 0.1
    model = build_model_from_config(preset("40M"))
    assert count_parameters(model) == 40_228_871


def test_registry_versions():
    assert {"baseline", "spatial-r1-v3.9.4", "spatial-r1-v4.0.1", "spatial-r1-v4.1"} <= set(MODEL_REGISTRY)
    cfg = preset("40M")
    cfg.model.model_version = "spatial-r1-v9"
    with pytest.raises(ValueError):
        build_model_from_config(cfg)


def test_validate_config_reports_every_problem_at_once():
    import pytest
    from dawn_srw_b200.config import preset, validate_config
    cfg = preset("40M")
    validate_config(cfg, world=8, pool_shards=1, on_gpu=True)               # the shipped shape is fine
    cfg.model.d_model, cfg.model.n_heads = 100, 3
    cfg.training.batch_size = 30
    cfg.model.dropout = 1.5
    with pytest.raises(ValueError) as e:
        validate_config(cfg, world=8, pool_shards=2, on_gpu=True)
    msg = str(e.value)
    assert "n_heads" in msg and "batch_size" in msg and "dropout" in msg and "multiple of 8" in msg
    cfg = preset("40M", d_model=384, n_heads=16)                             # head dimension 24
    validate_config(cfg, on_gpu=False)
    with pytest.raises(ValueError, match="head dimension 24"):
        validate_config(cfg, on_gpu=True)
    cfg = preset("40M")
    cfg.training.batch_size, cfg.training.seq_shard = 12, False
    validate_config(cfg, world=8, pool_shards=4)                             # 2 replicas share 12 sequences
    cfg.training.seq_shard = True
    with pytest.raises(ValueError, match="batch_size"):
        validate_config(cfg, world=8, pool_shards=4)                         # 8 ranks each take a slice
