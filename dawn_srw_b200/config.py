"""Typed view of the training YAML schema.

The YAML layout (sections ``seed``, ``data``, ``model``, ``training`` and the
top-level ``use_amp`` / ``checkpoint_dir`` / ``log_dir``) is the one the
reference trainer reads with ``dict.get`` (reference: scripts/train_jax.py:83-90,
116-168, 1660-1694, 2020, 2253-2285).  The reference config files load here
unchanged; unknown keys produce a warning instead of being silently ignored,
and the TPU mesh keys ``mesh_model`` / ``mesh_data`` are accepted as aliases of
``pool_shards`` / ``dp``.
"""
from __future__ import annotations

import dataclasses
import json
import warnings
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import yaml


@dataclass
class DataConfig:
    bin_train: Optional[str] = None
    bin_val: Optional[str] = None
    max_train_tokens: Optional[int] = None
    max_val_tokens: int = 10_000_000
    local_cache_dir: Optional[str] = None
    # additions: synthetic uniform-random token source (benchmarks, tests)
    synthetic: bool = False
    synthetic_sequences: int = 4096


@dataclass
class ModelConfig:
    model_version: str = "spatial-r1-v4.1"
    vocab_size: int = 30522
    d_model: int = 384
    n_layers: int = 12
    n_heads: int = 6
    max_seq_len: int = 512
    d_route: int = 128
    n_qk: int = 1580
    n_v: int = 2600
    n_know: int = 25200
    dropout: float = 0.1
    router_dropout: float = 0.1
    gradient_checkpointing: bool = False
    d_ff: int = 1536  # dense baseline only

    @property
    def d_head(self) -> int:
        return self.d_model // self.n_heads

    @property
    def is_spatial(self) -> bool:
        return self.model_version.startswith("spatial")


@dataclass
class TrainingConfig:
    batch_size: int = 128                # global batch (sequences)
    gradient_accumulation_steps: int = 1
    num_epochs: int = 1
    lr: float = 6.5e-4
    weight_decay: float = 0.1
    pool_weight_decay: float = 0.02
    warmup_ratio: float = 0.06
    orthogonality_weight: float = 0.01
    diversity_weight: float = 0.1
    load_balance_weight: float = 2e-5
    tau_reg_weight: float = 0.0
    entropy_weight: float = 0.0          # carried by the dense-baseline configs; no live loss term uses it
    process_norm_weight: float = 0.0     # likewise
    dead_penalty_weight: float = 0.0
    dead_penalty_threshold: float = 0.01
    sharpness: float = 500.0
    activation_threshold: float = 0.5
    activation_cutoff: float = 0.01
    epsilon: float = 1e-4
    max_intensity: float = 10.0
    exploration_weight: float = 0.0
    exploration_asymmetry: float = 0.15
    exploration_warmup_steps: int = 5000
    exploration_lower_bound: float = -0.5
    exploration_upper_bound: float = 2.0
    exploration_bound_eps: float = 1e-3
    # parallel layout.  pool_shards: ranks over which pool units are split;
    # dp: data-parallel replicas (0 = world / pool_shards); seq_shard: keep the
    # activations between pool ops sharded over the pool-shard group.
    pool_shards: int = 1
    dp: int = 0
    seq_shard: bool = True
    zero_pool_state: bool = False
    shard_pools: Optional[List[str]] = None   # pools split over pool_shards ranks (None: all); the rest are replicated
    fsdp: bool = False                   # dense baseline: Linear weights sharded by rows over the data-parallel ranks
    overlap_grad_reduce: bool = True     # replicated-parameter gradients are all-reduced during backward
    n_chunks_know: int = 0
    n_chunks_qk: int = 0
    n_chunks_v: int = 0
    max_chunk_size: int = 12500
    target_chunk_gb: float = 2.0
    checkpoint_interval: int = 5000
    val_interval: int = 5000
    log_interval: int = 100
    log_analysis_multiplier: int = 20
    max_steps: int = 0                   # 0 = run the configured epochs
    max_val_batches: int = 200
    keep_last_checkpoints: int = 3

    _ALIASES = {"learning_rate": "lr", "mesh_model": "pool_shards", "mesh_data": "dp"}


@dataclass
class Config:
    seed: int = 42
    data: DataConfig = field(default_factory=DataConfig)
    model: ModelConfig = field(default_factory=ModelConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    use_amp: bool = True
    checkpoint_dir: str = "checkpoints_b200"
    log_dir: Optional[str] = None

    # ------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        d = dataclasses.asdict(self)
        d["training"].pop("_ALIASES", None)
        return d

    def model_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self.model)

    def training_dict(self) -> Dict[str, Any]:
        d = dataclasses.asdict(self.training)
        d.pop("_ALIASES", None)
        return d


_MODEL_ALIASES = {"d_bottleneck": "d_route", "dropout_rate": "dropout"}


def _fill(dc_cls, raw: Dict[str, Any], aliases: Dict[str, str], section: str):
    names = {f.name for f in dataclasses.fields(dc_cls) if not f.name.startswith("_")}
    kwargs = {}
    for key, val in (raw or {}).items():
        name = aliases.get(key, key)
        if name in names:
            if key != name and name in kwargs:
                continue  # canonical key wins over its alias
            kwargs[name] = val
        else:
            warnings.warn(f"config: unknown key {section}.{key!r} ignored", stacklevel=3)
    obj = dc_cls(**kwargs)
    # coerce numeric strings such as "1.0e-4" that YAML 1.1 leaves as str
    for f in dataclasses.fields(dc_cls):
        v = getattr(obj, f.name, None)
        if isinstance(v, str) and f.type in ("float", "int"):
            setattr(obj, f.name, float(v) if f.type == "float" else int(float(v)))
    return obj


def config_from_dict(raw: Dict[str, Any]) -> Config:
    raw = dict(raw or {})
    cfg = Config(
        seed=int(raw.pop("seed", 42)),
        data=_fill(DataConfig, raw.pop("data", {}), {}, "data"),
        model=_fill(ModelConfig, raw.pop("model", {}), _MODEL_ALIASES, "model"),
        training=_fill(TrainingConfig, raw.pop("training", {}),
                       TrainingConfig._ALIASES, "training"),
        use_amp=bool(raw.pop("use_amp", True)),
        checkpoint_dir=raw.pop("checkpoint_dir", "checkpoints_b200"),
        log_dir=raw.pop("log_dir", None),
    )
    for key in raw:
        warnings.warn(f"config: unknown top-level key {key!r} ignored", stacklevel=2)
    return cfg


def validate_config(cfg: Config, world: int = 1, pool_shards: int = 1, on_gpu: bool = False) -> None:
    """Reject configurations that cannot run, with the reason, before any
    memory is allocated (the reference fails late inside XLA for most of these)."""
    m, t = cfg.model, cfg.training
    errs = []
    if m.d_model % m.n_heads != 0:
        errs.append(f"model.d_model ({m.d_model}) is not a multiple of model.n_heads ({m.n_heads})")
    elif on_gpu and ((m.d_model // m.n_heads) % 16 != 0 or m.d_model // m.n_heads > 128):
        errs.append(f"head dimension {m.d_model // m.n_heads} is outside what the attention kernels "
                    "take (a multiple of 16, at most 128)")
    if on_gpu and m.d_model % 8 != 0:
        errs.append(f"model.d_model ({m.d_model}) must be a multiple of 8 (16-byte rows for TMA)")
    if m.is_spatial:
        if on_gpu and m.d_route % 8 != 0:
            errs.append(f"model.d_route ({m.d_route}) must be a multiple of 8 (16-byte rows for TMA)")
        for name in ("n_qk", "n_v", "n_know"):
            if getattr(m, name) < max(1, pool_shards):
                errs.append(f"model.{name} ({getattr(m, name)}) is smaller than the number of pool shards")
    if world % max(1, pool_shards) != 0:
        errs.append(f"world size {world} is not a multiple of training.pool_shards ({pool_shards})")
    else:
        dp = world // max(1, pool_shards)
        batch_shards = world if (pool_shards == 1 or t.seq_shard) else dp
        if t.batch_size % max(1, batch_shards) != 0:
            errs.append(f"training.batch_size ({t.batch_size}) is not divisible by the {batch_shards} "
                        "ranks that each take a slice of the batch")
    if not (0.0 <= m.dropout < 1.0 and 0.0 <= m.router_dropout < 1.0):
        errs.append("dropout rates must be in [0, 1)")
    if t.gradient_accumulation_steps < 1:
        errs.append("training.gradient_accumulation_steps must be at least 1")
    if m.max_seq_len < 2:
        errs.append("model.max_seq_len must be at least 2 (next-token loss)")
    if errs:
        raise ValueError("invalid configuration:\n  - " + "\n  - ".join(errs))


def load_config(path: str) -> Config:
    """YAML from a local path or an fsspec URL."""
    from .utils.fileio import open_file
    with open_file(path, "r") as f:
        return config_from_dict(yaml.safe_load(f))


def apply_overrides(cfg: Config, *, epochs=None, batch_size=None, lr=None,
                    run_config: Optional[Dict[str, Any]] = None) -> Config:
    """Resume precedence: CLI > run-folder ``config.json`` > YAML
    (reference: scripts/train_jax.py:1842-1897)."""
    if run_config:
        for k, v in (run_config.get("training") or {}).items():
            name = TrainingConfig._ALIASES.get(k, k)
            if hasattr(cfg.training, name) and not name.startswith("_"):
                setattr(cfg.training, name, v)
    if epochs is not None:
        cfg.training.num_epochs = int(epochs)
    if batch_size is not None:
        cfg.training.batch_size = int(batch_size)
    if lr is not None:
        cfg.training.lr = float(lr)
    return cfg


def save_run_config(cfg: Config, path: str) -> None:
    with open(path, "w") as f:
        json.dump({"model": cfg.model_dict(), "training": cfg.training_dict()}, f, indent=2)


# ---------------------------------------------------------------------------
# Named model shapes used by the benchmarks.
MODEL_PRESETS: Dict[str, Dict[str, Any]] = {
    "40M": dict(model_version="spatial-r1-v4.1", d_model=384, n_layers=12, n_heads=6,
                d_route=128, n_qk=1580, n_v=2600, n_know=25200),
    "400M": dict(model_version="spatial-r1-v4.0.1", d_model=1280, n_layers=18, n_heads=16,
                 d_route=256, n_qk=6400, n_v=10400, n_know=100000),
    "1B": dict(model_version="spatial-r1-v3.9.4", d_model=2048, n_layers=18, n_heads=16,
               d_route=384, n_qk=9900, n_v=16100, n_know=158800),
}


def preset(name: str, **overrides) -> Config:
    cfg = Config()
    for k, v in {**MODEL_PRESETS[name], **overrides}.items():
        if hasattr(cfg.model, k):
            setattr(cfg.model, k, v)
        elif hasattr(cfg.training, k):
            setattr(cfg.training, k, v)
        else:
            raise KeyError(k)
    return cfg
