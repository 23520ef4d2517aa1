"""Model registry: ``model_version`` string -> class + constructor kwargs.

Registered (reference: scripts/train_jax.py:171-214 registers ``baseline``,
``spatial-r1-v3.9.4`` and ``spatial-r1-v4.1``; ``spatial-r1-v4.0.1`` is the
paper model whose file the reference keeps under models/legacy/).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict

from ..config import Config
from ..ops.gates import gate_spec_for
from .baseline import VanillaTransformer
from .dawn import DAWN


@dataclass
class ModelSpec:
    name: str
    cls: Any
    build_kwargs: Callable[[Config], Dict[str, Any]]
    supports_sharded: bool = False


def _baseline_kwargs(cfg: Config) -> Dict[str, Any]:
    m = cfg.model
    return dict(vocab_size=m.vocab_size, d_model=m.d_model, d_ff=m.d_ff, n_layers=m.n_layers,
                n_heads=m.n_heads, max_seq_len=m.max_seq_len, dropout_rate=m.dropout,
                gradient_checkpointing=m.gradient_checkpointing, seed=cfg.seed)


def _dawn_kwargs(cfg: Config) -> Dict[str, Any]:
    m = cfg.model
    return dict(vocab_size=m.vocab_size, d_model=m.d_model, n_layers=m.n_layers, n_heads=m.n_heads,
                max_seq_len=m.max_seq_len, d_route=m.d_route, n_qk=m.n_qk, n_v=m.n_v,
                n_know=m.n_know, dropout_rate=m.dropout, router_dropout=m.router_dropout,
                gradient_checkpointing=m.gradient_checkpointing, model_version=m.model_version,
                gate=gate_spec_for(m.model_version, cfg.training), seed=cfg.seed)


MODEL_REGISTRY: Dict[str, ModelSpec] = {
    "baseline": ModelSpec("baseline", VanillaTransformer, _baseline_kwargs),
    "spatial-r1-v3.9.4": ModelSpec("spatial-r1-v3.9.4", DAWN, _dawn_kwargs, True),
    "spatial-r1-v4.0.1": ModelSpec("spatial-r1-v4.0.1", DAWN, _dawn_kwargs, True),
    "spatial-r1-v4.1": ModelSpec("spatial-r1-v4.1", DAWN, _dawn_kwargs, True),
}


def build_model_from_config(cfg: Config, *, pool_shard=None, backend=None, sharded_pools=None):
    version = cfg.model.model_version
    if version not in MODEL_REGISTRY:
        raise ValueError(f"Unknown model_version: {version!r}. Known: {sorted(MODEL_REGISTRY)}")
    spec = MODEL_REGISTRY[version]
    kw = spec.build_kwargs(cfg)
    if spec.supports_sharded and pool_shard is not None:
        kw["pool_shard"] = pool_shard
        if sharded_pools is not None:
            kw["sharded_pools"] = list(sharded_pools)
    kw["backend"] = backend
    return spec.cls(**kw)


def count_parameters(model) -> int:
    return sum(p.numel() for p in model.parameters())
