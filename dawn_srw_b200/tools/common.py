"""Shared helpers for the command-line tools: build a model from a checkpoint
(native ``.pt`` or reference ``.flax``) or from a config file."""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from ..config import Config, config_from_dict, load_config
from ..models.registry import build_model_from_config
from ..utils import flax_convert as fc


def load_model(checkpoint: Optional[str] = None, config: Optional[str] = None, device=None,
               library: bool = False):
    """Returns (model, cfg, info).  ``checkpoint`` may be a ``.pt`` written by the
    trainer or a ``.flax`` blob of the reference; the model section of the
    checkpoint overrides the YAML's."""
    device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
    cfg = load_config(config) if config else Config()
    blob, sd = {}, None
    if checkpoint:
        if checkpoint.endswith(".flax"):
            blob = fc.load_flax_checkpoint(checkpoint)
            sd = blob["state_dict"]
        else:
            blob = torch.load(checkpoint, map_location="cpu", weights_only=False)
            sd = blob["params"]
        mc = blob.get("config") or {}
        for k, v in mc.items():
            k = {"d_bottleneck": "d_route", "dropout_rate": "dropout"}.get(k, k)
            if hasattr(cfg.model, k):
                setattr(cfg.model, k, v)
        if sd is not None and "token_emb.weight" in sd:
            cfg.model.vocab_size = sd["token_emb.weight"].shape[0]
    backend = None
    if library and device.type == "cuda":
        from ..ops.backend import ReferenceBackend
        backend = ReferenceBackend(torch.bfloat16, chunk_size=12500)
    model = build_model_from_config(cfg, backend=backend)
    if sd is not None:
        missing, unexpected = model.load_state_dict(sd, strict=False)
        if missing or unexpected:
            print(f"[load_model] missing {list(missing)[:5]} unexpected {list(unexpected)[:5]}")
    model.to(device).eval()
    info = {k: blob.get(k) for k in ("epoch", "step", "best_val_loss") if k in blob}
    return model, cfg, info


def tokenizer_or_none(name: str = "bert-base-uncased"):
    """The reference tokenises with ``bert-base-uncased`` (scripts/pretokenize_c4.py);
    it is only available when its files are in the local HF cache."""
    try:
        from transformers import AutoTokenizer
        return AutoTokenizer.from_pretrained(name, local_files_only=True)
    except Exception:
        return None
