"""Checkpoint save / load / retention / resume discovery.

Run folder layout (reference: scripts/train_jax.py:1096-1154, 283-361, 1774-1820):

    <checkpoint_dir>/run_v<version>_<YYYYMMDD_HHMMSS>_<rand4>/
        checkpoint_step<N>.pt      keep the newest ``keep_last`` of these
        checkpoint_epoch<E>.pt     kept
        best_model.pt              kept
        emergency_step<N>.pt       kept (written on preemption)
        config.json                {"model": ..., "training": ...}
        training_log_<ts>.txt, metrics_<ts>.jsonl

Each file is a ``torch.save`` dict with the reference's fields: ``params``
(state dict, names convertible 1:1 to the Flax tree), ``opt_state``, ``epoch``,
``step``, ``step_in_epoch``, ``steps_per_epoch``, ``best_val_loss``, ``config``
(model section), ``training_config``.  With sharded pools every shard rank
writes ``<name>.shard<k>of<n>.pt`` holding only its pool rows (no gather);
``consolidate`` rebuilds the single-file layout.

Resume picks the checkpoint with the highest *step*.  (The reference's file
sort puts ``best_model`` last, so its auto-resume prefers an older best model
over a newer step checkpoint; that is not reproduced.)
"""
from __future__ import annotations

import datetime
import glob
import json
import os
import random
import re
import string
from typing import Any, Dict, List, Optional, Tuple

import torch

KEEP_ALWAYS = ("best_model", "checkpoint_epoch", "emergency_step")


def new_run_dir(checkpoint_dir: str, version: str) -> str:
    kst = datetime.datetime.utcnow() + datetime.timedelta(hours=9)
    tag = "".join(random.choices(string.ascii_lowercase + string.digits, k=4))
    path = os.path.join(checkpoint_dir, f"run_v{version}_{kst.strftime('%Y%m%d_%H%M%S')}_{tag}")
    os.makedirs(path, exist_ok=True)
    return path


def _step_of(path: str) -> int:
    m = re.search(r"(?:checkpoint_step|emergency_step)(\d+)", os.path.basename(path))
    return int(m.group(1)) if m else -1


def _shard_set_complete(path: str) -> bool:
    """A sharded checkpoint ``<name>.shard0of<N>.pt`` counts only when all N
    shard files are present (each is written atomically by its own rank, so a
    job that died between two ranks' writes leaves an incomplete set)."""
    m = re.search(r"^(.*)\.shard0of(\d+)(\.[^.]+)$", path)
    if not m:
        return True
    base, n, ext = m.group(1), int(m.group(2)), m.group(3)
    return all(os.path.exists(f"{base}.shard{k}of{n}{ext}") for k in range(n))


def list_checkpoints(run_dir: str) -> List[str]:
    """Loadable checkpoints of a run folder: single files, and shard 0 of every
    sharded checkpoint whose shard set is complete."""
    files = [f for f in glob.glob(os.path.join(run_dir, "*.pt"))
             if ".shard" not in f or (".shard0of" in f and _shard_set_complete(f))]
    return sorted(files)


def peek_step(path: str) -> int:
    s = _step_of(path)
    if s >= 0:
        return s
    try:
        return int(torch.load(path, map_location="cpu", weights_only=False).get("step", -1))
    except Exception:
        return -1


def find_latest(checkpoint_dir: str) -> Optional[Tuple[str, str]]:
    """(run_dir, checkpoint_path) with the highest step in the newest run folder
    that has any checkpoint, else None."""
    runs = sorted(glob.glob(os.path.join(checkpoint_dir, "run_*")), key=os.path.getmtime,
                  reverse=True)
    for run in runs:
        ck = list_checkpoints(run)
        if ck:
            best = max(ck, key=peek_step)
            return run, best
    return None


def cleanup_old(run_dir: str, keep_last: int = 3) -> List[str]:
    """Delete all but the newest ``keep_last`` *complete* step checkpoints.
    Steps newer than the newest complete one are left alone (other ranks may
    still be writing their shard files); older incomplete sets are removed."""
    by_step: Dict[int, List[str]] = {}
    for f in glob.glob(os.path.join(run_dir, "checkpoint_step*.pt")):
        by_step.setdefault(_step_of(f), []).append(f)

    def complete(files: List[str]) -> bool:
        heads = [f for f in files if ".shard" not in f or ".shard0of" in f]
        return bool(heads) and all(_shard_set_complete(f) for f in heads)
    done = sorted(s for s, fs in by_step.items() if complete(fs))
    keep = set(done[-keep_last:]) if keep_last > 0 else set()
    newest_done = done[-1] if done else -1
    removed = []
    for s_, files in sorted(by_step.items()):
        if s_ in keep or s_ > newest_done:
            continue
        for f in files:
            os.remove(f)
            removed.append(f)
    return removed


def shard_suffix(index: int, count: int) -> str:
    return "" if count == 1 else f".shard{index}of{count}"


def save_checkpoint(path: str, model, optimizer, *, epoch: int, step: int, step_in_epoch: int,
                    steps_per_epoch: int, best_val_loss: float, config: Dict, training_config: Dict,
                    shard_index: int = 0, shard_count: int = 1, extra: Optional[Dict] = None) -> str:
    base, ext = os.path.splitext(path)
    path = f"{base}{shard_suffix(shard_index, shard_count)}{ext}"
    blob = {
        "params": {k: v.detach().cpu() for k, v in model.state_dict().items()},
        "opt_state": None if optimizer is None else _cpu_tree(optimizer.state_dict()),
        "epoch": epoch, "step": step, "step_in_epoch": step_in_epoch,
        "steps_per_epoch": steps_per_epoch, "best_val_loss": float(best_val_loss),
        "config": config, "training_config": training_config,
        "shard": {"index": shard_index, "count": shard_count},
    }
    if extra:
        blob.update(extra)
    tmp = path + ".tmp"
    torch.save(blob, tmp)
    os.replace(tmp, path)
    return path


def _cpu_tree(x):
    if isinstance(x, torch.Tensor):
        return x.detach().cpu()
    if isinstance(x, dict):
        return {k: _cpu_tree(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(_cpu_tree(v) for v in x)
    return x


def load_checkpoint(path: str, model=None, optimizer=None, *, shard_index: int = 0,
                    shard_count: int = 1, strict: bool = True) -> Dict[str, Any]:
    """Load ``path`` (or this rank's shard file next to it).  A corrupt or
    truncated file raises instead of yielding a half-restored state."""
    base, ext = os.path.splitext(path)
    base = re.sub(r"\.shard\d+of\d+$", "", base)
    cand = f"{base}{shard_suffix(shard_index, shard_count)}{ext}"
    if not os.path.exists(cand):
        raise FileNotFoundError(cand)
    try:
        blob = torch.load(cand, map_location="cpu", weights_only=False)
    except Exception as e:  # truncated zip, bad pickle, ...
        raise RuntimeError(f"checkpoint {cand} is unreadable: {e}") from e
    for key in ("params", "step"):
        if key not in blob:
            raise RuntimeError(f"checkpoint {cand} lacks field {key!r}")
    if model is not None:
        model.load_state_dict(blob["params"], strict=strict)
    if optimizer is not None and blob.get("opt_state") is not None:
        optimizer.load_state_dict(blob["opt_state"])
    return blob


def consolidate(paths: List[str], pool_sizes: Dict[str, int], out_path: str) -> str:
    """Merge per-shard files (ordered by shard index) into one full checkpoint:
    pool rows are concatenated with padding dropped, everything else is taken
    from shard 0."""
    blobs = [torch.load(p, map_location="cpu", weights_only=False) for p in sorted(
        paths, key=lambda p: int(re.search(r"\.shard(\d+)of", p).group(1)))]
    count = len(blobs)
    from ..parallel.topology import PoolShard
    merged = dict(blobs[0])
    row_blocks = blobs[0].get("fsdp_rows") or {}     # dense weights stored as per-rank row blocks
    sharded_pools = blobs[0].get("sharded_pools")    # None: every pool is split over the shards

    def merge_tree(trees):
        out = {}
        for k, v in trees[0].items():
            m = re.search(r"(qk|v|know)_(emb|read|write)$", k)
            if k in row_blocks and isinstance(v, torch.Tensor) and v.dim() == 2:
                out[k] = torch.cat([t[k] for t in trees], 0)[: row_blocks[k]]
            elif (m and isinstance(v, torch.Tensor) and v.dim() == 2
                  and (sharded_pools is None or m.group(1) in sharded_pools)):
                n = pool_sizes[m.group(1)]
                rows = []
                for i, t in enumerate(trees):
                    lo, hi, _ = PoolShard(i, count).slice_of(n)
                    rows.append(t[k][: hi - lo])
                out[k] = torch.cat(rows, 0)
            else:
                out[k] = v
        return out
    merged["params"] = merge_tree([b["params"] for b in blobs])
    if blobs[0].get("opt_state"):
        os0 = dict(blobs[0]["opt_state"])
        for key in ("exp_avg", "exp_avg_sq"):
            os0[key] = merge_tree([b["opt_state"][key] for b in blobs])
        merged["opt_state"] = os0
    merged["shard"] = {"index": 0, "count": 1}
    merged.pop("fsdp_rows", None)
    merged.pop("sharded_pools", None)
    torch.save(merged, out_path)
    return out_path
