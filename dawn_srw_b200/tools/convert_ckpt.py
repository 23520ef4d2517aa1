#!/usr/bin/env python
"""Checkpoint conversion and consolidation.

    python -m dawn_srw_b200.tools.convert_ckpt flax2pt  in.flax out.pt
    python -m dawn_srw_b200.tools.convert_ckpt pt2flax  in.pt   out.flax
    python -m dawn_srw_b200.tools.convert_ckpt consolidate out.pt shard0.pt shard1.pt ...

``flax2pt`` / ``pt2flax`` map between the reference's Flax parameter tree and
optax optimizer state (msgpack) and this framework's torch state dict and AdamW
state, so a run can be resumed on either side with its moments and step count
(see utils/flax_convert.py;
the reference's own converter, scripts/convert_flax_to_pt.py, covers only its
older model families).  ``consolidate`` merges per-shard checkpoints of a
pool-sharded run into the single-file layout.
"""
from __future__ import annotations

import sys

import torch

from ..train import checkpoint as ck
from ..utils import flax_convert as fc


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv:
        print(__doc__)
        return 2
    cmd = argv.pop(0)
    if cmd == "flax2pt":
        src, dst = argv
        blob = fc.load_flax_checkpoint(src)
        out = {k: v for k, v in blob.items() if k != "state_dict"}
        out["params"] = blob["state_dict"]
        out.setdefault("step", 0)
        torch.save(out, dst)
        has_opt = out.get("opt_state") is not None
        print(f"wrote {dst}: {len(out['params'])} tensors" +
              (f", Adam moments at optimizer step {out['opt_state']['count']}" if has_opt else
               ", no optimizer state"))
    elif cmd == "pt2flax":
        src, dst = argv
        blob = torch.load(src, map_location="cpu", weights_only=False)
        fields = {k: blob[k] for k in ("epoch", "step", "step_in_epoch", "steps_per_epoch",
                                       "best_val_loss", "config", "training_config") if k in blob}
        k = int((blob.get("training_config") or {}).get("gradient_accumulation_steps", 1) or 1)
        opt = blob.get("opt_state")
        if opt is not None and "exp_avg" not in opt:
            opt = None          # a partitioned optimizer's per-rank state is not convertible
        fc.save_flax_checkpoint(dst, blob["params"], opt_state=opt, accumulation_steps=k, **fields)
        print(f"wrote {dst}")
    elif cmd == "consolidate":
        dst, shards = argv[0], argv[1:]
        first = torch.load(shards[0], map_location="cpu", weights_only=False)
        cfg = first.get("config") or {}
        sizes = {"qk": cfg.get("n_qk"), "v": cfg.get("n_v"), "know": cfg.get("n_know")}
        ck.consolidate(shards, sizes, dst)
        print(f"wrote {dst} from {len(shards)} shards")
    else:
        print(__doc__)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main())
