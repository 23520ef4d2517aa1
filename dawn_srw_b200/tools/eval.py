#!/usr/bin/env python
"""Validation loss / perplexity / accuracy of a checkpoint on a token file.

    python -m dawn_srw_b200.tools.eval --checkpoint run/best_model.pt --bin-val val.bin
        [--config cfg.yaml] [--batch-size 32] [--max-batches 200] [--synthetic]
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from ..data.loaders import BinDataLoader, BinDataset, SyntheticDataset
from ..models.inference import vectorized_eval
from .common import load_model


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint")
    ap.add_argument("--config")
    ap.add_argument("--bin-val")
    ap.add_argument("--batch-size", type=int, default=32)
    ap.add_argument("--max-batches", type=int, default=200)
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--library", action="store_true")
    args = ap.parse_args(argv)
    model, cfg, info = load_model(args.checkpoint, args.config, library=args.library)
    S = cfg.model.max_seq_len
    if args.synthetic or not args.bin_val:
        ds = SyntheticDataset(args.batch_size * 4, S, cfg.model.vocab_size, seed=1)
    else:
        ds = BinDataset(args.bin_val, S, cfg.data.max_val_tokens)
    loader = BinDataLoader(ds, args.batch_size, pin=False)
    dev = next(model.parameters()).device

    def batches():
        for i, (ids, _) in enumerate(loader):
            if i >= args.max_batches:
                break
            yield ids.to(dev)
    loss, ppl, acc, n = vectorized_eval(model, batches())
    print(json.dumps({"val_loss": loss, "ppl": ppl, "accuracy_pct": acc, "valid_tokens": n, **info}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
