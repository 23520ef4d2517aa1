#!/usr/bin/env python
"""KV-cache text generation (temperature / top-k / top-p).

    python -m dawn_srw_b200.tools.generate --checkpoint run/best_model.pt --prompt "the cat"
        [--max-new-tokens 64] [--temperature 0.8] [--top-k 50] [--top-p 0.0] [--ids 101,2023,...]

Without a local ``bert-base-uncased`` tokenizer pass ``--ids`` and read ids back.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch

from ..models.inference import generate
from .common import load_model, tokenizer_or_none


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint")
    ap.add_argument("--config")
    ap.add_argument("--prompt", default="")
    ap.add_argument("--ids", default="")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=0)
    args = ap.parse_args(argv)
    model, cfg, _ = load_model(args.checkpoint, args.config)
    dev = next(model.parameters()).device
    tok = tokenizer_or_none()
    if args.ids:
        ids = [int(x) for x in args.ids.split(",")]
    elif tok is not None and args.prompt:
        ids = tok.encode(args.prompt, add_special_tokens=False)
    else:
        ids = [101]
    stop = [tok.sep_token_id, tok.pad_token_id] if tok is not None else []
    g = torch.Generator(device=dev).manual_seed(args.seed)
    seq, stats = generate(model, torch.tensor([ids], device=dev), args.max_new_tokens, args.temperature,
                          args.top_k, args.top_p, stop_ids=stop, generator=g)
    out = {"ids": seq[0].tolist(), **stats}
    if tok is not None:
        out["text"] = tok.decode(seq[0].tolist())
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
