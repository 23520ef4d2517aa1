#!/usr/bin/env python
"""Inference speed harness: full-sequence forward latency / throughput and
KV-cache generation speed of a model.

    python -m dawn_srw_b200.tools.bench_inference [--checkpoint run/best_model.pt | --config cfg.yaml]
        [--batch-sizes 1,8,32] [--seq-len 128] [--warmup 10] [--iters 100] [--new-tokens 32]

Method of the reference's harness (scripts/benchmark_speed.py:188-237): warm up,
then time ``iters`` forward passes with a device synchronisation per iteration
(latency mean / p50 / p95 in ms, tokens per second), plus tokens per second of
KV-cache sampling.  Prints one JSON line per batch size.
"""
from __future__ import annotations

import argparse
import json
import statistics
import sys
import time

import torch

from ..models.inference import generate, prefill
from .common import load_model


def _sync(dev):
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)


def run(model, vocab: int, batch: int, seq_len: int, warmup: int, iters: int, new_tokens: int):
    dev = next(model.parameters()).device
    g = torch.Generator(device="cpu").manual_seed(batch)
    ids = torch.randint(1, vocab, (batch, seq_len), generator=g).to(dev)
    for _ in range(warmup):
        prefill(model, ids)
    _sync(dev)
    lat = []
    for _ in range(iters):
        t0 = time.perf_counter()
        prefill(model, ids)
        _sync(dev)
        lat.append((time.perf_counter() - t0) * 1e3)
    lat.sort()
    mean = statistics.fmean(lat)
    rec = {"batch": batch, "seq_len": seq_len, "forward_ms_mean": mean,
           "forward_ms_p50": lat[len(lat) // 2], "forward_ms_p95": lat[min(len(lat) - 1, int(0.95 * len(lat)))],
           "forward_tokens_per_sec": batch * seq_len / (mean / 1e3)}
    if new_tokens > 0:
        prompt = ids[:, : max(1, min(8, seq_len - new_tokens))]
        generate(model, prompt, max_new_tokens=2)                      # warm-up
        _, stats = generate(model, prompt, max_new_tokens=new_tokens, temperature=1.0, top_k=50)
        rec["decode_tokens_per_sec"] = stats.get("steady_tokens_per_sec", stats["tokens_per_sec"])
        rec["decode_tokens_per_sec_with_first_step"] = stats["tokens_per_sec"]
        rec["decode_first_step_ms"] = 1e3 * stats["first_step_s"]
        rec["decode_graph"] = stats["graph"]
        rec["decode_new_tokens"] = stats["new_tokens"]
    return rec


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint")
    ap.add_argument("--config")
    ap.add_argument("--batch-sizes", default="1,8,32")
    ap.add_argument("--seq-len", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--new-tokens", type=int, default=32)
    ap.add_argument("--device")
    args = ap.parse_args(argv)
    model, cfg, _ = load_model(args.checkpoint, args.config, device=args.device)
    seq = min(args.seq_len, cfg.model.max_seq_len)
    for b in [int(x) for x in args.batch_sizes.split(",") if x]:
        print(json.dumps(run(model, cfg.model.vocab_size, b, seq, args.warmup, args.iters,
                             args.new_tokens)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
