#!/usr/bin/env python
"""CPU reference step: DAWN-SRW 40M (v4.1 config shapes), fp32, batch 2 x seq 128,
forward + backward + AdamW through the oracle backend, uniform-random tokens
from a seed, random init.

    python -m dawn_srw_b200.tools.bench_cpu [--steps 3] [--warmup 1] [--threads N]

Prints one JSON line (ms per step, tokens/s, parameter count, final loss).  This
is the configuration the CPU oracle tests use; it doubles as the timed CPU
baseline of the same math the kernels implement.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--threads", type=int, default=0)
    args = ap.parse_args(argv)
    if args.threads:
        torch.set_num_threads(args.threads)
    from ..config import preset
    from ..ops.backend import ReferenceBackend
    from ..train.trainer import Trainer
    cfg = preset("40M")
    cfg.model.max_seq_len = 128
    cfg.model.dropout = cfg.model.router_dropout = 0.0
    t = cfg.training
    t.batch_size, t.log_interval = 2, 0
    t.load_balance_weight, t.dead_penalty_weight, t.exploration_weight = 0.0, 0.05, 1e-3
    cfg.data.synthetic, cfg.data.synthetic_sequences = True, 16
    cfg.seed = 1
    dev = torch.device("cpu")
    tr = Trainer(cfg, device=dev, backend=ReferenceBackend(torch.float32), total_steps=1000)
    n_params = sum(p.numel() for p in tr.model.parameters())
    batches = [tr.train_loader.batch(i % len(tr.train_loader)) for i in range(4)]
    for i in range(args.warmup):
        tr.train_step(*batches[i % 4])
    t0 = time.perf_counter()
    for i in range(args.steps):
        m = tr.train_step(*batches[i % 4])
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    print(json.dumps({"metric": "CPU fp32 train step, DAWN-SRW 40M, batch 2 x seq 128",
                      "ms_per_step": dt * 1e3, "tokens_per_sec": 2 * 128 / dt, "parameters": n_params,
                      "threads": torch.get_num_threads(), "final_loss": float(m["total_loss"]),
                      "steps": args.steps, "warmup": args.warmup}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
