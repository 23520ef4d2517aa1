#!/usr/bin/env python
"""Training entry point.

    python -m dawn_srw_b200.tools.train --config configs/<file>.yaml [--from-scratch]
        [--resume-from PATH] [--epochs N] [--batch-size N] [--lr X] [--max-steps N] [--synthetic]

Multi-GPU: ``python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1
-m dawn_srw_b200.tools.train --config ...`` (one rank per GPU).

Resume (reference: scripts/train_jax.py:1774-1897): without ``--from-scratch``
rank 0 looks for the newest ``run_*`` folder under ``checkpoint_dir`` that holds
a checkpoint, picks the one with the highest step and broadcasts the choice, so
every rank resumes the same file; training hyper-parameters come from that
run's ``config.json`` unless overridden on the command line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from ..config import apply_overrides, load_config
from ..parallel.topology import init_topology
from ..train import checkpoint as ckpt
from ..train.trainer import Trainer


def broadcast_str(s: str, topo) -> str:
    """Rank 0's string to every rank (fixed 1 KiB buffer over the host group)."""
    if topo.world == 1:
        return s
    buf = torch.zeros(1024, dtype=torch.uint8)
    if topo.is_main:
        b = s.encode()[:1024]
        buf[: len(b)] = torch.tensor(list(b), dtype=torch.uint8)
    dist.broadcast(buf, src=0, group=topo.cpu_group)
    return bytes(buf.tolist()).rstrip(b"\0").decode()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--from-scratch", action="store_true")
    ap.add_argument("--resume-from")
    ap.add_argument("--epochs", type=int)
    ap.add_argument("--batch-size", type=int)
    ap.add_argument("--lr", type=float)
    ap.add_argument("--max-steps", type=int)
    ap.add_argument("--synthetic", action="store_true", help="uniform-random tokens instead of files")
    ap.add_argument("--library", action="store_true", help="library baseline backend (torch matmuls)")
    ap.add_argument("--checkpoint-dir", help="override the config's checkpoint_dir")
    ap.add_argument("--debug", action="store_true")
    ap.add_argument("--trace-steps", type=int, default=0,
                    help="after training, run this many extra steps with device-timed ranges "
                         "(forward blocks, backward, optimizer) and print the table; DAWN_NVTX=1 "
                         "additionally emits NVTX ranges for external profilers")
    ap.add_argument("--no-startup-check", action="store_true",
                    help="skip the start-up memory check and per-block timing table")
    args = ap.parse_args(argv)

    cfg = load_config(args.config)
    if args.checkpoint_dir:
        cfg.checkpoint_dir = args.checkpoint_dir
    t = cfg.training
    topo = init_topology(pool_shards=t.pool_shards, dp=t.dp, seq_shard=t.seq_shard)
    if args.synthetic:
        cfg.data.synthetic = True

    resume_path, run_dir = "", ""
    if args.resume_from:
        resume_path = args.resume_from
        run_dir = os.path.dirname(os.path.abspath(resume_path))
    elif not args.from_scratch and topo.is_main:
        found = ckpt.find_latest(cfg.checkpoint_dir)
        if found:
            run_dir, resume_path = found
    run_dir = broadcast_str(run_dir, topo)
    resume_path = broadcast_str(resume_path, topo)
    run_cfg = None
    if run_dir and os.path.exists(os.path.join(run_dir, "config.json")):
        run_cfg = json.load(open(os.path.join(run_dir, "config.json")))
    apply_overrides(cfg, epochs=args.epochs, batch_size=args.batch_size, lr=args.lr, run_config=run_cfg)
    if args.max_steps:
        t.max_steps = args.max_steps
    if not run_dir:
        if topo.is_main:
            run_dir = ckpt.new_run_dir(cfg.checkpoint_dir, cfg.model.model_version)
        run_dir = broadcast_str(run_dir, topo)

    backend = None
    if args.library and torch.cuda.is_available():
        from ..ops.backend import ReferenceBackend
        backend = ReferenceBackend(torch.bfloat16, chunk_size=t.max_chunk_size, use_checkpoint=True)
    trainer = Trainer(cfg, topo=topo, run_dir=run_dir, backend=backend)
    if resume_path:
        trainer.resume(resume_path)
        trainer.logger.message(f"Resumed from {resume_path} at step {trainer.global_step}")
    if not args.no_startup_check:
        from ..train.startup import startup_report
        startup_report(trainer, print_fn=trainer.logger.message)
    out = trainer.fit()
    if args.trace_steps > 0:
        from ..utils import tracing
        tracing.enable(timers=True)
        for i in range(args.trace_steps):
            trainer.train_step(*trainer.train_loader.batch(i % max(len(trainer.train_loader), 1)))
        rep = tracing.report()
        tracing.enable(timers=False)
        trainer.logger.message("[trace] %d steps\n%s" % (args.trace_steps, tracing.format_report(rep)))
    if topo.is_main:
        print(json.dumps({"final": out, "run_dir": run_dir}))
    if topo.world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
