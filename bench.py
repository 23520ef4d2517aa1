#!/usr/bin/env python
"""Flagship benchmark: DAWN-SRW training throughput (tokens/s, whole job).

    python bench.py --gpus N --steps K --warmup W [--model 400M] [--parallelism pool|dp]

For N > 1 launch one rank per GPU, e.g.
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

What is timed: full training steps (forward, loss assembly incl. auxiliary
losses, backward, gradient synchronisation, clip + AdamW) of the named model at
bf16 compute with fp32 master weights, on synthetic uniform-random tokens and
random-init weights.  Weak scaling: the per-GPU batch is fixed.

Two measurements of K steps each, both bracketed by barrier + synchronize:
  * device-timed (`value`): CUDA events on the launching stream, max over ranks;
    the step's inputs are already on the device.
  * end to end (`e2e`): the public ``Trainer.train_step`` API fed from pinned
    host memory every step (host-to-device copy of ids + mask) with a
    device-to-host read of the loss every step; wall clock between
    synchronizes, max over ranks.
SM clocks and throttle reasons are sampled with nvidia-smi during the timed
regions.  ``--impl reference`` reports whether the unmodified reference can run.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "library"])
    ap.add_argument("--model", default="400M", choices=["40M", "400M", "1B"])
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--batch-per-gpu", type=int, default=0, help="sequences per GPU per step")
    ap.add_argument("--parallelism", default="pool", choices=["pool", "dp"])
    ap.add_argument("--pool-shards", type=int, default=0,
                    help="with --parallelism pool: unit shards per pool (a divisor of --gpus); the "
                         "remaining factor is data parallel (e.g. --gpus 8 --pool-shards 4 = dp2 x pool4). "
                         "0 = all GPUs shard the pools")
    ap.add_argument("--shard-pools", default="",
                    help="comma-separated pools that are split over the pool shards (default: all "
                         "of qk,v,know); the others are kept whole on every rank, e.g. "
                         "--shard-pools know")
    ap.add_argument("--optimizer", default="auto", choices=["auto", "partitioned", "replicated"],
                    help="partitioned: reduce-scatter + AdamW on the owned slice + all-gather over "
                         "peer memory with sharded moments; auto = partitioned for --parallelism dp")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--log-step", action="store_true",
                    help="after the timed runs, also time steps that produce the full routing "
                         "diagnostics (what a logging step of the trainer costs)")
    ap.add_argument("--no-shard-check", action="store_true",
                    help="skip the one-off comparison of the sharded model's loss with the same "
                         "model unsharded on rank 0 (runs before the warm-up, N > 1 only)")
    ap.add_argument("--profile", metavar="FILE",
                    help="after the timed runs, profile one more step with torch.profiler and "
                         "write the per-kernel device-time table of rank 0 to FILE")
    return ap.parse_args()


def reference_arm(args):
    """The reference is a JAX/Flax program (scripts/train_jax.py); this image
    has no jax, flax or optax and no wheel for them offline."""
    root = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref")
    why = None
    if not os.path.isdir(root):
        why = "baseline/_ref is not installed"
    else:
        try:
            import jax  # noqa: F401
            import flax  # noqa: F401
            import optax  # noqa: F401
        except Exception as e:
            why = (f"the reference's train step needs jax+flax+optax ({type(e).__name__}: {e}); "
                   "none is installed or in the offline wheelhouse")
    if why is None:
        why = "reference import succeeded but no GPU runner for its TPU mesh code is wired up"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def parse_clock_csv(text: str):
    """Summary of `nvidia-smi --query-gpu=... --format=csv,noheader,nounits -lms` output
    (fields of ClockSampler.FIELDS): median SM clock under load, maximum SM clock and
    the throttle reasons that were active in any sample.  None if no line parses."""
    sm, smax, reasons = [], [], set()
    for line in text.splitlines():
        f = [x.strip() for x in line.split(",")]
        if len(f) < 9:
            continue
        try:
            sm.append(float(f[1]))
            smax.append(float(f[2]))
        except ValueError:
            continue
        for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                              "sw_power_cap"), f[5:9]):
            if val.lower().startswith("active"):
                reasons.add(name)
    if not sm:
        return None
    return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
            "samples": len(sm)}


class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.path = tempfile.mktemp(prefix="clocks_", suffix=".csv")
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.gpu), "-lms", "200"], stdout=open(self.path, "w"),
                stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            text = open(self.path).read()
            os.remove(self.path)
        except Exception:
            return out
        return parse_clock_csv(text) or out


def sharded_vs_unsharded(trainer, cfg, topo, dev, batch):
    """Before anything is timed: the deterministic (no dropout) cross-entropy of the
    sharded model on the global batch against the SAME model (same seed, so the same
    weights) built unsharded on rank 0 and fed all ranks' sequences.  Returns the two
    losses and their difference on rank 0 (None elsewhere)."""
    import copy
    import torch
    import torch.distributed as dist
    from dawn_srw_b200.parallel.topology import Topology
    from dawn_srw_b200.train.trainer import Trainer
    ids, mask = batch
    labels = torch.where(mask == 1, ids, torch.full_like(ids, -100))
    model = trainer.model
    was_training = model.training
    model.eval()
    with torch.no_grad():
        r = model(ids, labels=labels, attention_mask=mask, want_diag=False)
        acc = torch.stack([r["loss"].double() * r["valid_count"], r["valid_count"].double()])
    model.train(was_training)
    dist.all_reduce(acc)
    sharded = float(acc[0] / acc[1])
    all_ids = [torch.empty_like(ids) for _ in range(topo.world)] if topo.is_main else None
    all_mask = [torch.empty_like(mask) for _ in range(topo.world)] if topo.is_main else None
    dist.gather(ids, all_ids, dst=0)
    dist.gather(mask, all_mask, dst=0)
    out = None
    if topo.is_main:
        cfg1 = copy.deepcopy(cfg)
        cfg1.training.pool_shards, cfg1.training.seq_shard, cfg1.training.zero_pool_state = 1, False, False
        cfg1.training.dp = 1
        ref = Trainer(cfg1, topo=Topology(), device=dev, total_steps=10, build_data=False)
        ref.model.eval()
        tot = torch.zeros(2, dtype=torch.float64, device=dev)
        with torch.no_grad():
            for i_, m_ in zip(all_ids, all_mask):            # one rank's sequences at a time
                lab = torch.where(m_ == 1, i_, torch.full_like(i_, -100))
                rr = ref.model(i_, labels=lab, attention_mask=m_, want_diag=False)
                tot += torch.stack([rr["loss"].double() * rr["valid_count"], rr["valid_count"].double()])
        unsharded = float(tot[0] / tot[1])
        del ref
        torch.cuda.empty_cache()
        out = {"sharded": sharded, "unsharded": unsharded, "abs_diff": abs(sharded - unsharded),
               "ok": abs(sharded - unsharded) < 1e-2}
    dist.barrier()
    return out


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)
    import torch
    import torch.distributed as dist
    from dawn_srw_b200.config import preset
    from dawn_srw_b200.parallel.topology import init_topology
    from dawn_srw_b200.train.trainer import Trainer
    from dawn_srw_b200.ops import backend as B

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs a torchrun launch with {args.gpus} ranks "
                             f"(WORLD_SIZE={world})")
    pool_shards = world if (args.parallelism == "pool" and world > 1) else 1
    if pool_shards > 1 and args.pool_shards:
        if world % args.pool_shards != 0:
            raise SystemExit(f"--pool-shards {args.pool_shards} does not divide {world} GPUs")
        pool_shards = args.pool_shards
    topo = init_topology(pool_shards=pool_shards, seq_shard=True)
    dev = torch.device("cuda", topo.local_rank)
    torch.cuda.set_device(dev)

    bpg = args.batch_per_gpu or {"40M": 64, "400M": 32, "1B": 16}[args.model]
    cfg = preset(args.model)
    cfg.model.max_seq_len = args.seq_len
    cfg.model.gradient_checkpointing = False     # 180 GB HBM: nothing needs recomputing per layer
    t = cfg.training
    t.batch_size = bpg * world
    t.pool_shards, t.seq_shard = pool_shards, True
    if args.shard_pools and pool_shards > 1:
        t.shard_pools = [n.strip() for n in args.shard_pools.split(",") if n.strip()]
    t.log_interval = 0
    opt_mode = args.optimizer
    if opt_mode == "auto":
        opt_mode = "partitioned" if (args.parallelism == "dp" and world > 1) else "replicated"
    t.zero_pool_state = opt_mode == "partitioned" and world > 1
    cfg.data.synthetic = True
    cfg.data.synthetic_sequences = t.batch_size * 4
    # loss weights of the named reference configs
    if args.model == "400M":
        t.lr, t.warmup_ratio, t.load_balance_weight, t.diversity_weight = 3e-4, 0.08, 0.1, 0.1
    elif args.model == "1B":
        t.lr, t.load_balance_weight, t.diversity_weight = 2e-4, 0.1, 0.1
    else:
        t.load_balance_weight, t.dead_penalty_weight, t.exploration_weight = 0.0, 0.05, 1e-3
        cfg.model.dropout, cfg.model.router_dropout = 0.05, 0.02
    backend = None
    if args.impl == "library":
        backend = B.ReferenceBackend(torch.bfloat16, chunk_size=12500, use_checkpoint=True)
    trainer = Trainer(cfg, topo=topo, device=dev, backend=backend, total_steps=100000)

    # K distinct batches, staged in pinned host memory (cycled)
    host_batches = [trainer.train_loader.batch(i % len(trainer.train_loader)) for i in range(4)]
    dev_batches = [(a.to(dev), b.to(dev)) for a, b in host_batches]
    tokens_per_step = t.batch_size * args.seq_len

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    from dawn_srw_b200.ops import cuda_backend as CB
    shard_check = None
    if world > 1 and args.impl == "ours" and not args.no_shard_check:
        shard_check = sharded_vs_unsharded(trainer, cfg, topo, dev, dev_batches[0])
    for i in range(args.warmup):
        trainer.train_step(*dev_batches[i % 4])
    barrier()

    # ---- device-timed --------------------------------------------------
    launches0 = CB.launch_count() if args.impl == "ours" else 0
    sampler = ClockSampler(topo.local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        m = trainer.train_step(*dev_batches[i % 4])
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    launches = (CB.launch_count() - launches0) if args.impl == "ours" else 0
    loss_val = float(m["total_loss"])

    # ---- end to end through the public API -----------------------------
    e2e = None
    if not args.no_e2e:
        barrier()
        t0 = time.perf_counter()
        for i in range(args.steps):
            m = trainer.train_step(*host_batches[i % 4])      # H2D copy from pinned memory
            _ = float(m["total_loss"])                        # D2H read of the step's loss
        barrier()
        e2e_s = time.perf_counter() - t0
        h2d = sum(x.numel() * x.element_size() for x in host_batches[0])
        e2e = (e2e_s, h2d, 4)

    log_step = None
    if args.log_step:
        trainer.train_step(*dev_batches[0], want_diag=True)          # warm the diagnostic path
        barrier()
        l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0.record()
        for i in range(2):
            trainer.train_step(*dev_batches[i % 4], want_diag=True)
        l1.record()
        barrier()
        log_step = l0.elapsed_time(l1) / 2

    if args.profile:
        from torch.profiler import ProfilerActivity, profile
        barrier()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            trainer.train_step(*dev_batches[0])
            torch.cuda.synchronize()
        if topo.is_main:
            rows = sorted(((e.key, e.device_time_total / 1e3, e.count) for e in prof.key_averages()
                           if e.device_time_total > 0), key=lambda r: -r[1])
            with open(args.profile, "w") as f:
                f.write(f"# one training step, rank 0 of {world}; total device time "
                        f"{sum(r[1] for r in rows):.1f} ms\n")
                for k, t_ms, n in rows[:40]:
                    f.write(f"{t_ms:10.2f} ms {n:6d}x  {k[:120]}\n")

    trainer.backend.finish_run()          # raise now if any kernel reported a device-side failure
    vals = torch.tensor([ms, e2e[0] if e2e else 0.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms, e2e_s = vals.tolist()
    if topo.is_main:
        ms_per_step = ms / args.steps
        value = tokens_per_step / (ms_per_step / 1e3)
        out = {
            "metric": f"train tokens/s/box (device-timed, max over ranks) DAWN-SRW {args.model}",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform tokens, random init", "impl": args.impl,
            "config": {"model": f"DAWN-SRW {args.model} ({cfg.model.model_version})",
                       "global_batch": t.batch_size, "seq_len": args.seq_len,
                       "parallelism": ((f"dp{world // pool_shards}x" if pool_shards < world else "")
                                       + f"pool{pool_shards}"
                                       + (f"[{','.join(t.shard_pools)} only]" if t.shard_pools else "")
                                       + "+seqshard" if pool_shards > 1 else f"dp{world}"),
                       "l2": "inputs and weights per step exceed the 126 MB L2 (no flush needed)",
                       "layer_recompute": False,
                       "optimizer": type(trainer.optimizer).__name__},
            "clocks": clocks, "gpu_launches": launches, "final_loss": loss_val,
        }
        if log_step is not None:
            out["log_step"] = {"ms": log_step, "ratio_to_normal_step": log_step / ms_per_step}
        if shard_check is not None:
            out["sharded_vs_unsharded_ce"] = shard_check
        if e2e:
            out["e2e"] = {"value": tokens_per_step * args.steps / e2e_s, "unit": "tokens/s",
                          "h2d_bytes_per_step": e2e[1], "d2h_bytes_per_step": e2e[2]}
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
