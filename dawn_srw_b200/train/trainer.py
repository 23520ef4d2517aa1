"""Training runtime: model + optimizer + data + step + loop.

``Trainer.train_step(ids, mask)`` is the public per-step API: it takes the
step's token batch from (pinned) host memory, copies it to the device, runs
forward, loss assembly, backward, gradient synchronisation and the optimizer,
and returns the metrics as device tensors (``float(metrics["total_loss"])`` is
the single device-to-host read per step the reference also performs).

``Trainer.fit()`` is the loop (reference: scripts/train_jax.py:2884-3260):
per-step NaN guard, token-weighted window averages, two-cadence logging,
periodic validation and checkpoints, cooperative preemption (SIGTERM sets a
flag; every 10 steps the flag is OR-reduced over ranks on the host-side gloo
group so all ranks leave the loop together and write ``emergency_step<N>``),
resume with mid-epoch data position, and a post-resume check that every rank
agrees on the global step.
"""
from __future__ import annotations

import json
import math
import os
import signal
import time
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist

from ..config import Config, validate_config, save_run_config
from ..data.loaders import load_data
from ..models.registry import build_model_from_config, count_parameters
from ..ops.backend import default_backend
from ..parallel.grad_sync import GradSync
from ..parallel.topology import Topology
from . import checkpoint as ckpt
from . import logging as L
from .losses import total_loss
from ..utils.tracing import trace
from .optimizer import DawnAdamW, warmup_cosine


class NonFiniteLoss(ValueError):
    pass


class Trainer:
    def __init__(self, cfg: Config, *, topo: Optional[Topology] = None, device=None, backend=None,
                 run_dir: Optional[str] = None, total_steps: Optional[int] = None,
                 build_data: bool = True):
        self.cfg = cfg
        self.topo = topo or Topology()
        if device is None:
            device = torch.device("cuda", self.topo.local_rank) if torch.cuda.is_available() \
                else torch.device("cpu")
        self.device = torch.device(device)
        validate_config(cfg, world=self.topo.world, pool_shards=self.topo.pool_shards,
                        on_gpu=self.device.type == "cuda" and backend is None)
        self.backend = backend or default_backend(self.device)
        t, m = cfg.training, cfg.model
        self.is_baseline = not m.is_spatial
        self.train_loader = self.val_loader = None
        if build_data:
            self.train_loader, self.val_loader, vocab = load_data(
                cfg.data, m.max_seq_len, t.batch_size, m.vocab_size,
                batch_index=self.topo.batch_index, batch_replicas=self.topo.batch_replicas,
                seed=cfg.seed)
            m.vocab_size = vocab
        shard = self.topo.pool_shard if self.topo.pool_shards > 1 else None
        self.model = build_model_from_config(cfg, pool_shard=shard, backend=self.backend,
                                             sharded_pools=t.shard_pools).to(self.device)
        self.model.set_parallel(shard_group=self.topo.shard_group, dp_group=self.topo.dp_group,
                                seq_sharded=self.topo.seq_shard, world_group=self.topo.world_group)
        self.fsdp = bool(t.fsdp) and self.is_baseline and self.topo.world > 1
        if self.fsdp:
            # every rank built the same full weights (same seed); keep this rank's rows only
            from ..parallel.fsdp import shard_dense_weights
            shard_dense_weights(self.model, self.topo.world_group)
        self.steps_per_epoch = len(self.train_loader) if self.train_loader is not None else 0
        k = max(1, t.gradient_accumulation_steps)
        if total_steps is None:
            total_steps = max(1, t.num_epochs * (self.steps_per_epoch // k))
            if t.max_steps:
                # max_steps counts micro-steps (like global_step, the log / val / checkpoint
                # cadences and the reference's loop); the schedule runs on optimizer steps
                horizon = max(1, t.max_steps // k)
                total_steps = min(total_steps, horizon) if self.steps_per_epoch else horizon
        self.total_steps = total_steps
        warm = int(total_steps * t.warmup_ratio)
        self.schedule = lambda s: warmup_cosine(s, t.lr, warm, total_steps)
        if t.zero_pool_state and self.topo.world > 1 and not self.fsdp:
            # replicated parameters: reduce-scatter + AdamW on the owned slice + all-gather,
            # moments sharded over the replicas
            from ..parallel.zero import PartitionedAdamW
            self.optimizer = PartitionedAdamW(
                self.model.named_parameters(), self.topo, lr=t.lr, weight_decay=t.weight_decay,
                pool_weight_decay=t.pool_weight_decay, schedule=self.schedule,
                accumulation_steps=k)
        else:
            sync = GradSync(self.topo) if self.topo.world > 1 else None
            if sync is not None and k == 1 and t.overlap_grad_reduce:
                sync.attach(self.model.named_parameters())     # reduce while backward still runs
            self.optimizer = DawnAdamW(
                self.model.named_parameters(), lr=t.lr, weight_decay=t.weight_decay,
                pool_weight_decay=t.pool_weight_decay, schedule=self.schedule, accumulation_steps=k,
                grad_sync=sync)
        self.global_step = 0          # micro-steps taken
        self.epoch = 0
        self.step_in_epoch = 0
        self.best_val_loss = float("inf")
        self.run_dir = run_dir
        self.logger = L.RunLogger(run_dir, enabled=self.topo.is_main)
        self.heartbeat = L.Heartbeat(run_dir, self.topo.rank, self.topo.world)
        self._emb_snap = None
        self.preempt_requested = False
        self._t0 = time.time()

    # ------------------------------------------------------------------
    def describe(self) -> str:
        lines = list(self.model.get_model_info())
        lines.append(f"  parameters: {count_parameters(self.model):,} (this rank)")
        lines.append("  " + self.optimizer.describe_groups())
        lines.append(f"  backend: {self.backend.name}; world {self.topo.world} = dp {self.topo.dp} x "
                     f"pool_shards {self.topo.pool_shards}; seq_shard {self.topo.seq_shard}")
        return "\n".join(lines)

    def _to_device(self, ids, mask):
        ids = ids.to(self.device, non_blocking=True).long()
        mask = mask.to(self.device, non_blocking=True)
        return ids, mask

    def _snap_emb(self):
        p = self.model.neuron_pool
        self._emb_snap = {n: getattr(p, f"{n}_emb").detach().clone() for n in ("qk", "v", "know")}

    def train_step(self, ids: torch.Tensor, mask: torch.Tensor, *, want_diag: bool = False
                   ) -> Dict[str, Any]:
        t = self.cfg.training
        self.model.train()
        ids, mask = self._to_device(ids, mask)
        labels = torch.where(mask == 1, ids, torch.full_like(ids, -100))
        with trace("forward"):
            result = self.model(ids, labels=labels, attention_mask=mask, want_diag=want_diag)
        opt_step = self.optimizer.count
        total, parts = total_loss(result, self.model, t, opt_step, is_baseline=self.is_baseline,
                                  dp_group=self.topo.world_group if self.topo.world > 1 else None,
                                  backend=self.backend, want_stats=want_diag)
        with trace("backward"):
            total.backward()
        with trace("optimizer"):
            self.optimizer.step()     # consumes this micro-step's gradients (it keeps its own sum)
            self.optimizer.zero_grad()
        self.backend.finish_step()
        self.global_step += 1
        metrics: Dict[str, Any] = {"total_loss": total.detach()}
        metrics.update({k: (v.detach() if isinstance(v, torch.Tensor) else v) for k, v in parts.items()})
        metrics["correct"], metrics["valid_count"] = result["correct"], result["valid_count"]
        metrics["accuracy"] = result["correct"].float() / result["valid_count"].clamp(min=1).float()
        metrics["grad_norm"] = self.optimizer.last_grad_norm
        metrics["lr"] = self.optimizer.last_lr
        if want_diag and not self.is_baseline:
            metrics.update(self._diag_metrics(result, parts))
        return metrics

    def _diag_metrics(self, result, parts) -> Dict[str, Any]:
        t = self.cfg.training
        out = {k: v for k, v in result.items()
               if k not in ("per_token_ce", "valid_mask", "attn_tau_offset", "know_tau_offset", "logits")}
        out["aux_weighted"] = t.load_balance_weight * parts["aux_loss"]
        out["tau_reg_weighted"] = t.tau_reg_weight * parts["tau_reg"]
        out["orth_weighted"] = 0.0
        out["div_weighted"] = t.diversity_weight * parts["div_loss"]
        out["dead_penalty_weighted"] = t.dead_penalty_weight * parts["dead_penalty"]
        rt = self.model.router
        out["tau_know_bias"] = rt.tau_know.bias.detach()[0]
        for i in range(3):
            out[f"tau_attn_bias_{i}"] = rt.tau_attn.bias.detach()[i]
        if "attn_tau_std" in result:
            q, k, v = result["attn_tau_std"].tolist()
            out.update(attn_tau_std_q=q, attn_tau_std_k=k, attn_tau_std_v=v)
        if self._emb_snap is not None:
            p = self.model.neuron_pool
            for n in ("qk", "v", "know"):
                cur, prev = getattr(p, f"{n}_emb").detach(), self._emb_snap[n]
                out[f"drift_{n}_emb"] = (cur - prev).norm() / (prev.norm() + 1e-8)
        self._snap_emb()
        return out

    # ------------------------------------------------------------------
    @torch.no_grad()
    def evaluate(self, max_batches: Optional[int] = None) -> Dict[str, float]:
        """Deterministic forward over the validation stream; sums are kept on
        the device and read once (reference: scripts/train_jax.py:1042-1089)."""
        if self.val_loader is None:
            return {}
        self.model.eval()
        max_batches = max_batches or self.cfg.training.max_val_batches
        acc = torch.zeros(3, device=self.device, dtype=torch.float64)
        for i, (ids, mask) in enumerate(self.val_loader):
            if i >= max_batches:
                break
            ids, mask = self._to_device(ids, mask)
            labels = torch.where(mask == 1, ids, torch.full_like(ids, -100))
            r = self.model(ids, labels=labels, attention_mask=mask, want_diag=False)
            acc += torch.stack([r["loss"].double() * r["valid_count"], r["correct"].double(),
                                r["valid_count"].double()])
        if self.topo.world > 1:
            dist.all_reduce(acc, group=self.topo.world_group)
        loss_sum, correct, valid = acc.tolist()
        self.model.train()
        if valid == 0:
            return {}
        loss = loss_sum / valid
        return {"val_loss": loss, "val_acc": correct / valid, "val_ppl": math.exp(min(loss, 50.0))}

    # ------------------------------------------------------------------
    def save(self, name: str) -> Optional[str]:
        if self.run_dir is None:
            return None
        # a kernel that gave up on a wait must surface before its results are written out
        # (the per-step check reports one step late)
        if hasattr(self.backend, "finish_run"):
            self.backend.finish_run()
        t = self.topo
        writes = t.is_main or (t.pool_shards > 1 and t.dp_index == 0) or self.fsdp
        if hasattr(self.optimizer, "gather_state"):
            self.optimizer.gather_state()       # collective: sharded moments -> per-parameter form
        path = None
        if writes:
            si, sc = self._ckpt_shard()
            extra = None
            if t.pool_shards > 1 and self.cfg.training.shard_pools is not None:
                extra = {"sharded_pools": list(self.cfg.training.shard_pools)}
            if self.fsdp:     # which tensors hold row blocks, and of how many rows (for consolidate)
                extra = {"fsdp_rows": {n: p._fsdp_rows for n, p in self.model.named_parameters()
                                       if getattr(p, "_fsdp_rows", None) is not None}}
            path = ckpt.save_checkpoint(
                os.path.join(self.run_dir, name), self.model, self.optimizer, epoch=self.epoch,
                step=self.global_step, step_in_epoch=self.step_in_epoch,
                steps_per_epoch=self.steps_per_epoch, best_val_loss=self.best_val_loss,
                config=self.cfg.model_dict(), training_config=self.cfg.training_dict(),
                shard_index=si, shard_count=sc, extra=extra)
        if t.is_main and name.startswith("checkpoint_step"):
            ckpt.cleanup_old(self.run_dir, self.cfg.training.keep_last_checkpoints)
        return path

    def _ckpt_shard(self):
        """(index, count) of this rank's checkpoint file: pool shards, or the row
        blocks of a row-sharded dense model (one file per rank)."""
        if self.fsdp:
            return self.topo.rank, self.topo.world
        return self.topo.shard_index, self.topo.pool_shards

    def resume(self, path: str) -> None:
        err = None
        try:
            si, sc = self._ckpt_shard()
            blob = ckpt.load_checkpoint(path, self.model, self.optimizer,
                                        shard_index=si, shard_count=sc)
        except Exception as e:       # missing / unreadable shard file on this rank
            err, blob = e, None
        if self.topo.world > 1:
            # every rank learns whether all loads succeeded before anyone enters a collective
            ok = torch.tensor([0 if err is not None else 1], dtype=torch.int32)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.topo.cpu_group)
            if int(ok) == 0 and err is None:
                raise RuntimeError(f"another rank could not load its part of {path}")
        if err is not None:
            raise err
        self.global_step = int(blob["step"])
        self.epoch = int(blob.get("epoch", 0))
        self.best_val_loss = float(blob.get("best_val_loss", float("inf")))
        sie = int(blob.get("step_in_epoch", 0))
        same = int(blob.get("steps_per_epoch", -1)) == self.steps_per_epoch
        self.step_in_epoch = sie if same else 0
        self.check_step_consistency()

    def check_step_consistency(self) -> None:
        """After a resume every rank must be at the same global step."""
        if self.topo.world == 1:
            return
        v = torch.tensor([self.global_step], dtype=torch.int64)
        lo, hi = v.clone(), v.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=self.topo.cpu_group)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=self.topo.cpu_group)
        if int(lo) != int(hi):
            raise RuntimeError(f"ranks disagree on the resumed step: min {int(lo)} max {int(hi)}")

    # ------------------------------------------------------------------
    def _install_sigterm(self):
        def handler(signum, frame):
            if not self.preempt_requested:
                self.preempt_requested = True
                print(f"\n!!! SIGTERM (rank {self.topo.rank}) at step {self.global_step}: "
                      "flagging preemption", flush=True)
        try:
            signal.signal(signal.SIGTERM, handler)
        except ValueError:
            pass  # not the main thread

    def preemption_consensus(self) -> bool:
        """OR of every rank's preemption flag (host-side group)."""
        if self.topo.world == 1:
            return self.preempt_requested
        v = torch.tensor([1 if self.preempt_requested else 0], dtype=torch.int32)
        dist.all_reduce(v, op=dist.ReduceOp.MAX, group=self.topo.cpu_group)
        if int(v) and not self.preempt_requested:
            self.preempt_requested = True
        return self.preempt_requested

    def fit(self) -> Dict[str, Any]:
        cfg, t = self.cfg, self.cfg.training
        log = self.logger
        self._install_sigterm()
        if self.run_dir and self.topo.is_main:
            save_run_config(cfg, os.path.join(self.run_dir, "config.json"))
        log.message(self.describe())
        if not self.is_baseline:
            self._snap_emb()
        win = torch.zeros(4, device=self.device, dtype=torch.float64)  # loss*valid, ce*valid, correct, valid
        win_steps, win_t0 = 0, time.time()
        last: Dict[str, Any] = {}
        done = False
        while self.epoch < t.num_epochs and not done:
            ep_t0 = time.time()
            ep_acc = torch.zeros(3, device=self.device, dtype=torch.float64)
            self.train_loader.reset(self.step_in_epoch)
            for local_step, (ids, mask) in enumerate(self.train_loader, start=self.step_in_epoch):
                if local_step % 10 == 0 and self.preemption_consensus():
                    log.message("Preemption requested -- leaving the training loop.")
                    done = True
                    break
                nxt = self.global_step + 1
                is_log = L.is_log_step(nxt, t.log_interval)
                is_an = L.is_analysis_step(nxt, t.log_interval, t.log_analysis_multiplier)
                m = self.train_step(ids, mask, want_diag=is_log or is_an)
                self.heartbeat.beat(self.global_step)
                self.step_in_epoch = local_step + 1
                # the per-step device->host read.  The gradient norm is computed from the
                # globally reduced gradients, so it is identical on every rank and non-finite
                # on all of them as soon as one rank's loss is: all ranks leave together.
                gn = m.get("grad_norm")
                gn = gn.detach().float().reshape(()) if isinstance(gn, torch.Tensor) else \
                    torch.tensor(float(gn or 0.0), device=self.device)
                tl, gnv = torch.stack([m["total_loss"].detach().float().reshape(()),
                                       gn.to(self.device)]).tolist()
                if not (math.isfinite(tl) and math.isfinite(gnv)):
                    raise NonFiniteLoss(f"non-finite total_loss {tl} / grad_norm {gnv} at step "
                                        f"{self.global_step}")
                v = m["valid_count"].double()
                win += torch.stack([m["total_loss"].double() * v, m["ce_loss"].double() * v,
                                    m["correct"].double(), v])
                ep_acc += torch.stack([m["ce_loss"].double() * v, m["correct"].double(), v])
                win_steps += 1
                if is_log or is_an:
                    w = win.tolist()
                    dt = max(time.time() - win_t0, 1e-9)
                    rec_m = dict(m)
                    if w[3] > 0:
                        rec_m.update(total_loss=w[0] / w[3], ce_loss=w[1] / w[3], accuracy=w[2] / w[3])
                    for key in ("total_loss", "ce_loss", "aux_loss", "div_loss", "grad_norm"):
                        val = rec_m.get(key)
                        if isinstance(val, torch.Tensor):
                            val = val.detach()
                        val = float(val) if val is not None else 0.0
                        if not math.isfinite(val):
                            raise NonFiniteLoss(f"non-finite {key}={val} in the log window at step {self.global_step}")
                    rec = L.build_train_record(self.global_step, self.epoch, rec_m,
                                               steps_per_sec=win_steps / dt,
                                               elapsed=time.time() - self._t0, analysis=is_an)
                    log.message(L.format_regular(rec))
                    if is_an:
                        log.message(L.format_analysis(rec))
                    log.record(rec)
                    win.zero_()
                    win_steps, win_t0 = 0, time.time()
                if t.val_interval and self.global_step % t.val_interval == 0:
                    self._validate_and_maybe_save("val")
                if t.checkpoint_interval and self.global_step % t.checkpoint_interval == 0:
                    self.save(f"checkpoint_step{self.global_step}.pt")
                last = m
                if t.max_steps and self.global_step >= t.max_steps:
                    # a run cut short by max_steps still leaves a checkpoint to resume from
                    if not (t.checkpoint_interval and self.global_step % t.checkpoint_interval == 0):
                        self.save(f"checkpoint_step{self.global_step}.pt")
                    done = True
                    break
            if done:
                break
            vals = self.evaluate()
            ea = ep_acc.tolist()
            if vals:
                rec = {"type": "val_epoch", "step": self.global_step, "epoch": self.epoch, **vals,
                       "train_loss": ea[0] / max(ea[2], 1.0), "train_acc": ea[1] / max(ea[2], 1.0),
                       "epoch_time": time.time() - ep_t0}
                log.record(rec)
                log.message(f"[epoch {self.epoch}] val_loss {vals['val_loss']:.4f} val_acc {vals['val_acc']:.4f}")
                if vals["val_loss"] < self.best_val_loss:
                    self.best_val_loss = vals["val_loss"]
                    self.save("best_model.pt")
            self.save(f"checkpoint_epoch{self.epoch}.pt")
            self.epoch += 1
            self.step_in_epoch = 0
        if self.preempt_requested:
            self.save(f"emergency_step{self.global_step}.pt")
        self.backend.finish_run()
        return {k: (float(v) if isinstance(v, torch.Tensor) and v.numel() == 1 else v)
                for k, v in last.items() if k in ("total_loss", "ce_loss", "accuracy", "grad_norm", "lr")}

    def _validate_and_maybe_save(self, rec_type: str):
        vals = self.evaluate()
        if not vals:
            return
        self.logger.record({"type": rec_type, "step": self.global_step, "epoch": self.epoch,
                            "val_loss": vals["val_loss"], "val_acc": vals["val_acc"]})
        self.logger.message(f"[val @ {self.global_step}] loss {vals['val_loss']:.4f} "
                            f"acc {vals['val_acc']:.4f} ppl {vals['val_ppl']:.2f}")
        if vals["val_loss"] < self.best_val_loss:
            self.best_val_loss = vals["val_loss"]
            self.save("best_model.pt")
