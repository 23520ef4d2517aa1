"""Start-up self-benchmark: does a step fit in memory, how long does it take,
and where does the time go.

Run once before training (reference: scripts/train_jax.py:2352-2770, which
compiles and runs the real step twice on a dummy batch, reads the HBM
statistics, then times LayerNorm / router / QK / V / self-attention / knowledge
individually and prints a table with an ETA).  Here nothing needs compiling;
the report consists of

* two forward+backward passes of the real model on a synthetic batch (no
  optimizer step, gradients are dropped afterwards, so training state is
  untouched), timed with CUDA events, with the allocator's peak against the
  device capacity;
* forward timings (``n_runs`` each) of the building blocks of one layer at the
  training shapes;
* the ETA for the configured number of optimizer steps.
"""
from __future__ import annotations

import time
from typing import Any, Callable, Dict, List

import torch


def _timer(device) -> Callable[[Callable[[], Any], int], float]:
    """Returns time_ms(fn, runs): mean milliseconds per call (after one warm-up)."""
    cuda = device.type == "cuda"

    def time_ms(fn, runs):
        fn()
        if cuda:
            torch.cuda.synchronize(device)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(runs):
                fn()
            e1.record()
            torch.cuda.synchronize(device)
            return e0.elapsed_time(e1) / runs
        t0 = time.perf_counter()
        for _ in range(runs):
            fn()
        return (time.perf_counter() - t0) * 1e3 / runs
    return time_ms


def startup_report(trainer, n_runs: int = 5, print_fn=print) -> Dict[str, Any]:
    model, cfg, dev = trainer.model, trainer.cfg, trainer.device
    t, m = cfg.training, cfg.model
    be = trainer.backend
    time_ms = _timer(dev)
    ids, mask = trainer.train_loader.batch(0)
    ids = ids.to(dev).long()
    mask = mask.to(dev)
    labels = torch.where(mask == 1, ids, torch.full_like(ids, -100))
    B, S = ids.shape
    rep: Dict[str, Any] = {"batch_per_rank": B, "seq_len": S}

    # ---- whole step (forward + backward), memory -------------------------
    if dev.type == "cuda":
        torch.cuda.reset_peak_memory_stats(dev)
    was_training = model.training
    model.train()

    def fwd_bwd():
        res = model(ids, labels=labels, attention_mask=mask, want_diag=False)
        (res["loss"] + res.get("aux_loss", 0.0)).backward()
        sync = getattr(trainer.optimizer, "grad_sync", None)
        if sync is not None:
            sync.discard()                   # this backward's gradients are not used
        trainer.optimizer.zero_grad()
    try:
        rep["fwd_bwd_ms"] = time_ms(fwd_bwd, 2)
    except torch.cuda.OutOfMemoryError as e:             # pragma: no cover - needs a too-large config
        rep["oom"] = str(e).splitlines()[0]
        print_fn(f"[startup] OUT OF MEMORY on the first step: {rep['oom']}")
        raise
    trainer.optimizer.zero_grad()
    if dev.type == "cuda":
        free, total = torch.cuda.mem_get_info(dev)
        rep["hbm_peak_gb"] = torch.cuda.max_memory_allocated(dev) / 2 ** 30
        rep["hbm_total_gb"] = total / 2 ** 30
        rep["hbm_headroom_gb"] = rep["hbm_total_gb"] - rep["hbm_peak_gb"]
    tokens = B * S * trainer.topo.batch_replicas
    rep["tokens_per_sec_fwd_bwd"] = tokens / (rep["fwd_bwd_ms"] / 1e3)
    k = max(1, t.gradient_accumulation_steps)
    rep["eta_hours"] = trainer.total_steps * k * rep["fwd_bwd_ms"] / 3.6e6

    # ---- building blocks of one layer (forward only) ----------------------
    rows: List = []
    if m.is_spatial:
        with torch.no_grad():
            pools = model.prepare_pools(be)
            blk = model.layers[0]
            D, r, H = model.d_model, model.d_route, model.n_heads
            T = B * S
            x = torch.randn(B, S, D, device=dev)
            xf = x.reshape(T, D)
            rt = model.router
            n1 = be.layer_norm(x, blk.norm1.weight, blk.norm1.bias).reshape(T, D)
            h_all = be.linear(n1, rt.proj_attn.weight, rt.proj_attn.bias)
            tau_all = be.linear(n1, rt.tau_attn.weight, rt.tau_attn.bias).float()
            h_k = be.linear(n1, rt.proj_know.weight, rt.proj_know.bias)
            tau_k = be.linear(n1, rt.tau_know.weight, rt.tau_know.bias).float()
            heads = lambda z: z.reshape(B, S, H, D // H).transpose(1, 2)
            q = heads(torch.randn(T, D, device=dev))
            ops = [
                ("layer_norm", lambda: be.layer_norm(x, blk.norm1.weight, blk.norm1.bias)),
                ("router_proj", lambda: be.linear(n1, rt.proj_attn.weight, rt.proj_attn.bias)),
                ("srw_qk (2 routes)", lambda: be.srw(n1, h_all[:, :2 * r].reshape(T, 2, r), tau_all[:, 0:2],
                                                     pools["qk"], model.gate, pctx=model.pctx("qk"),
                                                     want_diag=False)),
                ("srw_v", lambda: be.srw(n1, h_all[:, 2 * r:].reshape(T, 1, r), tau_all[:, 2:3], pools["v"],
                                         model.gate, pctx=model.pctx("v"), want_diag=False)),
                ("self_attention", lambda: be.attention(q, q, q, 0.0, False)),
                ("expand_O", lambda: be.linear(xf, blk.attn.expand_O.weight, None)),
                ("srw_know", lambda: be.srw(n1, h_k.reshape(T, 1, r), tau_k, pools["know"], model.gate,
                                            pctx=model.pctx("know"), want_diag=False)),
            ]
            for name, fn in ops:
                rows.append((name, time_ms(fn, n_runs)))
    rep["ops_forward_ms"] = dict(rows)
    model.train(was_training)

    if trainer.topo.is_main:
        print_fn("[startup] forward+backward %.1f ms/step/rank, %.0f tokens/s (whole job), ETA %.2f h "
                 "for %d optimizer steps" % (rep["fwd_bwd_ms"], rep["tokens_per_sec_fwd_bwd"],
                                             rep["eta_hours"], trainer.total_steps))
        if "hbm_peak_gb" in rep:
            print_fn("[startup] device memory: peak %.1f GB of %.1f GB (headroom %.1f GB)"
                     % (rep["hbm_peak_gb"], rep["hbm_total_gb"], rep["hbm_headroom_gb"]))
        if rows:
            layer_ms = sum(v for _, v in rows)
            print_fn("[startup] one layer, forward, by building block:")
            for name, v in rows:
                print_fn("    %-20s %9.3f ms  %5.1f %%" % (name, v, 100.0 * v / max(layer_ms, 1e-9)))
    return rep
