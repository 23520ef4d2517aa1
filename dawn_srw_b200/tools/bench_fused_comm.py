#!/usr/bin/env python
"""Fused compute+collective kernels against their rooflines and against the
NCCL formulation of the same step.  Launch one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m dawn_srw_b200.tools.bench_fused_comm [--tokens-per-rank 16384] [--d-model 1280]
        [--d-route 256] [--units 100000,6400] [--opt-elems 100000000] [--iters 5] [--json out.json]

Three paths, each timed with CUDA events (max over ranks) after warm-up, on
operands larger than the L2:

1. all-gather -> gate GEMM: every rank contributes ``tokens-per-rank`` rows of
   x [.,D] and h [.,r]; the gate kernel runs over all tokens x U/N units while
   its gather warps pull the peers' rows (fused) vs NCCL all-gather followed by
   the same kernel without gathering.
2. write GEMM -> reduce-scatter: p [T,U/N] . write [U/N,D] with each output
   slab TMA-stored (bf16) into this rank's slot of the owner's receive buffer,
   barrier, slots summed in fp32 by the owner (fused) vs the plain GEMM
   followed by NCCL reduce-scatter (bf16, what the library path sends).
3. partitioned optimizer: gradient slices summed from the peers + AdamW +
   parameters stored to the peers (two kernels, two barriers) vs NCCL
   all-reduce + full AdamW on every rank.

Roofline of a fused path: the slower of FLOPs / sustained cuBLAS bf16 rate and
bytes that must cross NVLink / 770 GB/s per direction (both measured on this
pool; the rate comes from MEASURED_PEAKS.json when present).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def sustained_tflops() -> float:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        return float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
    except Exception:
        return 1400.0


def timed(fn, iters, world, dev):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens-per-rank", type=int, default=16384)
    ap.add_argument("--d-model", type=int, default=1280)
    ap.add_argument("--d-route", type=int, default=256)
    ap.add_argument("--units", default="100000,6400", help="total pool sizes (split over the ranks)")
    ap.add_argument("--opt-elems", type=int, default=100_000_000)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--json")
    args = ap.parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ..ops import cuda_backend as CB
    from ..ops.gates import gate_spec_for
    from ..parallel.symm import SymmWorkspace
    e = CB.ext()
    st = CB.status_word(dev)
    ws = SymmWorkspace(None, dev) if world > 1 else None
    peak = sustained_tflops()
    Tl, D, r = args.tokens_per_rank, args.d_model, args.d_route
    T = Tl * world
    g = torch.Generator(device=dev).manual_seed(rank)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    spec = gate_spec_for("spatial-r1-v4.0.1")
    gl = CB._gate_list(spec)
    bf = torch.bfloat16
    recs = []
    rows = slice(rank * Tl, (rank + 1) * Tl)
    for U_tot in [int(u) for u in args.units.split(",")]:
        U = (U_tot // world) // 8 * 8
        emb = torch.nn.functional.normalize(rn(U, r), dim=-1).to(bf)
        read = torch.nn.functional.normalize(rn(U, D), dim=-1).to(bf)
        write = torch.nn.functional.normalize(rn(U, D), dim=-1).to(bf)
        x_l, h_l = rn(Tl, D).to(bf), rn(Tl, r).to(bf)
        tau = torch.full((T,), 1.6, device=dev)
        isd = torch.ones(T, device=dev)
        p = torch.empty(T, U, dtype=bf, device=dev)
        den = torch.zeros(T, device=dev)
        # ---- 1. all-gather -> gate GEMM ---------------------------------
        flops = 2.0 * T * U * (r + D)
        if world > 1:
            xf = [ws.alloc(f"bx{i}", (T, D), bf) for i in range(2)]
            hf = [ws.alloc(f"bh{i}", (T, r), bf) for i in range(2)]
            ready = torch.zeros(T // 128, dtype=torch.int32, device=dev)
            state = {"b": 0, "ep": 0}

            def fused_ag():
                state["b"] ^= 1
                state["ep"] += 1
                b = state["b"]
                xf[b].local[rows].copy_(x_l)
                hf[b].local[rows].copy_(h_l)
                ws.barrier()
                e.srw_fwd_gate_gather(hf[b].local, emb, xf[b].local, read, p, tau, isd, den, gl, st,
                                      [xf[b].ptrs, hf[b].ptrs], rank, Tl, ready, state["ep"])
            xg, hg = torch.empty(T, D, dtype=bf, device=dev), torch.empty(T, r, dtype=bf, device=dev)

            def nccl_ag():
                dist.all_gather_into_tensor(xg, x_l)
                dist.all_gather_into_tensor(hg, h_l)
                e.srw_fwd_gate(hg, emb, xg, read, p, tau, isd, den, None, None, None, gl, st)
            t_f, t_n = timed(fused_ag, args.iters, world, dev), timed(nccl_ag, args.iters, world, dev)
        else:
            xg, hg = x_l, h_l
            t_f = t_n = timed(lambda: e.srw_fwd_gate(hg, emb, xg, read, p, tau, isd, den, None, None,
                                                     None, gl, st), args.iters, world, dev)
        t_local = timed(lambda: e.srw_fwd_gate(hg, emb, xg, read, p, tau, isd, den, None, None, None,
                                               gl, st), args.iters, world, dev)
        link_b = (world - 1) * Tl * (D + r) * 2.0
        roof = max(flops / (peak * 1e9), link_b / (NVLINK_GBS * 1e6))
        recs.append({"path": "all-gather -> gate GEMM", "units_per_rank": U, "fused_ms": t_f,
                     "nccl_ms": t_n, "kernel_without_comm_ms": t_local, "roofline_ms": roof,
                     "fraction_of_roofline": roof / t_f, "nvlink_mb_in": link_b / 1e6,
                     "tflops": flops / t_f / 1e9})
        # ---- 2. write GEMM -> reduce-scatter ------------------------------
        flops = 2.0 * T * U * D
        if world > 1:
            tgt = ws.alloc("rs_tgt", (world * Tl, D), bf)
            full32 = torch.empty(T, D, device=dev)
            fullbf = torch.empty(T, D, dtype=bf, device=dev)
            outbf = torch.empty(Tl, D, dtype=bf, device=dev)

            def fused_rs():
                e.gemm_scatter(p, False, write, True, tgt.ptrs, rank, Tl, D, True, 1.0, None, st, None, [])
                ws.barrier()
                e.sum_slabs(tgt.local, world, False)

            def nccl_rs():
                CB.gemm(p, False, write, True, out=fullbf)
                dist.reduce_scatter_tensor(outbf, fullbf)
            t_f, t_n = timed(fused_rs, args.iters, world, dev), timed(nccl_rs, args.iters, world, dev)
        else:
            full32 = torch.empty(T, D, device=dev)
            t_f = t_n = timed(lambda: CB.gemm(p, False, write, True, out=full32), args.iters, world, dev)
        t_local = timed(lambda: CB.gemm(p, False, write, True, out=full32), args.iters, world, dev)
        link_b = (world - 1) * Tl * D * 2.0              # bf16 slabs to the other owners
        roof = max(flops / (peak * 1e9), link_b / (NVLINK_GBS * 1e6))
        recs.append({"path": "write GEMM -> reduce-scatter", "units_per_rank": U, "fused_ms": t_f,
                     "nccl_ms": t_n, "kernel_without_comm_ms": t_local, "roofline_ms": roof,
                     "fraction_of_roofline": roof / t_f, "nvlink_mb_out": link_b / 1e6,
                     "tflops": flops / t_f / 1e9})
        del emb, read, write, p
    # ---- 3. partitioned optimizer ---------------------------------------
    if world > 1:
        from ..parallel.grad_sync import GradSync
        from ..parallel.topology import Topology
        from ..parallel.zero import PartitionedAdamW
        from ..train.optimizer import DawnAdamW
        topo = Topology(rank=rank, world=world, local_rank=local, pool_shards=1, dp=world,
                        seq_shard=False, shard_group=None, dp_group=dist.group.WORLD,
                        world_group=dist.group.WORLD, cpu_group=None)
        n = args.opt_elems
        pa = [("w.weight", torch.nn.Parameter(torch.randn(n, device=dev) * 0.02))]
        pb = [("w.weight", torch.nn.Parameter(pa[0][1].detach().clone()))]
        oa = PartitionedAdamW(pa, topo, lr=1e-3, peer_kernels=True)
        ob = DawnAdamW(pb, lr=1e-3, grad_sync=GradSync(topo), fused=True)
        gsrc = torch.randn(n, device=dev)

        def step_a():
            pa[0][1].grad.copy_(gsrc)
            oa.step()
            oa.zero_grad()

        def step_b():
            pb[0][1].grad = gsrc.clone()
            ob.step()
        t_f, t_n = timed(step_a, args.iters, world, dev), timed(step_b, args.iters, world, dev)
        link_b = n * 4.0 * (world - 1) / world
        roof = 2.0 * link_b / (NVLINK_GBS * 1e6)
        recs.append({"path": "partitioned AdamW (reduce-scatter + update + all-gather)",
                     "elements": n, "fused_ms": t_f, "nccl_ms": t_n, "roofline_ms": roof,
                     "fraction_of_roofline": roof / t_f, "nvlink_mb_each_way": link_b / 1e6})
    CB.check_status()
    if rank == 0:
        out = {"world": world, "tokens_per_rank": Tl, "d_model": D, "d_route": r,
               "bf16_tflops_sustained": peak, "nvlink_gbs": NVLINK_GBS, "records": recs}
        if args.json:
            with open(args.json, "w") as f:
                json.dump(out, f, indent=1)
        for rcd in recs:
            print("%-52s %s fused %7.3f ms | nccl %7.3f ms | roofline %6.3f ms -> %.2f of roofline" % (
                rcd["path"], ("U/N=%-6d" % rcd["units_per_rank"]) if "units_per_rank" in rcd else
                ("n=%-8d" % rcd["elements"]), rcd["fused_ms"], rcd["nccl_ms"], rcd["roofline_ms"],
                rcd["fraction_of_roofline"]))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
