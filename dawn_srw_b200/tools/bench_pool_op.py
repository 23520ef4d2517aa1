#!/usr/bin/env python
"""SRW pool-op microbenchmark, on one GPU or with the pool sharded over N GPUs.

    python -m dawn_srw_b200.tools.bench_pool_op [--tokens 4096,16384,65536]
        [--d-model 384,1024,2048] [--units 2600,25200,100000] [--version spatial-r1-v4.0.1]
        [--iters 5] [--calls 18] [--json out.json]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m dawn_srw_b200.tools.bench_pool_op ...

For every (tokens per GPU, d_model d, pool size U) it times, with CUDA events
after warm-up (max over ranks), the forward and forward+backward of one SRW
route through the sm_100a kernels: bf16 unit-norm e/r/w rows, threshold offset
chosen for about 5 % active units.  As in a model, where all layers share the
pools, the pool is prepared once (normalisation, Gram matrix) and then used by
``--calls`` route calls (18 = the layers of the 400M model; fewer when the kept
read scalars of that many calls would not fit); the reported time is per call.
With N ranks every rank holds U/N units and its own tokens; the op runs as the
fused all-gather -> gate GEMMs -> write GEMM -> reduce-scatter group.

Reported per case: time per call, executed TFLOP/s per GPU (forward
2*T*U*(r+2d); backward with kept read scalars 2*T*U*(3r+4d): S, dP and five
gradient GEMMs), and the fraction of the roofline, which is the slower of
FLOPs / sustained cuBLAS bf16 rate (MEASURED_PEAKS.json, fallback 1400) and,
for N > 1, the bytes that must cross NVLink per GPU and direction / 770 GB/s
(forward: in (N-1)*T*(d+r)*2, out (N-1)*T*d*2; backward: in (N-1)*T*(2d+r)*2,
out (N-1)*T*(d+r)*2, with T tokens per GPU).  An L2-flushing write runs
between timed iterations.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import sys

import torch

NVLINK_GBS = 770.0


def measured(key: str, fallback: float) -> float:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        return float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))[key])
    except Exception:
        return fallback


def run_case(T, d, U, r, version, iters, calls, topo, only_fwd=False):
    import torch.distributed as dist
    from ..ops.backend import ParallelCtx
    from ..ops.cuda_backend import CudaBackend, check_status
    from ..ops.gates import gate_spec_for
    dev = torch.device("cuda", topo.local_rank)
    G = topo.world
    spec = gate_spec_for(version)
    be = CudaBackend()
    Ul = (U + G - 1) // G                                        # units held by this rank
    n_valid = max(0, min(Ul, U - topo.rank * Ul))
    gen = torch.Generator(device=dev).manual_seed(1 + topo.rank)
    rn = lambda *s: torch.randn(*s, device=dev, generator=gen)
    nz = torch.nn.functional.normalize
    emb = nz(rn(Ul, r), dim=-1).requires_grad_(True)
    read = nz(rn(Ul, d), dim=-1).requires_grad_(True)
    write = nz(rn(Ul, d), dim=-1).requires_grad_(True)
    x = rn(T, d).requires_grad_(True)
    h = rn(T, 1, r).requires_grad_(True)
    off = torch.full((T, 1), 1.65, device=dev, requires_grad=True)   # ~5 % of a normal above mu + 1.65 sd
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    w = rn(T, 1, d)
    pctx = (ParallelCtx(shard_group=topo.shard_group, dp_group=topo.dp_group, n_total=U,
                        n_valid=n_valid, seq_sharded=True) if G > 1 else ParallelCtx())
    # the kept read scalars of all calls of one step stay alive until its backward
    calls = max(1, min(calls, int(24e9 // max(1, T * G * Ul * 2))))

    def step(backward):
        pool = be.prepare_pool(emb, read, write, spec, pctx)
        tot = None
        for _ in range(calls):
            (res,) = be.srw_group(x, [dict(h=h, tau_off=off, pool=pool, pctx=pctx)], spec,
                                  want_diag=False)
            if backward:
                t = (res.stacked() * w).sum()
                tot = t if tot is None else tot + t
        if backward:
            tot.backward()
        be.finish_step() if hasattr(be, "finish_step") else None

    times = {}
    for name, bwd in (("fwd", False), ("fwd_bwd", True)):
        if only_fwd and bwd:
            continue
        for _ in range(3):
            step(bwd)
        torch.cuda.synchronize()
        tot = 0.0
        for _ in range(iters):
            flush.zero_()
            if G > 1:
                dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step(bwd)
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        ms = torch.tensor([tot / iters / calls], device=dev)
        if G > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        times[name] = float(ms)
    check_status()
    sustained = measured("bf16_tflops_sustained", 1400.0)
    f_fwd = 2.0 * T * G * Ul * (r + 2 * d)
    f_bwd = 2.0 * T * G * Ul * (3 * r + 4 * d)
    link = lambda nbytes: nbytes / (NVLINK_GBS * 1e9) * 1e3          # ms
    roof_fwd = max(f_fwd / sustained / 1e9, link((G - 1) * T * (d + r) * 2.0))
    roof_bwd = max(f_bwd / sustained / 1e9, link((G - 1) * T * (2 * d + r) * 2.0))
    out = {"gpus": G, "tokens_per_gpu": T, "d_model": d, "units": U, "d_route": r, "version": version,
           "calls_per_prepared_pool": calls,
           "fwd_ms": times["fwd"], "fwd_tflops_per_gpu": f_fwd / times["fwd"] / 1e9,
           "fwd_frac_of_roofline": roof_fwd / times["fwd"]}
    if "fwd_bwd" in times:
        out.update(fwd_bwd_ms=times["fwd_bwd"],
                   fwd_bwd_tflops_per_gpu=(f_fwd + f_bwd) / times["fwd_bwd"] / 1e9,
                   fwd_bwd_frac_of_roofline=(roof_fwd + roof_bwd) / times["fwd_bwd"])
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="4096,16384,65536", help="tokens per GPU")
    ap.add_argument("--d-model", default="384,1024,2048")
    ap.add_argument("--units", default="2600,25200,100000")
    ap.add_argument("--version", default="spatial-r1-v4.0.1")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--calls", type=int, default=18, help="route calls per prepared pool")
    ap.add_argument("--only-fwd", action="store_true")
    ap.add_argument("--json")
    args = ap.parse_args(argv)
    from ..parallel.topology import Topology, init_topology
    world = int(os.environ.get("WORLD_SIZE", "1"))
    topo = init_topology(pool_shards=world, seq_shard=True) if world > 1 else Topology()
    torch.cuda.set_device(topo.local_rank)
    rows = []
    for T in map(int, args.tokens.split(",")):
        for d in map(int, args.d_model.split(",")):
            r = {384: 128, 1024: 256, 1280: 256, 2048: 384}.get(d, 128)
            for U in map(int, args.units.split(",")):
                Ul = (U + world - 1) // world
                if T * world * Ul * 2 * 4 > 100e9:     # [T_all, U/N] bf16 work tiles of one call
                    continue
                row = run_case(T, d, U, r, args.version, args.iters, args.calls, topo, args.only_fwd)
                # autograd graphs of a case can sit in reference cycles: free them before the next
                gc.collect()
                torch.cuda.empty_cache()
                row["allocated_gb_after"] = round(torch.cuda.memory_allocated() / 2 ** 30, 2)
                rows.append(row)
                if topo.is_main:
                    print(json.dumps(row), flush=True)
    if args.json and topo.is_main:
        json.dump({"bf16_tflops_sustained": measured("bf16_tflops_sustained", 1400.0),
                   "nvlink_gbs": NVLINK_GBS, "rows": rows}, open(args.json, "w"), indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
