#!/usr/bin/env python
"""SRW pool-op microbenchmark.

    python -m dawn_srw_b200.tools.bench_pool_op [--tokens 4096,16384] [--d-model 384,1280]
        [--units 2600,25200,100000] [--version spatial-r1-v4.0.1] [--iters 5] [--json out.json]

For every (tokens N, d_model d, pool size U) it times, with CUDA events after
warm-up, the forward and forward+backward of one SRW route through the sm_100a
kernels (bf16 normal(0, 0.02)-scaled e/r/w rows, threshold offset chosen for
about 5 % active units) and reports achieved TFLOP/s against the measured
cuBLAS bf16 peak in MEASURED_PEAKS.json (fallback 1590 TFLOP/s).  FLOPs counted:
forward 2*N*U*(r + 2d); backward 2*N*U*(2r + 5d) (score/read recompute, dP, and
the five gradient GEMMs).  Inputs exceed the 126 MB L2 for the larger shapes;
an L2-flushing write runs between timed iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def peak_tflops() -> float:
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        return float(json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        return 1590.0


def run_case(N, d, U, r, version, iters, only_fwd=False):
    from ..ops.backend import ParallelCtx
    from ..ops.cuda_backend import CudaBackend, check_status
    from ..ops.gates import gate_spec_for
    dev = torch.device("cuda")
    spec = gate_spec_for(version)
    be = CudaBackend()
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    emb = torch.nn.functional.normalize(rn(U, r), dim=-1).requires_grad_(True)
    read = torch.nn.functional.normalize(rn(U, d), dim=-1).requires_grad_(True)
    write = torch.nn.functional.normalize(rn(U, d), dim=-1).requires_grad_(True)
    x = rn(N, d).requires_grad_(True)
    h = rn(N, 1, r).requires_grad_(True)
    off = torch.full((N, 1), 1.65, device=dev, requires_grad=True)   # ~5 % of a normal above mu + 1.65 sd
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    w = rn(N, 1, d)

    def step(backward):
        pool = be.prepare_pool(emb, read, write, spec, ParallelCtx())
        res = be.srw(x, h, off, pool, spec, pctx=ParallelCtx(), want_diag=False)
        if backward:
            (res.stacked() * w).sum().backward()
        return res
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
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step(bwd)
            e1.record()
            torch.cuda.synchronize()
            tot += e0.elapsed_time(e1)
        times[name] = tot / iters
    check_status()
    f_fwd = 2.0 * N * U * (r + 2 * d)
    f_bwd = 2.0 * N * U * (2 * r + 5 * d)
    out = {"tokens": N, "d_model": d, "units": U, "d_route": r, "version": version,
           "fwd_ms": times["fwd"], "fwd_tflops": f_fwd / times["fwd"] / 1e9}
    if "fwd_bwd" in times:
        out.update(fwd_bwd_ms=times["fwd_bwd"], fwd_bwd_tflops=(f_fwd + f_bwd) / times["fwd_bwd"] / 1e9)
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="4096,16384")
    ap.add_argument("--d-model", default="384,1280")
    ap.add_argument("--units", default="2600,25200,100000")
    ap.add_argument("--version", default="spatial-r1-v4.0.1")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--only-fwd", action="store_true")
    ap.add_argument("--json")
    args = ap.parse_args(argv)
    peak = peak_tflops()
    rows = []
    for N in map(int, args.tokens.split(",")):
        for d in map(int, args.d_model.split(",")):
            r = {384: 128, 1024: 256, 1280: 256, 2048: 384}.get(d, 128)
            for U in map(int, args.units.split(",")):
                if N * U * 2 * 3 > 60e9:       # keep the [N,U] bf16 work tiles under ~60 GB
                    continue
                row = run_case(N, d, U, r, args.version, args.iters, args.only_fwd)
                row["fwd_frac_of_measured_peak"] = row["fwd_tflops"] / peak
                if "fwd_bwd_tflops" in row:
                    row["fwd_bwd_frac_of_measured_peak"] = row["fwd_bwd_tflops"] / peak
                rows.append(row)
                print(json.dumps(row), flush=True)
    if args.json:
        json.dump({"peak_tflops_measured": peak, "rows": rows}, open(args.json, "w"), indent=1)
    return 0


if __name__ == "__main__":
    sys.exit(main())
