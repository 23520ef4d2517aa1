#!/usr/bin/env python
"""Launch the four engine kernels of one SRW route back to back, for profilers.

    python -m dawn_srw_b200.tools.profile_kernels [--tokens 4096] [--units 25600]
        [--d-model 1280] [--d-route 256] [--kind 1] [--iters 2]

Per iteration, in this order: forward gate kernel, write GEMM (p . write),
backward gate kernel, pool-gradient GEMM (p^T . dy, reduce-add).  The default
shape holds < 2 GB on the device and its operands exceed the 126 MB L2, so an
``ncu --set full`` capture of one iteration finishes in about a minute:

    ncu --set full --clock-control none -k regex:gemm_engine_kernel -s 4 -c 4 \
        -o prof python -m dawn_srw_b200.tools.profile_kernels
"""
from __future__ import annotations

import argparse
import sys

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--units", type=int, default=25600)
    ap.add_argument("--d-model", type=int, default=1280)
    ap.add_argument("--d-route", type=int, default=256)
    ap.add_argument("--kind", type=int, default=1)
    ap.add_argument("--iters", type=int, default=2)
    args = ap.parse_args(argv)
    from ..ops import cuda_backend as CB
    from ..ops.gates import GateSpec
    dev = torch.device("cuda")
    e, st = CB.ext(), CB.status_word(dev)
    T, U, r, D = args.tokens, args.units, args.d_route, args.d_model
    gl = CB._gate_list(GateSpec(kind=args.kind))
    nz = torch.nn.functional.normalize
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *s: torch.randn(*s, device=dev, generator=g)
    h, x, dy = rn(T, r).bfloat16(), rn(T, D).bfloat16(), (rn(T, D) * 0.1).bfloat16()
    emb, read, write = (nz(rn(U, d), dim=-1).bfloat16() for d in (r, D, D))
    p = torch.empty(T, U, dtype=torch.bfloat16, device=dev)
    dxr, ds = torch.empty_like(p), torch.empty_like(p)
    den, dtau, dsz = (torch.zeros(T, device=dev) for _ in range(3))
    dden = torch.zeros(T, device=dev)
    tau = torch.full((T,), 1.0, device=dev)
    isd = torch.full((T,), 1.0, device=dev)
    raw = torch.empty(T, D, device=dev)
    gw = torch.zeros(U, D, device=dev)
    for _ in range(args.iters):
        e.srw_fwd_gate(h, emb, x, read, p, tau, isd, den, None, None, None, gl, st)
        CB.gemm(p, False, write, True, out=raw)
        e.srw_bwd_gate(h, emb, x, read, dy, write, p, dxr, ds, tau, isd, dden, dtau, dsz, gl, st)
        CB.gemm(p, True, dy, True, out=gw, accumulate=True)
    torch.cuda.synchronize()
    CB.check_status()
    print(f"ok: T={T} U={U} d={D} r={r} kind={args.kind} iters={args.iters}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
