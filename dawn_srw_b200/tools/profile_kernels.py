#!/usr/bin/env python
"""Launch the four engine kernels of one SRW route back to back, for profilers.

    python -m dawn_srw_b200.tools.profile_kernels [--tokens 4096] [--units 25600]
        [--d-model 1280] [--d-route 256] [--kind 1] [--iters 2]

Per iteration, in this order: forward gate kernel, write GEMM (p . write),
backward gate step, pool-gradient GEMM (p^T . dy, reduce-add); each is timed
with CUDA events (second half of the iterations) and printed with its TFLOP/s.  The default
shape holds < 2 GB on the device and its operands exceed the 126 MB L2, so an
``ncu --set full`` capture of one iteration finishes in about a minute:

    ncu --set full --clock-control none -k regex:gemm_engine_kernel -s 4 -c 4 \
        -o prof python -m dawn_srw_b200.tools.profile_kernels

``--attention`` launches the causal attention forward and backward kernels
instead (batch 8 x 16 heads x 512 tokens x head dimension 80 by default):

    ncu --set full --clock-control none -k regex:attn_ -s 2 -c 2 -o prof_attn \
        python -m dawn_srw_b200.tools.profile_kernels --attention
"""
from __future__ import annotations

import argparse
import sys

import torch


def attention(args):
    import time
    from ..ops import cuda_backend as CB
    dev = torch.device("cuda")
    B, H, S, dh = args.batch, args.heads, args.seq, args.head_dim
    g = torch.Generator(device=dev).manual_seed(0)
    q, k, v = (torch.randn(B, S, H * dh, device=dev, generator=g).bfloat16().requires_grad_(True)
               for _ in range(3))
    w = torch.randn(B, S, H * dh, device=dev, generator=g).bfloat16()
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    for it in range(args.iters):
        ev[0].record()
        out = CB.causal_attention(q, k, v, H, 0.1, 1234)
        ev[1].record()
        out.backward(w)
        ev[2].record()
        q.grad = k.grad = v.grad = None
    torch.cuda.synchronize()
    CB.check_status()
    fl = 4.0 * B * H * S * S * dh / 2            # causal: half of the S x S tiles
    f_ms, b_ms = ev[0].elapsed_time(ev[1]), ev[1].elapsed_time(ev[2])
    print(f"ok: attention B={B} H={H} S={S} dh={dh}: forward {f_ms:.3f} ms ({fl / f_ms / 1e9:.0f} TFLOP/s), "
          f"backward {b_ms:.3f} ms ({2.5 * fl / b_ms / 1e9:.0f} TFLOP/s)")
    return 0


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--units", type=int, default=25600)
    ap.add_argument("--d-model", type=int, default=1280)
    ap.add_argument("--d-route", type=int, default=256)
    ap.add_argument("--kind", type=int, default=1)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--recompute", action="store_true",
                    help="backward gate step without kept read scalars (recomputes S and XR)")
    ap.add_argument("--attention", action="store_true")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--head-dim", type=int, default=80)
    args = ap.parse_args(argv)
    if args.attention:
        return attention(args)
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
    Up = (U + 7) // 8 * 8
    p = torch.empty(T, Up, dtype=torch.bfloat16, device=dev)
    dxr, ds = torch.empty_like(p), torch.empty_like(p)
    keep = bool(e.srw_wide_tiles(U)) and not args.recompute
    xr = torch.empty_like(p) if keep else None
    den, dtau, dsz = (torch.zeros(T, device=dev) for _ in range(3))
    dden = torch.zeros(T, device=dev)
    tau = torch.full((T,), 1.0, device=dev)
    isd = torch.full((T,), 1.0, device=dev)
    raw = torch.empty(T, D, device=dev)
    gw = torch.zeros(U, D, device=dev)
    names = ["fwd_gate", "write_gemm", "bwd_gate", "dwrite_gemm"]
    flops = [2.0 * T * U * (r + D), 2.0 * T * U * D,
             2.0 * T * U * (r + D) * (1 if keep else 2), 2.0 * T * U * D]
    acc = [0.0] * 4
    for it in range(args.iters):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        ev[0].record()
        e.srw_fwd_gate_xr(h, emb, x, read, p, xr, tau, isd, None, den, None, None, None, gl, st, *CB.NO_GATHER)
        ev[1].record()
        CB.gemm(p[:, :U], False, write, True, out=raw)
        ev[2].record()
        if keep:
            # p overwrites the kept read scalars in place, as in training
            e.srw_bwd_gate_xr(h, emb, dy, write, xr, xr, dxr, ds, tau, isd, dden, None, dtau, gl, st,
                              *CB.NO_GATHER)
        else:
            e.srw_bwd_gate(h, emb, x, read, dy, write, p, dxr, ds, tau, isd, dden, dtau, dsz, gl, st)
        ev[3].record()
        CB.gemm(p[:, :U], True, dy, True, out=gw, accumulate=True)
        ev[4].record()
        torch.cuda.synchronize()
        if it >= args.iters // 2:                       # the first half warms up
            for k in range(4):
                acc[k] += ev[k].elapsed_time(ev[k + 1])
    CB.check_status()
    n = args.iters - args.iters // 2
    print(f"ok: T={T} U={U} d={D} r={r} kind={args.kind} iters={args.iters} "
          f"backward gate step: {'one launch on kept read scalars' if keep else 'recomputes S and XR'}")
    for k in range(4):
        ms = acc[k] / n
        print(f"  {names[k]:12s} {ms:8.3f} ms  {flops[k] / ms / 1e9:7.0f} TFLOP/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
