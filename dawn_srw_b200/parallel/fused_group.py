"""A group of SRW routes that read the same activations, sequence- and
pool-sharded, with every collective inside the kernels.

The Q, K and V routes of an attention block all consume the same normed ``x``
(and the Know route its own), so the per-route version of the fused path
(parallel/fused_srw.py) gathers ``x`` three times, pays two barriers per route
and sums the per-token denominators with a separate all-reduce between the
gate kernel and the write GEMM.  Here one group is

  forward (2 barriers, no other collective)
    1. each rank writes its rows of ``x``, of all routes' ``h`` and of the
       per-token statistics ``(tau, 1/sigma)`` into its slice of the symmetric
       full buffers; barrier;
    2. the first route's gate kernel pulls the peers' rows of ALL of them
       (gather warps: TMA for the bf16 tensors, plain 16-byte copies for the
       statistics); the other routes' gate kernels find them in place;
    3. every route's write GEMM stores its un-normalised bf16 partial rows into
       its slot of the owner's receive buffer and, in the same epilogue, its
       partial denominators into the owner's denominator slots; barrier;
    4. the owner sums slots and denominators and divides AFTER the reduction:
       ``out = scale * sum_w raw_w / max(sum_w den_w, 1)``.
  backward (2 barriers)
    the cotangents take the same road: ``dy`` rows and ``(tau, 1/sigma, dden)``
    are gathered by the first backward gate kernel together with ``x`` and
    ``h``; ``dx`` (all routes into one buffer of routes x ranks slabs), ``dh``
    and the partial ``dtau`` leave through the scatter epilogues.

Pool gradients stay on the rank that owns the units.  Requires the 256-wide
gate kernels (every pool's local unit count >= 512) and kept read scalars.
"""
from __future__ import annotations

from typing import List, Sequence

import torch

from ..ops.gates import GATE_GELU_Z
from .symm import SymmWorkspace

MAX_ROUTES = 3
# From this many ranks on, every kernel of a group gathers its own rows; below it the first
# kernel gathers for all.  Measured per 400M step: 2 ranks 780 vs 794 ms and 4 ranks 812 vs 837 ms
# in favour of the single gather (the other kernels keep their full operand ring), 8 ranks 902 vs
# 878 ms in favour of the spread one (1.35 GB would otherwise arrive in one 0.46 ms kernel).
kSpreadGatherRanks = int(__import__("os").environ.get("DSB_SPREAD_GATHER_RANKS", "8"))


class GroupShardComm:
    """Symmetric buffers shared by all route groups of a model (sized for up
    to three routes per group)."""

    def __init__(self, group, device, t_local: int, d_model: int, d_route: int):
        self.ws = SymmWorkspace(group, device)
        self.group = self.ws.group
        self.rank, self.world = self.ws.rank, self.ws.world
        if t_local % 256 != 0:
            raise ValueError(f"tokens per rank ({t_local}) must be a multiple of 256 for the fused path")
        self.t_local, self.t_total = t_local, t_local * self.world
        self.d_model, self.d_route = d_model, d_route
        bf, f32 = torch.bfloat16, torch.float32
        T, W, R = self.t_total, self.world, MAX_ROUTES
        a = self.ws.alloc
        # gathered operands, two of each (a buffer is rewritten two groups after it was read,
        # with a barrier in between that every reader passes only after its read)
        self.xfull = [a(f"g_x{i}", (T, d_model), bf) for i in range(2)]
        self.hfull = [a(f"g_h{i}", (T, R * d_route), bf) for i in range(2)]
        self.dyfull = [a(f"g_dy{i}", (T, R * d_model), bf) for i in range(2)]
        self.stats = [[a(f"g_st{i}_{j}", (T, 4), f32) for j in range(R)] for i in range(2)]
        # receive buffers of the reduce-scatters: [route][rank slot][local token]
        self.out_rs = [a(f"g_out{i}", (R * W * t_local, d_model), bf) for i in range(2)]
        self.dx_rs = [a(f"g_dx{i}", (R * W * t_local, d_model), bf) for i in range(2)]
        self.dh_rs = [a(f"g_dh{i}", (R * W * t_local, d_route), bf) for i in range(2)]
        self.aux_rs = [a(f"g_aux{i}", (R * W * t_local,), f32) for i in range(2)]   # den / dtau partials
        self.ready = torch.zeros(T // 128, dtype=torch.int32, device=device)
        self.epoch = 0
        self._parity = {"gather": 0, "out": 0, "dx": 0}
        self.rows = slice(self.rank * t_local, (self.rank + 1) * t_local)
        from . import collectives as C
        self.ws.enable_small_allreduce()
        C.register_small_allreduce(group, self.ws.all_reduce_small, self.ws.AR_CAP)
        if group is not self.group:
            C.register_small_allreduce(self.group, self.ws.all_reduce_small, self.ws.AR_CAP)

    def flip(self, which: str) -> int:
        self._parity[which] ^= 1
        return self._parity[which]

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    @staticmethod
    def offset_ptrs(buf, elems: int) -> List[int]:
        """Peer pointers of ``buf`` advanced by ``elems`` elements."""
        return [p + elems * buf.local.element_size() for p in buf.ptrs]


class _RouteGroupFn(torch.autograd.Function):
    """inputs:  x_bf [Tl, D] bf16, h_all [Tl, nR, r] bf16, tau [Tl, nR], inv_sd [Tl, nR],
                then the non-tensor arguments, anchors (one per call; they keep the
                pool-preparation node last in backward) and scales (one tensor per route)
       outputs: nR outputs [Tl, D] fp32 (normalised and scaled), nR denominators [Tl]."""

    @staticmethod
    def forward(ctx, x_bf, h_all, tau, inv_sd, comm, spec, holders, units, n_anchor, alives, masks,
                diags, tau_off, *rest):
        from ..ops import cuda_backend as CB
        anchors, scales = rest[:n_anchor], rest[n_anchor:]
        c: GroupShardComm = comm
        e, dev = CB.ext(), x_bf.device
        st = CB.status_word(dev)
        T, Tl, W = c.t_total, c.t_local, c.world
        D, r = c.d_model, c.d_route
        nR = h_all.shape[1]
        gl = CB._gate_list(spec)
        b = c.flip("gather")
        xf, hf, sf = c.xfull[b], c.hfull[b], c.stats[b]
        xf.local[c.rows].copy_(x_bf)
        hf.local[c.rows, : nR * r].copy_(h_all.reshape(Tl, nR * r))
        for i in range(nR):
            s_loc = sf[i].local[c.rows]
            s_loc[:, 0].copy_(tau[:, i])
            s_loc[:, 1].copy_(inv_sd[:, i])
            if tau_off is not None:                      # only the diagnostics read it back
                s_loc[:, 3].copy_(tau_off[:, i])
        c.ws.barrier()                                   # every rank's rows are in place
        ob = c.flip("out")
        out_t, aux_t = c.out_rs[ob], c.aux_rs[ob]
        xrs = []
        keep = any(ctx.needs_input_grad[:4])             # a backward pass will follow
        for i in range(nR):
            hd, U = holders[i], units[i]
            Up = CB._round_up(U, 8)
            p = torch.empty(T, Up, dtype=torch.bfloat16, device=dev)
            xr = torch.empty(T, Up, dtype=torch.bfloat16, device=dev) if keep else None
            den = torch.zeros(T, dtype=torch.float32, device=dev)
            h_i = hf.local[:, i * r:(i + 1) * r]
            if W >= kSpreadGatherRanks:
                # every kernel brings in what it needs and nobody has brought yet: the first
                # one x and its own h rows, the others only their h rows and statistics - the
                # copies of a group are spread over its kernels instead of all waiting on the
                # first (with many ranks the first kernel is far shorter than its gather)
                ptrs, lds, cols = [c.offset_ptrs(hf, i * r)], [hf.local.stride(0)], [r]
                if i == 0:
                    ptrs, lds, cols = [xf.ptrs] + ptrs, [xf.local.stride(0)] + lds, [D] + cols
                gather = (ptrs, lds, cols, [sf[i].ptrs], c.rank, Tl, c.ready, c.next_epoch())
            elif i == 0:                                 # few ranks: the first kernel brings everything in
                gather = ([xf.ptrs, hf.ptrs], [xf.local.stride(0), hf.local.stride(0)], [D, nR * r],
                          [sf[j].ptrs for j in range(nR)], c.rank, Tl, c.ready, c.next_epoch())
            else:
                gather = CB.NO_GATHER
            e.srw_fwd_gate_xr(h_i, hd.emb[:U], xf.local, hd.read[:U], p, xr, None, None, sf[i].local,
                              den, diags[i], alives[i], masks[i], gl, st, *gather)
            # un-normalised partial rows + partial denominators to the owners
            e.gemm_scatter(p[:, :U], False, hd.write[:U], True,
                           c.offset_ptrs(out_t, i * W * Tl * D), c.rank, Tl, D, True, 1.0, None, st,
                           den, c.offset_ptrs(aux_t, i * W * Tl))
            xrs.append(xr)
        CB.count_launches(2 * nR)
        c.ws.barrier()                                   # every rank's partial rows have landed
        outs, dens = [], []
        for i in range(nR):
            sc = scales[i].detach().float().reshape(1)
            o, d = e.sum_slabs_div(out_t.local[i * W * Tl:(i + 1) * W * Tl], W,
                                   aux_t.local[i * W * Tl:(i + 1) * W * Tl], sc)
            outs.append(o)
            dens.append(d)
        CB.count_launches(nR)
        ctx.save_for_backward(x_bf, h_all, tau, inv_sd, *outs, *dens, *scales)
        ctx.xrs = xrs
        ctx.meta = (c, spec, holders, units, nR, n_anchor)
        ctx.masked = any(m is not None for m in masks)
        ctx.mark_non_differentiable(*dens)
        return tuple(outs) + tuple(dens)

    @staticmethod
    def backward(ctx, *grads):
        from ..ops import cuda_backend as CB
        c, spec, holders, units, nR, n_anchor = ctx.meta
        if ctx.masked:
            raise RuntimeError("a unit-masked (ablation) forward has no backward on the fused path")
        sv = ctx.saved_tensors
        x_bf, h_all, tau, inv_sd = sv[:4]
        outs, dens, scales = sv[4:4 + nR], sv[4 + nR:4 + 2 * nR], sv[4 + 2 * nR:]
        xrs, ctx.xrs = ctx.xrs, None
        e, dev = CB.ext(), x_bf.device
        st = CB.status_word(dev)
        T, Tl, W = c.t_total, c.t_local, c.world
        D, r = c.d_model, c.d_route
        gl = CB._gate_list(spec)
        b = c.flip("gather")
        xf, hf, dyf, sf = c.xfull[b], c.hfull[b], c.dyfull[b], c.stats[b]
        xf.local[c.rows].copy_(x_bf)
        hf.local[c.rows, : nR * r].copy_(h_all.reshape(Tl, nR * r))
        d_scales = []
        for i in range(nR):
            d_out = grads[i]
            if d_out is None:
                d_out = torch.zeros_like(outs[i])
            den_l = dens[i].clamp(min=1.0)
            rs_l = (scales[i].detach().float() / den_l).contiguous()
            # one pass over (d_out, out): bf16 dy * scale / den and <d_out, out> per token, which
            # gives the denominator and scale gradients (out = scale * raw / den)
            dyb, rowdot = e.route_bwd_prologue(d_out.float().contiguous(), outs[i], rs_l)
            dyf.local[c.rows, i * D:(i + 1) * D].copy_(dyb)
            dden_l = torch.where(dens[i] > 1.0, -rowdot / den_l, torch.zeros_like(rowdot))
            s_loc = sf[i].local[c.rows]
            s_loc[:, 0].copy_(tau[:, i])
            s_loc[:, 1].copy_(inv_sd[:, i])
            s_loc[:, 2].copy_(dden_l)
            d_scales.append((rowdot.sum() / scales[i].detach().float()).reshape(scales[i].shape)
                            .to(scales[i].dtype) if ctx.needs_input_grad[13 + n_anchor + i] else None)
        CB.count_launches(nR)
        c.ws.barrier()
        xb = c.flip("dx")
        dx_t, dh_t, aux_t = c.dx_rs[xb], c.dh_rs[xb], c.aux_rs[xb]
        for i in range(nR):
            hd, U = holders[i], units[i]
            emb, read, write = hd.emb[:U], hd.read[:U], hd.write[:U]
            p = xrs[i]                                   # p overwrites the kept read scalars
            dxr, ds = torch.empty_like(p), torch.empty_like(p)
            dtau = torch.zeros(T, dtype=torch.float32, device=dev)
            h_i = hf.local[:, i * r:(i + 1) * r]
            dy_i = dyf.local[:, i * D:(i + 1) * D]
            if W >= kSpreadGatherRanks:
                # as in forward: each kernel gathers its own dy and h rows, the first one x too
                ptrs = [c.offset_ptrs(hf, i * r), c.offset_ptrs(dyf, i * D)]
                lds, cols = [hf.local.stride(0), dyf.local.stride(0)], [r, D]
                if i == 0:
                    ptrs, lds, cols = [xf.ptrs] + ptrs, [xf.local.stride(0)] + lds, [D] + cols
                gather = (ptrs, lds, cols, [sf[i].ptrs], c.rank, Tl, c.ready, c.next_epoch())
            elif i == 0:
                gather = ([xf.ptrs, hf.ptrs, dyf.ptrs],
                          [xf.local.stride(0), hf.local.stride(0), dyf.local.stride(0)],
                          [D, nR * r, nR * D], [sf[j].ptrs for j in range(nR)], c.rank, Tl, c.ready,
                          c.next_epoch())
            else:
                gather = CB.NO_GATHER
            e.srw_bwd_gate_xr(h_i, emb, dy_i, write, p, p, dxr, ds, None, None, None, sf[i].local, dtau,
                              gl, st, *gather)
            pv, dxrv, dsv = p[:, :U], dxr[:, :U], ds[:, :U]
            CB.gemm(pv, True, dy_i, True, out=hd.g_write[:U], accumulate=True)        # p^T dy
            CB.gemm(dxrv, True, xf.local, True, out=hd.g_read[:U], accumulate=True)   # dxr^T x
            CB.gemm(dsv, True, h_i, True, out=hd.g_emb[:U], accumulate=True)          # ds^T h
            e.gemm_scatter(dxrv, False, read, True, c.offset_ptrs(dx_t, i * W * Tl * D), c.rank, Tl,
                           D, True, 1.0, None, st, dtau, c.offset_ptrs(aux_t, i * W * Tl))   # dxr . read
            e.gemm_scatter(dsv, False, emb, True, c.offset_ptrs(dh_t, i * W * Tl * r), c.rank, Tl, r,
                           True, 1.0, None, st, None, [])                                   # ds . emb
            xrs[i] = None
        CB.count_launches(3 * nR)
        c.ws.barrier()
        dx = e.sum_slabs(dx_t.local[: nR * W * Tl], nR * W, True)          # bf16 [Tl, D], all routes
        dhs, dtaus, d_isds = [], [], []
        for i in range(nR):
            dh32 = e.sum_slabs(dh_t.local[i * W * Tl:(i + 1) * W * Tl], W, False)     # fp32 [Tl, r]
            dtau_l = aux_t.local[i * W * Tl:(i + 1) * W * Tl].view(W, Tl).sum(0)
            dhs.append(dh32.to(torch.bfloat16))
            dtaus.append(dtau_l)
            if spec.kind == GATE_GELU_Z:
                # sum_u ds_u z_u = (1/sigma)(<h, ds.emb> + tau * dtau) on the fully reduced values
                isd_l, tau_l = inv_sd[:, i], tau[:, i]
                dsz_l = isd_l * ((h_all[:, i].float() * dh32).sum(-1) + tau_l * dtau_l)
                d_isds.append(dsz_l / (isd_l * isd_l))
        CB.count_launches(1 + nR)
        d_h = torch.stack(dhs, dim=1)
        d_tau = torch.stack(dtaus, dim=1)
        d_isd = torch.stack(d_isds, dim=1) if d_isds else None
        zeros = tuple(torch.zeros(1, device=dev) for _ in range(n_anchor))
        return (dx, d_h, d_tau, d_isd, None, None, None, None, None, None, None, None, None) + \
            zeros + tuple(d_scales)


def route_group(x_bf, h_all, tau, inv_sd, comm, spec, holders: Sequence, units: Sequence[int],
                anchors: Sequence[torch.Tensor], scales: Sequence[torch.Tensor],
                alives: Sequence = None, masks: Sequence = None, diags: Sequence = None,
                tau_off=None):
    """One entry of holders / units / scales / alives / masks per ROUTE (a pool with two
    routes appears twice), one anchor per call.  ``alives``: uint8 [U] buffers that get a 1
    for every unit some token gates above the dead threshold (or None); ``masks``: fp32 [U]
    multipliers on the gate (ablation; forward only); ``diags``: zeroed fp32 [T * 12 + 2]
    buffers for the routing diagnostics of log steps (with ``tau_off`` [Tl, nR], which then
    travels in the spare slot of the per-token statistics so that every rank can finalise them).
    -> (outs: list of [Tl, D] fp32, dens: list of [Tl])."""
    nR = h_all.shape[1]
    alives = tuple(alives) if alives is not None else (None,) * nR
    masks = tuple(masks) if masks is not None else (None,) * nR
    diags = tuple(diags) if diags is not None else (None,) * nR
    res = _RouteGroupFn.apply(x_bf, h_all, tau, inv_sd, comm, spec, tuple(holders), tuple(units),
                              len(anchors), alives, masks, diags,
                              None if tau_off is None else tau_off.detach(), *anchors, *scales)
    return list(res[:nR]), list(res[nR:])
