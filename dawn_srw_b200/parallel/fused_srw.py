"""Sequence-sharded, pool-sharded SRW route with the collectives inside the kernels.

Layout (8 GPUs = one shard group): rank k stores ``U/8`` units of every pool and
``T/8`` tokens of the activations.  One SRW route then is

  forward
    1. each rank writes its bf16 ``x``/``h`` rows into its slice of the
       symmetric "full" buffers; bounded barrier;
    2. gate kernel with the all-gather fused in: gather warps pull the other
       ranks' row blocks over NVLink (TMA from peer memory) into the local full
       buffer while tcgen05 tiles on this rank's own tokens already run;
       writes ``p = gate * xr`` for all tokens x local units and the partial
       ``sum_U den_term`` per token;
    3. the per-token denominators are summed over ranks (``[T]`` fp32, NCCL);
    4. write GEMM with the reduce-scatter fused into its epilogue: each 32-row
       slab of ``scale * (p . write) / den`` is TMA-stored (bf16) into this
       rank's slot of the owner rank's receive buffer, locally or over NVLink;
       after a barrier the owner sums its slots in fp32.  (Plain stores cross
       NVLink at write bandwidth; remote fp32 reduce-adds measured 3-4x slower.)
  backward mirrors it: ``dy`` rows are gathered by the backward gate kernel
  together with ``x`` and ``h``; ``dx`` and ``dh`` leave through the same fused
  reduce-scatter epilogue; pool gradients stay on the rank that owns the units.

Against the reference's layout (activations replicated over the unit axis and a
bf16 all-reduce of the output, models/dawn_spatial_v41_exp.py:579-586) this
halves the output traffic and removes the redundant LayerNorm / router /
attention work across the group.
"""
from __future__ import annotations

from typing import Dict

import torch
import torch.distributed as dist

from ..ops.gates import GATE_GELU_Z
from . import collectives as C
from .symm import SymmWorkspace


class FusedShardComm:
    """Symmetric buffers + counters shared by all fused SRW calls of a model."""

    def __init__(self, group, device, t_local: int, d_model: int, d_route: int):
        self.ws = SymmWorkspace(group, device)
        self.group = self.ws.group
        self.rank, self.world = self.ws.rank, self.ws.world
        if t_local % 256 != 0:
            raise ValueError(f"tokens per rank ({t_local}) must be a multiple of 256 for the fused path")
        self.t_local, self.t_total = t_local, t_local * self.world
        bf, f32 = torch.bfloat16, torch.float32
        T = self.t_total
        self.xfull = [self.ws.alloc(f"xfull{i}", (T, d_model), bf) for i in range(2)]
        self.hfull = [self.ws.alloc(f"hfull{i}", (T, d_route), bf) for i in range(2)]
        self.dyfull = [self.ws.alloc(f"dyfull{i}", (T, d_model), bf) for i in range(2)]
        # reduce-scatter receive buffers: every rank stores its partial rows for this rank's
        # tokens into its own slot ([world, t_local, cols], bf16); the owner sums the slots.
        # Two of each: a buffer is next written two ops after it was read, with a barrier in
        # between that the reader only passes after its read, so no peer can overwrite early.
        W = self.world
        self.out_rs = [self.ws.alloc(f"out_rs{i}", (W * t_local, d_model), bf) for i in range(2)]
        self.dx_rs = [self.ws.alloc(f"dx_rs{i}", (W * t_local, d_model), bf) for i in range(2)]
        self.dh_rs = [self.ws.alloc(f"dh_rs{i}", (W * t_local, d_route), bf) for i in range(2)]
        self._rs_parity = {"out": 0, "dx": 0}
        self.ready = torch.zeros(T // 128, dtype=torch.int32, device=device)
        self.epoch = 0
        self.parity = 0
        self.rows = slice(self.rank * t_local, (self.rank + 1) * t_local)
        # small fp32 sums over this group (per-token statistics, denominators, loss terms)
        # go through one peer-memory kernel instead of a library all-reduce
        from . import collectives as C
        self.ws.enable_small_allreduce()
        C.register_small_allreduce(group, self.ws.all_reduce_small, self.ws.AR_CAP)
        if group is not self.group:
            C.register_small_allreduce(self.group, self.ws.all_reduce_small, self.ws.AR_CAP)

    def next_buffers(self):
        self.parity ^= 1
        return self.parity

    def next_rs(self, which: str) -> int:
        self._rs_parity[which] ^= 1
        return self._rs_parity[which]

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch


class _SRWRouteGatherFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_bf, h_bf, tau_full, inv_sd_full, anchor, holder, spec, U, comm, scale):
        from ..ops import cuda_backend as CB
        e, dev = CB.ext(), x_bf.device
        st = CB.status_word(dev)
        c: FusedShardComm = comm
        T, Tl, D = c.t_total, c.t_local, x_bf.shape[1]
        Up = CB._round_up(U, 8)
        b = c.next_buffers()
        xf, hf = c.xfull[b], c.hfull[b]
        xf.local[c.rows].copy_(x_bf)
        hf.local[c.rows].copy_(h_bf)
        c.ws.barrier()                                   # every rank's rows are in place
        p = torch.empty(T, Up, dtype=torch.bfloat16, device=dev)
        den = torch.zeros(T, dtype=torch.float32, device=dev)
        gl = CB._gate_list(spec)
        CB._LAUNCHES += 2
        e.srw_fwd_gate_gather(hf.local, holder.emb[:U], xf.local, holder.read[:U], p, tau_full,
                              inv_sd_full, den, gl, st, [xf.ptrs, hf.ptrs], c.rank, Tl, c.ready,
                              c.next_epoch())
        C._all_reduce_sum_(den, c.group)                 # [T] fp32: peer-memory kernel when it fits
        inv_den = (scale.detach().float() / den.clamp(min=1.0)).contiguous()   # pool scale folded in
        tgt = c.out_rs[c.next_rs("out")]
        e.gemm_scatter(p[:, :U], False, holder.write[:U], True, tgt.ptrs, c.rank, Tl, D, True, 1.0,
                       inv_den, st, None, [])
        c.ws.barrier()                                   # every rank's partial rows have landed
        out = e.sum_slabs(tgt.local, c.world, False)     # fp32 [Tl, D]
        CB.count_launches(1)
        ctx.save_for_backward(x_bf, h_bf, tau_full, inv_sd_full, den, out, scale)
        ctx.holder, ctx.spec, ctx.U, ctx.comm = holder, spec, U, c
        ctx.mark_non_differentiable(den)
        return out, den

    @staticmethod
    def backward(ctx, d_out, _d_den):
        from ..ops import cuda_backend as CB
        x_bf, h_bf, tau_full, inv_sd_full, den, out, scale = ctx.saved_tensors
        hd, spec, U, c = ctx.holder, ctx.spec, ctx.U, ctx.comm
        e, dev = CB.ext(), x_bf.device
        st = CB.status_word(dev)
        T, Tl, D, r = c.t_total, c.t_local, x_bf.shape[1], h_bf.shape[1]
        Up = CB._round_up(U, 8)
        den_l = den[c.rows]
        rs_l = (scale.detach().float() / den_l.clamp(min=1.0)).contiguous()
        b = c.next_buffers()
        xf, hf, dyf = c.xfull[b], c.hfull[b], c.dyfull[b]
        xf.local[c.rows].copy_(x_bf)
        hf.local[c.rows].copy_(h_bf)
        # one pass over (d_out, out): bf16 dy * scale / den, and <d_out, out> per token, which
        # gives the denominator and scale gradients (out = scale * raw / den)
        dyb, rowdot = e.route_bwd_prologue(d_out.float().contiguous(), out, rs_l)
        CB.count_launches(1)
        dyf.local[c.rows].copy_(dyb)
        dden_l = torch.where(den_l > 1.0, -rowdot / den_l.clamp(min=1.0), torch.zeros_like(rowdot))
        d_scale = (rowdot.sum() / scale.detach().float()).reshape(scale.shape).to(scale.dtype) \
            if ctx.needs_input_grad[9] else None
        dden = torch.empty(T, dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(dden, dden_l.contiguous(), group=c.group)
        c.ws.barrier()
        p = torch.empty(T, Up, dtype=torch.bfloat16, device=dev)
        dxr, ds = torch.empty_like(p), torch.empty_like(p)
        dtau = torch.zeros(T, dtype=torch.float32, device=dev)
        dsz = torch.zeros(T, dtype=torch.float32, device=dev)
        emb, read, write = hd.emb[:U], hd.read[:U], hd.write[:U]
        CB._LAUNCHES += 2
        ep = c.next_epoch()      # the wide kernel pair uses ep (x, h rows) and ep + 1 (dy rows)
        c.next_epoch()
        e.srw_bwd_gate_gather(hf.local, emb, xf.local, read, dyf.local, write, p, dxr, ds, tau_full,
                              inv_sd_full, dden, dtau, dsz, CB._gate_list(spec), st,
                              [xf.ptrs, hf.ptrs, dyf.ptrs], c.rank, Tl, c.ready, ep)
        pv, dxrv, dsv = p[:, :U], dxr[:, :U], ds[:, :U]
        CB.gemm(pv, True, dyf.local, True, out=hd.g_write[:U], accumulate=True)      # p^T dy
        CB.gemm(dxrv, True, xf.local, True, out=hd.g_read[:U], accumulate=True)      # dxr^T x
        CB.gemm(dsv, True, hf.local, True, out=hd.g_emb[:U], accumulate=True)        # ds^T h
        bi = c.next_rs("dx")
        dxt, dht = c.dx_rs[bi], c.dh_rs[bi]
        CB._LAUNCHES += 2
        e.gemm_scatter(dxrv, False, read, True, dxt.ptrs, c.rank, Tl, D, True, 1.0, None, st, None, [])   # dxr . read
        e.gemm_scatter(dsv, False, emb, True, dht.ptrs, c.rank, Tl, r, True, 1.0, None, st, None, [])     # ds . emb
        c.ws.barrier()
        dx = e.sum_slabs(dxt.local, c.world, True)       # bf16 [Tl, D]
        dh32 = e.sum_slabs(dht.local, c.world, False)    # fp32 [Tl, r]
        CB.count_launches(2)
        d_isd = None
        if spec.kind == GATE_GELU_Z:
            # sum_u ds_u z_u = (1/sigma)(<h, ds.emb> + tau * dtau), evaluated by the owner of
            # each token on the fully reduced ds.emb and dtau; other rows contribute zero
            dtau_l = torch.empty(Tl, dtype=torch.float32, device=dev)
            dist.reduce_scatter_tensor(dtau_l, dtau, group=c.group)
            isd_l, tau_l = inv_sd_full[c.rows], tau_full[c.rows]
            dsz_l = isd_l * ((h_bf.float() * dh32).sum(-1) + tau_l * dtau_l)
            d_isd = torch.zeros(T, dtype=torch.float32, device=dev)
            d_isd[c.rows] = dsz_l / (isd_l * isd_l)
        return (dx, dh32.to(torch.bfloat16), dtau, d_isd, torch.zeros(1, device=dev), None, None,
                None, None, d_scale)
