"""sm_100a backend: autograd wrappers around the hand-written kernels.

SRW pool op, one route (reference math: models/dawn_spatial_v41_exp.py:352-637;
the reference gets its backward from autodiff and recomputes per chunk):

  prepare (once per step, shared by all layers)
      emb_c/read_c/write_c = bf16(optionally row-normalised pool tensors)
      G = emb_c^T emb_c  [r,r],  e_sum = sum_u emb_c[u]      (fp32)
  per call
      mu    = h . e_sum / U            E[s^2] = h G h^T / U      (no pass over [T,U];
      sigma = sqrt(E[s^2] - mu^2) + 1e-8 ;  tau = mu + tau_off * sigma    ops/score_stats.py)
      kernel A (tcgen05):  S = h.emb^T, XR = x.read^T in TMEM; epilogue
                           p = gate(S) * XR -> bf16 [T,U];  den_sum[T]
      kernel B (tcgen05):  raw_out = p . write     [T,D]
      out = raw_out / max(den_sum, 1)
  backward
      kernel C (tcgen05):  S, XR, DP = dy.write^T in TMEM; epilogue writes
                           p, dxr = DP*g, ds and the per-token sums for tau, sigma
      five plain tcgen05 GEMMs: dwrite += p^T dy, dread += dxr^T x, demb += ds^T h
                           (TMA reduce-add into fp32 buffers shared by all layers),
                           dx = dxr . read, dh = ds . emb

The per-token score mean and variance over the pool are quadratic forms in
``h`` (sum_u (h.e_u)^2 = h (E^T E) h^T), so the reference's first pass over all
scores collapses to one r x r Gram matrix per step; its gradient reaches ``emb``
through G.  The per-unit mean score used by the load-balance and dead-unit
terms is likewise ``emb . mean_t(h)``.
"""
from __future__ import annotations

import math
from typing import Any, List, Optional

import torch
import torch.nn.functional as F

from . import build as _build
from . import reference as R
from .backend import ParallelCtx, PreparedPool
from .gates import GATE_GELU_Z, GateSpec
from .score_stats import score_stats, score_stats_rows
from .srw_ref import SRWResult, srw_pool_ref
from ..parallel import collectives as C

_EXT = None
_STATUS = {}
_LAUNCHES = 0


def launch_count() -> int:
    """How many kernels of this library have been launched by this process."""
    return _LAUNCHES


def ext():
    """The compiled extension; building or importing it must succeed on a GPU box."""
    global _EXT
    if _EXT is None:
        _EXT = _build.load()
    return _EXT


def status_word(device) -> torch.Tensor:
    device = torch.device(device)
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _STATUS:
        _STATUS[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _STATUS[key]


def check_status(device=None) -> None:
    """Raise if any kernel since the last check reported a device-side failure
    (a bounded wait that ran out).  Synchronises the device."""
    for key, st in list(_STATUS.items()):
        _PENDING.pop(key, None)
        code = int(st.item())
        if code != 0:
            st.zero_()
            raise RuntimeError(f"dawn_srw_b200 kernel reported status {code} on cuda:{key} "
                               "(1 = barrier wait timed out, 3 = peer wait timed out)")


_PENDING = {}


def check_status_deferred() -> None:
    """Per-step variant of ``check_status`` that does not stall the launching
    thread: it raises on the status word as it stood at the *previous* call
    (copied to pinned host memory asynchronously then) and queues the next
    copy.  A device-side failure is therefore reported one step late, while
    the CPU keeps running ahead of the GPU across step boundaries."""
    for key, st in list(_STATUS.items()):
        prev = _PENDING.get(key)
        if prev is not None:
            ev, host = prev
            ev.synchronize()
            code = int(host[0])
            if code != 0:
                st.zero_()
                _PENDING.pop(key, None)
                raise RuntimeError(f"dawn_srw_b200 kernel reported status {code} on cuda:{key} "
                                   "(1 = barrier wait timed out, 3 = peer wait timed out)")
            host_buf = host
        else:
            host_buf = torch.zeros(1, dtype=torch.int32).pin_memory()
        with torch.cuda.device(st.device):
            host_buf.copy_(st, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        _PENDING[key] = (ev, host_buf)


def _gate_list(spec: GateSpec) -> List[float]:
    return [spec.kind, spec.sharpness, spec.activation_threshold, spec.activation_cutoff,
            spec.epsilon, spec.max_intensity, spec.clip_max, spec.dead_threshold]


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class _XrBudget:
    """Accounting for the read scalars ``xr = x . read^T`` that forward passes keep
    for their backward pass (bf16 [T, U] per route and layer).  Keeping them
    removes the largest recomputed product from the backward gate step; the
    budget bounds how much device memory that may take.  ``limit`` defaults to
    half of the device memory (``DSB_XR_BUDGET_GB`` overrides it, 0 disables)."""

    def __init__(self):
        self.limit = {}
        self.live = {}

    def _limit(self, dev: torch.device) -> int:
        key = dev.index if dev.index is not None else torch.cuda.current_device()
        if key not in self.limit:
            import os
            env = os.environ.get("DSB_XR_BUDGET_GB")
            if env is not None:
                self.limit[key] = int(float(env) * (1 << 30))
            else:
                self.limit[key] = torch.cuda.get_device_properties(key).total_memory // 2
            self.live[key] = 0
        return key

    def acquire(self, dev: torch.device, nbytes: int) -> bool:
        key = self._limit(dev)
        if self.live[key] + nbytes > self.limit[key]:
            return False
        self.live[key] += nbytes
        return True

    def release(self, key: int, nbytes: int) -> None:
        self.live[key] = max(0, self.live.get(key, 0) - nbytes)


XR_BUDGET = _XrBudget()

# trailing arguments of the gate-kernel bindings when no all-gather is fused in:
# (ptr_lists, lds, cols, stat_lists, my_rank, rows_per_rank, ready, epoch)
NO_GATHER = ([], [], [], [], 0, 0, None, 0)


def _alloc_saved_xr(dev, T: int, Up: int, U: int, wanted: bool):
    """bf16 [T, Up] buffer for the read scalars of one route if the pool runs on
    the wide kernels and the budget allows it (``wanted``: a backward pass will
    follow and no unit mask is in play)."""
    if not wanted or not ext().srw_wide_tiles(U):
        return None
    nbytes = T * Up * 2
    if not XR_BUDGET.acquire(dev, nbytes):
        return None
    xr = torch.empty(T, Up, dtype=torch.bfloat16, device=dev)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    import weakref
    weakref.finalize(xr, XR_BUDGET.release, key, nbytes)
    return xr


def gemm(a, a_mn, b, b_mn, *, out=None, out_dtype=torch.float32, accumulate=False, alpha=1.0,
         row_scale=None, bias=None, block_n: Optional[int] = None):
    """out[M,N] (=|+=) alpha * row_scale * A.B^T + bias on the tcgen05 engine.
    a_mn / b_mn: the operand is stored transposed ([K, rows])."""
    M = a.shape[1] if a_mn else a.shape[0]
    N = b.shape[1] if b_mn else b.shape[0]
    if out is None:
        ld = _round_up(N, 8)
        buf = torch.empty(M, ld, dtype=out_dtype, device=a.device)
        out = buf[:, :N] if ld != N else buf
    if block_n is None:
        block_n = 128 if N <= 128 else 256
    global _LAUNCHES
    _LAUNCHES += 1
    if (M <= 4 and not a_mn and not b_mn and not accumulate and alpha == 1.0 and row_scale is None
            and out.dtype == torch.float32 and a.is_contiguous() and a.shape[1] % 8 == 0
            and a.shape[1] <= 8192):
        # a handful of rows (decoding): one SIMT pass over the weights instead of a 128-row MMA tile
        ext().gemv_rows(a, b, bias, out)
        return out
    ext().gemm(a, a_mn, b, b_mn, out, accumulate, float(alpha), row_scale, bias, block_n,
               status_word(a.device))
    return out


def _bf16_2d(t: torch.Tensor) -> torch.Tensor:
    """bf16, unit inner stride, 16-byte aligned rows."""
    if t.dtype != torch.bfloat16:
        t = t.to(torch.bfloat16)
    if t.stride(-1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        t = t.contiguous()
        if t.shape[1] % 8 != 0:
            buf = torch.zeros(t.shape[0], _round_up(t.shape[1], 8), dtype=t.dtype, device=t.device)
            buf[:, :t.shape[1]] = t
            t = buf[:, :t.shape[1]]
    return t


# ---------------------------------------------------------------------------
# dense layer:  y = x W^T + b   (W is [out, in])
class _LinearFn(torch.autograd.Function):
    """``w`` is the fp32 master weight (receives an fp32 gradient); ``w_bf`` is
    its bf16 compute copy, made once per optimizer step."""
    @staticmethod
    def forward(ctx, x, w, bias, w_bf, out_dtype):
        xb = _bf16_2d(x)
        ctx.save_for_backward(xb, w_bf)
        ctx.has_bias = bias is not None
        ctx.x_dtype = x.dtype
        return gemm(xb, False, w_bf, False, out_dtype=out_dtype, bias=bias)

    @staticmethod
    def backward(ctx, dy):
        xb, w_bf = ctx.saved_tensors
        dyb = _bf16_2d(dy)
        dx = gemm(dyb, False, w_bf, True, out_dtype=ctx.x_dtype) if ctx.needs_input_grad[0] else None
        dw = gemm(dyb, True, xb, True, out_dtype=torch.float32)           # dy^T . x
        db = dy.float().sum(0) if ctx.has_bias else None
        return dx, dw, db, None, None


class _DropoutFn(torch.autograd.Function):
    """y = res + dropout(x) (``res`` may be None).  The keep mask is a hash of
    (seed, element index): nothing is saved but the seed, backward regenerates it."""
    @staticmethod
    def forward(ctx, res, x, p):
        seed = int(torch.randint(0, 2 ** 62, (1,)).item())        # CPU generator: no device sync
        ctx.seed, ctx.p, ctx.has_res = seed, p, res is not None
        count_launches(1)
        return ext().dropout(None if res is None else res.contiguous(), x.contiguous(), seed, p)

    @staticmethod
    def backward(ctx, dy):
        count_launches(1)
        dx = ext().dropout(None, dy.contiguous(), ctx.seed, ctx.p) if ctx.needs_input_grad[1] else None
        return (dy if ctx.has_res else None), dx, None


class _LayerNormFn(torch.autograd.Function):
    """LayerNorm (eps 1e-6, population variance) with bf16 output: the only
    consumers of a normed activation are bf16 GEMM operands."""
    @staticmethod
    def forward(ctx, x, w, b):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1]).float().contiguous()
        y, mean, rstd = ext().layernorm_fwd(x2, w, b, 1e-6)
        ctx.save_for_backward(x2, w, mean, rstd)
        ctx.shape, ctx.x_dtype = shp, x.dtype
        return y.reshape(shp)

    @staticmethod
    def backward(ctx, dy):
        x2, w, mean, rstd = ctx.saved_tensors
        dy2 = dy.reshape(x2.shape).to(torch.bfloat16).contiguous()
        dx, dw, db = ext().layernorm_bwd(dy2, x2, w, mean, rstd)
        return dx.reshape(ctx.shape).to(ctx.x_dtype), dw, db


# ---------------------------------------------------------------------------
class _PoolTensors:
    """bf16 compute copies of a pool and the fp32 gradient accumulators of the current step."""
    __slots__ = ("emb", "read", "write", "g_emb", "g_read", "g_write", "emb_f", "__weakref__")

    def __init__(self):
        self.emb = self.read = self.write = None
        self.g_emb = self.g_read = self.g_write = None
        self.emb_f = None          # fp32 copy of emb for the per-unit mat-vecs (made on first use)


def _on_tensors(name):
    return property(lambda self: getattr(self.tensors, name),
                    lambda self, v: setattr(self.tensors, name, v))


class CudaPool(PreparedPool):
    """A prepared pool.  Its tensors live on a separate ``tensors`` object: the preparation
    node of the autograd graph (which the pool reaches through ``extra['anchor']``) keeps
    only that object, not the pool, so pool -> anchor -> graph node -> pool is not a cycle.
    Such a cycle runs through the C++ graph, where Python's collector cannot see it, and
    every forward pass that is not followed by a backward pass would leak its pools."""
    emb, read, write = _on_tensors("emb"), _on_tensors("read"), _on_tensors("write")
    g_emb, g_read, g_write = _on_tensors("g_emb"), _on_tensors("g_read"), _on_tensors("g_write")

    def __init__(self):
        self.tensors = _PoolTensors()
        self.extra = None


class _PoolPrepFn(torch.autograd.Function):
    """Once per forward: bf16 (row-normalised) pool copies, the Gram matrix and
    column sum of emb, and zeroed fp32 gradient accumulators that every SRW call
    of the step adds into.  Its backward runs after all of them (they depend on
    ``anchor``) and chains the accumulated gradients through the normalisation."""

    @staticmethod
    def forward(ctx, emb, read, write, holder, normalize, n_valid):
        ctx.normalize = normalize
        ctx.holder = holder
        U = n_valid

        def prep(w):
            if normalize:
                nrm = torch.linalg.vector_norm(w, dim=-1, keepdim=True) + 1e-8
                return (w / nrm).to(torch.bfloat16), nrm
            return w.to(torch.bfloat16), None
        emb_c, n_e = prep(emb)
        read_c, n_r = prep(read)
        write_c, n_w = prep(write)
        # E^T E on the tensor engine (bf16 inputs are exact, fp32 accumulation; the long K = U
        # is split over the SM pairs by the accumulating epilogue)
        r = emb.shape[1]
        if emb.is_cuda:
            gram = torch.zeros(r, r, dtype=torch.float32, device=emb.device)
            gemm(emb_c[:U], True, emb_c[:U], True, out=gram, accumulate=True)
        else:                                        # CPU: the algebra only (tests)
            ef = emb_c[:U].float()
            gram = ef.t() @ ef
        esum = emb_c[:U].sum(0, dtype=torch.float32)
        holder.emb, holder.read, holder.write = emb_c, read_c, write_c
        if any(ctx.needs_input_grad[:3]):
            holder.g_emb = torch.zeros_like(emb, dtype=torch.float32)
            holder.g_read = torch.zeros_like(read, dtype=torch.float32)
            holder.g_write = torch.zeros_like(write, dtype=torch.float32)
        ctx.save_for_backward(emb, read, write, n_e, n_r, n_w)
        ctx.U = U
        anchor = torch.zeros(1, device=emb.device)
        return anchor, gram, esum

    @staticmethod
    def backward(ctx, d_anchor, d_gram, d_esum):
        emb, read, write, n_e, n_r, n_w = ctx.saved_tensors
        hd = ctx.holder
        U = ctx.U
        g_emb, g_read, g_write = hd.g_emb, hd.g_read, hd.g_write
        if d_gram is not None:
            # d emb = E (dG + dG^T): engine GEMMs on a two-term bf16 split of the symmetric
            # factor, accumulated into the shared gradient buffer
            from .score_stats import split_bf16
            sym = (d_gram + d_gram.t()).float().contiguous()
            if sym.is_cuda:
                for part in split_bf16(sym):
                    gemm(hd.emb[:U], False, part, False, out=g_emb[:U], accumulate=True)
            else:
                g_emb[:U] += hd.emb[:U].float() @ sym
        if d_esum is not None:
            g_emb[:U] += d_esum.unsqueeze(0)

        def chain(g, w, nrm):
            if not ctx.normalize:
                return g
            n = w / nrm
            return (g - n * (n * g).sum(-1, keepdim=True)) / nrm
        out = (chain(g_emb, emb, n_e), chain(g_read, read, n_r), chain(g_write, write, n_w))
        hd.g_emb = hd.g_read = hd.g_write = None
        return out + (None, None, None)


def _emb_f32(holder):
    """fp32 copy of the prepared (bf16) embedding rows, made once per prepared pool: every
    layer's mat-vec, forward and backward, uses it."""
    t = holder.tensors if hasattr(holder, "tensors") else holder
    if t.emb_f is None:
        t.emb_f = t.emb.float()
    return t.emb_f


class _PoolMatVecFn(torch.autograd.Function):
    """m[u] = emb_c[u] . v  (per-unit mean score).  The emb gradient is added
    into the pool's shared accumulator."""
    @staticmethod
    def forward(ctx, v, anchor, holder, U):
        ctx.holder, ctx.U = holder, U
        ctx.save_for_backward(v)
        return _emb_f32(holder)[:U] @ v

    @staticmethod
    def backward(ctx, dm):
        (v,) = ctx.saved_tensors
        hd, U = ctx.holder, ctx.U
        hd.g_emb[:U].addr_(dm, v)
        return _emb_f32(hd)[:U].t() @ dm, torch.zeros_like(dm[:1]), None, None


def _route_backward_core(x_bf, h_bf, tau, inv_sd, dy, d_den, hd, spec, U, xr=None):
    """Backward of one local SRW route given the bf16 output cotangent ``dy``
    (already scaled by whatever multiplied ``p . write``) and the cotangent of
    the per-token denominator: the gate step and five engine GEMMs.  With the
    read scalars ``xr`` kept by the forward pass the gate step is one launch
    (S and DP = dy . write^T; p overwrites ``xr`` in place); otherwise S and XR
    are recomputed.  Either way it emits p, dxr, ds and dtau.  Pool gradients
    are accumulated into the holder's fp32 buffers.
    Returns (dx bf16, dh bf16, dtau, d_inv_sigma or None)."""
    e = ext()
    dev = x_bf.device
    T = x_bf.shape[0]
    Up = _round_up(U, 8)
    dtau = torch.zeros(T, dtype=torch.float32, device=dev)
    emb, read, write = hd.emb[:U], hd.read[:U], hd.write[:U]
    if xr is not None:
        p = xr
        dxr = torch.empty_like(p)
        ds = torch.empty_like(p)
        count_launches(1)
        e.srw_bwd_gate_xr(h_bf, emb, dy, write, xr, p, dxr, ds, tau, inv_sd, d_den, None, dtau,
                          _gate_list(spec), status_word(dev), *NO_GATHER)
    else:
        p = torch.empty(T, Up, dtype=torch.bfloat16, device=dev)
        dxr = torch.empty_like(p)
        ds = torch.empty_like(p)
        dsz = torch.zeros(T, dtype=torch.float32, device=dev)
        count_launches(2)
        e.srw_bwd_gate(h_bf, emb, x_bf, read, dy, write, p, dxr, ds, tau, inv_sd, d_den, dtau, dsz,
                       _gate_list(spec), status_word(dev))
    pv, dxrv, dsv = p[:, :U], dxr[:, :U], ds[:, :U]
    gemm(pv, True, dy, True, out=hd.g_write[:U], accumulate=True)       # p^T dy
    gemm(dxrv, True, x_bf, True, out=hd.g_read[:U], accumulate=True)    # dxr^T x
    gemm(dsv, True, h_bf, True, out=hd.g_emb[:U], accumulate=True)      # ds^T h
    dx = gemm(dxrv, False, read, True, out_dtype=torch.bfloat16)        # dxr . read
    dh32 = gemm(dsv, False, emb, True, out_dtype=torch.float32)         # ds . emb
    d_isd = None
    if spec.kind == GATE_GELU_Z:
        # sum_u ds_u z_u = (1/sigma) (<h, ds.emb> + tau * dtau): the sigma path needs no
        # reduction of its own in the kernel
        dsz = inv_sd * ((h_bf.float() * dh32).sum(-1) + tau * dtau)
        d_isd = dsz / (inv_sd * inv_sd)
    return dx, dh32.to(torch.bfloat16), dtau, d_isd


class _SRWRouteFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_bf, h_bf, tau, inv_sd, anchor, holder, spec, U, alive, unit_mask):
        e = ext()
        st = status_word(x_bf.device)
        T, D = x_bf.shape
        Up = _round_up(U, 8)
        p = torch.empty(T, Up, dtype=torch.bfloat16, device=x_bf.device)    # scratch
        den = torch.empty(T, dtype=torch.float32, device=x_bf.device)
        raw = torch.empty(T, D, dtype=torch.float32, device=x_bf.device)
        global _LAUNCHES
        _LAUNCHES += 2
        e.srw_forward(h_bf, holder.emb[:U], x_bf, holder.read[:U], holder.write[:U], tau, inv_sd,
                      p, raw, den, alive, unit_mask, _gate_list(spec), st)
        ctx.save_for_backward(x_bf, h_bf, tau, inv_sd)
        ctx.holder, ctx.spec, ctx.U = holder, spec, U
        return raw, den

    @staticmethod
    def backward(ctx, d_raw, d_den):
        x_bf, h_bf, tau, inv_sd = ctx.saved_tensors
        dev = x_bf.device
        d_den = d_den.contiguous().float() if d_den is not None else torch.zeros(x_bf.shape[0], device=dev)
        dx, dh, dtau, d_isd = _route_backward_core(x_bf, h_bf, tau, inv_sd, _bf16_2d(d_raw), d_den,
                                                   ctx.holder, ctx.spec, ctx.U)
        return (dx, dh, dtau, d_isd, torch.zeros(1, device=dev), None, None, None, None, None)


class _SRWRouteScaledFn(torch.autograd.Function):
    """One SRW route with the sum-normalisation and the pool scale folded into
    the write GEMM's epilogue: ``y = scale * (p . write) / max(den, 1)`` leaves
    the engine as the final fp32 output (no [T, D] pass for the divide or the
    scale).  Backward starts with one row kernel that produces the bf16
    ``dy * scale / max(den, 1)`` operand and ``<dy, y>`` per row, from which the
    denominator and scale gradients follow:
        d_den = -<dy, y> / den  (den > 1),   d_scale = sum_t <dy, y> / scale.
    Only for unsharded pools (the denominator is complete on this rank)."""

    @staticmethod
    def forward(ctx, x_bf, h_bf, tau, inv_sd, anchor, holder, spec, U, alive, unit_mask, scale,
                diag=None):
        e = ext()
        dev = x_bf.device
        T, D = x_bf.shape
        Up = _round_up(U, 8)
        p = torch.empty(T, Up, dtype=torch.bfloat16, device=dev)           # scratch
        den = torch.zeros(T, dtype=torch.float32, device=dev)
        xr = _alloc_saved_xr(dev, T, Up, U, getattr(holder, "keep_xr", True) and unit_mask is None
                             and any(ctx.needs_input_grad))
        count_launches(2)
        e.srw_fwd_gate_xr(h_bf, holder.emb[:U], x_bf, holder.read[:U], p, xr, tau, inv_sd, None, den,
                          diag, alive, unit_mask, _gate_list(spec), status_word(dev), *NO_GATHER)
        rs = (scale.detach().float() / den.clamp(min=1.0)).contiguous()
        y = gemm(p[:, :U], False, holder.write[:U], True, out_dtype=torch.float32, row_scale=rs)
        ctx.save_for_backward(x_bf, h_bf, tau, inv_sd, y, den, rs, scale)
        ctx.holder, ctx.spec, ctx.U = holder, spec, U
        ctx.xr = xr
        return y, den

    @staticmethod
    def backward(ctx, d_y, d_den_ext):
        x_bf, h_bf, tau, inv_sd, y, den, rs, scale = ctx.saved_tensors
        hd, spec, U = ctx.holder, ctx.spec, ctx.U
        dev = x_bf.device
        dy, rowdot = ext().route_bwd_prologue(d_y.contiguous().float(), y, rs)
        count_launches(1)
        d_den = torch.where(den > 1.0, -rowdot / den.clamp(min=1.0), torch.zeros_like(rowdot))
        if d_den_ext is not None:
            d_den = d_den + d_den_ext.float()
        d_scale = (rowdot.sum() / scale.detach().float()).reshape(scale.shape).to(scale.dtype) \
            if ctx.needs_input_grad[10] else None
        xr, ctx.xr = ctx.xr, None
        dx, dh, dtau, d_isd = _route_backward_core(x_bf, h_bf, tau, inv_sd, dy, d_den.contiguous(), hd,
                                                   spec, U, xr)
        return (dx, dh, dtau, d_isd, torch.zeros(1, device=dev), None, None, None, None, None,
                d_scale, None)


# ---------------------------------------------------------------------------
class _LMHeadCEFn(torch.autograd.Function):
    """Tied-embedding cross entropy with the softmax statistics taken in the logits
    GEMM's epilogue: the kernel emits per-tile (max, sum exp, arg-max, label logit)
    partials and bf16 logits, a row kernel merges the partials; no fp32 [T, V]
    tensor exists.  Backward rewrites the bf16 logits in place into
    ``d_nll * (softmax - onehot)`` and runs the two gradient GEMMs on them."""
    CHUNK = 65536

    @staticmethod
    def forward(ctx, x, emb, labels, emb_bf):
        T = x.shape[0]
        xb = _bf16_2d(x)
        e, st = ext(), status_word(x.device)
        V = emb_bf.shape[0]
        lab_c = labels.contiguous()
        parts = []
        for a in range(0, T, _LMHeadCEFn.CHUNK):
            b = min(a + _LMHeadCEFn.CHUNK, T)
            parts.append(e.lm_head_ce_fwd(xb[a:b], emb_bf, lab_c[a:b], st))
        count_launches(2 * len(parts))
        cat = lambda k: parts[0][k] if len(parts) == 1 else torch.cat([p_[k] for p_ in parts])
        lse, lab, pred = cat(1), cat(2), cat(3)
        ctx.save_for_backward(xb, emb_bf, lab_c, lse)
        ctx.logits = [p_[0] for p_ in parts]          # bf16, consumed (in place) by backward
        ctx.x_dtype, ctx.V = x.dtype, V
        ctx.mark_non_differentiable(pred)
        return lse - lab, pred

    @staticmethod
    def backward(ctx, d_nll, _d_pred):
        xb, emb_bf, labels, lse = ctx.saved_tensors
        logits, ctx.logits = ctx.logits, None
        T, V = xb.shape[0], ctx.V
        dx = torch.empty(T, xb.shape[1], dtype=ctx.x_dtype, device=xb.device)
        demb = torch.zeros(V, emb_bf.shape[1], dtype=torch.float32, device=xb.device)
        e = ext()
        scale = d_nll.float().contiguous()
        for i, a in enumerate(range(0, T, _LMHeadCEFn.CHUNK)):
            b = min(a + _LMHeadCEFn.CHUNK, T)
            lg = logits[i]
            e.lm_head_ce_bwd_inplace(lg, V, labels[a:b], lse[a:b], scale[a:b])
            dl = lg[:, :V]
            gemm(dl, False, emb_bf, True, out=dx[a:b])                         # dl . E
            gemm(dl, True, xb[a:b], True, out=demb, accumulate=True)           # dl^T x
            logits[i] = None
        count_launches(len(logits))
        return dx, demb, None, None


# ---------------------------------------------------------------------------
class _EmbedFn(torch.autograd.Function):
    """Token + position embedding gather; backward scatters with atomics into the
    token table and sums the batch for the position table."""

    @staticmethod
    def forward(ctx, ids, tok, pos):
        ids = ids.long().contiguous()
        ctx.save_for_backward(ids)
        ctx.sizes = (tok.shape[0], pos.shape[0])
        count_launches(1)
        return ext().embed_fwd(ids, tok.detach().contiguous(), pos.detach().contiguous())

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        count_launches(2)
        dtok, dpos = ext().embed_bwd(ids, dy.float().contiguous(), ctx.sizes[0], ctx.sizes[1])
        return None, dtok, dpos


class _OffDiagAbsCosFn(torch.autograd.Function):
    """sum_{i != j} |<n_i, n_j>| for unit rows ``n`` [m, d]: similarity matrix on
    the tcgen05 engine (bf16 operands), |.| reduction and sign matrix in one
    pass, gradient 2 * sign(sim) . n as a second engine GEMM."""

    @staticmethod
    def forward(ctx, n):
        nb = _bf16_2d(n.detach())
        sim = gemm(nb, False, nb, False, out_dtype=torch.float32)
        total, sgn = ext().offdiag_abs(sim)
        count_launches(1)
        ctx.save_for_backward(nb, sgn)
        ctx.n_dtype = n.dtype
        return total

    @staticmethod
    def backward(ctx, g):
        nb, sgn = ctx.saved_tensors
        dn = gemm(sgn, False, nb, True, out_dtype=torch.float32)          # sign(sim) . n
        return (dn * (2.0 * g)).to(ctx.n_dtype)


def pool_diversity_cuda(tensors, max_sample: int = 4096):
    """Mean |cos| between distinct rows per pool tensor, averaged over tensors
    (same sampling rule as ops/reference.pool_diversity)."""
    total = 0.0
    for w in tensors:
        n_rows = w.shape[0]
        if n_rows > max_sample:
            w = w[:: n_rows // max_sample][:max_sample]
        wf = w.float()
        n = wf / (torch.linalg.vector_norm(wf, dim=-1, keepdim=True) + 1e-8)
        m = n.shape[0]
        total = total + _OffDiagAbsCosFn.apply(n) / float(m * m - m)
    return total / len(tensors)


# ---------------------------------------------------------------------------
class _AttentionFn(torch.autograd.Function):
    """Causal attention on token-major [B, S, H*dh] tensors (tcgen05 kernels,
    ops/csrc/attention_kernels.cu).  Dropout acts on the softmax weights and is
    regenerated in backward from ``seed``."""

    @staticmethod
    def forward(ctx, q, k, v, n_heads, p_drop, seed):
        qb, kb, vb = (t.detach().to(torch.bfloat16).contiguous() for t in (q, k, v))
        out, lse = ext().attention_fwd(qb, kb, vb, n_heads, float(p_drop), int(seed),
                                       status_word(q.device))
        count_launches(1)
        ctx.save_for_backward(qb, kb, vb, out, lse)
        ctx.meta = (n_heads, float(p_drop), int(seed), q.dtype, k.dtype, v.dtype)
        return out

    @staticmethod
    def backward(ctx, d_out):
        qb, kb, vb, out, lse = ctx.saved_tensors
        n_heads, p_drop, seed, dq_t, dk_t, dv_t = ctx.meta
        dq, dk, dv = ext().attention_bwd(qb, kb, vb, out, d_out.to(torch.bfloat16).contiguous(),
                                         lse, n_heads, p_drop, seed, status_word(qb.device))
        count_launches(2)
        return dq.to(dq_t), dk.to(dk_t), dv.to(dv_t), None, None, None


def causal_attention(q, k, v, n_heads: int, dropout_p: float = 0.0, seed: int = 0):
    """q, k, v [B, S, H*dh] -> bf16 [B, S, H*dh]."""
    return _AttentionFn.apply(q, k, v, n_heads, dropout_p, seed)


# ---------------------------------------------------------------------------
def fused_adamw(params, grads, exp_avg, exp_avg_sq, clip_scale, lr, b1, b2, eps, wd, bc1, bc2):
    """Multi-tensor AdamW step with the clip factor applied on the fly
    (``clip_scale`` is a device scalar so no host sync is needed)."""
    e = ext()
    if hasattr(e, "adamw_multi") and all(p.dtype == torch.float32 and p.is_contiguous() for p in params):
        global _LAUNCHES
        _LAUNCHES += len(params)
        cs = clip_scale.detach().float().reshape(1).contiguous()
        e.adamw_multi([p.data for p in params], [g.float().contiguous() for g in grads], exp_avg,
                      exp_avg_sq, cs, lr, b1, b2, eps, wd, bc1, bc2)
        mark_updated(params)
        return
    g = torch._foreach_mul(grads, clip_scale)
    torch._foreach_mul_(exp_avg, b1)
    torch._foreach_add_(exp_avg, g, alpha=1.0 - b1)
    torch._foreach_mul_(exp_avg_sq, b2)
    torch._foreach_addcmul_(exp_avg_sq, g, g, value=1.0 - b2)
    den = torch._foreach_div(exp_avg_sq, bc2)
    torch._foreach_sqrt_(den)
    torch._foreach_add_(den, eps)
    upd = torch._foreach_div(exp_avg, bc1)
    torch._foreach_div_(upd, den)
    if wd != 0.0:
        torch._foreach_add_(upd, params, alpha=wd)
    torch._foreach_add_(params, upd, alpha=-lr)


def count_launches(n: int) -> None:
    """Account for kernels launched outside this module (communication kernels)."""
    global _LAUNCHES
    _LAUNCHES += int(n)


def mark_updated(params) -> None:
    """Bump the autograd version of tensors a kernel rewrote through raw
    pointers, so caches keyed on ``_version`` (the bf16 compute copies of the
    master weights) see the change."""
    torch._C._increment_version([p for p in params])


def grad_sq_norm(grads) -> torch.Tensor:
    """sum of squares over a list of fp32 gradient tensors (one pass each)."""
    return ext().grad_sq_norm([g.float().contiguous() for g in grads])


DIAG_COLS = 12      # per-token accumulators the gate kernels keep on log steps (csrc: DiagCol)


def diag_from_kernel(spec, dg, tau, inv_sd, tau_off, U_tot: int, alive, shard_group):
    """Routing diagnostics of a pool-op call from the accumulators its gate kernels filled.
    ``dg``: [R, T * DIAG_COLS + 2] fp32 (per token: gate sum, active, strong, band, z sum, two
    narrower bands, sum g log g, sum s^3, sum s^4, gate max; then max intensity and the count
    of capped intensities), partial over this rank's units for ALL T tokens; ``tau``,
    ``inv_sd``, ``tau_off``: [T, R] for the same tokens.  The sums over the shard group are
    taken here (log steps only)."""
    from .srw_ref import finalize_diag
    R, T = dg.shape[0], tau.shape[0]
    cols = dg[:, : T * DIAG_COLS].reshape(R, T, DIAG_COLS).permute(1, 0, 2)       # [T,R,12]
    col = lambda k: cols[..., k:k + 1].contiguous()
    acc = {"active": col(1), "strong": col(2), "band": col(3), "zsum": col(4), "b075": col(5),
           "b030": col(6), "glogg": col(7)}
    gsum = C.all_reduce_nograd(col(0), shard_group, "sum")
    den_sum = C.all_reduce_nograd(col(4), shard_group, "sum")      # two-stage gate: sum of intensities
    sd = (1.0 / inv_sd).unsqueeze(-1)
    tau3 = tau.unsqueeze(-1)
    mu = tau3 - tau_off.unsqueeze(-1) * sd
    scal = dg[:, T * DIAG_COLS:]
    dead_cnt = (alive == 0).float().sum() if alive is not None else tau.new_zeros(())
    return finalize_diag(spec, acc, col(10), col(8), col(9), gsum, den_sum, mu, sd, tau3, U_tot,
                         dead_cnt, scal[:, 0].max(), scal[:, 1].sum(), shard_group)


# ---------------------------------------------------------------------------
class CudaBackend:
    name = "sm100a"
    compute_dtype = torch.bfloat16

    def __init__(self, diag_chunk: int = 12500, fused_comm: bool = True, keep_xr: bool = True):
        ext()
        self.diag_chunk = diag_chunk
        # keep the read scalars x . read^T of every route for the backward pass while the
        # budget (XR_BUDGET) lasts; False always recomputes them
        self.keep_xr = keep_xr
        self._wcache = {}
        self.fused_comm = fused_comm     # in-kernel all-gather / reduce-scatter when sharded
        self._comm = {}

    # ---- dense ops -----------------------------------------------------
    def _w(self, w):
        """bf16 compute copy of a master weight, refreshed when the weight changes."""
        key = id(w)
        hit = self._wcache.get(key)
        if hit is None or hit[0] != w._version or hit[1].device != w.device:
            hit = (w._version, w.detach().to(torch.bfloat16))
            self._wcache[key] = hit
        return hit[1]

    def layer_norm(self, x, w, b):
        return _LayerNormFn.apply(x, w, b)

    def linear(self, x, w, b=None):
        n = w.shape[0]
        if n % 8 != 0:
            # tiny heads (the tau projections): pad the output dimension to the engine's
            # 8-column granularity; the padding rows are zero and sliced away again
            pad = _round_up(n, 8) - n
            wp = F.pad(w, (0, 0, 0, pad))
            bp = F.pad(b, (0, pad)) if b is not None else None
            y = _LinearFn.apply(x, wp, bp, wp.detach().to(torch.bfloat16), torch.float32)
            return y[:, :n]
        return _LinearFn.apply(x, w, b, self._w(w), torch.float32)

    @torch.no_grad()
    def linear_cat(self, x, layers):
        """Forward-only: several ``nn.Linear`` layers on the same input as ONE GEMM over
        their concatenated (and 8-padded) weights; the bf16 weight and the bias are cached
        until a parameter changes.  Returns one output view per layer."""
        key = tuple((l.weight.data_ptr(), l.weight._version,
                     0 if l.bias is None else l.bias._version) for l in layers)
        cache = self.__dict__.setdefault("_cat_cache", {})
        hit = cache.get(id(layers[0]))
        if hit is None or hit[0] != key:
            ws, bs, cuts, n0 = [], [], [], 0
            for l in layers:
                n = l.weight.shape[0]
                ws.append(l.weight.detach().float())
                bs.append(l.bias.detach().float() if l.bias is not None
                          else torch.zeros(n, device=l.weight.device))
                cuts.append((n0, n0 + n))
                n0 += n
            pad = _round_up(n0, 8) - n0
            w = F.pad(torch.cat(ws, 0), (0, 0, 0, pad)).to(torch.bfloat16).contiguous()
            b = F.pad(torch.cat(bs, 0), (0, pad)).contiguous()
            hit = (key, w, b, cuts)
            cache[id(layers[0])] = hit
        _, w, b, cuts = hit
        y = gemm(_bf16_2d(x), False, w, False, out_dtype=torch.float32, bias=b)
        return [y[:, a:e] for a, e in cuts]

    @torch.no_grad()
    def decode_attention(self, q, k, v, cache_k, cache_v, pos, n_heads: int):
        """One new token per sequence: q, k, v [B, D] fp32; k and v are written into the
        fp32 caches [B, H, S_max, dh] at the device-scalar position ``pos`` and the token
        attends over positions 0..pos.  One launch (the position stays on the device, so
        the call can be captured in a graph).  Returns [B, D] fp32."""
        f = lambda t: t.float().contiguous()
        count_launches(1)
        return ext().kv_decode_attention(f(q), f(k), f(v), cache_k, cache_v, pos, int(n_heads))

    def embed(self, ids, tok, pos):
        if tok.shape[1] % 4 != 0 or tok.dtype != torch.float32:
            return R.embed(ids, tok, pos)
        return _EmbedFn.apply(ids, tok, pos)

    def dropout(self, x, p, training):
        if not training or p == 0.0:
            return x
        if not x.is_cuda or x.dtype != torch.float32 or x.numel() % 4 != 0:
            return R.dropout(x, p, training)
        return _DropoutFn.apply(None, x, float(p))

    def dropout_add(self, res, x, p, training):
        """res + dropout(x): one kernel forward (and one for the gradient of x)."""
        if not training or p == 0.0:
            return res + x
        if (not x.is_cuda or x.dtype != torch.float32 or res.dtype != torch.float32
                or x.numel() % 4 != 0 or res.shape != x.shape):
            return res + R.dropout(x, p, training)
        return _DropoutFn.apply(res, x, float(p))

    def attention(self, q, k, v, dropout_p, training):
        """q, k, v [B, H, S, dh] (head-major views of token-major projections)."""
        B, H, S, dh = q.shape
        if dh % 16 != 0 or dh > 128:
            raise ValueError(f"head dimension {dh} is not supported by the attention kernels "
                             "(multiple of 16, at most 128)")
        tok = lambda t: t.transpose(1, 2).reshape(B, S, H * dh)
        p = float(dropout_p) if training else 0.0
        seed = int(torch.randint(0, 2 ** 62, (1,)).item()) if p > 0.0 else 0
        o = causal_attention(tok(q), tok(k), tok(v), H, p, seed)
        # bf16, as the kernel writes it: the only consumer is the bf16 operand of the O projection
        return o.view(B, S, H, dh).transpose(1, 2)

    def lm_head_ce(self, x, tok_emb, labels):
        B, S, D = x.shape
        sx = x[:, :-1, :].reshape(-1, D)
        sl = labels[:, 1:].reshape(-1).long()
        valid = sl != -100
        nll, pred = _LMHeadCEFn.apply(sx, tok_emb, sl, self._w(tok_emb))
        per_tok = (nll * valid).reshape(B, S - 1)
        loss = per_tok.sum() / (valid.sum() + 1e-8)
        correct = ((pred == sl) & valid).sum()
        return loss, per_tok, correct, valid.sum(), valid.reshape(B, S - 1)

    def logits(self, x, tok_emb):
        shp = x.shape
        lg = gemm(_bf16_2d(x.reshape(-1, shp[-1])), False, self._w(tok_emb), False,
                  out_dtype=torch.float32)
        return lg.reshape(*shp[:-1], -1)

    def diversity(self, tensors):
        return pool_diversity_cuda(tensors)

    # ---- SRW pool op ---------------------------------------------------
    def prepare_pool(self, emb, read, write, spec: GateSpec, pctx: Optional[ParallelCtx] = None):
        pctx = pctx or ParallelCtx()
        U = pctx.n_valid if pctx.n_valid is not None else emb.shape[0]
        pool = CudaPool()
        pool.keep_xr = self.keep_xr
        anchor, gram, esum = _PoolPrepFn.apply(emb, read, write, pool.tensors, spec.normalize_pool, U)
        gram = C.sum_over_shards(gram, pctx.shard_group)
        esum = C.sum_over_shards(esum, pctx.shard_group)
        from .score_stats import split_bf16
        pool.extra = {"anchor": anchor, "gram": gram, "esum": esum, "U": U,
                      "gram_split": split_bf16(gram.detach())}
        return pool

    def srw(self, x, h, tau_off, pool: CudaPool, spec: GateSpec, *,
            pctx: Optional[ParallelCtx] = None, want_diag: bool = True,
            return_gates: bool = False, unit_mask=None, out_scale=None) -> SRWResult:
        """``out_scale`` (float or 0-dim tensor): the pool's output scale; when
        given, the returned route outputs are already multiplied by it."""
        pctx = pctx or ParallelCtx()
        nsh0 = C.group_size(pctx.shard_group)
        if return_gates or nsh0 > 1:
            res, scaled = self._srw_unscaled(x, h, tau_off, pool, spec, pctx, want_diag,
                                             return_gates, unit_mask, out_scale)
            if out_scale is not None and not scaled:
                res.out = res.out * out_scale
            return res
        return self._srw_local(x, h, tau_off, pool, spec, pctx, want_diag, unit_mask, out_scale)

    @torch.no_grad()
    def srw_infer(self, x, h, tau_off, pool: CudaPool, spec: GateSpec, *, n_total=None,
                  out_scale=None):
        """Forward-only SRW call for generation (unsharded pools): no load-balance or dead-unit
        statistics, nothing kept for a backward pass, and the write GEMM cuts its long K = U
        into splits that meet in the fp32 reduce-add epilogue, so that with a handful of token
        rows (decoding: T = batch) every SM pair still streams a share of the pool instead of
        five row tiles streaming all of it (reference: _srw_inference,
        models/dawn_spatial_v41_exp.py:1713-1739).  Returns the per-route outputs [T, D] fp32,
        normalised and scaled."""
        ex = pool.extra
        U = ex["U"]
        U_tot = n_total if n_total is not None else U
        T, Rr, r = h.shape
        e, dev = ext(), x.device
        st = status_word(dev)
        x_bf = _bf16_2d(x)
        Up = _round_up(U, 8)
        D = x.shape[1]
        if out_scale is None:
            scale = 1.0
        else:
            scale = out_scale.detach().float() if isinstance(out_scale, torch.Tensor) else float(out_scale)
        gl = _gate_list(spec)
        wide = bool(e.srw_wide_tiles(U))
        # Routes of one pool are independent token rows as far as the kernels care: with few
        # tokens (decoding) they are stacked into one call, so the pool is streamed once.
        stack = Rr * T <= 128
        if Rr * T <= e.srw_rows_max(D):
            # one to four rows: a single streaming pass over the pool (SIMT, bound by HBM)
            tau, inv_sd, h_rm = score_stats_rows(h, tau_off, ex["gram"], ex["esum"], U_tot)
            x_rm = (x_bf.repeat(Rr, 1) if Rr > 1 else x_bf).contiguous()
            sc_t = scale.reshape(1) if isinstance(scale, torch.Tensor) else None
            out, _ = e.srw_rows(h_rm, x_rm, tau, inv_sd, pool.emb[:U], pool.read[:U], pool.write[:U],
                                None, _gate_list(spec), 1.0 if sc_t is not None else float(scale), sc_t)
            count_launches(2)
            return list(out.reshape(Rr, T, D).unbind(0))
        if stack:
            tau, inv_sd, h_rm = score_stats_rows(h, tau_off, ex["gram"], ex["esum"], U_tot)
            calls = [(h_rm, x_bf.repeat(Rr, 1) if Rr > 1 else x_bf, tau, inv_sd)]
        else:
            tau, inv_sd, _, h_bf3 = score_stats(h, tau_off, ex["gram"], ex["esum"], U_tot,
                                                ex["gram_split"])
            calls = [(_bf16_2d(h_bf3[:, ri]), x_bf, tau[:, ri].contiguous(), inv_sd[:, ri].contiguous())
                     for ri in range(Rr)]
        outs = []
        for h_r, x_r, tau_r, isd_r in calls:
            Tr = h_r.shape[0]
            p = torch.empty(Tr, Up, dtype=torch.bfloat16, device=dev)
            work = torch.zeros(Tr * (D + 1), dtype=torch.float32, device=dev)   # y and den, one fill
            y, den = work[:Tr * D].view(Tr, D), work[Tr * D:]
            if wide:
                e.srw_fwd_gate_xr(h_r, pool.emb[:U], x_r, pool.read[:U], p, None, tau_r, isd_r, None,
                                  den, None, None, None, gl, st, *NO_GATHER)
            else:
                e.srw_fwd_gate(h_r, pool.emb[:U], x_r, pool.read[:U], p, tau_r, isd_r, den, None, None,
                               None, gl, st)
            gemm(p[:, :U], False, pool.write[:U], True, out=y, accumulate=True)
            outs.append(y * (scale / den.clamp(min=1.0)).unsqueeze(-1))
        count_launches(len(calls))
        if stack:
            return list(outs[0].reshape(Rr, T, D).unbind(0))
        return outs

    def srw_group(self, x, calls, spec: GateSpec, *, want_diag: bool = True):
        """Several SRW calls on the same ``x``.  Sequence- and pool-sharded calls on
        the wide kernels run as ONE group through parallel/fused_group.py: ``x`` is
        gathered once, two barriers per direction for the whole group, per-token
        statistics and denominators travel inside the kernels (no library
        collective).  Everything else runs call by call."""
        if self._group_ok(x, calls, spec):
            return self._srw_group_fused(x, calls, spec, want_diag)
        return [self.srw(x, c["h"], c["tau_off"], c["pool"], spec, pctx=c.get("pctx"),
                         want_diag=want_diag, unit_mask=c.get("unit_mask"),
                         out_scale=c.get("out_scale")) for c in calls]

    def _group_ok(self, x, calls, spec) -> bool:
        if not self.fused_comm or not calls:
            return False
        from .gates import GATE_GELU_Z  # noqa: F401
        pc0 = calls[0].get("pctx") or ParallelCtx()
        nsh = C.group_size(pc0.shard_group)
        if nsh <= 1 or nsh > 8 or not pc0.seq_sharded:
            return False
        n_routes = sum(c["h"].shape[1] for c in calls)
        if n_routes > 3 or x.shape[0] % 256 != 0 or x.shape[1] % 64 != 0:
            return False
        for c in calls:
            pc = c.get("pctx") or ParallelCtx()
            if pc.shard_group is not pc0.shard_group or not pc.seq_sharded:
                return False
            if c["h"].shape[-1] % 64 != 0:
                return False
            # the same answer on every rank: judge by the padded rows per rank and by what the
            # last rank holds, not by this rank's own unit count
            per = c["pool"].emb.shape[0]
            n_total = pc.n_total if pc.n_total is not None else per * nsh
            if per < 512 or n_total - (nsh - 1) * per < 8:
                return False
            if c.get("unit_mask") is not None and torch.is_grad_enabled():
                return False            # masked (ablation) forwards have no backward on this path
        return True

    def _srw_group_fused(self, x, calls, spec, want_diag):
        from ..parallel.fused_group import GroupShardComm, route_group
        pc0 = calls[0]["pctx"]
        grp = pc0.shard_group
        nsh = C.group_size(grp)
        Tl, D = x.shape
        r = calls[0]["h"].shape[-1]
        key = ("group", id(grp), Tl, D, r)
        comm = self._comm.get(key)
        if comm is None:
            comm = self._comm[key] = GroupShardComm(grp, x.device, Tl, D, r)
        x_bf = _bf16_2d(x)
        hs, taus, isds, offs, holders, units, anchors, scales, alives, masks, diags, per_call = \
            [], [], [], [], [], [], [], [], [], [], [], []
        T_all = Tl * nsh
        hsums = []
        for c in calls:
            pool, pctx = c["pool"], c["pctx"]
            ex = pool.extra
            U = ex["U"]
            U_tot = pctx.n_total if pctx.n_total is not None else U * nsh
            tau, inv_sd, hsum, h_bf3 = score_stats(c["h"], c["tau_off"], ex["gram"], ex["esum"], U_tot,
                                                   ex["gram_split"])
            Rr = h_bf3.shape[1]
            hs.append(h_bf3)
            taus.append(tau)
            isds.append(inv_sd)
            offs.append(c["tau_off"].detach().float())
            hsums.append(hsum)
            anchors.append(ex["anchor"])
            sc = c.get("out_scale")
            if sc is None:
                sc = torch.ones((), device=x.device)
            elif not isinstance(sc, torch.Tensor):
                sc = torch.full((), float(sc), device=x.device)
            alive = torch.zeros(U, dtype=torch.uint8, device=x.device) if spec.has_dead_penalty else None
            um = c.get("unit_mask")
            um = None if um is None else um[:U].float().contiguous()
            for _ in range(Rr):
                holders.append(pool)
                units.append(U)
                scales.append(sc)
                alives.append(alive)
                masks.append(um)
                diags.append(torch.zeros(T_all * DIAG_COLS + 2, dtype=torch.float32, device=x.device)
                             if want_diag else None)
            per_call.append((Rr, U, U_tot, alive))
        # per-unit mean scores need the column sums of h over ALL tokens of the group: one
        # small all-reduce for every pool of the group
        hsum_all = C.sum_over_shards(torch.stack(hsums), grp)
        outs, dens = route_group(x_bf, torch.cat(hs, dim=1), torch.cat(taus, dim=1),
                                 torch.cat(isds, dim=1), comm, spec, holders, units, anchors, scales,
                                 alives, masks, diags, torch.cat(offs, dim=1) if want_diag else None)
        m_us, parts = [], []
        for k, (c, (Rr, U, U_tot, alive)) in enumerate(zip(calls, per_call)):
            hbar = hsum_all[k] / float(Tl * nsh * Rr)
            m_u = _PoolMatVecFn.apply(hbar, anchors[k], c["pool"], U)
            m_us.append(m_u)
            parts.append(torch.stack([C.mean_over_group(m_u.sum(), c["pctx"].dp_group),
                                      C.mean_over_group((m_u * m_u).sum(), c["pctx"].dp_group)]))
        ns = C.sum_over_shards(torch.stack(parts), grp)          # [calls, 2], one all-reduce
        results, i0 = [], 0
        for k, (c, (Rr, U, U_tot, alive)) in enumerate(zip(calls, per_call)):
            mean_score = ns[k, 0] / U_tot
            var_score = ns[k, 1] / U_tot - mean_score ** 2
            lb = var_score / (mean_score ** 2 + var_score + 1e-2)
            dead_pen = x.new_zeros(())
            if spec.has_dead_penalty:
                # a unit is alive if any token of the whole batch gates it: every rank of the
                # shard group sees all tokens of its own units, so only data-parallel replicas
                # need to be combined
                al = C.all_reduce_nograd(alive.float(), c["pctx"].dp_group, "max")
                dead = (al < 0.5).float()
                ms = C.mean_over_group(m_us[k], c["pctx"].dp_group)
                dead_pen = C.sum_over_shards((torch.relu(-ms) * dead).sum(), grp)
            o = outs[i0:i0 + Rr]
            den = torch.stack(dens[i0:i0 + Rr], dim=1).clamp(min=1.0)
            diag = {}
            if want_diag:
                with torch.no_grad():
                    # thresholds, 1/sigma and offsets of ALL tokens sit in the gathered
                    # statistics buffers of this group's forward
                    st_all = [comm.stats[comm._parity["gather"]][i0 + j].local for j in range(Rr)]
                    pick = lambda k: torch.stack([t[:, k] for t in st_all], dim=1)
                    diag = diag_from_kernel(spec, torch.stack(diags[i0:i0 + Rr]), pick(0), pick(1),
                                            pick(3), U_tot, alive, grp)
            results.append(SRWResult(out=o[0].unsqueeze(1) if Rr == 1 else None, lb=lb,
                                     dead_penalty=dead_pen, diag=diag, den=den, outs=list(o)))
            i0 += Rr
        return results

    def _srw_local(self, x, h, tau_off, pool, spec, pctx, want_diag, unit_mask, out_scale):
        """Unsharded pools: statistics, then per route the gate kernel and the
        write GEMM with normalisation and scale in its epilogue."""
        ex = pool.extra
        U, anchor = ex["U"], ex["anchor"]
        U_tot = pctx.n_total if pctx.n_total is not None else U
        T, Rr, r = h.shape
        x_bf = _bf16_2d(x)
        tau, inv_sd, hsum, h_bf3 = score_stats(h, tau_off, ex["gram"], ex["esum"], U_tot,
                                               ex["gram_split"])
        hbar = hsum / float(T * Rr)
        m_u = _PoolMatVecFn.apply(hbar, anchor, pool, U)
        ns_sum = C.mean_over_group(m_u.sum(), pctx.dp_group)
        ns_sq = C.mean_over_group((m_u * m_u).sum(), pctx.dp_group)
        mean_score = ns_sum / U_tot
        var_score = ns_sq / U_tot - mean_score ** 2
        lb = var_score / (mean_score ** 2 + var_score + 1e-2)
        alive = torch.zeros(U, dtype=torch.uint8, device=x.device) if spec.has_dead_penalty else None
        um = None if unit_mask is None else unit_mask[:U].float().contiguous()
        if out_scale is None:
            scale = torch.ones((), device=x.device)
        elif isinstance(out_scale, torch.Tensor):
            scale = out_scale
        else:
            scale = torch.full((), float(out_scale), device=x.device)
        outs, dens = [], []
        # routing diagnostics ride in the gate kernel's epilogue (wide kernels); pools too
        # small for those take the library path below
        dg = torch.zeros(Rr, T * DIAG_COLS + 2, dtype=torch.float32, device=x.device) \
            if want_diag and ext().srw_wide_tiles(U) else None
        for ri in range(Rr):
            y, den = _SRWRouteScaledFn.apply(x_bf, _bf16_2d(h_bf3[:, ri]), tau[:, ri].contiguous(),
                                             inv_sd[:, ri].contiguous(), anchor, pool, spec, U,
                                             alive, um, scale, None if dg is None else dg[ri])
            outs.append(y)
            dens.append(den)
        den = torch.stack(dens, dim=1).clamp(min=1.0)
        dead_pen = x.new_zeros(())
        if spec.has_dead_penalty:
            al = C.all_reduce_nograd(alive.float(), pctx.dp_group, "max")
            dead = (al < 0.5).float()
            ms = C.mean_over_group(m_u, pctx.dp_group)
            dead_pen = (torch.relu(-ms) * dead).sum()
        diag = {}
        if want_diag:
            with torch.no_grad():
                if dg is not None:
                    diag = diag_from_kernel(spec, dg, tau.detach(), inv_sd.detach(), tau_off.detach(),
                                            U_tot, alive, None)
                else:
                    diag = self._srw_library(x.detach(), h.detach(), tau_off.detach(), pool, spec,
                                             ParallelCtx(None, pctx.dp_group, pctx.n_total,
                                                         pctx.n_valid, False), True, False,
                                             unit_mask).diag
        out = outs[0].unsqueeze(1) if Rr == 1 else None
        return SRWResult(out=out, lb=lb, dead_penalty=dead_pen, diag=diag, den=den, outs=outs)

    def _srw_unscaled(self, x, h, tau_off, pool, spec, pctx, want_diag, return_gates, unit_mask,
                      out_scale=None):
        """Sharded pools (and gate dumps).  Returns (result, scale_applied)."""
        if return_gates:
            return self._srw_library(x, h, tau_off, pool, spec, pctx, True, True, unit_mask), False
        ex = pool.extra
        U, anchor = ex["U"], ex["anchor"]
        nsh = C.group_size(pctx.shard_group)
        U_tot = pctx.n_total if pctx.n_total is not None else U * nsh
        seq = bool(pctx.seq_sharded and nsh > 1)
        if seq and self.fused_comm and unit_mask is None and not spec.has_dead_penalty \
                and x.shape[0] % 256 == 0 and x.shape[1] % 64 == 0 and h.shape[-1] % 64 == 0 \
                and nsh <= 8:
            return self._srw_fused_sharded(x, h, tau_off, pool, spec, pctx, want_diag,
                                           out_scale), True
        if seq:
            x = C.gather_tokens(x, pctx.shard_group)
            h = C.gather_tokens(h, pctx.shard_group)
            tau_off = C.gather_tokens(tau_off, pctx.shard_group)
        T, Rr, r = h.shape
        x_bf = _bf16_2d(x)
        tau, inv_sd, hsum, h_bf3 = score_stats(h, tau_off, ex["gram"], ex["esum"], U_tot,
                                               ex["gram_split"])
        # per-unit mean score over the local tokens and routes -> LB / dead statistics
        hbar = hsum / float(T * Rr)
        m_u = _PoolMatVecFn.apply(hbar, anchor, pool, U)
        ns_sum = C.sum_over_shards(C.mean_over_group(m_u.sum(), pctx.dp_group), pctx.shard_group)
        ns_sq = C.sum_over_shards(C.mean_over_group((m_u * m_u).sum(), pctx.dp_group),
                                     pctx.shard_group)
        mean_score = ns_sum / U_tot
        var_score = ns_sq / U_tot - mean_score ** 2
        lb = var_score / (mean_score ** 2 + var_score + 1e-2)
        alive = None
        if spec.has_dead_penalty:
            alive = torch.zeros(U, dtype=torch.uint8, device=x.device)
        um = None if unit_mask is None else unit_mask[:U].float().contiguous()
        outs, dens = [], []
        for ri in range(Rr):
            h_r = _bf16_2d(h_bf3[:, ri])
            raw, den = _SRWRouteFn.apply(x_bf, h_r, tau[:, ri].contiguous(),
                                         inv_sd[:, ri].contiguous(), anchor, pool, spec, U, alive, um)
            outs.append(raw)
            dens.append(den)
        raw = torch.stack(outs, dim=1)                                     # [T,R,D]
        den_sum = C.sum_over_shards(torch.stack(dens, dim=1), pctx.shard_group)
        den = den_sum.clamp(min=1.0)
        out = raw / den.unsqueeze(-1)
        if seq:
            out = C.scatter_tokens_sum(out.to(torch.bfloat16), pctx.shard_group).float()
            r_, n_ = C.group_rank(pctx.shard_group), out.shape[0]
            den = den[r_ * n_:(r_ + 1) * n_]
        elif nsh > 1:
            out = C.sum_over_shards(out.to(torch.bfloat16), pctx.shard_group).float()
        dead_pen = x.new_zeros(())
        dead_cnt = x.new_zeros(())
        if spec.has_dead_penalty:
            al = C.all_reduce_nograd(alive.float(), pctx.dp_group, "max")
            dead = (al < 0.5).float()
            ms = C.mean_over_group(m_u, pctx.dp_group)
            dead_pen = C.sum_over_shards((torch.relu(-ms) * dead).sum(), pctx.shard_group)
            dead_cnt = dead.sum()
        diag = {}
        if want_diag:
            with torch.no_grad():
                lib = self._srw_library(x.detach(), h.detach(), tau_off.detach(), pool, spec,
                                        ParallelCtx(pctx.shard_group, pctx.dp_group, pctx.n_total,
                                                    pctx.n_valid, False), True, False, unit_mask)
                diag = lib.diag
        return SRWResult(out=out, lb=lb, dead_penalty=dead_pen, diag=diag, den=den), False

    def _srw_fused_sharded(self, x, h, tau_off, pool, spec, pctx, want_diag, out_scale=None):
        """Sequence- and pool-sharded route through the kernels with fused
        collectives (parallel/fused_srw.py).  x/h/tau_off hold this rank's tokens."""
        from ..parallel.fused_srw import FusedShardComm, _SRWRouteGatherFn
        ex = pool.extra
        U, anchor = ex["U"], ex["anchor"]
        grp = pctx.shard_group
        nsh = C.group_size(grp)
        U_tot = pctx.n_total if pctx.n_total is not None else U * nsh
        Tl, Rr, r = h.shape
        key = (id(grp), Tl, x.shape[1], r)
        comm = self._comm.get(key)
        if comm is None:
            comm = self._comm[key] = FusedShardComm(grp, x.device, Tl, x.shape[1], r)
        x_bf = _bf16_2d(x)
        tau, inv_sd, hsum, h_bf3 = score_stats(h, tau_off, ex["gram"], ex["esum"], U_tot,
                                               ex["gram_split"])                # [Tl,R]
        # per-unit mean score over ALL tokens of the group (they share one batch)
        hbar = C.sum_over_shards(hsum, grp) / float(Tl * nsh * Rr)
        m_u = _PoolMatVecFn.apply(hbar, anchor, pool, U)
        ns_sum = C.sum_over_shards(C.mean_over_group(m_u.sum(), pctx.dp_group), grp)
        ns_sq = C.sum_over_shards(C.mean_over_group((m_u * m_u).sum(), pctx.dp_group), grp)
        mean_score = ns_sum / U_tot
        var_score = ns_sq / U_tot - mean_score ** 2
        lb = var_score / (mean_score ** 2 + var_score + 1e-2)
        if out_scale is None:
            scale = torch.ones((), device=x.device)
        elif isinstance(out_scale, torch.Tensor):
            scale = out_scale
        else:
            scale = torch.full((), float(out_scale), device=x.device)
        outs, dens = [], []
        # one all-gather for the thresholds and 1/sigma of every route of this call
        stats_f = C.gather_tokens(torch.stack([tau, inv_sd], dim=0).permute(1, 0, 2).contiguous(), grp)
        for ri in range(Rr):
            tau_f = stats_f[:, 0, ri].contiguous()
            isd_f = stats_f[:, 1, ri].contiguous()
            o, d = _SRWRouteGatherFn.apply(x_bf, _bf16_2d(h_bf3[:, ri]), tau_f, isd_f, anchor, pool,
                                           spec, U, comm, scale)
            outs.append(o)
            dens.append(d[comm.rows])
        out = outs[0].unsqueeze(1) if Rr == 1 else None       # [Tl,R,D], normalised and scaled
        den = torch.stack(dens, dim=1).clamp(min=1.0)
        dead_pen = x.new_zeros(())     # gates with a dead-unit penalty take the NCCL path
        diag = {}
        if want_diag:
            with torch.no_grad():
                lib = self._srw_library(x.detach(), h.detach(), tau_off.detach(), pool, spec, pctx,
                                        True, False, None)
                diag = lib.diag
        return SRWResult(out=out, lb=lb, dead_penalty=dead_pen, diag=diag, den=den, outs=outs)

    def _srw_library(self, x, h, tau_off, pool, spec, pctx, want_diag, return_gates, unit_mask):
        """The same op through torch matmuls (diagnostics / gate dumps only)."""
        return srw_pool_ref(x, h, tau_off, pool.emb, pool.read, pool.write, spec,
                            compute_dtype=torch.bfloat16, chunk_size=self.diag_chunk,
                            n_valid=pctx.n_valid, n_total=pctx.n_total,
                            shard_group=pctx.shard_group, dp_group=pctx.dp_group,
                            unit_mask=unit_mask, want_diag=want_diag, return_gates=return_gates,
                            seq_sharded=pctx.seq_sharded)

    def finish_step(self):
        check_status_deferred()

    def finish_run(self):
        """Synchronise and raise on any device-side failure not yet reported."""
        check_status()
