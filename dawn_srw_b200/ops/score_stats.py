"""Per-token score statistics of the SRW pool op from a Gram matrix.

For scores ``s_u = <h, e_u>`` over a pool of ``U`` units

    mean_U s   = <h, esum> / U,          esum = sum_u e_u            [r]
    mean_U s^2 = h G h^T / U,            G = E^T E                   [r, r]

so ``mu``, ``sigma = sqrt(var) + 1e-8``, the threshold ``tau = mu + tau_off * sigma``
and ``1 / sigma`` of every token need no pass over the ``[T, U]`` scores (the
reference computes them from a first sweep over all scores:
models/dawn_spatial_v41_exp.py:433-464).  ``score_stats`` is one autograd node:

    inputs   h [T, R, r] (router output), tau_off [T, R], G, esum
    outputs  tau [T, R], inv_sigma [T, R], hsum [r] (column sums of bf16(h), for
             the per-unit mean score ``emb . mean_t h``), h_bf [T, R, r] (the bf16
             copy of h that the gate kernels consume)

Its backward adds, in one pass, the cotangent that reaches ``h`` through the
statistics, through ``hsum`` and through ``h_bf`` (the gate kernels' ``dh``).

On CUDA ``h . G`` and ``dG`` run on the tcgen05 engine (G split into two bf16
terms, so the product of the bf16 ``h`` with it is fp32-accurate) and the row
parts are the kernels of ops/csrc/stats_kernels.cu; on CPU the same algebra
runs in plain torch (which is how the formulas are tested without a GPU).

The variance is floored at 1e-12 under the square root and its gradient is
zero where the floor is active (an all-zero ``h`` row, padded rows), so no
``0 * inf`` can appear.
"""
from __future__ import annotations

import torch

VAR_FLOOR = 1e-12
SD_EPS = 1e-8


def split_bf16(g: torch.Tensor):
    """g ~= hi + lo with both terms bf16 (relative error about 2^-17)."""
    hi = g.to(torch.bfloat16)
    lo = (g - hi.float()).to(torch.bfloat16)
    return hi, lo


class _ScoreStatsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, off, gram, esum, inv_u, gram_split):
        T, Rr, r = h.shape
        N = T * Rr
        hb = h.detach().to(torch.bfloat16).reshape(N, r).contiguous()
        off_f = off.detach().float().reshape(N).contiguous()
        esum_f = esum.detach().float().contiguous()
        if h.is_cuda:
            from . import cuda_backend as CB
            hi, lo = gram_split if gram_split is not None else split_bf16(gram.detach().float())
            hg = CB.gemm(hb, False, hi, False, out_dtype=torch.float32)     # G is symmetric
            CB.gemm(hb, False, lo, False, out=hg, accumulate=True)
            tau, isd, mu, sd, hsum = CB.ext().score_stats_fwd(hg, hb, esum_f, off_f, float(inv_u))
            CB.count_launches(1)
        else:
            hf = hb.float()
            hg = hf @ gram.detach().float()
            mu = (hf @ esum_f) * inv_u
            m2 = (hg * hf).sum(-1) * inv_u
            sd = torch.sqrt((m2 - mu * mu).clamp_min(VAR_FLOOR)) + SD_EPS
            tau = mu + off_f * sd
            isd = 1.0 / sd
            hsum = hf.sum(0)
        ctx.save_for_backward(hb, off_f, mu, sd, hg, esum_f)
        ctx.inv_u, ctx.shape, ctx.h_dtype, ctx.off_dtype = float(inv_u), (T, Rr, r), h.dtype, off.dtype
        ctx.set_materialize_grads(False)
        return tau.view(T, Rr), isd.view(T, Rr), hsum, hb.view(T, Rr, r)

    @staticmethod
    def backward(ctx, d_tau, d_isd, d_hsum, d_hb):
        hb, off_f, mu, sd, hg, esum_f = ctx.saved_tensors
        T, Rr, r = ctx.shape
        N, inv_u = T * Rr, ctx.inv_u
        flat = lambda t: None if t is None else t.detach().float().reshape(N).contiguous()
        d_tau, d_isd = flat(d_tau), flat(d_isd)
        d_hsum = None if d_hsum is None else d_hsum.detach().float().contiguous()
        if hb.is_cuda:
            from . import cuda_backend as CB
            dhb = None if d_hb is None else d_hb.detach().to(torch.bfloat16).reshape(N, r).contiguous()
            dh, w, d_off, d_esum = CB.ext().score_stats_bwd(d_tau, d_isd, d_hsum, dhb, off_f, mu, sd,
                                                            hg, hb, esum_f, inv_u)
            CB.count_launches(1)
            d_gram = torch.zeros(r, r, dtype=torch.float32, device=hb.device)
            CB.gemm(w, True, hb, True, out=d_gram, accumulate=True, alpha=inv_u)    # w^T h / U
        else:
            zero = torch.zeros(N, dtype=torch.float32, device=hb.device)
            dt = d_tau if d_tau is not None else zero
            di = d_isd if d_isd is not None else zero
            hf = hb.float()
            d_sd = dt * off_f - di / (sd * sd)
            sq = sd - SD_EPS
            d_var = torch.where(sq > 1.5e-6, d_sd / (2.0 * sq.clamp_min(1e-30)), torch.zeros_like(sq))
            d_mu = dt - 2.0 * mu * d_var
            dh = (2.0 * inv_u) * d_var[:, None] * hg + (inv_u * d_mu)[:, None] * esum_f[None, :]
            if d_hsum is not None:
                dh = dh + d_hsum[None, :]
            if d_hb is not None:
                dh = dh + d_hb.detach().float().reshape(N, r)
            d_off = dt * sd
            d_esum = inv_u * (d_mu[:, None] * hf).sum(0)
            d_gram = inv_u * ((d_var[:, None] * hf).t() @ hf)
        return (dh.view(T, Rr, r).to(ctx.h_dtype), d_off.view(T, Rr).to(ctx.off_dtype), d_gram,
                d_esum, None, None)


def score_stats(h, tau_off, gram, esum, n_units: int, gram_split=None):
    """-> (tau [T,R], inv_sigma [T,R], hsum [r], h_bf [T,R,r]); see the module docstring."""
    return _ScoreStatsFn.apply(h, tau_off, gram, esum, 1.0 / float(n_units), gram_split)


@torch.no_grad()
def score_stats_rows(h, tau_off, gram, esum, n_units: int):
    """Forward-only statistics of a handful of rows (generation) in one launch:
    h [T, R, r], tau_off [T, R] -> route-major (row ``ri * T + t``) tau [R*T],
    inv_sigma [R*T] and the bf16 copy of h [R*T, r]."""
    T, Rr, r = h.shape
    inv_u = 1.0 / float(n_units)
    if h.is_cuda:
        from . import cuda_backend as CB
        hf = h if h.dtype == torch.float32 and h.stride(2) == 1 else h.float().contiguous()
        off = tau_off if tau_off.dtype == torch.float32 else tau_off.float()
        tau, isd, hb = CB.ext().score_stats_rows(hf, off, gram.detach().float().contiguous(),
                                                 esum.detach().float().contiguous(), inv_u)
        CB.count_launches(1)
        return tau, isd, hb
    hb = h.detach().to(torch.bfloat16).transpose(0, 1).reshape(Rr * T, r)
    hf = hb.float()
    mu = (hf @ esum.float()) * inv_u
    m2 = ((hf @ gram.float()) * hf).sum(-1) * inv_u
    sd = torch.sqrt((m2 - mu * mu).clamp_min(VAR_FLOOR)) + SD_EPS
    return mu + tau_off.float().t().reshape(-1) * sd, 1.0 / sd, hb
