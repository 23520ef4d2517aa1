"""Gate policies of the SRW pool op.

Three registered variants (reference: models/dawn_spatial_v394_exp.py:213-243,
models/legacy/dawn_spatial_v401_exp.py:296-342,
models/dawn_spatial_v41_exp.py:503-511,579-586):

==========  =====================================  ==================  ===========
version     gate g(s)                              denominator term    pool norm
==========  =====================================  ==================  ===========
v3.9.4      clip(relu(s - tau), 0, 10)             g                   emb,read,write unit rows
v4.0.1      z*Phi(z) for z>0, z=(s-tau)/sigma      g                   emb,read,write unit rows
v4.1        sigmoid(k*m)*(eps+min(max(m-c,0),M))   intensity           none
            with m = s - tau - thr
==========  =====================================  ==================  ===========

``GateSpec.kind`` is the integer the CUDA kernels switch on.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

GATE_RELU_CLIP = 0   # v3.9.4
GATE_GELU_Z = 1      # v4.0.1
GATE_TWO_STAGE = 2   # v4.1

_INV_SQRT2 = 0.7071067811865476
_INV_SQRT2PI = 0.3989422804014327


@dataclass(frozen=True)
class GateSpec:
    kind: int = GATE_TWO_STAGE
    normalize_pool: bool = False       # unit-norm rows of emb/read/write in forward
    learnable_scale: bool = True       # {qk,v,know}_scale parameters exist
    tau_reg_in_aux: bool = True        # 0.01*mean(relu(tau)) folded into aux
    has_dead_penalty: bool = False
    sharpness: float = 500.0
    activation_threshold: float = 0.5
    activation_cutoff: float = 0.01
    epsilon: float = 1e-4
    max_intensity: float = 10.0
    dead_threshold: float = 0.01
    clip_max: float = 10.0             # v3.9.4 gate ceiling

    @property
    def name(self) -> str:
        return {GATE_RELU_CLIP: "v3.9.4", GATE_GELU_Z: "v4.0.1", GATE_TWO_STAGE: "v4.1"}[self.kind]


def gate_spec_for(version: str, training_cfg=None) -> GateSpec:
    """Gate policy for a registered ``model_version`` string.  v4.1 reads its
    constants from the ``training`` section (reference: scripts/train_jax.py:153-168)."""
    t = training_cfg
    g = (lambda k, d: getattr(t, k, d) if t is not None and not isinstance(t, dict)
         else (t or {}).get(k, d))
    if version.endswith("v3.9.4"):
        return GateSpec(kind=GATE_RELU_CLIP, normalize_pool=True, learnable_scale=False,
                        tau_reg_in_aux=False)
    if version.endswith("v4.0.1"):
        return GateSpec(kind=GATE_GELU_Z, normalize_pool=True, learnable_scale=True,
                        tau_reg_in_aux=True)
    if version.endswith("v4.1"):
        return GateSpec(kind=GATE_TWO_STAGE, normalize_pool=False, learnable_scale=True,
                        tau_reg_in_aux=True, has_dead_penalty=True,
                        sharpness=float(g("sharpness", 500.0)),
                        activation_threshold=float(g("activation_threshold", 0.5)),
                        activation_cutoff=float(g("activation_cutoff", 0.01)),
                        epsilon=float(g("epsilon", 1e-4)),
                        max_intensity=float(g("max_intensity", 10.0)),
                        dead_threshold=float(g("dead_penalty_threshold", 0.01)))
    raise ValueError(f"no gate policy for model_version {version!r}")


def gate_forward(spec: GateSpec, s: torch.Tensor, tau: torch.Tensor, sigma: torch.Tensor):
    """Differentiable gate in plain torch.

    s [..., U] fp32 scores, tau/sigma [..., 1].  Returns ``(gate, den_term, aux)``
    where ``aux`` holds the per-element quantities the diagnostics need
    (``activation``/``intensity`` for v4.1, ``z``/``phi`` for v4.0.1).
    """
    if spec.kind == GATE_RELU_CLIP:
        raw = s - tau
        gate = raw.clamp(min=0.0).clamp(max=spec.clip_max)
        return gate, gate, {"raw": raw}
    if spec.kind == GATE_GELU_Z:
        z = (s - tau) / sigma
        phi = 0.5 * (1.0 + torch.erf(z * _INV_SQRT2))
        gate = torch.where(z > 0, z * phi, torch.zeros_like(z))
        return gate, gate, {"z": z, "phi": phi}
    m = (s - tau) - spec.activation_threshold
    act = torch.sigmoid(spec.sharpness * m)
    am = (m - spec.activation_cutoff).clamp(min=0.0)
    inten = spec.epsilon + am.clamp(max=spec.max_intensity)
    return act * inten, inten, {"activation": act, "intensity": inten}


def gate_backward(spec: GateSpec, s, tau, sigma, dgate, dden_term):
    """Manual derivative used by the fused kernels (and mirrored here in torch
    so the math is testable on CPU): returns ``(ds_local, dtau_rows, dsigma_rows)``
    where ``ds_local`` is the gradient on the scores through the gate alone and
    the row terms are the sums over units that flow to ``tau`` and ``sigma``.

    ``dgate`` is the gradient on the gate values, ``dden_term`` (broadcast
    [..., 1]) the gradient on the per-unit denominator term.
    """
    if spec.kind == GATE_RELU_CLIP:
        raw = s - tau
        inside = ((raw > 0) & (raw < spec.clip_max)).to(s.dtype)
        ds = (dgate + dden_term) * inside
        return ds, -ds.sum(-1, keepdim=True), torch.zeros_like(tau)
    if spec.kind == GATE_GELU_Z:
        z = (s - tau) / sigma
        phi = 0.5 * (1.0 + torch.erf(z * _INV_SQRT2))
        pdf = _INV_SQRT2PI * torch.exp(-0.5 * z * z)
        dz = (dgate + dden_term) * (phi + z * pdf) * (z > 0).to(s.dtype)
        ds = dz / sigma
        return ds, -ds.sum(-1, keepdim=True), -(ds * z).sum(-1, keepdim=True)
    m = (s - tau) - spec.activation_threshold
    act = torch.sigmoid(spec.sharpness * m)
    amr = m - spec.activation_cutoff
    inten = spec.epsilon + amr.clamp(min=0.0).clamp(max=spec.max_intensity)
    dact = dgate * inten
    dint = dgate * act + dden_term
    lin = ((amr > 0) & (amr < spec.max_intensity)).to(s.dtype)
    ds = dact * spec.sharpness * act * (1.0 - act) + dint * lin
    return ds, -ds.sum(-1, keepdim=True), torch.zeros_like(tau)


def sqrt_d(d_model: int) -> float:
    return math.sqrt(float(d_model))
