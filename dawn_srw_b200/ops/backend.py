"""Op backends.

``ReferenceBackend`` runs every op through plain PyTorch (CPU oracle in fp32;
on a GPU with ``compute_dtype=bfloat16`` it is the library baseline: cuBLAS
GEMMs + NCCL).  ``CudaBackend`` (ops/cuda_backend.py) replaces the hot ops with
the hand-written sm_100a kernels.  There is exactly one product path on a GPU:
``default_backend`` raises if the compiled extension is missing instead of
falling back silently.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Optional

import torch

from . import reference as R
from .gates import GateSpec
from .srw_ref import SRWResult, prepare_pool_ref, srw_pool_ref


@dataclass
class ParallelCtx:
    """Where a pool op runs: which process group splits the units, which group
    is data-parallel, and the true (unpadded) unit counts."""
    shard_group: Any = None
    dp_group: Any = None
    n_total: Optional[int] = None     # global units in the pool
    n_valid: Optional[int] = None     # real (non-padding) units held locally
    seq_sharded: bool = False         # activations between pool ops are token-sharded


@dataclass
class PreparedPool:
    emb: torch.Tensor
    read: torch.Tensor
    write: torch.Tensor
    extra: Any = None                 # backend-specific (Gram matrix, grad buffers, ...)


class ReferenceBackend:
    name = "reference"

    def __init__(self, compute_dtype=torch.float32, chunk_size: Optional[int] = None,
                 use_checkpoint: bool = False):
        self.compute_dtype = compute_dtype
        self.chunk_size = chunk_size
        self.use_checkpoint = use_checkpoint

    # ---- dense ops -----------------------------------------------------
    def layer_norm(self, x, w, b):
        return R.layer_norm(x, w, b)

    def linear(self, x, w, b=None):
        return R.linear(x, w, b, None if self.compute_dtype == torch.float32 else self.compute_dtype)

    def embed(self, ids, tok, pos):
        return R.embed(ids, tok, pos)

    def dropout(self, x, p, training):
        return R.dropout(x, p, training)

    def dropout_add(self, res, x, p, training):
        return res + R.dropout(x, p, training)

    def attention(self, q, k, v, dropout_p, training):
        if self.compute_dtype == torch.float32 or not q.is_cuda:
            return R.causal_attention(q, k, v, dropout_p, training)
        cd = self.compute_dtype
        o = torch.nn.functional.scaled_dot_product_attention(
            q.to(cd), k.to(cd), v.to(cd), dropout_p=dropout_p if training else 0.0, is_causal=True)
        return o.float()

    def lm_head_ce(self, x, tok_emb, labels):
        return R.lm_head_ce(x, tok_emb, labels,
                            None if self.compute_dtype == torch.float32 else self.compute_dtype)

    def logits(self, x, tok_emb):
        return R.logits_from_hidden(x, tok_emb,
                                    None if self.compute_dtype == torch.float32 else self.compute_dtype)

    def diversity(self, tensors):
        return R.pool_diversity(tensors)

    # ---- SRW pool op ---------------------------------------------------
    def prepare_pool(self, emb, read, write, spec: GateSpec, pctx: Optional[ParallelCtx] = None):
        e, r, w = prepare_pool_ref(emb, read, write, spec, self.compute_dtype)
        return PreparedPool(e, r, w)

    def srw(self, x, h, tau_off, pool: PreparedPool, spec: GateSpec, *,
            pctx: Optional[ParallelCtx] = None, want_diag: bool = True,
            return_gates: bool = False, unit_mask=None, out_scale=None) -> SRWResult:
        """``out_scale`` (float or 0-dim tensor): the pool's output scale; when
        given, ``SRWResult.out`` / ``route(i)`` are already multiplied by it."""
        pctx = pctx or ParallelCtx()
        res = self._srw(x, h, tau_off, pool, spec, pctx, want_diag, return_gates, unit_mask)
        if out_scale is not None:
            res.out = res.out * out_scale
        return res

    def srw_group(self, x, calls, spec: GateSpec, *, want_diag: bool = True):
        """Several SRW calls on the same activations ``x`` (the Q/K and V calls of
        an attention block).  ``calls``: dicts with the keyword arguments of
        ``srw`` (h, tau_off, pool, pctx, out_scale, unit_mask).  Backends that can
        share work between the calls override this; the default runs them in turn."""
        return [self.srw(x, c["h"], c["tau_off"], c["pool"], spec, pctx=c.get("pctx"),
                         want_diag=want_diag, unit_mask=c.get("unit_mask"),
                         out_scale=c.get("out_scale")) for c in calls]

    def _srw(self, x, h, tau_off, pool, spec, pctx, want_diag, return_gates, unit_mask):
        return srw_pool_ref(
            x, h, tau_off, pool.emb, pool.read, pool.write, spec,
            compute_dtype=self.compute_dtype, chunk_size=self.chunk_size,
            n_valid=pctx.n_valid, n_total=pctx.n_total, shard_group=pctx.shard_group,
            dp_group=pctx.dp_group, unit_mask=unit_mask, want_diag=want_diag,
            return_gates=return_gates, use_checkpoint=self.use_checkpoint,
            seq_sharded=pctx.seq_sharded)

    def finish_run(self):
        pass

    def finish_step(self):
        pass


_EXT_ERROR: Optional[str] = None


def load_cuda_backend(**kw):
    from .cuda_backend import CudaBackend
    return CudaBackend(**kw)


def default_backend(device: torch.device, *, allow_library: Optional[bool] = None, **kw):
    """Backend for ``device``.  CPU -> fp32 reference.  CUDA -> the sm_100a
    kernels; a missing or unbuildable extension is an error unless the caller
    (or ``DAWN_B200_LIBRARY=1``) explicitly asks for the library baseline."""
    device = torch.device(device)
    if device.type != "cuda":
        return ReferenceBackend(torch.float32)
    if allow_library is None:
        allow_library = os.environ.get("DAWN_B200_LIBRARY", "0") == "1"
    if allow_library:
        return ReferenceBackend(torch.bfloat16, chunk_size=kw.pop("chunk_size", 12500),
                                use_checkpoint=True)
    return load_cuda_backend(**kw)
