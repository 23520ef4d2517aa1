"""Symmetric (peer-mapped) device memory for the in-kernel communication paths.

Buffers are allocated with ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations mapped into every rank of the group), which hands back raw peer
pointers; the kernels then read and write those addresses directly over
NVLink (TMA loads from a peer, TMA reduce-adds into a peer, release/acquire
flag words).  No NCCL call is involved after set-up.

``SymmWorkspace`` owns
* one signal pad per rank (uint32 slots) for ``barrier()`` — a bounded
  all-to-all flag exchange (ops/csrc/comm_kernels.cu); a peer that never shows
  up produces status 3 on the host instead of a hang;
* named data buffers, each visible as a local tensor and as peer pointers.

The reference has no counterpart: its collectives are implicit in XLA SPMD
(reference: scripts/train_jax.py:728-729).
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch
import torch.distributed as dist


class SymmBuffer:
    def __init__(self, local: torch.Tensor, ptrs: List[int], handle):
        self.local, self.ptrs, self.handle = local, ptrs, handle

    def peer(self, rank: int, shape, dtype, offset_elems: int = 0) -> torch.Tensor:
        """Tensor view of rank ``rank``'s copy (peer-mapped memory)."""
        return self.handle.get_buffer(rank, shape, dtype, offset_elems)


class SymmWorkspace:
    PAD_SLOTS = 1024

    def __init__(self, group, device):
        import torch.distributed._symmetric_memory as sm
        self._sm = sm
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.device = torch.device(device)
        self.buffers: Dict[str, SymmBuffer] = {}
        pad = self.alloc("__pads__", (self.PAD_SLOTS,), torch.int32)
        pad.local.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        self.pads_dev = torch.tensor(pad.ptrs, dtype=torch.int64, device=self.device)
        self._epoch: Dict[int, int] = {}

    def alloc(self, name: str, shape, dtype) -> SymmBuffer:
        """Collective: every rank of the group must call it with the same arguments."""
        if name in self.buffers:
            b = self.buffers[name]
            if tuple(b.local.shape) == tuple(shape) and b.local.dtype == dtype:
                return b
            raise ValueError(f"symmetric buffer {name!r} exists with another shape")
        t = self._sm.empty(*shape, dtype=dtype, device=self.device)
        hdl = self._sm.rendezvous(t, self.group)
        buf = SymmBuffer(t, [int(p) for p in hdl.buffer_ptrs], hdl)
        self.buffers[name] = buf
        return buf

    def barrier(self, channel: int = 0, wait_cycles: int = 0) -> None:
        """Enqueue a bounded cross-GPU barrier on the current stream.  Channels
        use disjoint pad slots, so barriers on different streams do not mix."""
        from ..ops import cuda_backend as CB
        ep = self._epoch.get(channel, 0) + 1
        self._epoch[channel] = ep
        CB.ext().peer_barrier(self.pads_dev, self.rank, self.world, ep, channel * self.world,
                              CB.status_word(self.device), wait_cycles)
