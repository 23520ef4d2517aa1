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
        self._ar_stage, self._ar_stage_dev, self._ar_epoch = None, None, 0

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

    AR_SLOT_BASE = 512          # pad slots [512, 1024) belong to all_reduce_small
    AR_CAP = 131072             # largest vector (fp32 elements) it takes: 32 CTAs x 8 ranks of slots

    def all_reduce_small(self, x: torch.Tensor) -> torch.Tensor:
        """In-place sum over the group of a contiguous fp32 tensor of at most
        ``AR_CAP`` elements, by one kernel over peer memory (no library call)."""
        from ..ops import cuda_backend as CB
        if self._ar_stage is None:
            raise RuntimeError("enable_small_allreduce() was not called (it is collective)")
        self._ar_epoch += 1
        CB.ext().small_allreduce(self._ar_stage_dev, self.pads_dev, self.rank, self.world,
                                 self._ar_epoch, self.AR_SLOT_BASE, x, x, self.AR_CAP,
                                 CB.status_word(self.device), 0)
        CB.count_launches(1)
        return x

    def enable_small_allreduce(self) -> None:
        """Collective: allocate the staging buffers of ``all_reduce_small``."""
        if self._ar_stage is None:
            self._ar_stage = self.alloc("__ar_stage__", (2 * self.AR_CAP,), torch.float32)
            self._ar_stage_dev = torch.tensor(self._ar_stage.ptrs, dtype=torch.int64,
                                              device=self.device)

    def barrier(self, channel: int = 0, wait_cycles: int = 0) -> None:
        """Enqueue a bounded cross-GPU barrier on the current stream.  Channels
        use disjoint pad slots, so barriers on different streams do not mix."""
        from ..ops import cuda_backend as CB
        ep = self._epoch.get(channel, 0) + 1
        self._epoch[channel] = ep
        CB.ext().peer_barrier(self.pads_dev, self.rank, self.world, ep, channel * self.world,
                              CB.status_word(self.device), wait_cycles)
