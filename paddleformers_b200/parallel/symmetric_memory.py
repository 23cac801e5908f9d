"""Symmetric device buffers: the same allocation on every rank of a group, each mapped into every peer.

A ``SymmetricBuffer`` is what the fused compute + collective kernels address other GPUs through: ``peer_ptrs[i]`` is
the device address (valid on *this* GPU) of rank i's copy, reachable with ordinary loads / stores / reductions and
non-multicast TMA over NVLink. The handles travel through ``torch.distributed`` once at construction; nothing is
exchanged on the step path. ``FlagPad`` is a small symmetric int32 array used for epoch flags between ranks.

Role in the reference: the NVLink buffers DeepEP sets up (paddleformers/transformers/fused_a2a.py:49-78) and the
comm buffers Flux uses for its all-gather GEMM (paddleformers/cli/train/ernie_pretrain/models/
sequence_parallel_utils.py:179-236).
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import functional as F


class SymmetricBuffer:
    def __init__(self, nbytes: int, group, device: Optional[torch.device] = None):
        ops = F._ops()
        self.group = group
        self.nbytes = int((nbytes + 255) // 256 * 256)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        # a one-rank group (or no process group at all): the only peer is this rank itself, nothing to exchange
        self._solo = not dist.is_initialized() or not isinstance(group, (dist.ProcessGroup, type(None)))
        self.world = 1 if self._solo else dist.get_world_size(group)
        self.rank = 0 if self._solo else dist.get_rank(group)
        self.local_ptr, handle = ops.symm_alloc(self.nbytes)
        handles: List[Optional[torch.Tensor]] = [None] * self.world
        if not self._solo:
            dist.all_gather_object(handles, handle, group=group)
        self.peer_ptrs: List[int] = []
        for r, h in enumerate(handles):
            self.peer_ptrs.append(self.local_ptr if r == self.rank else int(ops.symm_open(h)))
        self.peer_ptrs_tensor = torch.tensor(self.peer_ptrs, dtype=torch.int64, device=self.device)
        if not self._solo:
            dist.barrier(group=group)

    def tensor(self, shape: Sequence[int], dtype: torch.dtype, byte_offset: int = 0) -> torch.Tensor:
        """View of the LOCAL copy."""
        n = 1
        for s in shape:
            n *= s
        assert byte_offset + n * torch.empty((), dtype=dtype).element_size() <= self.nbytes
        return F._ops().symm_tensor(self.local_ptr + byte_offset, list(shape), dtype, self.device.index or 0)

    def close(self):
        ops = F._ops()
        for r, p in enumerate(self.peer_ptrs):
            if r != self.rank:
                ops.symm_close(p)
        if not self._solo:
            dist.barrier(group=self.group)
        ops.symm_free(self.local_ptr)


class FlagPad(SymmetricBuffer):
    """Symmetric array of int32 epoch flags (zero-initialised)."""

    def __init__(self, n_flags: int, group, device=None):
        super().__init__(n_flags * 4, group, device)
        self.n_flags = n_flags
        self.flags = self.tensor((n_flags,), torch.int32)

    def signal_all(self, slot: int, value: int):
        """Write ``value`` into ``flags[slot]`` of every rank (stream-ordered after this rank's earlier work)."""
        F._ops().peer_signal(self.peer_ptrs_tensor, slot, value)

    def wait(self, slot0: int, n: int, value: int, timeout_s: float = 2.0):
        """Block the stream until ``flags[slot0 : slot0 + n] >= value`` on this rank, or record a timeout status."""
        F._ops().peer_wait(self.local_ptr, slot0, n, value, timeout_s)


def device_barrier(pad: FlagPad, epoch: int, base_slot: int = 0, timeout_s: float = 2.0):
    """Stream-ordered barrier over the group through peer flags: rank r raises flag ``base_slot + r`` on everyone, then
    waits for all of them."""
    F._ops().peer_signal(pad.peer_ptrs_tensor, base_slot + pad.rank, epoch)
    pad.wait(base_slot, pad.world, epoch, timeout_s)
