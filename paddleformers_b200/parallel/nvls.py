"""All-reduce through NVSwitch multicast memory (``csrc/nvls.cu``): the switch forms the sum (``multimem.ld_reduce``) and
fans the result out (``multimem.st``), so every GPU moves 1/tp of the tensor per direction instead of a ring's 2(tp-1)/tp.

The multicast binding of the buffers is plumbing and comes from ``torch.distributed._symmetric_memory`` (one symmetric
allocation per process group, bound to a multicast object when the fabric supports it); the reduction kernel, its
barriers and their bounded waits are this library's. Used by the tensor-parallel linears without sequence parallelism
(``ReduceFromTP`` / ``CopyToTP``) for bf16 tensors up to ``PFB_NVLS_MAX_MB`` (default 64 MB); anything else, and every
group without multicast support, stays on NCCL. ``PFB_NVLS=0`` switches it off.

A rank must not exit while its peers still use the multicast object: ``release()`` (called by ``Trainer`` shutdown paths
and at interpreter exit) drops the buffers after a barrier.
"""
from __future__ import annotations

import atexit
import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

STATS = {"nvls_all_reduce": 0}
_STATE: Dict[int, Optional["NvlsAllReduce"]] = {}


class NvlsAllReduce:
    def __init__(self, group, max_bytes: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        dev = torch.device("cuda", torch.cuda.current_device())
        self.flag_bytes = int(torch.ops.pfb200.nvls_flag_bytes())
        self.capacity = max_bytes // 2                       # bf16 elements
        self.buf = symm_mem.empty(self.flag_bytes + max_bytes, dtype=torch.uint8, device=dev)
        self.buf.zero_()
        torch.cuda.synchronize()
        self.handle = symm_mem.rendezvous(self.buf, group=group)
        self.mc_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        if self.mc_ptr == 0:
            raise RuntimeError("the process group's symmetric memory has no multicast binding")
        self.peer_ptrs = torch.tensor([int(p) for p in self.handle.buffer_ptrs], dtype=torch.int64)
        self.data = self.buf[self.flag_bytes:].view(torch.bfloat16)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        dist.barrier(group=group)                            # every rank's flags are zero before anyone signals

    def all_reduce_(self, x: torch.Tensor) -> torch.Tensor:
        n = x.numel()
        padded = (n + 7) // 8 * 8
        flat = x.reshape(-1)
        self.data[:n].copy_(flat)
        self.epoch.add_(1)
        torch.ops.pfb200.nvls_allreduce_bf16(self.mc_ptr, self.peer_ptrs, padded, self.rank, self.epoch)
        flat.copy_(self.data[:n])
        STATS["nvls_all_reduce"] += 1
        return x


def _get(group) -> Optional[NvlsAllReduce]:
    key = id(group)
    if key not in _STATE:
        st = None
        if (os.environ.get("PFB_NVLS", "1") != "0" and torch.cuda.is_available() and hasattr(torch.ops.pfb200, "nvls_allreduce_bf16")
                and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0" and dist.get_backend(group) == "nccl"):
            try:
                st = NvlsAllReduce(group, int(float(os.environ.get("PFB_NVLS_MAX_MB", "64")) * (1 << 20)))
            except Exception as e:  # noqa: BLE001  no multicast on this fabric / torch build: NCCL does the all-reduce
                from ..utils.log import logger

                logger.info(f"NVLS all-reduce unavailable ({type(e).__name__}: {e}); using NCCL")
                st = None
        _STATE[key] = st
    return _STATE[key]


def all_reduce_(x: torch.Tensor, group) -> torch.Tensor:
    """In-place sum over ``group``: the multicast kernel when it applies, NCCL otherwise."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous():
        st = _get(group)
        if st is not None and 0 < x.numel() <= st.capacity:
            return st.all_reduce_(x)
    dist.all_reduce(x, group=group)
    return x


def release() -> None:
    """Drop the multicast-bound buffers; all ranks call it (it synchronises the device and the group first)."""
    for key, st in list(_STATE.items()):
        if st is not None:
            try:
                torch.cuda.synchronize()
                if dist.is_initialized():
                    dist.barrier(group=st.group)
            except Exception:  # noqa: BLE001  the group is already gone
                pass
            st.data = st.buf = st.handle = None
        _STATE.pop(key, None)


atexit.register(release)
