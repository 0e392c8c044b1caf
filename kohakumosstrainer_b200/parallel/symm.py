"""Symmetric memory: buffers every rank of a group has mapped, plus the flag words the
peer-memory kernels synchronise on.

Allocation and handle exchange go through `torch.distributed._symmetric_memory` (CUDA
virtual-memory handles exchanged over the process group's store; an NVLS multicast mapping
when the fabric supports it). The collectives themselves are this package's kernels
(`csrc/comm.cu`), which read and write the peers' mappings directly.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist
from torch import Tensor


# NVLS multicast mappings are opt-in (KMOSS_NVLS=1): a rank that dies while its memory is bound
# to a multicast object can fault its peers' GPUs, and the peer load / store path needs none.
if os.environ.get("KMOSS_NVLS", "0") != "1":
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")


def available(device) -> bool:
    if torch.device(device).type != "cuda" or not dist.is_initialized():
        return False
    try:
        from torch.distributed import _symmetric_memory  # noqa: F401
    except ImportError:
        return False
    return dist.get_backend() == "nccl"


class SymmetricBuffer:
    """A flat tensor mapped on every rank of `group`: `local` is this rank's memory,
    `ptrs[r]` the device address of rank r's copy as seen from here, `mc_ptr` the multicast
    address (0 without NVLS)."""

    def __init__(self, numel: int, dtype: torch.dtype, device, group=None, zero: bool = True):
        import torch.distributed._symmetric_memory as sm

        group = group or dist.group.WORLD
        self.local: Tensor = sm.empty(numel, dtype=dtype, device=device)
        if zero:
            self.local.zero_()
        self.handle = sm.rendezvous(self.local, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.mc_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.rank, self.world = self.handle.rank, self.handle.world_size


class PeerFlags:
    """Zero-initialised flag words for the all-reduce kernels, one allocation per process
    group, with the strictly increasing epoch the kernels compare against."""

    def __init__(self, device, group=None):
        from ..ops import native

        words = native.load().allreduce_flag_words()
        self.buffer = SymmetricBuffer(words, torch.int32, device, group, zero=True)
        torch.cuda.synchronize(device)
        dist.barrier(group)  # nobody signals before every rank's flags are zero
        self.epoch = 0

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch
