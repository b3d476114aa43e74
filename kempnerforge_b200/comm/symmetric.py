"""Symmetric (peer-mapped) memory for the data-parallel engine.

Every rank allocates the same buffer from the CUDA virtual-memory pool that PyTorch's symmetric-memory
module manages; after a rendezvous each rank holds the device address of every peer's copy and, when the
fabric supports it, one NVSwitch multicast address that fans a store out to (or reduces a load over) all
copies.  Our kernels take those addresses directly (``kempnerforge_b200.ops.cuda.symm_*``).

Ordering between ranks is a signal-pad barrier on the stream (``SymmBuffer.barrier``); it is bounded by a
timeout, so a rank that never arrives produces an error instead of a hang.  ``KF_SYMM_MULTIMEM=0`` keeps the
kernels on plain peer loads / stores (the mode used by fault-handling tests), ``1`` forces the multicast
instructions, the default ``auto`` uses them from four ranks on.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

BARRIER_TIMEOUT_MS = int(os.environ.get("KF_SYMM_BARRIER_TIMEOUT_MS", "30000"))


class SymmBuffer:
    """A flat tensor in symmetric memory plus the addresses of every peer's copy."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
        self.tensor.zero_()
        self.handle = symm_mem.rendezvous(self.tensor, group)
        self.world = self.handle.world_size
        self.rank = self.handle.rank
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.peer_ptrs = (ctypes.c_longlong * 8)(*(ptrs + [0] * (8 - len(ptrs))))
        # NVSwitch multicast (multimem.ld_reduce / multimem.st) pays once the in-switch reduction / fan-out saves bytes on
        # this GPU's links: with two ranks it saves nothing and measured 1.8x slower than plain peer loads / stores
        # (0.685 vs 0.375 ms for one block's reduce-scatter), so "auto" uses it from four ranks on
        mode = os.environ.get("KF_SYMM_MULTIMEM", "auto")
        use_mc = mode == "1" or (mode == "auto" and self.world >= 4)
        mc = int(self.handle.multicast_ptr) if use_mc and getattr(self.handle, "multicast_ptr", 0) else 0
        self.multicast_ptr = mc or None

    def barrier(self, channel: int = 0) -> None:
        """All ranks of the group reach this point of their current streams (bounded wait)."""
        self.handle.barrier(channel=channel, timeout_ms=BARRIER_TIMEOUT_MS)


_REGISTRY: dict[int, SymmBuffer] = {}


def lookup(t: torch.Tensor) -> SymmBuffer | None:
    return _REGISTRY.get(t.data_ptr())


def make_allocator(group):
    """Allocator for ``FlatParamGroup``: flat buffers are placed in symmetric memory of ``group``."""
    if group is None:
        group = dist.group.WORLD

    def alloc(numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        buf = SymmBuffer(numel, dtype, device, group)
        _REGISTRY[buf.tensor.data_ptr()] = buf
        return buf.tensor

    return alloc
