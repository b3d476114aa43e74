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


class SymmSlice:
    """A sub-range of an arena: the same interface as :class:`SymmBuffer` (tensor, peer addresses, multicast address,
    barrier), with every address advanced by the slice's byte offset.  Barriers of a slice use the arena's signal pad
    on the slice's channel."""

    def __init__(self, arena: SymmBuffer, byte_offset: int, numel: int, dtype: torch.dtype, channel: int) -> None:
        elem = torch.empty((), dtype=dtype).element_size()
        raw = arena.tensor.view(torch.uint8)[byte_offset : byte_offset + numel * elem]
        self.tensor = raw.view(dtype)
        self.arena, self.world, self.rank, self.channel = arena, arena.world, arena.rank, channel
        ptrs = [int(arena.peer_ptrs[i]) + byte_offset if i < arena.world else 0 for i in range(8)]
        self.peer_ptrs = (ctypes.c_longlong * 8)(*ptrs)
        self.multicast_ptr = (arena.multicast_ptr + byte_offset) if arena.multicast_ptr else None
        self.handle = arena.handle

    def barrier(self, channel: int | None = None) -> None:
        self.arena.barrier(self.channel if channel is None else channel)


_REGISTRY: dict[int, object] = {}


def lookup(t: torch.Tensor):
    return _REGISTRY.get(t.data_ptr())


ARENA_ALIGN = 256
ARENA_MIN_BYTES = int(os.environ.get("KF_SYMM_ARENA_MIN_MB", "256")) << 20
ARENA_MAX_BYTES = int(os.environ.get("KF_SYMM_ARENA_MAX_MB", "8192")) << 20


def make_allocator(group):
    """Allocator for ``FlatParamGroup``: flat buffers are placed in symmetric memory of ``group``.

    Buffers are carved out of a few large arenas (each one rendezvous: 256 MB first, doubling up to 8 GB, or as large
    as a single request needs) instead of one rendezvous per buffer: a 32-block model needs a handful of exchanges of
    peer addresses at start-up, not 66.  Requests alternate between two barrier channels (parameters / gradients are
    allocated alternately), so the two kinds never share a signal slot."""
    if group is None:
        group = dist.group.WORLD
    state = {"arena": None, "used": 0, "next": ARENA_MIN_BYTES, "count": 0}

    def alloc(numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        elem = torch.empty((), dtype=dtype).element_size()
        need = -(-numel * elem // ARENA_ALIGN) * ARENA_ALIGN
        arena = state["arena"]
        if arena is None or state["used"] + need > arena.tensor.numel():
            size = max(need, min(state["next"], ARENA_MAX_BYTES))
            state["next"] = min(2 * size, ARENA_MAX_BYTES)
            arena = state["arena"] = SymmBuffer(size, torch.uint8, device, group)
            state["used"] = 0
        piece = SymmSlice(arena, state["used"], numel, dtype, channel=state["count"] % 2)
        state["used"] += need
        state["count"] += 1
        _REGISTRY[piece.tensor.data_ptr()] = piece
        return piece.tensor

    return alloc
