"""Buffers behind the fused tensor-parallel GEMM + collective kernels.

``GemmRSContext`` owns, per tensor-parallel group, a staging buffer and a counter array in symmetric memory:
the GEMM epilogue of every rank stores finished tiles into the owner's staging slice and bumps the owner's
per-tile counter; the owner sums the slices once a tile's counter shows all contributions.  The buffers are
sized for the largest (T, D) seen and shared by every row-parallel Linear of the model (calls are serialised
on the stream; staging and counters alternate by call parity).
"""

from __future__ import annotations

import ctypes

import torch

from kempnerforge_b200.comm.symmetric import SymmBuffer


class GemmRSContext:
    def __init__(self, group, device: torch.device, max_tokens: int, max_dim: int) -> None:
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.max_tokens, self.max_dim = max_tokens, max_dim
        # [2 parities][world sources][T / world][D] bf16  ==  2 * T * D elements
        self.stage = SymmBuffer(2 * max_tokens * max_dim, torch.bfloat16, device, group)
        tiles = (max_tokens // self.world // 128 + 1) * ((max_dim + 255) // 256)
        self.flags = SymmBuffer(2 * tiles, torch.int32, device, group)
        self.stage_ptrs = (ctypes.c_longlong * 8)(*self.stage.peer_ptrs)
        self.flag_ptrs = (ctypes.c_longlong * 8)(*self.flags.peer_ptrs)
        self.calls = 0
        self.shape: tuple[int, int] | None = None
        self.stage.barrier()

    def reserve(self, tokens: int, dim: int) -> None:
        """Counters are laid out for one (T, D); a different shape restarts them (all ranks do so together)."""
        if tokens > self.max_tokens or dim > self.max_dim:
            raise ValueError(f"fused GEMM+reduce-scatter buffers sized for ({self.max_tokens}, {self.max_dim}), "
                             f"got ({tokens}, {dim})")
        if self.shape != (tokens, dim):
            if self.shape is not None:
                torch.cuda.current_stream().synchronize()
                self.stage.barrier()  # nobody is still pushing for the old layout
            self.flags.tensor.zero_()
            self.calls = 0
            self.shape = (tokens, dim)
            self.stage.barrier()

    def next_call(self) -> int:
        n = self.calls
        self.calls += 1
        return n


class AgGemmContext(GemmRSContext):
    """Gather buffer ([2 parities][T][K] bf16) and per-(source, row block) counters for the fused
    all-gather + GEMM kernel; same life cycle as ``GemmRSContext``."""

    def __init__(self, group, device: torch.device, max_tokens: int, max_dim: int) -> None:
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.max_tokens, self.max_dim = max_tokens, max_dim
        self.stage = SymmBuffer(2 * max_tokens * max_dim, torch.bfloat16, device, group)
        self.flags = SymmBuffer(2 * self.world * (max_tokens // self.world // 128 + 1), torch.int32, device, group)
        self.stage_ptrs = (ctypes.c_longlong * 8)(*self.stage.peer_ptrs)
        self.flag_ptrs = (ctypes.c_longlong * 8)(*self.flags.peer_ptrs)
        self.calls = 0
        self.shape = None
        self.stage.barrier()
