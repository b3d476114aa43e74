"""Buffers behind the fused tensor-parallel GEMM + collective kernels.

``GemmRSContext`` owns, per tensor-parallel group, a staging buffer and a counter array in symmetric memory:
the GEMM epilogue of every rank stores finished tiles into the owner's staging slice and bumps the owner's
per-tile counter; the owner sums the slices once a tile's counter shows all contributions.  The buffers are
sized for the largest (T, D) seen and shared by every row-parallel Linear of the model (calls are serialised
on the stream; staging and counters alternate by call parity).

Why two parities are enough (no fence between call n and call n + 2).  A rank writes into a peer's parity-p buffer
only from inside its own call n (n = p mod 2).  For rank A to *start* call n + 2 it has finished call n + 1 on its
stream, and its call n + 1 could only finish after it had received every peer's contribution to call n + 1 (the
all-gather GEMM consumes every owner's rows; the reduce-scatter GEMM sums every source's tiles, each behind a
bounded counter wait).  Peer B issues its contribution to call n + 1 from its own call n + 1 kernel, which is ordered
on B's stream after B's call n kernel — the last reader of B's parity-p buffer of call n.  Hence
"B finished reading parity p of call n"  happens-before  "B contributes to n + 1"  happens-before  "A finishes n + 1"
happens-before  "A overwrites B's parity p in call n + 2".  The argument needs (i) every call of a context to involve
every rank of the group, (ii) calls of one context to be issued on one stream per rank in the same order on all ranks
— both hold for the layers of a tensor-parallel model — and (iii) the counters to be monotonic (they are: the expected
value is derived from the call number), so a stale counter can never satisfy a later call.
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
