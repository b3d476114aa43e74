"""Rotary position embedding with half-split pairing.

Tables are fp32 (S, head_dim/2); element i of a head is paired with element
i + head_dim/2.  Parity: kempnerforge/model/position.py:12-71.
"""

from __future__ import annotations

import torch

from kempnerforge_b200.ops import functional as F
from kempnerforge_b200.ops import ref


def precompute_rope_frequencies(head_dim: int, max_seq_len: int, theta: float = 10000.0, device=None):
    """Returns (cos, sin), each of shape (max_seq_len, head_dim // 2), fp32."""
    return ref.rope_tables(head_dim, max_seq_len, theta, device)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: (batch, seq, heads, head_dim); cos/sin: (seq, head_dim/2) or (batch, seq, head_dim/2)."""
    return F.rope(x, cos, sin)
