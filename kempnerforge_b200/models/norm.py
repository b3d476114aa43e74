"""Normalisation layers.  ``RMSNorm`` runs the fused sm_100a kernel on bf16 CUDA inputs.

Parity: kempnerforge/model/norm.py:11-45 (fp32 compute, cast back; registry keys
``rmsnorm`` / ``layernorm``).
"""

from __future__ import annotations

import torch
from torch import nn

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.ops import functional as F


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.rmsnorm(x, self.weight, self.eps)

    def extra_repr(self) -> str:
        return f"{self.weight.shape[0]}, eps={self.eps}"


registry.register("norm", "rmsnorm", lambda dim, eps=1e-5: RMSNorm(dim, eps))
registry.register("norm", "layernorm", lambda dim, eps=1e-5: nn.LayerNorm(dim, eps=eps))


def build_norm(norm_type: str, dim: int, eps: float = 1e-5) -> nn.Module:
    return registry.get("norm", str(norm_type))(dim, eps)
