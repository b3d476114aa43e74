"""Feed-forward blocks.

``SwiGLUMLP`` issues one GEMM for gate and up (their weights sit back to back in
the block's flat parameter buffer, so the stacked (2H, D) matrix is a view), a
fused SwiGLU kernel, and the down GEMM.
Parity: kempnerforge/model/mlp.py:12-77 (module/parameter names, registry keys
``swiglu`` / ``standard_gelu`` / ``standard_relu``, ``build_mlp`` dispatch).
"""

from __future__ import annotations

import torch
from torch import nn

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.ops import functional as F


class SwiGLUMLP(nn.Module):
    def __init__(self, dim: int, hidden_dim: int) -> None:
        super().__init__()
        self.gate_proj = nn.Linear(dim, hidden_dim, bias=False)
        self.up_proj = nn.Linear(dim, hidden_dim, bias=False)
        self.down_proj = nn.Linear(hidden_dim, dim, bias=False)
        self.tp = None  # TPContext when gate/up are column-sharded and down row-sharded

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp is not None:
            gu = self.tp.column_linear(x, [self.gate_proj.weight, self.up_proj.weight])
            return self.tp.row_linear(F.swiglu_stacked(gu), self.down_proj.weight)
        gu = F.fused_linear(x, [self.gate_proj.weight, self.up_proj.weight])
        return F.linear(F.swiglu_stacked(gu), self.down_proj.weight)


_ACTS = {"gelu": nn.GELU, "relu": nn.ReLU, "silu": nn.SiLU}


class StandardMLP(nn.Module):
    def __init__(self, dim: int, hidden_dim: int, activation: str = "gelu") -> None:
        super().__init__()
        self.up_proj = nn.Linear(dim, hidden_dim, bias=False)
        self.down_proj = nn.Linear(hidden_dim, dim, bias=False)
        self.act = _ACTS[activation]()
        self.tp = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp is not None:
            x = self.tp.before_column_parallel(x)
        y = F.linear(self.act(F.linear(x, self.up_proj.weight)), self.down_proj.weight)
        return self.tp.after_row_parallel(y) if self.tp is not None else y


registry.register("mlp", "swiglu", lambda dim, hidden: SwiGLUMLP(dim, hidden))
registry.register("mlp", "standard_gelu", lambda dim, hidden: StandardMLP(dim, hidden, "gelu"))
registry.register("mlp", "standard_relu", lambda dim, hidden: StandardMLP(dim, hidden, "relu"))


def build_mlp(dim: int, hidden_dim: int, activation: str = "silu") -> nn.Module:
    """silu -> SwiGLU (three matrices); gelu / relu -> two-matrix MLP."""
    key = {"silu": "swiglu", "gelu": "standard_gelu", "relu": "standard_relu"}.get(str(activation))
    if key is None:
        raise ValueError(f"Unknown activation: {activation!r}")
    return registry.get("mlp", key)(dim, hidden_dim)
