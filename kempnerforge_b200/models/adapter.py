"""Adapters from vision features (B, N, F) to decoder embeddings (B, N', D).

  mlp_2layer        Linear -> activation -> Linear (with biases; hidden defaults to the output width)
  linear            one Linear
  avgpool           mean over window x window patches of the square token grid (ragged edges averaged over the
                    patches that exist), then Linear
  attentional_pool  one query per window (the window mean) attends over the window's patches (multi-head), then
                    Linear; the grid side must be divisible by the window

Parity: kempnerforge/model/adapter.py:54-383 (types, ``output_num_tokens``, ``pooled_token_count``).
"""

from __future__ import annotations

import math

import torch
from torch import nn

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.config.vlm import DIVISIBLE_ONLY_POOL_TYPES, POOLING_ADAPTER_TYPES, pooled_token_count  # noqa: F401

_ACT = {"gelu": nn.GELU, "silu": nn.SiLU, "relu": nn.ReLU}


class VisionAdapter(nn.Module):
    def output_num_tokens(self, num_input_tokens: int) -> int:
        return num_input_tokens

    def reset_parameters(self) -> None:
        """Re-run the default initialisation of every Linear (after ``to_empty`` on a meta-device build)."""
        for m in self.modules():
            if isinstance(m, nn.Linear):
                m.reset_parameters()


def _check_dims(kind: str, in_dim: int, out_dim: int) -> None:
    if in_dim <= 0 or out_dim <= 0:
        raise ValueError(f"{kind} in_dim and out_dim must be positive (got {in_dim}, {out_dim})")


class MLP2LayerAdapter(VisionAdapter):
    def __init__(self, in_dim: int, out_dim: int, hidden_dim: int | None = None, activation: str = "gelu", **_) -> None:
        super().__init__()
        _check_dims("MLP2LayerAdapter", in_dim, out_dim)
        if activation not in _ACT:
            raise ValueError(f"Unknown adapter activation {activation!r}; known: {sorted(_ACT)}")
        hidden = hidden_dim or out_dim
        self.proj1 = nn.Linear(in_dim, hidden)  # parameter names are the checkpoint keys of the reference
        self.act = _ACT[activation]()
        self.proj2 = nn.Linear(hidden, out_dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj2(self.act(self.proj1(x)))


class LinearAdapter(VisionAdapter):
    def __init__(self, in_dim: int, out_dim: int, **_) -> None:
        super().__init__()
        _check_dims("LinearAdapter", in_dim, out_dim)
        self.proj = nn.Linear(in_dim, out_dim)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.proj(x)


def _to_windows(x: torch.Tensor, window: int):
    """(B, N, F) on a square grid -> (B, windows, window*window, F) plus a validity mask for ragged edges."""
    b, n, f = x.shape
    side = math.isqrt(n)
    if side * side != n:
        raise ValueError(f"pooling adapters need a square patch grid (got {n} tokens)")
    out_side = -(-side // window)
    pad = out_side * window - side
    grid = x.reshape(b, side, side, f)
    valid = torch.ones(side, side, dtype=torch.bool, device=x.device)
    if pad:
        grid = torch.nn.functional.pad(grid, (0, 0, 0, pad, 0, pad))
        valid = torch.nn.functional.pad(valid, (0, pad, 0, pad))
    grid = grid.reshape(b, out_side, window, out_side, window, f).permute(0, 1, 3, 2, 4, 5)
    grid = grid.reshape(b, out_side * out_side, window * window, f)
    valid = valid.reshape(out_side, window, out_side, window).permute(0, 2, 1, 3).reshape(out_side * out_side, window * window)
    return grid, valid


class AvgPoolAdapter(VisionAdapter):
    def __init__(self, in_dim: int, out_dim: int, pool_window: int = 2, **_) -> None:
        super().__init__()
        _check_dims("AvgPoolAdapter", in_dim, out_dim)
        if pool_window <= 0:
            raise ValueError(f"pool_window must be positive (got {pool_window})")
        self.window = self.pool_window = pool_window
        self.proj = nn.Linear(in_dim, out_dim)

    def output_num_tokens(self, num_input_tokens: int) -> int:
        return pooled_token_count(num_input_tokens, self.window)

    def forward(self, x: torch.Tensor, pool_window: int | None = None) -> torch.Tensor:
        """``pool_window`` overrides the configured window for this call (the projection is shared)."""
        window = self.window if pool_window is None else pool_window
        if window <= 0:
            raise ValueError(f"pool_window must be positive (got {window})")
        win, valid = _to_windows(x, window)
        w = valid.to(x.dtype)[None, :, :, None]
        pooled = (win * w).sum(dim=2) / w.sum(dim=2).clamp_min(1)
        return self.proj(pooled)


class AttentionalPoolAdapter(VisionAdapter):
    def __init__(self, in_dim: int, out_dim: int, pool_window: int = 2, pool_heads: int = 16, **_) -> None:
        super().__init__()
        _check_dims("AttentionalPoolAdapter", in_dim, out_dim)
        if in_dim % pool_heads:
            raise ValueError(f"feature dim {in_dim} is not divisible by pool_heads {pool_heads}")
        if pool_window <= 0:
            raise ValueError(f"pool_window must be positive (got {pool_window})")
        self.window, self.heads = pool_window, pool_heads
        self.pool_window, self.pool_heads, self.head_dim = pool_window, pool_heads, in_dim // pool_heads
        self.q_proj = nn.Linear(in_dim, in_dim)
        self.k_proj = nn.Linear(in_dim, in_dim)
        self.v_proj = nn.Linear(in_dim, in_dim)
        self.o_proj = nn.Linear(in_dim, in_dim)
        self.out_proj = nn.Linear(in_dim, out_dim)

    def output_num_tokens(self, num_input_tokens: int) -> int:
        return pooled_token_count(num_input_tokens, self.window, require_divisible=True)

    def forward(self, x: torch.Tensor, pool_window: int | None = None) -> torch.Tensor:
        """``pool_window`` overrides the configured window for this call (images 2x2, video 3x3 share the weights)."""
        window = self.window if pool_window is None else pool_window
        if window <= 0:
            raise ValueError(f"pool_window must be positive (got {window})")
        side = math.isqrt(x.shape[1])
        if side % window:
            raise ValueError(f"ragged grid: token grid side {side} is not divisible by pool_window {window}")
        win, _ = _to_windows(x, window)  # (B, W, P, F)
        b, w, p, f = win.shape
        hd = f // self.heads
        q = self.q_proj(win.mean(dim=2)).reshape(b * w, 1, self.heads, hd).transpose(1, 2)
        k = self.k_proj(win).reshape(b * w, p, self.heads, hd).transpose(1, 2)
        v = self.v_proj(win).reshape(b * w, p, self.heads, hd).transpose(1, 2)
        att = torch.nn.functional.scaled_dot_product_attention(q, k, v)  # tiny: P keys per window
        pooled = self.o_proj(att.transpose(1, 2).reshape(b, w, f))
        return self.out_proj(pooled)


registry.register("adapter", "mlp_2layer", MLP2LayerAdapter)
registry.register("adapter", "linear", LinearAdapter)
registry.register("adapter", "avgpool", AvgPoolAdapter)
registry.register("adapter", "attentional_pool", AttentionalPoolAdapter)


def build_adapter(adapter_config, in_dim: int, out_dim: int) -> VisionAdapter:
    return registry.get("adapter", adapter_config.type)(in_dim, out_dim, **adapter_config.extra_kwargs())
