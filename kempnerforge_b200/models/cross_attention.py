"""Cross-attention blocks for the ``cross_attention`` vision-language architecture.

Text hidden states query image features (keys / values); no rotary embedding, no causal mask.  The block's two
output projections (``attn.o_proj`` and ``mlp.down_proj``) start at zero, so a freshly inserted block is the
identity and a text-only checkpoint keeps its behaviour.  ``image_mask`` marks valid image positions; a sample
whose mask is empty attends to everything instead of producing NaNs.

Parity: kempnerforge/model/cross_attention.py:36-156 (module names ``attn_norm`` / ``attn`` / ``mlp_norm`` / ``mlp``).
"""

from __future__ import annotations

import torch
from torch import nn

from kempnerforge_b200.models.mlp import build_mlp
from kempnerforge_b200.models.norm import build_norm
from kempnerforge_b200.ops import functional as F
from kempnerforge_b200.ops import ref


class CrossAttention(nn.Module):
    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, head_dim: int | None = None) -> None:
        super().__init__()
        self.n_heads, self.n_kv_heads = n_heads, n_kv_heads
        self.head_dim = head_dim or dim // n_heads
        self.n_rep = n_heads // n_kv_heads
        hd = self.head_dim
        self.q_proj = nn.Linear(dim, n_heads * hd, bias=False)
        self.k_proj = nn.Linear(dim, n_kv_heads * hd, bias=False)
        self.v_proj = nn.Linear(dim, n_kv_heads * hd, bias=False)
        self.o_proj = nn.Linear(n_heads * hd, dim, bias=False)
        self.o_proj.weight._kf_zero_init = True
        nn.init.zeros_(self.o_proj.weight)

    def forward(self, x: torch.Tensor, image_features: torch.Tensor, image_mask: torch.Tensor | None = None) -> torch.Tensor:
        b, s, _ = x.shape
        n = image_features.shape[1]
        hd = self.head_dim
        q = F.linear(x, self.q_proj.weight).view(b, s, -1, hd)
        kv = F.fused_linear(image_features, [self.k_proj.weight, self.v_proj.weight]).view(b, n, -1, hd)
        hkv = kv.shape[2] // 2
        k, v = kv[:, :, :hkv], kv[:, :, hkv:]
        if image_mask is None:
            out = F.attention(q, k, v, causal=False)
        else:
            out = ref.attention(q, k, v, causal=False, key_padding_mask=image_mask)
        return F.linear(out.reshape(b, s, -1), self.o_proj.weight)


class CrossAttentionBlock(nn.Module):
    """Two ways to build one: from a model config (``CrossAttentionBlock(config, n_heads=, n_kv_heads=)``) or from loose
    dimensions as in the reference (``CrossAttentionBlock(dim=, n_heads=, n_kv_heads=, ffn_hidden_dim=, norm_type=,
    activation=)``)."""

    def __init__(self, config=None, n_heads: int | None = None, n_kv_heads: int | None = None, ffn_hidden_dim: int | None = None,
                 norm_type: str = "rmsnorm", activation: str = "silu", *, dim: int | None = None) -> None:
        super().__init__()
        if config is None or isinstance(config, int):          # loose dimensions
            dim = dim if dim is not None else config
            if dim is None or n_heads is None or ffn_hidden_dim is None:
                raise TypeError("CrossAttentionBlock needs a model config, or dim, n_heads and ffn_hidden_dim")
            eps, hidden = 1e-5, ffn_hidden_dim
        else:
            dim, norm_type, activation, eps = config.dim, config.norm_type, config.activation, config.norm_eps
            n_heads = n_heads or config.n_heads
            hidden = ffn_hidden_dim or config.computed_ffn_hidden_dim
        n_kv_heads = n_kv_heads or n_heads
        self.attn_norm = build_norm(norm_type, dim, eps)
        self.attn = CrossAttention(dim, n_heads, n_kv_heads)
        self.mlp_norm = build_norm(norm_type, dim, eps)
        self.mlp = build_mlp(dim, hidden, activation)
        self.mlp.down_proj.weight._kf_zero_init = True
        nn.init.zeros_(self.mlp.down_proj.weight)

    def forward(self, x: torch.Tensor, image_features: torch.Tensor, image_mask: torch.Tensor | None = None) -> torch.Tensor:
        x = x + self.attn(self.attn_norm(x), image_features, image_mask)
        return x + self.mlp(self.mlp_norm(x))
