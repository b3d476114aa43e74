"""Token embedding and output head.

Attribute names (``embedding``, ``proj``) fix the checkpoint keys
``token_embedding.embedding.weight`` and ``output_head.proj.weight``.
Parity: kempnerforge/model/embedding.py:9-55.
"""

from __future__ import annotations

import torch
from torch import nn

from kempnerforge_b200.ops import functional as F


class TokenEmbedding(nn.Module):
    def __init__(self, vocab_size: int, dim: int) -> None:
        super().__init__()
        self.embedding = nn.Embedding(vocab_size, dim)

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        return F.embedding(tokens, self.embedding.weight)


class OutputHead(nn.Module):
    def __init__(self, dim: int, vocab_size: int) -> None:
        super().__init__()
        self.proj = nn.Linear(dim, vocab_size, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return F.linear(x, self.proj.weight)

    def tie_weights(self, embedding: TokenEmbedding) -> None:
        """Share the embedding matrix with the projection (one Parameter, two uses)."""
        self.proj.weight = embedding.embedding.weight
