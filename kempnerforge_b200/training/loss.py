"""Losses on (logits, labels): cross entropy, token-chunked cross entropy, z-loss.

``ignore_index`` is -100; when every label is ignored the loss is 0.  The fused head +
loss path (no logits tensor at all) is ``Transformer.compute_loss``; these functions
serve callers that already hold logits (evaluation, vision-language wrappers, hooks).

Parity: kempnerforge/training/loss.py:19-127.
"""

from __future__ import annotations

from collections.abc import Callable

import torch

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.ops import ref

IGNORE_INDEX = ref.IGNORE_INDEX


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    return ref.cross_entropy(logits, labels)


def chunked_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, chunk_size: int = 4096) -> torch.Tensor:
    """Same value as ``cross_entropy``; the fp32 work is done ``chunk_size`` tokens at a time."""
    flat = logits.reshape(-1, logits.shape[-1])
    lab = labels.reshape(-1)
    total = flat.new_zeros((), dtype=torch.float32)
    for lo in range(0, flat.shape[0], max(1, chunk_size)):
        nll, _, _ = ref.cross_entropy_parts(flat[lo : lo + chunk_size], lab[lo : lo + chunk_size])
        total = total + nll
    return total / (lab != IGNORE_INDEX).sum().clamp_min(1).float()


cross_entropy_loss = cross_entropy
chunked_cross_entropy_loss = chunked_cross_entropy


def z_loss(logits: torch.Tensor, weight: float = 1e-4) -> torch.Tensor:
    """weight * mean(logsumexp(logits)^2) over all positions."""
    return weight * torch.logsumexp(logits.float(), dim=-1).pow(2).mean()


registry.register("loss", "cross_entropy", cross_entropy)
registry.register("loss", "chunked_cross_entropy", chunked_cross_entropy)


def build_loss_fn(config) -> Callable[[torch.Tensor, torch.Tensor], torch.Tensor]:
    name = config.loss_fn
    base = registry.get("loss", name)
    if name == "chunked_cross_entropy":
        chunk = config.ce_chunk_size or 4096
        inner = base
        base = lambda lg, lb: inner(lg, lb, chunk_size=chunk)  # noqa: E731
    zw = config.z_loss_weight
    if zw > 0:
        return lambda lg, lb: base(lg, lb) + z_loss(lg, zw)
    return base
