"""``ModalityContext``: the bundle of optional vision-language inputs of ``Transformer.forward``.

Parity: kempnerforge/model/modality.py:35-95 (fields and mutual-exclusion rules).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class ModalityContext:
    inputs_embeds: torch.Tensor | None = None  # replaces the token embedding
    prefix_embeds: torch.Tensor | None = None  # prepended to the token embedding
    output_slice: slice | None = None  # positions whose logits are returned
    image_features: torch.Tensor | None = None  # cross-attention side channel
    image_mask: torch.Tensor | None = None  # validity of image_features positions
    modality_ids: torch.Tensor | None = None  # per-position modality tag (MoT / MoMa)
    key_padding_mask: torch.Tensor | None = None  # validity of residual-stream keys

    def __post_init__(self) -> None:
        routes = [self.inputs_embeds, self.prefix_embeds, self.image_features]
        if sum(r is not None for r in routes) > 1:
            raise ValueError(
                "ModalityContext: inputs_embeds, prefix_embeds and image_features are mutually exclusive (at most one may be set)"
            )
        if self.image_mask is not None and self.image_features is None:
            raise ValueError("ModalityContext: image_mask requires image_features to be set")
        extends_residual = self.prefix_embeds is not None or self.inputs_embeds is not None
        if self.modality_ids is not None and not extends_residual:
            raise ValueError("ModalityContext: modality_ids requires prefix_embeds OR inputs_embeds to be set")
        if self.key_padding_mask is not None and not extends_residual:
            raise ValueError("ModalityContext: key_padding_mask requires prefix_embeds OR inputs_embeds to be set")
