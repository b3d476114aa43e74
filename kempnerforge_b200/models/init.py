"""Weight initialisation.

Every parameter with two or more dimensions is drawn from N(0, init_std);
residual-branch output projections (``o_proj``, ``down_proj`` and the packed
``down_w``) use init_std / sqrt(2 * n_layers); one-dimensional parameters keep
their constructor values (norm weights 1, router bias 0).  Cross-attention and
MoT output projections that must start as identity branches are zeroed.

Parity: kempnerforge/model/init.py:26-63.  Deviation: the packed expert
``down_w`` is scaled like the unpacked ``experts.j.down_proj.weight`` so packed
and unpacked models are initialised the same way.
"""

from __future__ import annotations

import math

import torch
from torch import nn

_RESIDUAL_SUFFIXES = ("o_proj.weight", "down_proj.weight", "down_w")


def init_weights(model: nn.Module, n_layers, init_std: float = 0.02) -> None:
    """``n_layers`` is the layer count, or a model config carrying ``n_layers`` and ``init_std``."""
    if not isinstance(n_layers, int):
        n_layers, init_std = n_layers.n_layers, getattr(n_layers, "init_std", init_std)
    scaled = init_std / math.sqrt(2 * max(1, n_layers))
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() < 2:
                continue
            if getattr(p, "_kf_zero_init", False):
                p.zero_()
                continue
            std = scaled if name.endswith(_RESIDUAL_SUFFIXES) else init_std
            p.normal_(mean=0.0, std=std)
