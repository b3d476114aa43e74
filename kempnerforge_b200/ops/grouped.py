"""Ragged grouped GEMMs for mixture-of-experts layers.

Rows of the activation matrix are grouped by expert; ``counts[e]`` consecutive
rows belong to expert ``e``.  On CUDA the segment boundaries stay on the device
(no ``.tolist()``), on CPU a plain loop over experts runs.

Parity: replaces the padded ``torch._grouped_mm`` path and the Python
pack/unpack loops of kempnerforge/model/moe.py:20-145.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from kempnerforge_b200.ops import cuda as _cuda_binding


def stack_expert_weights(weights: list[torch.Tensor]) -> torch.Tensor:
    """(E, out, in) over per-expert Linear weights: a view when they are adjacent in one buffer."""
    if len(weights) > 1 and all(w.is_cuda for w in weights) and _cuda_binding.rows_adjacent(weights):
        first = weights[0]
        e = len(weights)
        view = torch.as_strided(first, (e, *first.shape), (first.numel(), *first.stride()))
        if not torch.is_grad_enabled() or not any(w.requires_grad for w in weights):
            return view
    return torch.stack(weights)


def grouped_linear(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, layout: str) -> torch.Tensor:
    """y[rows of expert e] = x[rows of expert e] @ W_e, W_e = w[e] ('kn': (in, out)) or w[e].T ('nk')."""
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and hasattr(torch, "_grouped_mm"):
        offs = counts.cumsum(0).to(torch.int32)
        wb = w if layout == "kn" else w.transpose(1, 2)
        if x.shape[1] % 8 == 0 and wb.shape[2] % 8 == 0:
            return torch._grouped_mm(x, wb, offs=offs)
    out = x.new_empty(x.shape[0], w.shape[2] if layout == "kn" else w.shape[1])
    start = 0
    for e, n in enumerate(counts.tolist()):
        if n:
            we = w[e] if layout == "kn" else w[e].t()
            out[start : start + n] = x[start : start + n] @ we
        start += n
    if start < x.shape[0]:
        out[start:] = 0
    return out


def grouped_ffn(x_sorted, counts, gate_w, up_w, down_w, layout: str, activation=None) -> torch.Tensor:
    """Expert feed-forward over expert-sorted rows: SwiGLU when ``gate_w`` is given, else act(up) -> down."""
    up = grouped_linear(x_sorted, up_w, counts, layout)
    if gate_w is not None:
        hidden = F.silu(grouped_linear(x_sorted, gate_w, counts, layout)) * up
    else:
        hidden = activation(up)
    return grouped_linear(hidden, down_w, counts, layout)
