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


class _GroupedLinearFn(torch.autograd.Function):
    """Ragged grouped Linear on the tcgen05 grouped GEMMs: forward, input gradient and weight gradient (a reduction
    over each expert's ragged token range, its tail rows masked inside the kernel)."""

    @staticmethod
    def forward(ctx, x, w, offsets, layout):
        kc = _cuda_binding
        ctx.save_for_backward(x, w, offsets)
        ctx.layout = layout
        return kc.grouped_gemm(x, w, offsets, b_mn=(layout == "kn"))

    @staticmethod
    def backward(ctx, dy):
        kc = _cuda_binding
        x, w, offsets = ctx.saved_tensors
        layout = ctx.layout
        if not dy.is_contiguous():
            dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # 'nk': W_e is (N, K): dx = dy @ W_e reads W with the output dim (K) contiguous; 'kn': W_e is (K, N): dx = dy @ W_e^T
            dx = kc.grouped_gemm(dy, w, offsets, b_mn=(layout == "nk"))
        if ctx.needs_input_grad[1]:
            a, b = (x, dy) if layout == "kn" else (dy, x)         # (E, K, N) or (E, N, K)
            if kc.grouped_wgrad_supported(a, b):
                dw = kc.grouped_wgrad(a, b, offsets)
            else:
                dw = torch._grouped_mm(a.t(), b, offs=offsets[1:])
        return dx, dw, None, None


def _native_ok(x: torch.Tensor, w: torch.Tensor, layout: str) -> bool:
    from kempnerforge_b200.ops import functional as _F

    if _F._FORCE_REF or not (x.is_cuda and x.dtype == torch.bfloat16 and w.dim() == 3 and w.is_contiguous()):
        return False
    kc = _cuda_binding
    fwd_mn, bwd_mn = layout == "kn", layout == "nk"
    n = w.shape[2] if fwd_mn else w.shape[1]
    # the input-gradient GEMM reduces over n: its MN-major form needs n % 64
    return (kc.available() and kc.grouped_gemm_supported(x, w, fwd_mn) and (not bwd_mn or n % 64 == 0)
            and hasattr(torch, "_grouped_mm"))


def grouped_linear(x: torch.Tensor, w: torch.Tensor, counts: torch.Tensor, layout: str) -> torch.Tensor:
    """y[rows of expert e] = x[rows of expert e] @ W_e, W_e = w[e] ('kn': (in, out)) or w[e].T ('nk')."""
    if _native_ok(x, w, layout):
        offsets = torch.zeros(counts.numel() + 1, dtype=torch.int32, device=x.device)
        offsets[1:] = counts.cumsum(0)
        return _GroupedLinearFn.apply(x if x.is_contiguous() else x.contiguous(), w, offsets, layout)
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
