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


class _GroupedSwiGLUFn(torch.autograd.Function):
    """silu(x @ Wg_e) * (x @ Wu_e) over ragged expert rows: one grouped GEMM with the activation in its epilogue
    forward; backward = one ragged SwiGLU-gradient kernel, two input-gradient grouped GEMMs (the second accumulating
    into the first's output) and two ragged weight-gradient reductions over the strided halves of d[gate | up].
    Nothing reads a row count on the host: buffers may be sized by an upper bound, ``offsets`` bounds the work."""

    @staticmethod
    def forward(ctx, x, wg, wu, offsets, layout):
        kc = _cuda_binding
        h, gu = kc.grouped_swiglu(x, wg, wu, offsets, b_mn=(layout == "kn"), want_gu=True)
        ctx.save_for_backward(x, wg, wu, offsets, gu)
        ctx.layout = layout
        return h

    @staticmethod
    def backward(ctx, dh):
        kc = _cuda_binding
        x, wg, wu, offsets, gu = ctx.saved_tensors
        layout = ctx.layout
        f = dh.shape[1]
        dgu = kc.swiglu_bwd_ragged(dh.contiguous(), gu, offsets)
        dgate, dup = dgu[:, :f], dgu[:, f:]
        dx = dwg = dwu = None
        if ctx.needs_input_grad[0]:
            dx = kc.grouped_gemm(dgate, wg, offsets, b_mn=(layout == "nk"))
            kc.grouped_gemm(dup, wu, offsets, b_mn=(layout == "nk"), out=dx, accumulate=True)
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            def wgrad(d):
                a, b = (x, d) if layout == "kn" else (d, x)
                if kc.grouped_wgrad_supported(a, b):
                    return kc.grouped_wgrad(a, b, offsets)
                return torch._grouped_mm(a.contiguous().t(), b.contiguous(), offs=offsets[1:])
            dwg, dwu = wgrad(dgate), wgrad(dup)
        return dx, dwg, dwu, None, None


class _GroupedFFNFn(torch.autograd.Function):
    """The whole expert feed-forward, down(silu(x @ Wg_e) * (x @ Wu_e)), over ragged expert rows as one node.

    Forward: the gate / up grouped GEMM with the SwiGLU epilogue, then the down projection.  Backward: the down
    projection's input-gradient product with the SwiGLU gradient in its epilogue (the gradient of the hidden
    activation never reaches memory; d[gate | up] overwrites the saved pre-activations), two input-gradient grouped
    GEMMs (the second accumulating into the first's output) and three ragged weight-gradient reductions."""

    @staticmethod
    def forward(ctx, x, wg, wu, wd, offsets, layout):
        kc = _cuda_binding
        kn = layout == "kn"
        h, gu = kc.grouped_swiglu(x, wg, wu, offsets, b_mn=kn, want_gu=True)
        y = kc.grouped_gemm(h, wd, offsets, b_mn=kn)
        ctx.save_for_backward(x, wg, wu, wd, offsets, gu, h)
        ctx.layout = layout
        return y

    @staticmethod
    def backward(ctx, dy):
        kc = _cuda_binding
        x, wg, wu, wd, offsets, gu, h = ctx.saved_tensors
        layout = ctx.layout
        kn = layout == "kn"
        f = h.shape[1]
        if not dy.is_contiguous():
            dy = dy.contiguous()

        def wgrad(a, b):   # per-expert a_e^T b_e in the weight's own layout
            a, b = (a, b) if kn else (b, a)
            if kc.grouped_wgrad_supported(a, b):
                return kc.grouped_wgrad(a, b, offsets)
            return torch._grouped_mm(a.contiguous().t(), b.contiguous(), offs=offsets[1:])

        dwd = wgrad(h, dy) if ctx.needs_input_grad[3] else None
        # dh = dy @ Wd_e^T: 'kn' stores Wd_e as (F, D), read with the reduction index D contiguous
        dgu = kc.grouped_swiglu_bwd(dy, wd, gu, offsets, b_mn=not kn)   # gu is dead after this; reuse its storage
        dgate, dup = dgu[:, :f], dgu[:, f:]
        dx = dwg = dwu = None
        if ctx.needs_input_grad[0]:
            dx = kc.grouped_gemm(dgate, wg, offsets, b_mn=not kn)
            kc.grouped_gemm(dup, wu, offsets, b_mn=not kn, out=dx, accumulate=True)
        if ctx.needs_input_grad[1] or ctx.needs_input_grad[2]:
            dwg, dwu = wgrad(x, dgate), wgrad(x, dup)
        return dx, dwg, dwu, dwd, None, None


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


def offsets_of(counts: torch.Tensor) -> torch.Tensor:
    off = torch.zeros(counts.numel() + 1, dtype=torch.int32, device=counts.device)
    off[1:] = counts.cumsum(0)
    return off


def grouped_ffn(x_sorted, counts, gate_w, up_w, down_w, layout: str, activation=None, offsets=None) -> torch.Tensor:
    """Expert feed-forward over expert-sorted rows: SwiGLU when ``gate_w`` is given, else act(up) -> down.
    ``offsets`` (int32 (E + 1) on the device) may be passed instead of being derived from ``counts``; ``x_sorted`` may
    then have more rows than ``offsets[-1]`` (the extra rows are ignored)."""
    if (gate_w is not None and _native_ok(x_sorted, up_w, layout) and _native_ok(x_sorted, gate_w, layout)
            and _cuda_binding.grouped_swiglu_supported(x_sorted, gate_w, layout == "kn")):
        f = up_w.shape[2] if layout == "kn" else up_w.shape[1]
        down_ok = down_w.dim() == 3 and down_w.is_contiguous() and _cuda_binding.grouped_gemm_supported(
            torch.empty((0, f), dtype=x_sorted.dtype, device=x_sorted.device), down_w, layout == "kn")
        if down_ok and (layout != "nk" or (down_w.shape[1] % 64 == 0)):
            off = offsets if offsets is not None else offsets_of(counts)
            xs = x_sorted if x_sorted.is_contiguous() else x_sorted.contiguous()
            # the output gradient has the shape of the input (dim -> hidden -> dim)
            if _cuda_binding.grouped_swiglu_bwd_supported(xs, down_w, layout != "kn"):
                return _GroupedFFNFn.apply(xs, gate_w, up_w, down_w, off, layout)
            hidden = _GroupedSwiGLUFn.apply(xs, gate_w, up_w, off, layout)
            return _GroupedLinearFn.apply(hidden, down_w, off, layout)
    up = grouped_linear(x_sorted, up_w, counts, layout)
    if gate_w is not None:
        hidden = F.silu(grouped_linear(x_sorted, gate_w, counts, layout)) * up
    else:
        hidden = activation(up)
    return grouped_linear(hidden, down_w, counts, layout)
