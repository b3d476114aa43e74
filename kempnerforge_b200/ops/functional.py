"""Differentiable front-ends of the hot ops.

Every function takes ordinary tensors.  CUDA tensors in bf16 go to the
hand-written sm_100a kernels (``kempnerforge_b200.ops.cuda``); everything else
(CPU, fp32 debugging, exotic shapes) runs the PyTorch formulas of
``kempnerforge_b200.ops.ref``.  There is no silent downgrade on a GPU: if the
native library is missing, importing the CUDA binding raises.

Weights that belong to a flat parameter group carry ``_kf_grad`` (a view into
the group's flat gradient buffer).  For those, the weight-gradient GEMM writes
(or accumulates) straight into that view and autograd receives ``None`` —
the optimizer and the reduce-scatter read the flat buffer directly.
"""

from __future__ import annotations

import math

import torch

from kempnerforge_b200.ops import ref

_cuda_mod = None


def _cuda():
    global _cuda_mod
    if _cuda_mod is None:
        from kempnerforge_b200.ops import cuda as _m

        _cuda_mod = _m
    return _cuda_mod


def use_native(*tensors: torch.Tensor) -> bool:
    """True when the native kernels handle these tensors (CUDA + bf16)."""
    t = tensors[0]
    return t.is_cuda and t.dtype == torch.bfloat16 and not _FORCE_REF


_FORCE_REF = False


class force_reference:
    """Context manager that routes CUDA tensors through the PyTorch formulas (tests / debugging)."""

    def __enter__(self):
        global _FORCE_REF
        self._old, _FORCE_REF = _FORCE_REF, True

    def __exit__(self, *exc):
        global _FORCE_REF
        _FORCE_REF = self._old


# --------------------------------------------------------------------------- flat-gradient plumbing
def _deposit_weight_grad(weight: torch.Tensor, compute, shape):
    """Run ``compute(out, accumulate)`` into the weight's flat-gradient view if it has one.

    Returns the tensor autograd should see (None when the flat buffer took it).
    """
    slot = getattr(weight, "_kf_grad", None)
    if slot is None:
        out = torch.empty(shape, dtype=weight.dtype, device=weight.device)
        compute(out, False)
        return out
    live = getattr(weight, "_kf_grad_live", False)
    compute(slot, live)
    weight._kf_grad_live = True
    return None


# --------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
    """y = x @ Wᵀ for one weight or for several weights stacked along the output dim."""

    @staticmethod
    def forward(ctx, x, *weights):
        cu = _cuda()
        w = cu.stack_rows(weights)
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = cu.gemm(x2, w, a_kmajor=True, b_kmajor=True)
        ctx.save_for_backward(x2, *weights)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        cu = _cuda()
        x2, *weights = ctx.saved_tensors
        w = cu.stack_rows(weights)
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = cu.gemm(dy2, w, a_kmajor=True, b_kmajor=False).view(ctx.x_shape)
        wgrads = _linear_weight_grads(cu, dy2, x2, weights, ctx.needs_input_grad[1:])
        return (dx, *wgrads)


def _linear_weight_grads(cu, dy2, x2, weights, needs):
    if not any(needs):
        return [None] * len(weights)
    slots = [getattr(w, "_kf_grad", None) for w in weights]
    fused_slot = cu.stack_rows(slots) if all(s is not None for s in slots) and cu.rows_adjacent(slots) else None
    if fused_slot is not None and all(needs):
        live = [getattr(w, "_kf_grad_live", False) for w in weights]
        if all(live) or not any(live):
            cu.gemm(dy2, x2, a_kmajor=False, b_kmajor=False, out=fused_slot, accumulate=live[0])
            for w in weights:
                w._kf_grad_live = True
            return [None] * len(weights)
    # generic: one GEMM over the stacked rows, then hand out row blocks
    total = sum(w.shape[0] for w in weights)
    dw = cu.gemm(dy2, x2, a_kmajor=False, b_kmajor=False)
    out, row = [], 0
    for w, need, slot in zip(weights, needs, slots):
        piece = dw[row : row + w.shape[0]]
        row += w.shape[0]
        if not need:
            out.append(None)
        elif slot is not None:
            if getattr(w, "_kf_grad_live", False):
                slot.add_(piece)
            else:
                slot.copy_(piece)
                w._kf_grad_live = True
            out.append(None)
        else:
            out.append(piece)
    assert row == total
    return out


def _stack_weight_rows(weights) -> torch.Tensor:
    """The weights as one (sum(out_i), in) matrix: a zero-copy view when they are adjacent rows of a flat
    buffer on the GPU, a concatenation otherwise."""
    if len(weights) == 1:
        return weights[0]
    if weights[0].is_cuda:
        return _cuda().stack_rows(weights)
    return torch.cat(list(weights), dim=0)


def _deposit_stacked_weight_grads(weights, needs, compute):
    """Run ``compute(out, accumulate)`` for the stacked weight gradient and hand the row blocks to the flat
    gradient buffers (or to autograd when a weight has none)."""
    slots = [getattr(w, "_kf_grad", None) for w in weights]
    if all(needs) and all(s is not None for s in slots) and weights[0].is_cuda and _cuda().rows_adjacent(slots):
        live = [getattr(w, "_kf_grad_live", False) for w in weights]
        if all(live) or not any(live):
            compute(_cuda().stack_rows(slots), live[0])
            for w in weights:
                w._kf_grad_live = True
            return [None] * len(weights)
    total = sum(w.shape[0] for w in weights)
    dw = torch.empty(total, weights[0].shape[1], dtype=weights[0].dtype, device=weights[0].device)
    compute(dw, False)
    out, row = [], 0
    for w, need, slot in zip(weights, needs, slots):
        piece = dw[row : row + w.shape[0]]
        row += w.shape[0]
        if not need:
            out.append(None)
        elif slot is not None:
            if getattr(w, "_kf_grad_live", False):
                slot.add_(piece)
            else:
                slot.copy_(piece)
                w._kf_grad_live = True
            out.append(None)
        else:
            out.append(piece)
    return out


def _fp8_route(x: torch.Tensor, weights) -> bool:
    if not getattr(weights[0], "_kf_fp8", False):
        return False
    from kempnerforge_b200.ops import fp8

    return (x.is_cuda or x.dtype == torch.bfloat16) and fp8.supported(x, list(weights))


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    if _fp8_route(x, [weight]):
        from kempnerforge_b200.ops import fp8

        y = fp8.linear(x, [weight])
        return y if bias is None else y + bias
    if use_native(x) and weight.dtype == torch.bfloat16 and _gemm_friendly(x, weight):
        y = _LinearFn.apply(x, weight)
        return y if bias is None else y + bias
    return torch.nn.functional.linear(x, weight, bias)


def fused_linear(x: torch.Tensor, weights: list[torch.Tensor]) -> torch.Tensor:
    """One GEMM against several (out_i, in) weights; output columns are [out_0 | out_1 | ...]."""
    if _fp8_route(x, weights):
        from kempnerforge_b200.ops import fp8

        return fp8.linear(x, list(weights))
    if use_native(x) and all(w.dtype == torch.bfloat16 for w in weights) and all(
        _gemm_friendly(x, w) for w in weights
    ):
        return _LinearFn.apply(x, *weights)
    return torch.cat([torch.nn.functional.linear(x, w) for w in weights], dim=-1)


def _gemm_friendly(x: torch.Tensor, w: torch.Tensor) -> bool:
    # TMA needs 16-byte aligned row pitches: in/out features multiples of 8 bf16 elements
    return w.dim() == 2 and w.shape[1] % 8 == 0 and w.shape[0] % 8 == 0 and x.shape[-1] == w.shape[1]


# --------------------------------------------------------------------------- rmsnorm
class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        cu = _cuda()
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y, rstd = cu.rmsnorm_fwd(x2, weight, eps)
        ctx.save_for_backward(x2, weight, rstd)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        cu = _cuda()
        x2, weight, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx, dw = cu.rmsnorm_bwd(dy2, x2, weight, rstd)
        slot = getattr(weight, "_kf_grad", None)
        if slot is not None:
            if getattr(weight, "_kf_grad_live", False):
                slot.add_(dw)
            else:
                slot.copy_(dw)
                weight._kf_grad_live = True
            dw = None
        else:
            dw = dw.to(weight.dtype)
        return dx.view(dy.shape), dw, None


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    if use_native(x) and weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, weight, eps)
    return ref.rmsnorm(x, weight, eps)


# --------------------------------------------------------------------------- rope
class _RopeFn(torch.autograd.Function):
    """Half-split rotation of the first ``n_rot_heads`` heads of a (B, S, Htot, hd) tensor (out of place)."""

    @staticmethod
    def forward(ctx, x, cos, sin, n_rot_heads):
        cu = _cuda()
        ctx.save_for_backward(cos, sin)
        ctx.n_rot = n_rot_heads
        return cu.rope(x, cos, sin, n_rot_heads, inverse=False)

    @staticmethod
    def backward(ctx, dy):
        cu = _cuda()
        cos, sin = ctx.saved_tensors
        if not dy.is_contiguous():
            dy = dy.contiguous()
        return cu.rope(dy, cos, sin, ctx.n_rot, inverse=True), None, None, None


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int | None = None):
    """Rotate heads [0, n_rot_heads) of x (B, S, H, hd); the remaining heads pass through."""
    n_heads = x.shape[2]
    n_rot = n_heads if n_rot_heads is None else n_rot_heads
    if use_native(x) and cos.dim() == 2 and x.is_contiguous() and x.shape[-1] % 16 == 0:
        return _RopeFn.apply(x, cos.contiguous(), sin.contiguous(), n_rot)
    if n_rot == n_heads:
        return ref.apply_rope(x, cos, sin)
    return torch.cat([ref.apply_rope(x[:, :, :n_rot], cos, sin), x[:, :, n_rot:]], dim=2)


# --------------------------------------------------------------------------- attention
class _FlashAttnFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, doc_ids, scale):
        cu = _cuda()
        out, lse = cu.attn_fwd(q, k, v, causal, doc_ids, scale)
        ctx.save_for_backward(q, k, v, out, lse, doc_ids if doc_ids is not None else torch.empty(0))
        ctx.causal, ctx.scale, ctx.has_doc = causal, scale, doc_ids is not None
        return out

    @staticmethod
    def backward(ctx, dout):
        cu = _cuda()
        q, k, v, out, lse, doc = ctx.saved_tensors
        dq, dk, dv = cu.attn_bwd(
            dout, q, k, v, out, lse, ctx.causal, doc if ctx.has_doc else None, ctx.scale
        )
        return dq, dk, dv, None, None, None


def attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    causal: bool = True,
    doc_ids: torch.Tensor | None = None,
    key_padding_mask: torch.Tensor | None = None,
    scale: float | None = None,
) -> torch.Tensor:
    """q (B, Sq, H, hd), k/v (B, Sk, Hkv, hd) -> (B, Sq, H, hd); grouped KV heads are never expanded."""
    hd = q.shape[-1]
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    if use_native(q) and key_padding_mask is None:
        cu = _cuda()
        needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
        policy = cu.attn_policy()
        want = policy == "native" or (policy == "auto" and (not needs_grad or doc_ids is not None))
        if want and (doc_ids is None or q.shape[1] == k.shape[1]) and cu.attn_supported(q, k, v, causal, needs_grad):
            if not needs_grad:
                return cu.attn_fwd(q, k, v, causal, doc_ids, scale)[0]
            return _FlashAttnFn.apply(q, k, v, causal, doc_ids, scale)
    if q.is_cuda and doc_ids is None and key_padding_mask is None and q.dtype != torch.float32:
        # library attention for shapes the native kernel does not cover
        out = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
            is_causal=causal and q.shape[1] > 1, scale=scale, enable_gqa=k.shape[2] != q.shape[2],
        )
        return out.transpose(1, 2)
    return ref.attention(q, k, v, causal, doc_ids, key_padding_mask, scale)


# --------------------------------------------------------------------------- swiglu
class _SwiGLUFn(torch.autograd.Function):
    """h = silu(gu[:, :H]) * gu[:, H:] for a stacked (T, 2H) gate|up tensor."""

    @staticmethod
    def forward(ctx, gu):
        cu = _cuda()
        ctx.save_for_backward(gu)
        return cu.swiglu_fwd(gu)

    @staticmethod
    def backward(ctx, dh):
        cu = _cuda()
        (gu,) = ctx.saved_tensors
        if not dh.is_contiguous():
            dh = dh.contiguous()
        return cu.swiglu_bwd(dh, gu)


def swiglu_stacked(gu: torch.Tensor) -> torch.Tensor:
    """gu (..., 2H) holding [gate | up] -> silu(gate) * up of shape (..., H)."""
    h = gu.shape[-1] // 2
    if use_native(gu) and gu.is_contiguous() and h % 8 == 0:
        return _SwiGLUFn.apply(gu)
    return ref.swiglu(gu[..., :h], gu[..., h:])


# --------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        cu = _cuda()
        ctx.save_for_backward(ids)
        ctx.table = table
        return cu.embedding_fwd(ids, table)

    @staticmethod
    def backward(ctx, dy):
        cu = _cuda()
        (ids,) = ctx.saved_tensors
        table = ctx.table
        if not dy.is_contiguous():
            dy = dy.contiguous()

        def compute(out, accumulate):
            cu.embedding_bwd(dy, ids, out, accumulate)

        return None, _deposit_weight_grad(table, compute, table.shape)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    if use_native(table) and table.shape[1] % 8 == 0:
        return _EmbeddingFn.apply(ids, table)
    return torch.nn.functional.embedding(ids, table)


# --------------------------------------------------------------------------- head + cross entropy
class _LinearCrossEntropyFn(torch.autograd.Function):
    """Output head GEMM fused with cross entropy, token-chunked so (T, V) logits never exist.

    Forward computes, chunk by chunk, logits = h Wᵀ, the per-token logsumexp and
    picked logit, and immediately the logits gradient (softmax - onehot, plus the
    z-loss term) which feeds the dgrad and wgrad GEMMs of that chunk; the
    gradients are for an upstream factor of one.  Backward multiplies them by the
    incoming scalar and deposits the weight gradient.
    """

    @staticmethod
    def forward(ctx, h, weight, labels, z_weight, chunk):
        cu = _cuda()
        h2 = h.reshape(-1, h.shape[-1])
        if not h2.is_contiguous():
            h2 = h2.contiguous()
        lab = labels.reshape(-1).contiguous()
        t = h2.shape[0]
        inv_n = torch.reciprocal((lab != ref.IGNORE_INDEX).sum().clamp_min(1).float())
        stats = torch.zeros(2, dtype=torch.float32, device=h.device)  # [sum nll, sum lse^2]
        dh = torch.empty_like(h2)
        dw = torch.empty_like(weight)
        for lo in range(0, t, chunk):
            hi = min(t, lo + chunk)
            logits = cu.gemm(h2[lo:hi], weight, a_kmajor=True, b_kmajor=True)
            # in place: logits <- d(loss)/dlogits ; stats accumulate
            cu.ce_fwd_bwd(logits, lab[lo:hi], stats, inv_n, z_weight)
            cu.gemm(logits, weight, a_kmajor=True, b_kmajor=False, out=dh[lo:hi])
            cu.gemm(logits, h2[lo:hi], a_kmajor=False, b_kmajor=False, out=dw, accumulate=lo > 0)
        ctx.save_for_backward(dh, dw)
        ctx.h_shape = h.shape
        ctx.weight = weight
        return (stats[0] + z_weight * stats[1]) * inv_n

    @staticmethod
    def backward(ctx, dloss):
        dh, dw = ctx.saved_tensors
        factor = dloss.to(dh.dtype)
        dh = dh.mul_(factor).view(ctx.h_shape)

        def compute(out, accumulate):
            if accumulate:
                out.addcmul_(dw, factor)
            else:
                torch.mul(dw, factor, out=out)

        return dh, _deposit_weight_grad(ctx.weight, compute, dw.shape), None, None, None


def linear_cross_entropy(
    h: torch.Tensor,
    weight: torch.Tensor,
    labels: torch.Tensor,
    z_loss_weight: float = 0.0,
    chunk_tokens: int = 4096,
) -> torch.Tensor:
    """Mean cross entropy of (h @ weightᵀ) against labels (+ z-loss), without materialising all logits."""
    if (
        use_native(h)
        and weight.dtype == torch.bfloat16
        and _gemm_friendly(h, weight)
        and torch.is_grad_enabled()
    ):
        return _LinearCrossEntropyFn.apply(h, weight, labels, float(z_loss_weight), int(chunk_tokens))
    h2 = h.reshape(-1, h.shape[-1])
    lab = labels.reshape(-1)
    total_nll = h2.new_zeros((), dtype=torch.float32)
    total_z = h2.new_zeros((), dtype=torch.float32)
    for lo in range(0, h2.shape[0], chunk_tokens):
        logits = linear(h2[lo : lo + chunk_tokens], weight)
        nll, z, _ = ref.cross_entropy_parts(logits, lab[lo : lo + chunk_tokens])
        total_nll = total_nll + nll
        total_z = total_z + z
    n = (lab != ref.IGNORE_INDEX).sum().clamp_min(1).float()
    loss = total_nll / n
    if z_loss_weight:
        loss = loss + z_loss_weight * total_z / n
    return loss
