"""Autograd wrappers of the native mixture-of-experts kernels: fused router, stable sort by expert, row gather and
weighted combine.  Every piece stays on the device; the router's backward is a handful of element-wise PyTorch ops
on the (tokens, experts) score matrix, everything else has a native backward.

Parity: kempnerforge/model/router.py:45-72,157-200 and kempnerforge/model/moe.py:256-349 (same mathematics: softmax
or sigmoid(+bias) scores, top-k, renormalised weights, Switch load-balancing loss E * sum(f_e * P_e), z-loss
mean(logsumexp²), sort by expert, weighted sum over the k expert outputs).
"""

from __future__ import annotations

import torch

from kempnerforge_b200.ops import cuda as kc


def native_ok(x: torch.Tensor, num_experts: int, top_k: int) -> bool:
    from kempnerforge_b200.ops import functional as F

    if F._FORCE_REF:
        return False
    return (x.is_cuda and kc.available() and getattr(kc.lib(), "kf_router_topk", None) is not None
            and num_experts <= 256 and top_k <= 8 and top_k <= num_experts)


class _RouterFn(torch.autograd.Function):
    """(weights, indices, counts, score_mean, z_loss) from logits.  ``score_mean`` (mean score per expert) and
    ``z_loss`` are differentiable, like ``weights``; ``indices`` and ``counts`` are not."""

    @staticmethod
    def forward(ctx, logits, bias, sigmoid, k):
        logits = logits.contiguous()
        w, idx, counts, prob_sum, lse_sq = kc.router_topk(logits, bias, sigmoid, k)
        t = logits.shape[0]
        # the sigmoid router nudges its bias in place right after routing: keep a private copy for the backward
        ctx.save_for_backward(logits, bias.detach().clone() if bias is not None else torch.empty(0), idx, w)
        ctx.sigmoid, ctx.has_bias = sigmoid, bias is not None
        ctx.mark_non_differentiable(idx, counts)
        return w, idx, counts, prob_sum / t, lse_sq.reshape(()) / t

    @staticmethod
    def backward(ctx, dw, _didx, _dcounts, dmean, dz):
        logits, bias, idx, w = ctx.saved_tensors
        lf = logits.float()
        t = lf.shape[0]
        if ctx.sigmoid:
            scores = torch.sigmoid(lf + bias.float()) if ctx.has_bias else torch.sigmoid(lf)
        else:
            scores = torch.softmax(lf, dim=-1)
        sel = scores.gather(1, idx)
        ssum = sel.sum(dim=1, keepdim=True)
        # w = sel / ssum
        dsel = (dw - (dw * w).sum(dim=1, keepdim=True)) / ssum
        dscores = torch.zeros_like(scores).scatter_(1, idx, dsel)
        if dmean is not None:
            dscores = dscores + dmean.float()[None, :] / t
        if ctx.sigmoid:
            dlogits = dscores * scores * (1.0 - scores)
        else:
            dlogits = scores * (dscores - (dscores * scores).sum(dim=1, keepdim=True))
        if dz is not None:
            lse = torch.logsumexp(lf, dim=-1, keepdim=True)
            dlogits = dlogits + (dz.float() * 2.0 / t) * lse * torch.softmax(lf, dim=-1)
        # expert_bias is nudged by its own rule, never by gradients through the scores (the reference detaches
        # nothing here either, but its bias update overwrites any gradient step); keep autograd's answer
        dbias = dlogits.sum(dim=0).to(bias.dtype) if (ctx.has_bias and ctx.needs_input_grad[1]) else None
        return dlogits.to(logits.dtype), dbias, None, None


def route(logits: torch.Tensor, bias: torch.Tensor | None, sigmoid: bool, k: int):
    return _RouterFn.apply(logits, bias, sigmoid, k)


class _GatherFn(torch.autograd.Function):
    """x_sorted[row] = x[token of row]; backward sums the k rows of every token."""

    @staticmethod
    def forward(ctx, x, slot_of_row, row_of_slot, k):
        ctx.save_for_backward(row_of_slot)
        ctx.k, ctx.tokens = k, x.shape[0]
        return kc.moe_gather(x.contiguous(), slot_of_row, k)

    @staticmethod
    def backward(ctx, dy):
        (row_of_slot,) = ctx.saved_tensors
        return kc.moe_combine(dy.contiguous(), row_of_slot, None, ctx.tokens, ctx.k), None, None, None


class _CombineFn(torch.autograd.Function):
    """out[t] = sum_j w[t, j] * y_sorted[row_of_slot[t, j]]."""

    @staticmethod
    def forward(ctx, y, w, row_of_slot, slot_of_row):
        t, k = w.shape
        wf = w.float().contiguous()
        ctx.save_for_backward(y, wf, row_of_slot, slot_of_row)
        ctx.w_dtype = w.dtype
        return kc.moe_combine(y.contiguous(), row_of_slot, wf, t, k)

    @staticmethod
    def backward(ctx, dout):
        y, wf, row_of_slot, slot_of_row = ctx.saved_tensors
        t, k = wf.shape
        dy, dw_rows = kc.moe_combine_bwd(dout.contiguous(), y.contiguous(), slot_of_row, wf.reshape(-1), k)
        # dw comes out per sorted row (indexed by slot inside the kernel): it is already in slot order
        return dy, dw_rows.view(t, k).to(ctx.w_dtype), None, None


def sort_by_expert(indices: torch.Tensor, num_experts: int):
    return kc.moe_sort(indices.contiguous(), num_experts)


def gather_rows(x, slot_of_row, row_of_slot, k):
    return _GatherFn.apply(x, slot_of_row, row_of_slot, k)


def combine_rows(y, w, row_of_slot, slot_of_row):
    return _CombineFn.apply(y, w, row_of_slot, slot_of_row)
