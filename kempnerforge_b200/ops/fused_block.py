"""One autograd node for a whole dense transformer block on the native kernels.

Forward:  x -> RMSNorm -> fused QKV GEMM (rotary embedding in its epilogue) -> tcgen05 flash attention
            -> O GEMM (+x in its epilogue) -> RMSNorm -> fused gate|up GEMM (SwiGLU in its epilogue)
            -> down GEMM (+residual in its epilogue)
With ``recompute=True`` (full activation checkpointing) only the block input is kept; backward
re-runs the forward *except the down projection* (its output is not needed for any gradient),
which removes one of the four large GEMMs from the recomputation.  Without recomputation the
intermediates are kept and backward starts immediately.

Backward is written out by hand: every weight-gradient GEMM writes (or accumulates) straight
into the parameter's flat gradient buffer, the two residual-gradient additions are folded into
the RMSNorm backward kernel, and no autograd graph is built for the block's interior.  The
attention backward writes dq | dk | dv into the three head ranges of ONE fused gradient buffer and
applies the inverse rotary embedding on the way out (dq in its fp32 -> bf16 pass, dk in its
epilogue), so neither a copy nor a separate rotary pass exists in either direction.

``KF_AC_KEEP_ATTN=1`` additionally keeps each block's attention output and log-sum-exp (66 MB per
block at the 8B shape) so that the recomputation skips the attention forward; the default keeps
only the block input, which is what "full" checkpointing means in the reference.

Semantics are those of kempnerforge/model/transformer.py:82-103 with the activation
checkpointing of kempnerforge/distributed/parallel.py:90-122.
"""

from __future__ import annotations

import math
import os

import torch

from kempnerforge_b200.ops import cuda as kc


def _wgrad(dy2: torch.Tensor, x2: torch.Tensor, weights) -> list:
    """dW for row-stacked weights; deposits into flat gradient views when present, else returns tensors."""
    slots = [getattr(w, "_kf_grad", None) for w in weights]
    if all(s is not None for s in slots) and kc.rows_adjacent(slots):
        live = [getattr(w, "_kf_grad_live", False) for w in weights]
        if all(live) or not any(live):
            kc.gemm(dy2, x2, a_kmajor=False, b_kmajor=False, out=kc.stack_rows(slots), accumulate=live[0])
            for w in weights:
                w._kf_grad_live = True
            return [None] * len(weights)
    dw = kc.gemm(dy2, x2, a_kmajor=False, b_kmajor=False)
    out, row = [], 0
    for w, slot in zip(weights, slots):
        piece = dw[row : row + w.shape[0]]
        row += w.shape[0]
        if slot is None:
            out.append(piece)
        else:
            if getattr(w, "_kf_grad_live", False):
                slot.add_(piece)
            else:
                slot.copy_(piece)
                w._kf_grad_live = True
            out.append(None)
    return out


def _norm_wgrad(weight, dw):
    slot = getattr(weight, "_kf_grad", None)
    if slot is None:
        return dw.to(weight.dtype)
    if getattr(weight, "_kf_grad_live", False):
        slot.add_(dw)
    else:
        slot.copy_(dw)
        weight._kf_grad_live = True
    return None


def _attention_fwd(q, k, v, causal, scale, need_ctx: bool = True):
    """(out, ctx) with ctx holding what the backward needs (None when ``need_ctx`` is False: the
    first forward of a recomputed block only wants the output)."""
    if kc.attn_policy() == "native" and kc.attn_supported(q, k, v, causal, needs_grad=True):
        out, lse = kc.attn_fwd(q, k, v, causal, None, scale)
        return out, ("native", lse)
    if not need_ctx:
        o = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal, scale=scale,
            enable_gqa=k.shape[2] != q.shape[2]).transpose(1, 2)
        return o, None
    with torch.enable_grad():
        ql, kl, vl = (t.detach().requires_grad_(True) for t in (q, k, v))
        o = torch.nn.functional.scaled_dot_product_attention(
            ql.transpose(1, 2), kl.transpose(1, 2), vl.transpose(1, 2), is_causal=causal, scale=scale,
            enable_gqa=kl.shape[2] != ql.shape[2]).transpose(1, 2)
    return o.detach(), ("library", (ql, kl, vl, o))


def _attention_bwd(dout, q, k, v, out, actx, causal, scale):
    kind, saved = actx
    if kind == "native":
        return kc.attn_bwd(dout, q, k, v, out, saved, causal, None, scale)
    ql, kl, vl, o = saved
    return torch.autograd.grad(o, (ql, kl, vl), dout)


def _sharded_unit(w):
    """The sharded flat unit (ZeRO-3) that owns parameter ``w``, or None."""
    g = getattr(w, "_kf_flat", None)
    return g if g is not None and getattr(g, "sharded", False) else None


def _gather_plan(g, key: str, weights, x2):
    """Plan for the weight-gathering GEMM when the unit is sharded, the weights are not yet in the staging buffer
    and the shapes fit the kernel; otherwise the weights are made valid by a plain pull and None is returned."""
    if g is None:
        return None
    eng = g.engine
    if eng._stage_owner is not g:
        eng.acquire(g)
    if key in g.valid or "all" in g.valid:
        return None
    plan = eng.gather_plan(g, weights, x2.shape[1]) if (x2.shape[0] >= 256 and x2.stride(0) % 8 == 0) else None
    if plan is None:
        eng.ensure(g, key, weights)
        return None
    g.valid.add(key)  # the kernel launched next leaves the whole operand in the staging buffer
    return plan


def _rope_fused(n1, w_qkv, cos, sin, s: int, hd: int) -> bool:
    """The rotary epilogue of the CTA-pair GEMM applies: fp32 (S, hd / 2) tables, whole sequences per row block,
    and a problem large enough for that kernel (small ones keep the separate in-place pass)."""
    return (os.environ.get("KF_ROPE_EPILOGUE", "1") != "0" and cos.dtype == torch.float32 and cos.is_contiguous()
            and sin.is_contiguous() and cos.dim() == 2 and cos.shape[0] >= s and cos.shape[1] == hd // 2
            and n1.shape[0] % s == 0 and n1.shape[0] >= 256 and w_qkv.shape[0] % 256 == 0
            and kc.gemm_rope_supported(n1, w_qkv, hd))


class DenseBlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, wn1, wq, wk, wv, wo, wn2, wg, wu, wd, eps, head_dim, recompute):
        b, s, d = x.shape
        x2 = x.reshape(b * s, d)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.meta = (b, s, d, eps, head_dim, recompute)
        ctx.weights = (wn1, wq, wk, wv, wo, wn2, wg, wu, wd)
        keep_attn = recompute and os.environ.get("KF_AC_KEEP_ATTN", "0") == "1"
        inter = DenseBlockFn._run_forward(x2, cos, sin, ctx.weights, ctx.meta, need_output=True, keep=not recompute,
                                          keep_attn=keep_attn)
        y = inter.pop("y")
        ctx.attn_saved = None
        if recompute:
            ctx.save_for_backward(x2, cos, sin)
            ctx.inter = None
            if keep_attn and inter.get("actx") is not None and inter["actx"][0] == "native":
                ctx.attn_saved = (inter["attn2"], inter["actx"])
        else:
            ctx.save_for_backward(x2, cos, sin)
            ctx.inter = inter
        return y.view(b, s, d)

    @staticmethod
    def _run_forward(x2, cos, sin, weights, meta, need_output: bool, keep: bool, keep_attn: bool = False,
                     attn_saved=None) -> dict:
        wn1, wq, wk, wv, wo, wn2, wg, wu, wd = weights
        b, s, d, eps, hd, _ = meta
        h, hkv = wq.shape[0] // hd, wk.shape[0] // hd
        unit = _sharded_unit(wq)
        if unit is not None and unit.engine._stage_owner is not unit:
            unit.engine.acquire(unit)   # norm weights are pulled here; matrices by the GEMMs that read them
        n1, rstd1 = kc.rmsnorm_fwd(x2, wn1, eps)
        w_qkv = kc.stack_rows([wq, wk, wv])
        rope_ok = _rope_fused(n1, w_qkv, cos, sin, s, hd)
        plan = _gather_plan(unit, "qkv", [wq, wk, wv], n1)
        if plan is not None:
            qkv = kc.gemm_gather(n1, plan, w_qkv.shape[0], epi=2 if rope_ok else 0,
                                 rope=(cos, sin, s, (h + hkv) * hd, hd) if rope_ok else None)
            qkv4 = qkv.view(b, s, h + 2 * hkv, hd)
            if not rope_ok:
                kc.rope(qkv4, cos, sin, h + hkv, inverse=False, out=qkv4)
        elif rope_ok:
            qkv = kc.gemm(n1, w_qkv, rope=(cos, sin, s, (h + hkv) * hd, hd), mode=2)  # rotation in the GEMM epilogue
            qkv4 = qkv.view(b, s, h + 2 * hkv, hd)
        else:
            qkv = kc.gemm(n1, w_qkv)
            qkv4 = qkv.view(b, s, h + 2 * hkv, hd)
            kc.rope(qkv4, cos, sin, h + hkv, inverse=False, out=qkv4)  # in place: each element is read and written by one thread
        q, k, v = qkv4[:, :, :h], qkv4[:, :, h : h + hkv], qkv4[:, :, h + hkv :]
        scale = 1.0 / math.sqrt(hd)
        if attn_saved is not None:       # kept from the first forward: the recomputation skips the attention kernel
            attn2, actx = attn_saved
        else:
            attn, actx = _attention_fwd(q, k, v, True, scale, need_ctx=keep or keep_attn)
            attn2 = attn.reshape(b * s, h * hd)
        plan = _gather_plan(unit, "o", [wo], attn2)
        if plan is not None:
            h1 = kc.gemm_gather(attn2, plan, wo.shape[0], epi=0, residual=x2)
        else:
            h1 = kc.gemm(attn2, wo, residual=x2)  # residual add in the GEMM epilogue
        n2, rstd2 = kc.rmsnorm_fwd(h1, wn2, eps)
        w_gu = kc.stack_rows([wg, wu])
        plan = _gather_plan(unit, "gu", [wg, wu], n2) if kc.gemm_swiglu_supported(n2, w_gu) else None
        if plan is None and unit is not None:
            unit.engine.ensure(unit, "gu", [wg, wu])
        if plan is not None:
            hmid, gu = kc.gemm_gather(n2, plan, wg.shape[0], epi=1, want_gu=keep)
        elif kc.gemm_swiglu_supported(n2, w_gu):
            # activation in the GEMM epilogue; the pre-activations are written only when the backward will need them
            hmid, gu = kc.gemm_swiglu(n2, w_gu, want_gu=keep)
        else:
            gu = kc.gemm(n2, w_gu)
            hmid = kc.swiglu_fwd(gu)
        out = {}
        if need_output:
            plan = _gather_plan(unit, "d", [wd], hmid)
            if plan is not None:
                y = kc.gemm_gather(hmid, plan, wd.shape[0], epi=0, residual=h1)
            else:
                y = kc.gemm(hmid, wd, residual=h1)
            out["y"] = y
        if keep:
            out.update(n1=n1, rstd1=rstd1, qkv4=qkv4, attn2=attn2, actx=actx, h1=h1, n2=n2, rstd2=rstd2, gu=gu, hmid=hmid)
        elif keep_attn:
            out.update(attn2=attn2, actx=actx)
        return out

    @staticmethod
    def backward(ctx, dy):
        x2, cos, sin = ctx.saved_tensors
        b, s, d, eps, hd, recompute = ctx.meta
        wn1, wq, wk, wv, wo, wn2, wg, wu, wd = ctx.weights
        unit = _sharded_unit(wq)
        if unit is not None:
            unit.engine.prepare_backward(unit)  # parameter staging is ours again; gradient staging slot is free
        it = ctx.inter
        if it is None:
            it = DenseBlockFn._run_forward(x2, cos, sin, ctx.weights, ctx.meta, need_output=False, keep=True,
                                           attn_saved=ctx.attn_saved)
            ctx.attn_saved = None
        dy2 = dy.reshape(b * s, d)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        h, hkv = wq.shape[0] // hd, wk.shape[0] // hd
        if unit is not None:  # whatever the recomputation did not gather (the down projection; everything without AC)
            eng = unit.engine
            eng.ensure(unit, "d", [wd])
            eng.ensure(unit, "gu", [wg, wu])
            eng.ensure(unit, "o", [wo])
            eng.ensure(unit, "qkv", [wq, wk, wv])
        # ---- feed-forward branch
        (g_wd,) = _wgrad(dy2, it["hmid"], [wd])
        if kc.gemm_swiglu_bwd_supported(dy2, wd, it["gu"]):
            dgu = kc.gemm_swiglu_bwd(dy2, wd, it["gu"])  # SwiGLU gradient in the GEMM epilogue, written over gu
        else:
            dhmid = kc.gemm(dy2, wd, a_kmajor=True, b_kmajor=False)
            dgu = kc.swiglu_bwd(dhmid, it["gu"], out=it["gu"])  # gu is dead after this; reuse its storage
            del dhmid
        dn2 = kc.gemm(dgu, kc.stack_rows([wg, wu]), a_kmajor=True, b_kmajor=False)
        g_wg, g_wu = _wgrad(dgu, it["n2"], [wg, wu])
        dh1, dwn2 = kc.rmsnorm_bwd(dn2, it["h1"], wn2, it["rstd2"], residual_grad=dy2, out=dn2)
        g_wn2 = _norm_wgrad(wn2, dwn2)
        # ---- attention branch
        dattn = kc.gemm(dh1, wo, a_kmajor=True, b_kmajor=False)
        (g_wo,) = _wgrad(dh1, it["attn2"], [wo])
        qkv4 = it["qkv4"]
        q, k, v = qkv4[:, :, :h], qkv4[:, :, h : h + hkv], qkv4[:, :, h + hkv :]
        attn = it["attn2"].view(b, s, h, hd)
        dqkv4 = torch.empty_like(qkv4)
        if it["actx"][0] == "native":
            # dq | dk | dv land in their head ranges of the fused gradient, already through the inverse rotation
            fused_rope = hd == 128 and cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
            kc.attn_bwd(dattn.view(b, s, h, hd), q, k, v, attn, it["actx"][1], True, None, 1.0 / math.sqrt(hd),
                        dq=dqkv4[:, :, :h], dk=dqkv4[:, :, h : h + hkv], dv=dqkv4[:, :, h + hkv :],
                        rope=(cos, sin) if fused_rope else None)
            if not fused_rope:
                kc.rope(dqkv4, cos, sin, h + hkv, inverse=True, out=dqkv4)
        else:
            dq, dk, dv = _attention_bwd(dattn.view(b, s, h, hd), q, k, v, attn, it["actx"], True, 1.0 / math.sqrt(hd))
            dqkv4[:, :, :h].copy_(dq)
            dqkv4[:, :, h : h + hkv].copy_(dk)
            dqkv4[:, :, h + hkv :].copy_(dv)
            del dq, dk, dv
            kc.rope(dqkv4, cos, sin, h + hkv, inverse=True, out=dqkv4)
        dqkv = dqkv4.view(b * s, (h + 2 * hkv) * hd)
        dn1 = kc.gemm(dqkv, kc.stack_rows([wq, wk, wv]), a_kmajor=True, b_kmajor=False)
        g_wq, g_wk, g_wv = _wgrad(dqkv, it["n1"], [wq, wk, wv])
        dx, dwn1 = kc.rmsnorm_bwd(dn1, x2, wn1, it["rstd1"], residual_grad=dh1, out=dn1)
        g_wn1 = _norm_wgrad(wn1, dwn1)
        ctx.inter = None
        return (dx.view(b, s, d), None, None, g_wn1, g_wq, g_wk, g_wv, g_wo, g_wn2, g_wg, g_wu, g_wd, None, None, None)


class AttnHalfFn(torch.autograd.Function):
    """x + Attention(RMSNorm(x)) as one autograd node: the first half of a block whose second half is not the plain
    SwiGLU MLP (mixture-of-experts layers).  Same kernels as the dense block: rotary embedding in the QKV GEMM
    epilogue, tcgen05 flash attention, the residual in the O GEMM epilogue; backward with dq | dk | dv written through
    the inverse rotation into one fused gradient and the residual gradient folded into the RMSNorm backward.

    Everything the backward needs goes through ``save_for_backward``, so an enclosing non-reentrant
    ``torch.utils.checkpoint`` (full activation checkpointing of the block) drops and recomputes it like any other op.
    Parity: kempnerforge/model/transformer.py:82-103 (attention sub-layer)."""

    @staticmethod
    def forward(ctx, x, cos, sin, wn1, wq, wk, wv, wo, eps, hd):
        b, s, d = x.shape
        x2 = x.reshape(b * s, d)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        h, hkv = wq.shape[0] // hd, wk.shape[0] // hd
        n1, rstd1 = kc.rmsnorm_fwd(x2, wn1, eps)
        w_qkv = kc.stack_rows([wq, wk, wv])
        fused_rope = _rope_fused(n1, w_qkv, cos, sin, s, hd)
        if fused_rope:
            qkv = kc.gemm(n1, w_qkv, rope=(cos, sin, s, (h + hkv) * hd, hd), mode=2)
            qkv4 = qkv.view(b, s, h + 2 * hkv, hd)
        else:
            qkv = kc.gemm(n1, w_qkv)
            qkv4 = qkv.view(b, s, h + 2 * hkv, hd)
            kc.rope(qkv4, cos, sin, h + hkv, inverse=False, out=qkv4)
        q, k, v = qkv4[:, :, :h], qkv4[:, :, h : h + hkv], qkv4[:, :, h + hkv :]
        attn, lse = kc.attn_fwd(q, k, v, True, None, 1.0 / math.sqrt(hd))
        attn2 = attn.reshape(b * s, h * hd)
        h1 = kc.gemm(attn2, wo, residual=x2)  # residual add in the GEMM epilogue
        ctx.save_for_backward(x2, cos, sin, n1, rstd1, qkv, attn2, lse)
        ctx.weights = (wn1, wq, wk, wv, wo)
        ctx.meta = (b, s, d, hd)
        return h1.view(b, s, d)

    @staticmethod
    def backward(ctx, dh):
        x2, cos, sin, n1, rstd1, qkv, attn2, lse = ctx.saved_tensors
        wn1, wq, wk, wv, wo = ctx.weights
        b, s, d, hd = ctx.meta
        h, hkv = wq.shape[0] // hd, wk.shape[0] // hd
        dh1 = dh.reshape(b * s, d)
        if not dh1.is_contiguous():
            dh1 = dh1.contiguous()
        dattn = kc.gemm(dh1, wo, a_kmajor=True, b_kmajor=False)
        (g_wo,) = _wgrad(dh1, attn2, [wo])
        qkv4 = qkv.view(b, s, h + 2 * hkv, hd)
        q, k, v = qkv4[:, :, :h], qkv4[:, :, h : h + hkv], qkv4[:, :, h + hkv :]
        dqkv4 = torch.empty_like(qkv4)
        fused_rope = hd == 128 and cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
        kc.attn_bwd(dattn.view(b, s, h, hd), q, k, v, attn2.view(b, s, h, hd), lse, True, None, 1.0 / math.sqrt(hd),
                    dq=dqkv4[:, :, :h], dk=dqkv4[:, :, h : h + hkv], dv=dqkv4[:, :, h + hkv :],
                    rope=(cos, sin) if fused_rope else None)
        if not fused_rope:
            kc.rope(dqkv4, cos, sin, h + hkv, inverse=True, out=dqkv4)
        dqkv = dqkv4.view(b * s, (h + 2 * hkv) * hd)
        dn1 = kc.gemm(dqkv, kc.stack_rows([wq, wk, wv]), a_kmajor=True, b_kmajor=False)
        g_wq, g_wk, g_wv = _wgrad(dqkv, n1, [wq, wk, wv])
        dx, dwn1 = kc.rmsnorm_bwd(dn1, x2, wn1, rstd1, residual_grad=dh1, out=dn1)
        g_wn1 = _norm_wgrad(wn1, dwn1)
        return dx.view(b, s, d), None, None, g_wn1, g_wq, g_wk, g_wv, g_wo, None, None


def attn_half_supported(block, x, kv_cache, doc_ids, key_padding_mask) -> bool:
    """The fused attention sub-layer covers bf16 causal self-attention with head dim 128 on a GPU, without masks,
    caches, q/k norms, tensor parallelism, fp8 or hooks; the feed-forward half of the block may be anything."""
    att = block.attention
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 3 and kv_cache is None and doc_ids is None
            and key_padding_mask is None and torch.is_grad_enabled()):
        return False
    if os.environ.get("KF_DISABLE_FUSED_ATTN_HALF"):
        return False
    unit = getattr(att.q_proj.weight, "_kf_flat", None)
    return (
        getattr(att, "tp", None) is None
        and att.q_norm is None
        and not att.capture_attention_weights
        and type(block.attention_norm).__name__ == "RMSNorm"
        and not getattr(block, "fp8", False)
        and not getattr(block, "_kf_fp8_block", False)
        and not (unit is not None and getattr(unit, "sharded", False))
        and att.head_dim == 128
        and x.shape[-1] % 8 == 0
        and x.shape[0] * x.shape[1] >= 128
        and kc.attn_policy() == "native"
        and getattr(kc.lib(), "kf_attn_bwd_bf16", None) is not None
        and att.q_proj.weight.dtype == torch.bfloat16
        and not block._forward_hooks
        and not att._forward_hooks
        and not block.attention_norm._forward_hooks
    )


def attn_half(block, x, cos, sin):
    att = block.attention
    return AttnHalfFn.apply(x, cos, sin, block.attention_norm.weight, att.q_proj.weight, att.k_proj.weight,
                            att.v_proj.weight, att.o_proj.weight, block.attention_norm.eps, att.head_dim)


def dense_block_supported(block, x, kv_cache, doc_ids, key_padding_mask) -> bool:
    """The fused node covers the plain dense pre-norm SwiGLU block in bf16 on a GPU."""
    att, mlp = block.attention, block.mlp
    return (
        x.is_cuda
        and x.dtype == torch.bfloat16
        and kv_cache is None
        and doc_ids is None
        and key_padding_mask is None
        and torch.is_grad_enabled()
        and getattr(att, "tp", None) is None
        and att.q_norm is None
        and not att.capture_attention_weights
        and type(mlp).__name__ == "SwiGLUMLP"
        and getattr(mlp, "tp", None) is None
        and type(block.attention_norm).__name__ == "RMSNorm"
        and not getattr(block, "fp8", False)
        and block.ac_mode in ("none", "full")
        and x.shape[-1] % 8 == 0
        and att.head_dim % 16 == 0
        and not block._forward_hooks
        and not att._forward_hooks
        and not mlp._forward_hooks
        and not block.attention_norm._forward_hooks
        and not block.mlp_norm._forward_hooks
    )


def dense_block(block, x, cos, sin):
    att, mlp = block.attention, block.mlp
    recompute = block.ac_mode == "full" and block.training
    return DenseBlockFn.apply(
        x, cos, sin, block.attention_norm.weight, att.q_proj.weight, att.k_proj.weight, att.v_proj.weight,
        att.o_proj.weight, block.mlp_norm.weight, mlp.gate_proj.weight, mlp.up_proj.weight, mlp.down_proj.weight,
        block.attention_norm.eps, att.head_dim, recompute,
    )
