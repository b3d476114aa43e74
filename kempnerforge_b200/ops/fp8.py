"""FP8 training for dense Linear layers: tensorwise dynamic scaling, e4m3 activations / weights and e5m2
gradients, bf16 master weights, fp32 accumulation on tcgen05 ``kind::f8f6f4`` tensor cores.

``convert_model`` tags the weights of the selected ``nn.Linear`` modules; ``ops.functional.linear`` /
``fused_linear`` route tagged weights through ``_Fp8LinearFn``:

    forward   y  = (q4(x) @ q4(W)ᵀ)            / (s_x s_w)
    backward  dx = (q5(dy) @ q4(W))             / (s_g s_w)      q4 = e4m3, q5 = e5m2,
              dW = (q5(dy)ᵀ @ q4(x))            / (s_g s_x)      s = fp8_max / absmax (device scalars)

Scales never visit the host.  The cast kernel emits the transposed copies dgrad / wgrad need in the same pass,
so all three GEMMs run with the reduction dimension contiguous.  On a CPU (tests) the same arithmetic is
emulated with ``torch.float8_*`` dtypes.

Parity: kempnerforge/distributed/parallel.py:125-174 (torchao ``convert_to_float8_training`` with tensorwise
recipes; the module filter skips experts, shared experts and routers; dims must be multiples of 16).
"""

from __future__ import annotations

import torch
from torch import nn

from kempnerforge_b200.metrics.logger import get_logger

log = get_logger(__name__)

E4M3_MAX = 448.0
E5M2_MAX = 57344.0


def _eligible(linear: nn.Linear) -> bool:
    return linear.in_features % 16 == 0 and linear.out_features % 16 == 0


def convert_model(model: nn.Module, skip: tuple[str, ...] = ("experts", "shared_expert", "router")) -> int:
    """Tag every eligible ``nn.Linear`` outside ``skip`` for fp8 GEMMs.  Returns the number tagged."""
    n = 0
    for name, mod in model.named_modules():
        if not isinstance(mod, nn.Linear) or any(part in skip for part in name.split(".")):
            continue
        if name.split(".")[-1] == "proj" and "output_head" in name:
            continue  # the vocabulary projection stays bf16: it is fused with the loss
        if not _eligible(mod):
            continue
        mod.weight._kf_fp8 = True
        n += 1
    for m in model.modules():
        if hasattr(m, "ac_mode"):
            m._kf_fp8_block = True  # the fused bf16 block node is bypassed
    log.info("fp8: %d Linear layers use e4m3/e5m2 tensor-core GEMMs", n)
    return n


def is_fp8_weight(w: torch.Tensor) -> bool:
    return bool(getattr(w, "_kf_fp8", False))


# --------------------------------------------------------------------------- quantisation
def quantize(x2: torch.Tensor, e5m2: bool = False, want_row: bool = True, want_t: bool = False,
             scale: torch.Tensor | None = None):
    """(scale, row-major fp8 bytes or None, transposed fp8 bytes or None) of a 2-D bf16 tensor."""
    from kempnerforge_b200.ops import cuda as cu

    if x2.is_cuda:
        if scale is None:
            scale = cu.fp8_scale(x2, e5m2)
        row, t = cu.fp8_cast(x2, scale, e5m2, want_row, want_t)
        return scale, row, t
    fmax = E5M2_MAX if e5m2 else E4M3_MAX
    dt = torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn
    if scale is None:
        scale = (fmax / x2.float().abs().max().clamp_min(1e-12)).reshape(1)
    q = (x2.float() * scale).clamp(-fmax, fmax).to(dt)
    return scale, (q if want_row else None), (q.t().contiguous() if want_t else None)


def scaled_mm(a8, b8, sa, sb, a_e5m2=False, b_e5m2=False, out=None, accumulate=False) -> torch.Tensor:
    """(a8 @ b8ᵀ) / (sa * sb) -> bf16; both operands (rows, K) with K contiguous."""
    from kempnerforge_b200.ops import cuda as cu

    if a8.is_cuda:
        return cu.gemm_fp8(a8, b8, sa, sb, a_e5m2, b_e5m2, out=out, accumulate=accumulate)
    y = (a8.float() @ b8.float().t()) / (sa * sb)
    if out is None:
        return y.to(torch.bfloat16)
    if accumulate:
        out.add_(y.to(out.dtype))
    else:
        out.copy_(y.to(out.dtype))
    return out


def quantized_weight(weights, want_t: bool):
    """(scale, row-major fp8, transposed fp8 or None) of the weights stacked along the output dimension.

    The quantised copies are kept on the first weight tensor and reused until a weight is modified in place (the
    tensors' version counters change on every optimizer step), so the micro-batches, the recomputation and the
    backward pass of one step quantise each weight once instead of once per use."""
    from kempnerforge_b200.ops import functional as F

    versions = tuple(w._version for w in weights) + tuple(w.data_ptr() for w in weights)
    holder = weights[0]
    cached = getattr(holder, "_kf_fp8_cache", None)
    if cached is None or cached[0] != versions:
        sw, w8, _ = quantize(F._stack_weight_rows(weights).detach())
        cached = [versions, sw, w8, None]
        holder._kf_fp8_cache = cached
    if want_t and cached[3] is None:
        cached[3] = quantize(F._stack_weight_rows(weights).detach(), want_row=False, want_t=True, scale=cached[1])[2]
    return cached[1], cached[2], cached[3]


class _Fp8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, *weights):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        sx, x8, _ = quantize(x2)
        sw, w8, _ = quantized_weight(weights, want_t=False)
        y = scaled_mm(x8, w8, sx, sw)
        ctx.save_for_backward(x2, sx, sw, *weights)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w8.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from kempnerforge_b200.ops import functional as F

        x2, sx, sw, *weights = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        need_dx = ctx.needs_input_grad[0]
        need_dw = any(ctx.needs_input_grad[1:])
        sg, g8, g8t = quantize(dy2, e5m2=True, want_row=need_dx, want_t=need_dw)
        dx = None
        if need_dx:
            _, _, w8t = quantized_weight(weights, want_t=True)                      # (K, N)
            dx = scaled_mm(g8, w8t, sg, sw, a_e5m2=True).view(ctx.x_shape)
        wgrads = [None] * len(weights)
        if need_dw:
            _, _, x8t = quantize(x2, want_row=False, want_t=True, scale=sx)          # (K, T)
            wgrads = F._deposit_stacked_weight_grads(
                weights, ctx.needs_input_grad[1:],
                lambda out, acc: scaled_mm(g8t, x8t, sg, sx, a_e5m2=True, out=out, accumulate=acc))
        return (dx, *wgrads)


def linear(x: torch.Tensor, weights: list[torch.Tensor]) -> torch.Tensor:
    """fp8 Linear against one weight or several weights stacked along the output dimension."""
    return _Fp8LinearFn.apply(x, *weights)


def supported(x: torch.Tensor, weights: list[torch.Tensor]) -> bool:
    t = x.numel() // x.shape[-1]
    return (x.dtype == torch.bfloat16 and t % 16 == 0 and all(is_fp8_weight(w) for w in weights)
            and all(w.shape[0] % 16 == 0 and w.shape[1] % 16 == 0 for w in weights))
