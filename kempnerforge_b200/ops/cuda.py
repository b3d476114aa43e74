"""ctypes binding of ``libkfb200.so`` — the hand-written sm_100a kernels.

Tensors are passed as raw device pointers together with the current CUDA
stream, so every launch is ordered like an ordinary PyTorch op.  Importing this
module on a machine with a GPU but without the built library raises: there is
no silent fallback to library kernels.
"""

from __future__ import annotations

import ctypes
import math
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from kempnerforge_b200.ops.build import LIB_PATH

_lib = None
GEMM_MODE = int(os.environ.get("KF_GEMM_MODE", "0"))  # 0 = automatic, 1 = single CTA tiles, 2 = CTA pairs
LAUNCH_COUNT = 0  # number of native kernel launches issued through this module (bench bookkeeping)


class NativeKernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise NativeKernelError(
                f"native library {LIB_PATH} is missing; run `python -m kempnerforge_b200.ops.build`"
            )
        _lib = ctypes.CDLL(str(LIB_PATH))
        _declare(_lib)
        if os.environ.get("KF_ATTN_BWD_DQ", "") == "red" and hasattr(_lib, "kf_attn_bwd_dq_mode"):
            _lib.kf_attn_bwd_dq_mode(0)
        if os.environ.get("KF_GROUPED_PAIR", "1") == "0" and hasattr(_lib, "kf_grouped_pair_mode"):
            _lib.kf_grouped_pair_mode(0)
    return _lib


def available() -> bool:
    return torch.cuda.is_available() and LIB_PATH.exists()


def _declare(L: ctypes.CDLL) -> None:
    vp, i, ll, f = c_void_p, c_int, c_longlong, c_float
    sigs = {
        "kf_gemm_bf16": [vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, i, i, i, i, vp],
        "kf_gemm_swiglu_bf16": [vp, vp, vp, vp, i, i, i, i, i, i, i, i, vp],
        "kf_gemm_rope_bf16": [vp, vp, vp, i, i, i, i, i, i, vp, vp, i, i, i, i, vp],
        "kf_gemm_swiglu_bwd_bf16": [vp, vp, vp, vp, i, i, i, i, i, i, i, vp],
        "kf_gemm_symm_bf16": [i, vp, vp, vp, i, i, i, i, i, f, f, f, i, vp],
        "kf_rmsnorm_fwd_bf16": [vp, vp, vp, vp, i, i, f, vp],
        "kf_rmsnorm_bwd_blocks": [i],
        "kf_rmsnorm_bwd_bf16": [vp, vp, vp, vp, vp, vp, vp, vp, i, i, vp, vp],
        "kf_rope_bf16": [vp, vp, vp, vp, ll, i, i, i, i, i, vp],
        "kf_swiglu_fwd_bf16": [vp, vp, ll, i, vp],
        "kf_swiglu_bwd_bf16": [vp, vp, vp, ll, i, vp],
        "kf_embedding_fwd_bf16": [vp, vp, vp, ll, i, i, vp],
        "kf_embedding_bwd_bf16": [vp, vp, vp, ll, i, i, vp],
        "kf_ce_fwd_bwd_bf16": [vp, vp, vp, vp, vp, f, i, i, i, vp],
        "kf_ce_vp_stats_bf16": [vp, vp, ll, vp, vp, vp, i, i, i, vp],
        "kf_ce_vp_bwd_bf16": [vp, vp, ll, vp, vp, vp, f, i, i, i, vp],
        "kf_adamw_flat": [vp, vp, vp, vp, ll, ll, f, f, f, f, f, f, f, vp, vp, i, i, i, vp],
        "kf_sumsq": [vp, ll, i, vp, vp, i, vp],
        "kf_test_flag_timeout": [vp, i, ll],
        "kf_gemm_fp8": [vp, vp, vp, i, i, i, ll, ll, i, i, i, vp, vp, i, i, vp],
        "kf_fp8_scale_bf16": [vp, ll, i, vp, vp, vp],
        "kf_fp8_cast_bf16": [vp, i, i, ll, vp, i, vp, ll, vp, ll, vp],
        "kf_lion": [vp, vp, vp, ll, i, f, f, f, f, vp],
        "kf_sf_adamw": [vp, vp, vp, vp, vp, ll, i, f, f, f, f, f, f, f, i, vp],
        "kf_ep_put_bf16": [vp, vp, i, vp, i, i, i, i, ll, vp, vp, i, vp],
        "kf_ep_layout": [vp, i, i, vp, vp, vp, vp, vp],
        "kf_ep_move_bf16": [vp, vp, vp, vp, vp, i, i, i, ll, i, vp, vp],
        "kf_router_topk": [vp, i, vp, i, i, i, i, vp, vp, vp, vp, vp, vp],
        "kf_moe_sort": [vp, i, i, vp, vp, vp, vp, vp],
        "kf_moe_capacity_mask": [vp, i, i, i, i, vp, vp],
        "kf_moe_gather_bf16": [vp, vp, i, i, i, vp, vp],
        "kf_moe_combine_bf16": [vp, vp, vp, i, i, i, vp, vp],
        "kf_moe_combine_bwd_bf16": [vp, vp, vp, vp, i, i, i, vp, vp, vp],
        "kf_grouped_gemm_bf16": [vp, vp, vp, vp, i, i, i, i, ll, ll, i, i, vp],
        "kf_grouped_gemm_acc_bf16": [vp, vp, vp, vp, i, i, i, i, ll, ll, i, i, i, vp],
        "kf_grouped_swiglu_bf16": [vp, vp, vp, vp, vp, vp, i, i, i, i, ll, ll, ll, i, i, vp],
        "kf_grouped_swiglu_bwd_bf16": [vp, vp, vp, vp, vp, i, i, i, i, ll, ll, i, i, vp],
        "kf_swiglu_bwd_ragged_bf16": [vp, vp, vp, ll, vp, i, vp],
        "kf_grouped_wgrad_bf16": [vp, vp, vp, vp, i, i, i, i, ll, ll, i, vp],
        "kf_ag_gemm_bf16": [vp, vp, vp, vp, vp, i, i, i, i, ll, ll, ll, i, i, i, i, i, vp],
        "kf_gemm_rs_bf16": [vp, vp, vp, vp, vp, vp, i, i, i, i, ll, ll, i, i, i, i, i, vp],
        "kf_attn_bwd_bf16": [vp] * 12 + [i] * 6 + [ll] * 8 + [f, i, vp],
        "kf_attn_bwd_rope_bf16": [vp] * 12 + [i] * 6 + [ll] * 8 + [f, i, vp, vp, vp],
        "kf_attn_bwd_dq_mode": [i],
        "kf_grouped_pair_mode": [i],
        "kf_attn_fwd2_bf16": [vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, ll, ll, ll, ll, f, i, vp],
        "kf_attn_fwd_bf16": [vp, vp, vp, vp, vp, vp, i, i, i, i, i, i, ll, ll, ll, ll, f, i, vp],
        "kf_symm_rs_norm_bf16": [vp, vp, i, i, ll, ll, vp, vp, i, i, vp],
        "kf_symm_adamw_bcast_bf16": [vp, vp, i, i, vp, vp, vp, ll, ll, ll, f, f, f, f, f, f, f, vp, vp, i, vp],
        "kf_symm_gather_bf16": [vp, vp, i, i, ll, ll, i, vp],
        "kf_symm_pull_bf16": [vp, i, i, vp, vp, vp, vp, i, vp],
        "kf_symm_rs_shard_bf16": [vp, vp, i, i, i, vp, vp, vp, vp, i, i, vp],
        "kf_gemm_gather_bf16": [i, vp, vp, vp, i, i, i, i, i, i, vp, i, i, i, vp, vp, vp, vp, vp, vp, i, i, i, i, vp],
        "kf_read_status": [],
        "kf_clear_status": [],
        "kf_status_device_ptr": [],
    }
    for name, args in sigs.items():
        fn = getattr(L, name, None)
        if fn is None:
            continue
        fn.argtypes = args
        fn.restype = c_void_p if name == "kf_status_device_ptr" else c_int
    if hasattr(L, "kf_clear_status"):
        L.kf_clear_status.restype = None


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(code: int, what: str) -> None:
    global LAUNCH_COUNT
    LAUNCH_COUNT += 1
    if code != 0:
        raise NativeKernelError(f"{what} failed with code {code}")


_SM_COUNT: dict[int, int] = {}


def sm_count() -> int:
    dev = torch.cuda.current_device()
    if dev not in _SM_COUNT:
        _SM_COUNT[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _SM_COUNT[dev]


def read_status() -> int:
    """Status word of the library on the current device (0 = no kernel gave up a wait). Synchronises."""
    return int(lib().kf_read_status())


def clear_status() -> None:
    lib().kf_clear_status()


# --------------------------------------------------------------------------- row stacking of adjacent views
def rows_adjacent(tensors) -> bool:
    """True when 2-D tensors with equal width sit back to back in one storage (so they form one matrix)."""
    first = tensors[0]
    if first is None or not first.is_contiguous():
        return False
    ptr = first.data_ptr() + first.numel() * first.element_size()
    for t in tensors[1:]:
        if (
            t is None
            or not t.is_contiguous()
            or t.shape[1:] != first.shape[1:]
            or t.dtype != first.dtype
            or t.data_ptr() != ptr
            or t.untyped_storage().data_ptr() != first.untyped_storage().data_ptr()
        ):
            return False
        ptr += t.numel() * t.element_size()
    return True


def stack_rows(tensors):
    """One (sum rows, cols) matrix over the given row blocks: a zero-copy view when adjacent, else a copy."""
    tensors = list(tensors)
    if len(tensors) == 1:
        return tensors[0]
    if rows_adjacent(tensors):
        first = tensors[0]
        rows = sum(t.shape[0] for t in tensors)
        return torch.as_strided(first.detach(), (rows, *first.shape[1:]), first.stride())
    return torch.cat([t.detach() for t in tensors], dim=0)


# --------------------------------------------------------------------------- GEMM
def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    a_kmajor: bool = True,
    b_kmajor: bool = True,
    out: torch.Tensor | None = None,
    accumulate: bool = False,
    out_dtype: torch.dtype | None = None,
    residual: torch.Tensor | None = None,
    mode: int | None = None,
    rope: tuple | None = None,
) -> torch.Tensor:
    """out[M,N] = A * Bᵀ (+ out if ``accumulate``) (+ ``residual``) on the tcgen05 tensor cores.

    ``rope = (cos, sin, seq_len, rope_cols, head_dim)``: rotary position embedding in the epilogue (fused Q | K | V
    projection): the heads inside the first ``rope_cols`` output columns are rotated by the angle of position
    ``row % seq_len``; ``cos`` / ``sin`` are fp32 (seq_len, head_dim / 2).  Needs K-major operands, bf16 output.

    ``mode``: None/0 = automatic, 1 = single-CTA 128x256 tiles, 2 = CTA pairs (cta_group::2) on 256x256 tiles.

    ``a_kmajor``: a is stored (M, K); otherwise (K, M).  ``b_kmajor``: b is stored (N, K); otherwise (K, N).
    Rows may be strided (row pitch a multiple of 8 elements); columns must be contiguous.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = (a.shape[0], a.shape[1]) if a_kmajor else (a.shape[1], a.shape[0])
    N, Kb = (b.shape[0], b.shape[1]) if b_kmajor else (b.shape[1], b.shape[0])
    assert K == Kb, f"inner dimensions differ: {K} vs {Kb}"
    lda, ldb = a.stride(0), b.stride(0)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or torch.bfloat16, device=a.device)
        accumulate = False
    assert out.shape == (M, N) and out.stride(1) == 1
    ldc = out.stride(0)
    out_f32 = out.dtype == torch.float32
    assert out_f32 or out.dtype == torch.bfloat16
    if lda % 8 or ldb % 8 or ldc % (4 if out_f32 else 8) or a.data_ptr() % 16 or b.data_ptr() % 16 or out.data_ptr() % 16:
        raise NativeKernelError(
            f"gemm operands must have 16-byte aligned bases and row pitches (lda={lda}, ldb={ldb}, ldc={ldc})"
        )
    if rope is not None:
        cos, sin, seq_len, rope_cols, hd = rope
        assert a_kmajor and b_kmajor and not out_f32 and not accumulate and residual is None
        assert cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
        assert cos.shape[-1] == hd // 2 and cos.numel() >= seq_len * (hd // 2) and M % seq_len == 0
        code = lib().kf_gemm_rope_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, lda, ldb, ldc, cos.data_ptr(),
                                       sin.data_ptr(), int(seq_len), int(rope_cols), int(hd), sm_count(), _stream())
        _check(code, "kf_gemm_rope_bf16")
        return out
    ldr = 0
    if residual is not None:
        assert residual.shape == (M, N) and residual.dtype == out.dtype and residual.stride(1) == 1
        ldr = residual.stride(0)
        if ldr % (4 if out_f32 else 8) or residual.data_ptr() % 16:
            raise NativeKernelError("gemm residual must be 16-byte aligned")
    code = lib().kf_gemm_bf16(
        a.data_ptr(), b.data_ptr(), out.data_ptr(), residual.data_ptr() if residual is not None else None,
        M, N, K, lda, ldb, ldc, ldr, 0 if a_kmajor else 1, 0 if b_kmajor else 1, int(out_f32), int(accumulate),
        GEMM_MODE if mode is None else mode, sm_count(), _stream(),
    )
    _check(code, "kf_gemm_bf16")
    return out


# --------------------------------------------------------------------------- norm / rope / swiglu / embedding
def rmsnorm_fwd(x: torch.Tensor, w: torch.Tensor, eps: float):
    rows, d = x.shape
    y = torch.empty_like(x)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    _check(
        lib().kf_rmsnorm_fwd_bf16(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, d, eps, _stream()),
        "kf_rmsnorm_fwd_bf16",
    )
    return y, rstd


def rmsnorm_bwd(dy, x, w, rstd, residual_grad: torch.Tensor | None = None, out: torch.Tensor | None = None,
                dw_out: torch.Tensor | None = None):
    """Returns (dx, dw).  ``residual_grad`` is added to dx inside the kernel (it may be the same tensor as ``out``)."""
    rows, d = x.shape
    nb = lib().kf_rmsnorm_bwd_blocks(rows)
    partial = torch.empty(nb * d, dtype=torch.float32, device=x.device)
    dx = out if out is not None else torch.empty_like(x)
    dw = dw_out if dw_out is not None else torch.empty(d, dtype=torch.bfloat16, device=x.device)
    _check(
        lib().kf_rmsnorm_bwd_bf16(
            dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), partial.data_ptr(),
            dw.data_ptr(), None, rows, d, residual_grad.data_ptr() if residual_grad is not None else None, _stream(),
        ),
        "kf_rmsnorm_bwd_bf16",
    )
    return dx, dw


def rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot: int, inverse: bool, out=None):
    b, s, h, hd = x.shape
    y = torch.empty_like(x) if out is None else out
    assert cos.dtype == torch.float32 and cos.shape[0] >= s and cos.shape[1] == hd // 2
    _check(
        lib().kf_rope_bf16(x.data_ptr(), y.data_ptr(), cos.data_ptr(), sin.data_ptr(), b * s, s, h, n_rot, hd, int(inverse), _stream()),
        "kf_rope_bf16",
    )
    return y


def swiglu_fwd(gu: torch.Tensor) -> torch.Tensor:
    h = gu.shape[-1] // 2
    rows = gu.numel() // (2 * h)
    out = torch.empty((*gu.shape[:-1], h), dtype=gu.dtype, device=gu.device)
    _check(lib().kf_swiglu_fwd_bf16(gu.data_ptr(), out.data_ptr(), rows, h, _stream()), "kf_swiglu_fwd_bf16")
    return out


def swiglu_bwd(dh: torch.Tensor, gu: torch.Tensor, out=None) -> torch.Tensor:
    h = gu.shape[-1] // 2
    rows = gu.numel() // (2 * h)
    dgu = torch.empty_like(gu) if out is None else out
    _check(lib().kf_swiglu_bwd_bf16(dh.data_ptr(), gu.data_ptr(), dgu.data_ptr(), rows, h, _stream()), "kf_swiglu_bwd_bf16")
    return dgu


def embedding_fwd(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    ids = ids.contiguous()
    if ids.dtype != torch.int64:
        ids = ids.long()
    v, d = table.shape
    out = torch.empty((*ids.shape, d), dtype=table.dtype, device=table.device)
    _check(lib().kf_embedding_fwd_bf16(ids.data_ptr(), table.data_ptr(), out.data_ptr(), ids.numel(), d, v, _stream()), "kf_embedding_fwd_bf16")
    return out


def embedding_bwd(dy: torch.Tensor, ids: torch.Tensor, dtable: torch.Tensor, accumulate: bool) -> None:
    ids = ids.contiguous()
    if ids.dtype != torch.int64:
        ids = ids.long()
    v, d = dtable.shape
    if not accumulate:
        dtable.zero_()
    _check(lib().kf_embedding_bwd_bf16(ids.data_ptr(), dy.data_ptr(), dtable.data_ptr(), ids.numel(), d, v, _stream()), "kf_embedding_bwd_bf16")


# --------------------------------------------------------------------------- cross entropy
def ce_fwd_bwd(logits: torch.Tensor, labels: torch.Tensor, stats: torch.Tensor, inv_n: torch.Tensor, z_weight: float) -> None:
    """Overwrites ``logits`` (rows, V) with d loss / d logits and adds [sum nll, sum lse²] into ``stats``."""
    rows, v = logits.shape
    assert logits.stride(1) == 1
    row_nll = torch.empty(rows, dtype=torch.float32, device=logits.device)
    row_lse2 = torch.empty(rows, dtype=torch.float32, device=logits.device)
    labels = labels.contiguous()
    _check(
        lib().kf_ce_fwd_bwd_bf16(
            logits.data_ptr(), labels.data_ptr(), row_nll.data_ptr(), row_lse2.data_ptr(), inv_n.data_ptr(),
            float(z_weight), rows, v, logits.stride(0), _stream(),
        ),
        "kf_ce_fwd_bwd_bf16",
    )
    stats[0] += row_nll.sum()
    stats[1] += row_lse2.sum()


# --------------------------------------------------------------------------- optimizer
_DT = {torch.bfloat16: 0, torch.float32: 1}


def adamw_flat(p, g, m, v, n_decay: int, lr: float, beta1: float, beta2: float, eps: float, wd: float,
               step: int, grad_scale: torch.Tensor | None = None, skip: torch.Tensor | None = None) -> None:
    """One fused AdamW update over flat 1-D buffers; elements [0, n_decay) are weight-decayed."""
    n = p.numel()
    bc1 = 1.0 - beta1**step
    bc2_sqrt = math.sqrt(1.0 - beta2**step)
    _check(
        lib().kf_adamw_flat(
            p.data_ptr(), g.data_ptr(), m.data_ptr(), v.data_ptr(), n, n_decay, lr, beta1, beta2, eps, wd,
            bc1, bc2_sqrt, grad_scale.data_ptr() if grad_scale is not None else None,
            skip.data_ptr() if skip is not None else None, _DT[p.dtype], _DT[g.dtype], _DT[m.dtype], _stream(),
        ),
        "kf_adamw_flat",
    )


def sumsq(x: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """out[0] (+)= sum(x²) in fp32 with a fixed reduction order."""
    partial = torch.empty(1024, dtype=torch.float32, device=x.device)
    _check(lib().kf_sumsq(x.data_ptr(), x.numel(), _DT[x.dtype], partial.data_ptr(), out.data_ptr(), int(accumulate), _stream()), "kf_sumsq")
    return out


def gemm_swiglu(x2: torch.Tensor, w_gate_up: torch.Tensor, want_gu: bool = True):
    """(h, gu): h = silu(x Wgᵀ) * (x Wuᵀ) computed in the epilogue of one tcgen05 GEMM over the stacked weight
    ``w_gate_up`` = [Wg ; Wu] of shape (2F, K); ``gu`` (M, 2F) holds the pre-activations when ``want_gu``."""
    m, k = x2.shape
    f = w_gate_up.shape[0] // 2
    h = torch.empty((m, f), dtype=torch.bfloat16, device=x2.device)
    gu = torch.empty((m, 2 * f), dtype=torch.bfloat16, device=x2.device) if want_gu else None
    _check(lib().kf_gemm_swiglu_bf16(x2.data_ptr(), w_gate_up.data_ptr(), h.data_ptr(), gu.data_ptr() if want_gu else None,
                                     m, f, k, x2.stride(0), w_gate_up.stride(0), f, 2 * f, sm_count(), _stream()),
           "kf_gemm_swiglu_bf16")
    return h, gu


def gemm_swiglu_bwd(dy2: torch.Tensor, w_down: torch.Tensor, gu: torch.Tensor) -> torch.Tensor:
    """d[gate | up] (M, 2F), written over ``gu``: the input-gradient GEMM of the down projection (``dy2`` (M, K) times
    ``w_down`` (K, F) as stored) with the SwiGLU gradient in its epilogue; the gradient of the hidden activation is
    never written to memory."""
    m, k = dy2.shape
    f = w_down.shape[1]
    assert w_down.shape[0] == k and gu.shape == (m, 2 * f) and gu.is_contiguous() and w_down.stride(1) == 1
    _check(lib().kf_gemm_swiglu_bwd_bf16(dy2.data_ptr(), w_down.data_ptr(), gu.data_ptr(), gu.data_ptr(), m, f, k,
                                         dy2.stride(0), w_down.stride(0), 2 * f, sm_count(), _stream()),
           "kf_gemm_swiglu_bwd_bf16")
    return gu


def gemm_symm(x: torch.Tensor, tall: bool = False, residual: torch.Tensor | None = None, alpha: float = 1.0,
              beta: float = 0.0, diag: float = 0.0) -> torch.Tensor:
    """bf16 (n, n) = alpha * x xᵀ + beta * residual + diag * I for x (n, K), or alpha * xᵀ x + ... for ``tall`` x (K, n).

    Only the tiles on and above the diagonal go through the tensor cores; the kernel stores each of them a second time
    transposed, so the result is exactly symmetric.  ``residual`` must be symmetric."""
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    n, k = (x.shape[1], x.shape[0]) if tall else x.shape
    out = torch.empty((n, n), dtype=torch.bfloat16, device=x.device)
    if residual is not None:
        assert residual.shape == (n, n) and residual.dtype == torch.bfloat16 and residual.stride(1) == 1
    _check(lib().kf_gemm_symm_bf16(int(tall), x.data_ptr(), out.data_ptr(), residual.data_ptr() if residual is not None else None,
                                   n, k, x.stride(0), n, residual.stride(0) if residual is not None else 0, float(alpha),
                                   float(beta), float(diag), sm_count(), _stream()), "kf_gemm_symm_bf16")
    return out


def gemm_symm_supported(x: torch.Tensor, tall: bool = False) -> bool:
    n, k = (x.shape[1], x.shape[0]) if tall else x.shape
    return (getattr(lib(), "kf_gemm_symm_bf16", None) is not None and os.environ.get("KF_GEMM_SYMM", "1") == "1"
            and x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.stride(0) % 8 == 0 and n % 8 == 0 and n >= 256
            and k % 64 == 0)


def gemm_swiglu_bwd_supported(dy2: torch.Tensor, w_down: torch.Tensor, gu: torch.Tensor | None) -> bool:
    return (gu is not None and getattr(lib(), "kf_gemm_swiglu_bwd_bf16", None) is not None
            and not os.environ.get("KF_DISABLE_SWIGLU_EPILOGUE") and os.environ.get("KF_SWIGLU_BWD_EPILOGUE", "1") == "1" and dy2.shape[0] >= 256 and dy2.shape[1] % 64 == 0
            and w_down.shape[1] % 256 == 0 and dy2.stride(0) % 8 == 0 and w_down.stride(0) % 8 == 0 and gu.is_contiguous()
            and dy2.dtype == torch.bfloat16)


def gemm_swiglu_supported(x2: torch.Tensor, w_gate_up: torch.Tensor) -> bool:
    f = w_gate_up.shape[0] // 2
    return (getattr(lib(), "kf_gemm_swiglu_bf16", None) is not None and not os.environ.get("KF_DISABLE_SWIGLU_EPILOGUE")
            and f % 128 == 0 and x2.shape[0] >= 256 and x2.stride(1) == 1 and w_gate_up.stride(1) == 1
            and x2.stride(0) % 8 == 0 and w_gate_up.stride(0) % 8 == 0 and x2.dtype == torch.bfloat16)


# --------------------------------------------------------------------------- fp8
def fp8_scale(x2: torch.Tensor, e5m2: bool = False) -> torch.Tensor:
    """Device scalar fp8_max / absmax(x) (fp32, shape (1,))."""
    scratch = torch.empty(2, dtype=torch.float32, device=x2.device)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    _check(lib().kf_fp8_scale_bf16(x2.data_ptr(), x2.numel(), int(e5m2), scratch[1:].data_ptr(), scratch.data_ptr(),
                                   _stream()), "kf_fp8_scale_bf16")
    return scratch[:1]


def fp8_cast(x2: torch.Tensor, scale: torch.Tensor, e5m2: bool, want_row: bool = True, want_t: bool = False):
    """fp8 bytes of x * scale: (rows, cols) and / or the transposed (cols, rows) copy, as uint8 tensors."""
    rows, cols = x2.shape
    assert x2.stride(1) == 1
    row = torch.empty((rows, cols), dtype=torch.uint8, device=x2.device) if want_row else None
    t = torch.empty((cols, rows), dtype=torch.uint8, device=x2.device) if want_t else None
    _check(lib().kf_fp8_cast_bf16(x2.data_ptr(), rows, cols, x2.stride(0), scale.data_ptr(), int(e5m2),
                                  row.data_ptr() if want_row else None, cols, t.data_ptr() if want_t else None, rows,
                                  _stream()), "kf_fp8_cast_bf16")
    return row, t


def gemm_fp8(a8: torch.Tensor, b8: torch.Tensor, sa: torch.Tensor, sb: torch.Tensor, a_e5m2: bool = False,
             b_e5m2: bool = False, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """bf16 (M, N) = a8 (M, K) @ b8 (N, K)ᵀ / (sa * sb) on the fp8 tensor cores."""
    m, k = a8.shape
    n = b8.shape[0]
    assert b8.shape[1] == k and a8.stride(1) == 1 and b8.stride(1) == 1
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=a8.device)
        accumulate = False
    assert out.stride(1) == 1
    _check(lib().kf_gemm_fp8(a8.data_ptr(), b8.data_ptr(), out.data_ptr(), m, n, k, a8.stride(0), b8.stride(0),
                             out.stride(0), int(a_e5m2), int(b_e5m2), sa.data_ptr(), sb.data_ptr(), int(accumulate),
                             sm_count(), _stream()), "kf_gemm_fp8")
    return out


# --------------------------------------------------------------------------- attention
def attn_policy() -> str:
    """``KF_ATTN``: "native" (default) = the tcgen05 kernels wherever they apply (training blocks included; shapes
    they do not cover fall back to the library call); "library" = never."""
    v = os.environ.get("KF_ATTN", "native")
    return "native" if v == "auto" else v


def _attn_rows_ok(t: torch.Tensor) -> bool:
    """(B, S, heads, hd) whose (b, s) pairs form evenly pitched rows with the heads side by side."""
    b, s, _, hd = t.shape
    return (t.stride(-1) == 1 and t.stride(2) == hd and (b == 1 or t.stride(0) == s * t.stride(1))
            and t.stride(1) % 8 == 0 and t.data_ptr() % 16 == 0)


def attn_supported(q, k, v, causal: bool, needs_grad: bool = False) -> bool:
    """Shapes the tcgen05 attention kernels cover: bf16, head dim 64 or 128, grouped KV heads, causal or full,
    optional document ids; q / k / v may be strided views of one fused projection output."""
    L = lib()
    if getattr(L, "kf_attn_fwd_bf16", None) is None or attn_policy() == "library":
        return False
    if needs_grad and (getattr(L, "kf_attn_bwd_bf16", None) is None or q.shape[-1] != 128):
        return False
    if q.dtype != torch.bfloat16 or q.shape[-1] not in (64, 128) or q.shape[2] % k.shape[2] != 0:
        return False
    if causal and q.shape[1] != k.shape[1]:
        return False
    return _attn_rows_ok(q) and _attn_rows_ok(k) and _attn_rows_ok(v)


def attn_fwd(q, k, v, causal: bool, doc_ids, scale: float):
    """q (B, Sq, H, hd), k / v (B, Sk, Hkv, hd) -> out (B, Sq, H, hd) bf16 and lse (B, H, Sq) fp32."""
    b, sq, h, hd = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    out = torch.empty((b, sq, h, hd), dtype=q.dtype, device=q.device)
    lse = torch.empty((b, h, sq), dtype=torch.float32, device=q.device)
    doc = None
    if doc_ids is not None:
        doc = doc_ids.to(torch.int32).contiguous()
    # two query tiles per CTA (interleaved softmax) once there are at least two tiles; KF_ATTN_FWD=1 forces the
    # single-tile kernel
    L = lib()
    two = sq > 128 and getattr(L, "kf_attn_fwd2_bf16", None) is not None and os.environ.get("KF_ATTN_FWD", "2") != "1"
    fn = L.kf_attn_fwd2_bf16 if two else L.kf_attn_fwd_bf16
    _check(
        fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                               doc.data_ptr() if doc is not None else None, b, sq, sk, h, hkv, hd, q.stride(1),
           k.stride(1), v.stride(1), h * hd, float(scale), int(causal), _stream()),
        "kf_attn_fwd2_bf16" if two else "kf_attn_fwd_bf16",
    )
    return out, lse


# --------------------------------------------------------------------------- Lion / schedule-free AdamW
def _same_flat(*ts: torch.Tensor) -> bool:
    d = ts[0].dtype
    return d in _DT and all(t.is_cuda and t.dtype == d and t.is_contiguous() and t.numel() == ts[0].numel() for t in ts)


def lion_step(p, g, m, lr: float, b1: float, b2: float, wd: float) -> bool:
    """In-place Lion update of one tensor; False when the tensors do not qualify (mixed dtypes, strided)."""
    if getattr(lib(), "kf_lion", None) is None or not _same_flat(p, g, m):
        return False
    _check(lib().kf_lion(p.data_ptr(), g.data_ptr(), m.data_ptr(), p.numel(), _DT[p.dtype], lr, b1, b2, wd, _stream()), "kf_lion")
    return True


def sf_adamw_step(y, g, z, v, x, lr, b1, b2, eps, wd, bc2, ck, first: bool) -> bool:
    """In-place schedule-free AdamW update: y is the tensor the model reads, z / x the base and averaged iterates."""
    if getattr(lib(), "kf_sf_adamw", None) is None or not _same_flat(y, g, z, v, x):
        return False
    _check(lib().kf_sf_adamw(y.data_ptr(), g.data_ptr(), z.data_ptr(), v.data_ptr(), x.data_ptr(), y.numel(), _DT[y.dtype],
                             lr, b1, b2, eps, wd, bc2, ck, int(first), _stream()), "kf_sf_adamw")
    return True


# --------------------------------------------------------------------------- mixture of experts
def router_topk(logits: torch.Tensor, bias: torch.Tensor | None, sigmoid: bool, k: int):
    """(weights fp32 (T, k), indices int64 (T, k), counts fp32 (E), prob_sum fp32 (E), sum of logsumexp² fp32 (1))."""
    t, e = logits.shape
    assert logits.is_contiguous() and logits.dtype in (torch.bfloat16, torch.float32)
    idx = torch.empty((t, k), dtype=torch.int64, device=logits.device)
    w = torch.empty((t, k), dtype=torch.float32, device=logits.device)
    acc = torch.zeros(2 * e + 1, dtype=torch.float32, device=logits.device)
    b = bias.float().contiguous() if bias is not None else None
    _check(lib().kf_router_topk(logits.data_ptr(), 0 if logits.dtype == torch.bfloat16 else 1,
                                b.data_ptr() if b is not None else None, int(sigmoid), t, e, k, idx.data_ptr(),
                                w.data_ptr(), acc.data_ptr(), acc[e:].data_ptr(), acc[2 * e:].data_ptr(), _stream()),
           "kf_router_topk")
    return w, idx, acc[:e], acc[e:2 * e], acc[2 * e:]


def moe_capacity_mask(indices: torch.Tensor, num_experts: int, cap: int) -> torch.Tensor:
    """fp32 (T, k) mask: 1 for the first ``cap`` tokens (sequence order) of every (slot, expert) pair, else 0."""
    t, k = indices.shape
    assert indices.dtype == torch.int64 and indices.is_contiguous()
    keep = torch.empty((t, k), dtype=torch.float32, device=indices.device)
    _check(lib().kf_moe_capacity_mask(indices.data_ptr(), t, k, num_experts, int(cap), keep.data_ptr(), _stream()),
           "kf_moe_capacity_mask")
    return keep


def moe_sort(indices: torch.Tensor, num_experts: int):
    """Stable sort of the (token, k) assignments by expert: (offsets int32 (E + 1), row_of_slot int32, slot_of_row int32)."""
    flat = indices.reshape(-1)
    assert flat.dtype == torch.int64 and flat.is_contiguous()
    slots = flat.numel()
    nb = (slots + 255) // 256
    scratch = torch.empty(max(nb, 1) * num_experts, dtype=torch.int32, device=flat.device)
    offsets = torch.empty(num_experts + 1, dtype=torch.int32, device=flat.device)
    row_of_slot = torch.empty(slots, dtype=torch.int32, device=flat.device)
    slot_of_row = torch.empty(slots, dtype=torch.int32, device=flat.device)
    _check(lib().kf_moe_sort(flat.data_ptr(), slots, num_experts, scratch.data_ptr(), offsets.data_ptr(),
                             row_of_slot.data_ptr(), slot_of_row.data_ptr(), _stream()), "kf_moe_sort")
    return offsets, row_of_slot, slot_of_row


def moe_gather(x: torch.Tensor, slot_of_row: torch.Tensor, k: int) -> torch.Tensor:
    rows, cols = slot_of_row.numel(), x.shape[1]
    out = torch.empty((rows, cols), dtype=x.dtype, device=x.device)
    _check(lib().kf_moe_gather_bf16(x.data_ptr(), slot_of_row.data_ptr(), rows, k, cols, out.data_ptr(), _stream()),
           "kf_moe_gather_bf16")
    return out


def moe_combine(y: torch.Tensor, row_of_slot: torch.Tensor, w: torch.Tensor | None, tokens: int, k: int) -> torch.Tensor:
    cols = y.shape[1]
    out = torch.empty((tokens, cols), dtype=y.dtype, device=y.device)
    _check(lib().kf_moe_combine_bf16(y.data_ptr(), row_of_slot.data_ptr(), w.data_ptr() if w is not None else None,
                                     tokens, k, cols, out.data_ptr(), _stream()), "kf_moe_combine_bf16")
    return out


def moe_combine_bwd(dout: torch.Tensor, y: torch.Tensor, slot_of_row: torch.Tensor, w: torch.Tensor, k: int):
    rows, cols = y.shape
    dy = torch.empty_like(y)
    dw = torch.empty(rows, dtype=torch.float32, device=y.device)
    _check(lib().kf_moe_combine_bwd_bf16(dout.data_ptr(), y.data_ptr(), slot_of_row.data_ptr(), w.data_ptr(), rows, k, cols,
                                         dy.data_ptr(), dw.data_ptr(), _stream()), "kf_moe_combine_bwd_bf16")
    return dy, dw


def grouped_swiglu(a: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, offsets: torch.Tensor, b_mn: bool,
                   want_gu: bool = True):
    """(h, gu): h = silu(a @ Wg_e) * (a @ Wu_e) over the ragged expert row ranges in ONE grouped GEMM (activation in
    its epilogue); ``gu`` (rows, 2F) keeps the bf16 pre-activations (gate | up) when ``want_gu``.  Weights (E, F, K)
    or, with ``b_mn``, (E, K, F).  Rows past ``offsets[E]`` are left untouched."""
    rows, k = a.shape
    e = wg.shape[0]
    f = wg.shape[2] if b_mn else wg.shape[1]
    assert wg.shape == wu.shape and wg.is_contiguous() and wu.is_contiguous() and a.stride(1) == 1
    h = torch.empty((rows, f), dtype=torch.bfloat16, device=a.device)
    gu = torch.empty((rows, 2 * f), dtype=torch.bfloat16, device=a.device) if want_gu else None
    _check(lib().kf_grouped_swiglu_bf16(a.data_ptr(), wg.data_ptr(), wu.data_ptr(), h.data_ptr(),
                                        gu.data_ptr() if gu is not None else None, offsets.data_ptr(), rows, e, f, k,
                                        a.stride(0), f, 2 * f, int(b_mn), sm_count(), _stream()), "kf_grouped_swiglu_bf16")
    return h, gu


def grouped_swiglu_supported(a: torch.Tensor, wg: torch.Tensor, b_mn: bool) -> bool:
    return getattr(lib(), "kf_grouped_swiglu_bf16", None) is not None and grouped_gemm_supported(a, wg, b_mn) \
        and not os.environ.get("KF_DISABLE_GROUPED_SWIGLU")


def grouped_swiglu_bwd(dy: torch.Tensor, w_down: torch.Tensor, gu: torch.Tensor, offsets: torch.Tensor, b_mn: bool) -> torch.Tensor:
    """d[gate | up] (rows, 2F), written over ``gu``: the input-gradient product of the experts' down projection
    (``dy`` (rows, K) times ``w_down``: (E, F, K), or (E, K, F) with ``b_mn``) with the SwiGLU gradient in its epilogue;
    the gradient of the hidden activation is never written to memory.  Rows past ``offsets[E]`` stay untouched."""
    rows, k = dy.shape
    e = w_down.shape[0]
    f = w_down.shape[2] if b_mn else w_down.shape[1]
    assert gu.shape == (rows, 2 * f) and gu.is_contiguous() and w_down.is_contiguous() and dy.stride(1) == 1
    _check(lib().kf_grouped_swiglu_bwd_bf16(dy.data_ptr(), w_down.data_ptr(), gu.data_ptr(), gu.data_ptr(), offsets.data_ptr(),
                                            rows, e, f, k, dy.stride(0), 2 * f, int(b_mn), sm_count(), _stream()),
           "kf_grouped_swiglu_bwd_bf16")
    return gu


def grouped_swiglu_bwd_supported(dy: torch.Tensor, w_down: torch.Tensor, b_mn: bool) -> bool:
    return (getattr(lib(), "kf_grouped_swiglu_bwd_bf16", None) is not None and grouped_gemm_supported(dy, w_down, b_mn)
            and os.environ.get("KF_SWIGLU_BWD_EPILOGUE", "1") == "1" and not os.environ.get("KF_DISABLE_GROUPED_SWIGLU")
            and dy.shape[0] >= 256 and sm_count() >= 2)


def swiglu_bwd_ragged(dh: torch.Tensor, gu: torch.Tensor, offsets: torch.Tensor) -> torch.Tensor:
    """dgu (rows, 2F) of h = silu(gate) * up for the rows below ``offsets[-1]`` (a device int; later rows untouched)."""
    rows, f = dh.shape
    assert gu.shape == (rows, 2 * f) and dh.is_contiguous() and gu.is_contiguous()
    dgu = torch.empty_like(gu)
    _check(lib().kf_swiglu_bwd_ragged_bf16(dh.data_ptr(), gu.data_ptr(), dgu.data_ptr(), rows, offsets[-1:].data_ptr(), f,
                                           _stream()), "kf_swiglu_bwd_ragged_bf16")
    return dgu


def grouped_gemm(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor, b_mn: bool, out: torch.Tensor | None = None,
                 accumulate: bool = False):
    """Ragged grouped GEMM: rows ``offsets[e]:offsets[e+1]`` of ``a`` (rows, K) are multiplied by expert e's matrix.
    ``b`` is (E, N, K) when ``b_mn`` is False and (E, K, N) when True; ``offsets`` is int32 (E + 1) on the device.
    ``accumulate``: add to ``out``."""
    rows, k = a.shape
    e = b.shape[0]
    n = b.shape[2] if b_mn else b.shape[1]
    assert (b.shape[1] if b_mn else b.shape[2]) == k and b.is_contiguous() and a.stride(1) == 1
    assert offsets.dtype == torch.int32 and offsets.numel() == e + 1
    if out is None:
        out = torch.empty((rows, n), dtype=torch.bfloat16, device=a.device)
    _check(lib().kf_grouped_gemm_acc_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), offsets.data_ptr(), rows, e, n, k,
                                          a.stride(0), out.stride(0), int(b_mn), int(accumulate), sm_count(), _stream()),
           "kf_grouped_gemm_acc_bf16")
    return out


def grouped_gemm_supported(a: torch.Tensor, b: torch.Tensor, b_mn: bool) -> bool:
    if getattr(lib(), "kf_grouped_gemm_bf16", None) is None or a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        return False
    k = a.shape[1]
    n = b.shape[2] if b_mn else b.shape[1]
    return (b.shape[0] <= 256 and k % 8 == 0 and n % 8 == 0 and (not b_mn or k % 64 == 0) and a.stride(1) == 1
            and a.stride(0) % 8 == 0 and b.is_contiguous())


def grouped_wgrad(a: torch.Tensor, b: torch.Tensor, offsets: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Per-expert ``a_e^T @ b_e`` over the ragged row ranges ``offsets[e]:offsets[e+1]``: (E, a.shape[1], b.shape[1])
    in bf16.  The weight gradient of :func:`grouped_gemm`; experts without rows get zeros."""
    rows, m = a.shape
    n = b.shape[1]
    e = offsets.numel() - 1
    assert b.shape[0] == rows and a.stride(1) == 1 and b.stride(1) == 1 and offsets.dtype == torch.int32
    if out is None:
        out = torch.empty((e, m, n), dtype=torch.bfloat16, device=a.device)
    assert out.shape == (e, m, n) and out.is_contiguous() and out.dtype == torch.bfloat16
    _check(lib().kf_grouped_wgrad_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), offsets.data_ptr(), rows, e, m, n,
                                       a.stride(0), b.stride(0), sm_count(), _stream()), "kf_grouped_wgrad_bf16")
    return out


def grouped_wgrad_supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    if os.environ.get("KF_GROUPED_WGRAD", "1") == "0":  # escape hatch: weight gradients through torch._grouped_mm
        return False
    if getattr(lib(), "kf_grouped_wgrad_bf16", None) is None or a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        return False
    return (a.shape[0] > 0 and a.shape[1] % 8 == 0 and b.shape[1] % 8 == 0 and a.stride(1) == 1 and b.stride(1) == 1
            and a.stride(0) % 8 == 0 and b.stride(0) % 8 == 0)


def all_gather_gemm(x_shard: torch.Tensor, w: torch.Tensor, ctx, seq_len: int, out: torch.Tensor | None = None,
                    w_kn: bool = False) -> torch.Tensor:
    """out[T, N] = gather over the ranks of ``ctx`` (along the sequence) of x_shard[T/tp, K], times the weight: w is
    (N, K) or, with ``w_kn``, (K, N) (the layout the input-gradient GEMM of a row-parallel Linear needs).  The shard is
    pushed to the peers by copy warps of the GEMM kernel itself.  ``ctx`` is a ``comm.fused_tp.AgGemmContext``."""
    tl, k = x_shard.shape
    t = tl * ctx.world
    n = w.shape[1] if w_kn else w.shape[0]
    assert x_shard.stride(1) == 1 and w.stride(1) == 1 and (w.shape[0] if w_kn else w.shape[1]) == k
    if out is None:
        out = torch.empty((t, n), dtype=torch.bfloat16, device=x_shard.device)
    ctx.reserve(t, k)
    _check(
        lib().kf_ag_gemm_bf16(x_shard.data_ptr(), w.data_ptr(), ctx.stage_ptrs, ctx.flag_ptrs, out.data_ptr(), t, n, k,
                              seq_len, x_shard.stride(0), w.stride(0), out.stride(0), ctx.world, ctx.rank, ctx.next_call(),
                              int(w_kn), sm_count(), _stream()),
        "kf_ag_gemm_bf16",
    )
    return out


def gemm_reduce_scatter(x2: torch.Tensor, w: torch.Tensor, ctx, seq_len: int, out: torch.Tensor | None = None,
                        residual: torch.Tensor | None = None, w_kn: bool = False) -> torch.Tensor:
    """out[T/tp, D] = reduce-scatter over the ranks of ``ctx`` of x2[T, K_local] times the weight (+ residual): w is
    (D, K_local) or, with ``w_kn``, (K_local, D) (the input-gradient GEMM of a column-parallel Linear).  Tiles are pushed
    to their owners from the GEMM epilogue.  ``ctx`` is a ``comm.fused_tp.GemmRSContext``."""
    t, k = x2.shape
    d = w.shape[1] if w_kn else w.shape[0]
    assert x2.stride(1) == 1 and w.stride(1) == 1 and (w.shape[0] if w_kn else w.shape[1]) == k
    tl = t // ctx.world
    if out is None:
        out = torch.empty((tl, d), dtype=torch.bfloat16, device=x2.device)
    ctx.reserve(t, d)
    _check(
        lib().kf_gemm_rs_bf16(x2.data_ptr(), w.data_ptr(), ctx.stage_ptrs, ctx.flag_ptrs, out.data_ptr(),
                              residual.data_ptr() if residual is not None else None, t, d, k, seq_len, x2.stride(0),
                              w.stride(0), ctx.world, ctx.rank, ctx.next_call(), int(w_kn), sm_count(), _stream()),
        "kf_gemm_rs_bf16",
    )
    return out


def grouped_pair_mode(mode: int) -> None:
    """1: the ragged grouped GEMMs run on CTA-pair tiles (default); 0: single-CTA 128 x 256 tiles."""
    lib().kf_grouped_pair_mode(int(mode))


def attn_bwd_dq_mode(mode: int) -> int:
    """How the attention backward adds its dQ tiles to the fp32 accumulator: 0 = one ``red.global`` per element,
    1 = one bulk tensor reduction (TMA) per tile staged in shared memory (default, 1.75x faster on the 8B shape).
    Returns the previous mode.  ``KF_ATTN_BWD_DQ=red`` selects 0 at load time."""
    return int(lib().kf_attn_bwd_dq_mode(int(mode)))


def gemm_rope_supported(x2: torch.Tensor, w: torch.Tensor, hd: int) -> bool:
    """The rotary epilogue lives in the CTA-pair kernel: bf16, head dim 64 / 128 / 256, whole heads per weight."""
    return (getattr(lib(), "kf_gemm_rope_bf16", None) is not None and hd in (64, 128, 256) and w.shape[0] % hd == 0
            and x2.dtype == torch.bfloat16 and x2.stride(0) % 8 == 0 and w.stride(0) % 8 == 0)


def attn_bwd(dout, q, k, v, out, lse, causal: bool, doc_ids, scale: float, dq=None, dk=None, dv=None, rope=None):
    """Gradients of ``attn_fwd``.  ``dq`` / ``dk`` / ``dv`` may be preallocated (strided) destinations, e.g. the
    three head ranges of one fused projection gradient; otherwise contiguous tensors are returned.
    ``rope = (cos, sin)`` (fp32 (S, 64)): dq and dk leave through the inverse rotary embedding, i.e. they are the
    gradients of the un-rotated projections when q and k were rotated after the projection."""
    b, sq, h, hd = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    if dout.stride(-1) != 1 or dout.stride(2) != hd or (b > 1 and dout.stride(0) != sq * dout.stride(1)):
        dout = dout.contiguous()
    dq = torch.empty((b, sq, h, hd), dtype=q.dtype, device=q.device) if dq is None else dq
    dk = torch.empty((b, sk, hkv, hd), dtype=q.dtype, device=q.device) if dk is None else dk
    dv = torch.empty((b, sk, hkv, hd), dtype=q.dtype, device=q.device) if dv is None else dv
    for t in (dq, dk, dv, out, dout):
        assert _attn_rows_ok(t), "attention gradients need evenly pitched rows with adjacent heads"
    dsum = torch.empty((b, h, sq), dtype=torch.float32, device=q.device)
    dq_acc = torch.empty((b, sq, h, hd), dtype=torch.float32, device=q.device)
    doc = doc_ids.to(torch.int32).contiguous() if doc_ids is not None else None
    cos = sin = None
    if rope is not None:
        cos, sin = rope
        assert sq == sk and cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()
        assert cos.shape[-1] == hd // 2 and cos.numel() >= sq * (hd // 2)
    _check(
        lib().kf_attn_bwd_rope_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), dout.data_ptr(),
                                    lse.data_ptr(), dsum.data_ptr(), dq_acc.data_ptr(), dq.data_ptr(), dk.data_ptr(),
                                    dv.data_ptr(), doc.data_ptr() if doc is not None else None, b, sq, sk, h, hkv, hd,
                                    q.stride(1), k.stride(1), v.stride(1), out.stride(1), dout.stride(1), dq.stride(1),
                                    dk.stride(1), dv.stride(1), float(scale), int(causal),
                                    cos.data_ptr() if cos is not None else None,
                                    sin.data_ptr() if sin is not None else None, _stream()),
        "kf_attn_bwd_rope_bf16",
    )
    return dq, dk, dv


# --------------------------------------------------------------------------- fused communication kernels
SYMM_RS_BLOCKS = int(os.environ.get("KF_SYMM_RS_BLOCKS", "296"))        # grid cap of the fused reduce-scatter kernel
SYMM_ADAMW_BLOCKS = int(os.environ.get("KF_SYMM_ADAMW_BLOCKS", "592"))  # grid cap of the fused AdamW + publication kernel


def symm_rs_norm(buf, lo: int, n: int, sumsq_out: torch.Tensor, accumulate: bool, max_blocks: int | None = None) -> None:
    """Average this rank's shard [lo, lo+n) of a symmetric gradient buffer over all ranks (in place, own copy)
    and add the squared norm of the result to ``sumsq_out[0]``.  The kernel runs beside the backward GEMMs on a side
    stream; ``max_blocks`` (default ``KF_SYMM_RS_BLOCKS``) bounds how many SMs it shares with them."""
    max_blocks = SYMM_RS_BLOCKS if max_blocks is None else max_blocks
    partial = torch.empty(1024, dtype=torch.float32, device=buf.tensor.device)
    _check(
        lib().kf_symm_rs_norm_bf16(buf.peer_ptrs, buf.multicast_ptr, buf.world, buf.rank, lo, n, partial.data_ptr(),
                                   sumsq_out.data_ptr(), int(accumulate), max_blocks, _stream()),
        "kf_symm_rs_norm_bf16",
    )


def symm_adamw_bcast(param_buf, grad_shard, m, v, lo: int, n: int, n_decay_global: int, lr, beta1, beta2, eps, wd,
                     step: int, grad_scale=None, skip=None, max_blocks: int | None = None) -> None:
    """AdamW on the shard [lo, lo+n) and store of the new parameters into every rank's parameter buffer."""
    max_blocks = SYMM_ADAMW_BLOCKS if max_blocks is None else max_blocks
    bc1 = 1.0 - beta1**step
    bc2_sqrt = math.sqrt(1.0 - beta2**step)
    _check(
        lib().kf_symm_adamw_bcast_bf16(
            param_buf.peer_ptrs, param_buf.multicast_ptr, param_buf.world, param_buf.rank, grad_shard.data_ptr(),
            m.data_ptr(), v.data_ptr(), lo, n, n_decay_global, lr, beta1, beta2, eps, wd, bc1, bc2_sqrt,
            grad_scale.data_ptr() if grad_scale is not None else None, skip.data_ptr() if skip is not None else None,
            max_blocks, _stream()),
        "kf_symm_adamw_bcast_bf16",
    )


def symm_gather(buf, lo: int, n: int, max_blocks: int = 592) -> None:
    _check(lib().kf_symm_gather_bf16(buf.peer_ptrs, buf.multicast_ptr, buf.world, buf.rank, lo, n, max_blocks, _stream()),
           "kf_symm_gather_bf16")


# --------------------------------------------------------------------------- vocabulary-parallel cross entropy
def ce_vp_stats(logits: torch.Tensor, labels: torch.Tensor, vocab_start: int):
    """Per row of this rank's vocabulary shard (T, V_local) bf16: (max, sum of exp relative to that max, logit of the
    label if the label is in [vocab_start, vocab_start + V_local) else 0), three fp32 (T,) vectors."""
    t, v = logits.shape
    out = torch.empty((3, t), dtype=torch.float32, device=logits.device)
    _check(lib().kf_ce_vp_stats_bf16(logits.data_ptr(), labels.data_ptr(), int(vocab_start), out[0].data_ptr(),
                                     out[1].data_ptr(), out[2].data_ptr(), t, v, logits.stride(0), _stream()),
           "kf_ce_vp_stats_bf16")
    return out[0], out[1], out[2]


def ce_vp_bwd(logits: torch.Tensor, labels: torch.Tensor, vocab_start: int, lse: torch.Tensor, inv_n: torch.Tensor,
              upstream: torch.Tensor | None, z_weight: float) -> torch.Tensor:
    """In place: logits <- gradient of the mean (over valid rows) cross entropy (+ z-loss) given the global
    log-sum-exp ``lse`` (T,); ``inv_n`` and ``upstream`` are device scalars."""
    t, v = logits.shape
    _check(lib().kf_ce_vp_bwd_bf16(logits.data_ptr(), labels.data_ptr(), int(vocab_start), lse.data_ptr(), inv_n.data_ptr(),
                                   upstream.data_ptr() if upstream is not None else None, float(z_weight), t, v,
                                   logits.stride(0), _stream()), "kf_ce_vp_bwd_bf16")
    return logits


# --------------------------------------------------------------------------- sharded parameters (ZeRO-3)
def _ll_array(values):
    return (ctypes.c_longlong * len(values))(*[int(v) for v in values])


def symm_pull(shard_buf, full_offsets, lengths, shard_offsets, dst: torch.Tensor, max_blocks: int = 592) -> None:
    """All-gather of up to 16 parameters of a sharded unit into the full-layout buffer ``dst``: parameter i
    (``lengths[i]`` elements, cut into ``world`` equal pieces) is assembled at ``dst[full_offsets[i]:]`` from every
    rank's piece at ``shard_offsets[i]`` of its shard (``shard_buf``: the symmetric shard buffer)."""
    _check(lib().kf_symm_pull_bf16(shard_buf.peer_ptrs, shard_buf.world, len(lengths), _ll_array(full_offsets),
                                   _ll_array(lengths), _ll_array(shard_offsets), dst.data_ptr(), max_blocks, _stream()),
           "kf_symm_pull_bf16")


def symm_rs_shard(grad_buf, full_offsets, lengths, shard_offsets, shard_grad: torch.Tensor, accumulate: bool,
                  max_blocks: int | None = None) -> None:
    """Reduce-scatter of full-layout gradient staging buffers (``grad_buf``: symmetric) into this rank's gradient
    shard: the mean over ranks of this rank's piece of every listed parameter is written (or added) to
    ``shard_grad[shard_offsets[i]:]``."""
    max_blocks = SYMM_RS_BLOCKS if max_blocks is None else max_blocks
    _check(lib().kf_symm_rs_shard_bf16(grad_buf.peer_ptrs, grad_buf.multicast_ptr, grad_buf.world, grad_buf.rank,
                                       len(lengths), _ll_array(full_offsets), _ll_array(lengths), _ll_array(shard_offsets),
                                       shard_grad.data_ptr(), int(accumulate), max_blocks, _stream()),
           "kf_symm_rs_shard_bf16")


def gemm_gather(x2: torch.Tensor, plan: dict, n: int, *, epi: int = 0, residual: torch.Tensor | None = None,
                rope: tuple | None = None, want_gu: bool = True):
    """GEMM whose weight operand is gathered from the data-parallel ranks' parameter shards inside the kernel.

    ``plan`` comes from ``ShardedDataParallelEngine.gather_plan`` (shard buffer, segment rows / shard offsets, the
    staging view that receives the operand, scratch flags).  ``epi`` 0: ``x W^T (+ residual)`` -> (M, n);
    1: SwiGLU over W = [gate ; up] with hidden size ``n`` -> (h (M, n), gu (M, 2n) or None); 2: rotary epilogue
    (``rope`` as in :func:`gemm`) -> (M, n).  Afterwards the staging view holds the whole weight."""
    m, k = x2.shape
    symm = plan["symm"]
    out = torch.empty((m, n), dtype=torch.bfloat16, device=x2.device)
    r_ptr, ldr, gu = None, 0, None
    if epi == 1 and want_gu:
        gu = torch.empty((m, 2 * n), dtype=torch.bfloat16, device=x2.device)
        r_ptr, ldr = gu.data_ptr(), 2 * n
    elif epi == 0 and residual is not None:
        assert residual.shape == (m, n) and residual.stride(1) == 1
        r_ptr, ldr = residual.data_ptr(), residual.stride(0)
    cos_p = sin_p = None
    s_len = rope_cols = hd = 0
    if epi == 2:
        cos, sin, s_len, rope_cols, hd = rope
        cos_p, sin_p = cos.data_ptr(), sin.data_ptr()
    code = lib().kf_gemm_gather_bf16(
        epi, x2.data_ptr(), out.data_ptr(), r_ptr, m, n, k, x2.stride(0), n, ldr, symm.peer_ptrs, symm.world, symm.rank,
        len(plan["seg_rows"]), _ll_array(plan["seg_rows"]), _ll_array(plan["seg_src"]), plan["stage"].data_ptr(),
        plan["flags"].data_ptr(), cos_p, sin_p, int(s_len), int(rope_cols), int(hd), sm_count(), _stream())
    _check(code, "kf_gemm_gather_bf16")
    return (out, gu) if epi == 1 else out
