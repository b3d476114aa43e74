"""Plain PyTorch implementations of every hot op.

They serve three purposes: the CPU execution path (tests, gloo runs), the fp32
oracle that each CUDA kernel is checked against, and the definition of the
numerics the kernels must reproduce.

Semantics follow the reference model code:
  RMSNorm fp32 compute then cast back ... kempnerforge/model/norm.py:11-27
  RoPE half-split rotation ............... kempnerforge/model/position.py:12-71
  GQA causal / document-masked attention . kempnerforge/model/attention.py:116-236
  SwiGLU .................................. kempnerforge/model/mlp.py:12-26
  cross entropy (ignore_index=-100) ....... kempnerforge/training/loss.py:19-102
  Newton-Schulz quintic ................... kempnerforge/training/optimizer.py:291-318
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

IGNORE_INDEX = -100


# --------------------------------------------------------------------------- norm
def _wide(x: torch.Tensor) -> torch.Tensor:
    """fp32 for the arithmetic of half-precision inputs; float64 stays float64 (gradient checks run in double)."""
    return x if x.dtype == torch.float64 else x.float()


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    xf = _wide(x)
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * inv * weight.to(xf.dtype)).to(x.dtype)


# --------------------------------------------------------------------------- rope
def rope_tables(head_dim: int, max_seq_len: int, theta: float = 10000.0, device=None):
    """(cos, sin), each (max_seq_len, head_dim // 2) in fp32."""
    half = head_dim // 2
    inv_freq = theta ** (-torch.arange(0, half, dtype=torch.float32, device=device) * 2.0 / head_dim)
    ang = torch.outer(torch.arange(max_seq_len, dtype=torch.float32, device=device), inv_freq)
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate pairs (x[..., i], x[..., i + hd/2]).  x: (B, S, H, hd); cos/sin: (S, hd/2) or (B, S, hd/2)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    if cos.dim() == 2:
        c, s = cos[None, :, None, :], sin[None, :, None, :]
    else:
        c, s = cos[:, :, None, :], sin[:, :, None, :]
    c, s = c.to(x.dtype), s.to(x.dtype)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)


# --------------------------------------------------------------------------- attention
def attention_mask(
    s_q: int,
    s_k: int,
    causal: bool,
    doc_ids: torch.Tensor | None = None,
    key_padding_mask: torch.Tensor | None = None,
    device=None,
) -> torch.Tensor | None:
    """Boolean (B or 1, 1, s_q, s_k) mask, True = may attend; None when nothing is masked."""
    mask = None
    if causal:
        offset = s_k - s_q
        i = torch.arange(s_q, device=device)[:, None]
        j = torch.arange(s_k, device=device)[None, :]
        mask = (j <= i + offset)[None, None]
    if doc_ids is not None:
        same = (doc_ids[:, :, None] == doc_ids[:, None, :])[:, None]
        mask = same if mask is None else (mask & same)
    if key_padding_mask is not None:
        keep = key_padding_mask[:, None, None, :].bool()
        mask = keep if mask is None else (mask & keep)
        # rows with no visible key would produce NaN; let them see everything instead
        dead = ~mask.any(dim=-1, keepdim=True)
        mask = mask | dead
    return mask


def attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    causal: bool = True,
    doc_ids: torch.Tensor | None = None,
    key_padding_mask: torch.Tensor | None = None,
    scale: float | None = None,
    return_weights: bool = False,
):
    """softmax(q kᵀ * scale + mask) v with grouped KV heads.

    q: (B, Sq, H, hd); k, v: (B, Sk, Hkv, hd) with H % Hkv == 0.  Query head h
    reads KV head h // (H // Hkv).  Returns (B, Sq, H, hd).
    """
    b, sq, h, hd = q.shape
    sk, hkv = k.shape[1], k.shape[2]
    group = h // hkv
    scale = 1.0 / math.sqrt(hd) if scale is None else scale
    qf = _wide(q.transpose(1, 2)).reshape(b, hkv, group, sq, hd)
    kf = _wide(k.transpose(1, 2))[:, :, None]
    vf = _wide(v.transpose(1, 2))[:, :, None]
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale  # (B, Hkv, G, Sq, Sk)
    mask = attention_mask(sq, sk, causal, doc_ids, key_padding_mask, device=q.device)
    if mask is not None:
        scores = scores.masked_fill(~mask[:, :, None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    out = torch.matmul(probs, vf).reshape(b, h, sq, hd).transpose(1, 2).to(q.dtype)
    if return_weights:
        return out, probs.reshape(b, h, sq, sk)
    return out


# --------------------------------------------------------------------------- mlp
def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate) * up


# --------------------------------------------------------------------------- loss
def cross_entropy_parts(logits: torch.Tensor, labels: torch.Tensor):
    """Returns (sum of nll over valid tokens, sum of logsumexp², valid count), all fp32 scalars."""
    lf = _wide(logits)
    lse = torch.logsumexp(lf, dim=-1)
    valid = labels != IGNORE_INDEX
    safe = labels.clamp_min(0)
    picked = lf.gather(-1, safe[..., None]).squeeze(-1)
    nll = torch.where(valid, lse - picked, torch.zeros_like(lse))
    z = torch.where(valid, lse * lse, torch.zeros_like(lse))
    return nll.sum(), z.sum(), valid.sum()


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, z_loss_weight: float = 0.0):
    """Mean NLL over labels != -100 (0 when all are ignored) + z_loss_weight * mean(lse²)."""
    nll, z, n = cross_entropy_parts(logits.reshape(-1, logits.shape[-1]), labels.reshape(-1))
    denom = n.clamp_min(1).float()
    loss = nll / denom
    if z_loss_weight:
        loss = loss + z_loss_weight * z / denom
    return loss


# --------------------------------------------------------------------------- optimizers
def adamw_step_(p, g, m, v, step: int, lr: float, b1: float, b2: float, eps: float, wd: float):
    """In-place decoupled-weight-decay Adam, same update order as ``torch.optim.AdamW``."""
    gf = g.float()
    pf = p.float() * (1.0 - lr * wd)
    mf = m.float().mul_(b1).add_(gf, alpha=1.0 - b1)
    vf = v.float().mul_(b2).addcmul_(gf, gf, value=1.0 - b2)
    bc1 = 1.0 - b1**step
    bc2 = 1.0 - b2**step
    denom = (vf.sqrt() / math.sqrt(bc2)).add_(eps)
    pf.addcdiv_(mf, denom, value=-lr / bc1)
    p.copy_(pf)
    m.copy_(mf)
    v.copy_(vf)


NS_COEFFS = (3.4445, -4.7750, 2.0315)


def newton_schulz(g: torch.Tensor, steps: int = 5, eps: float = 1e-7) -> torch.Tensor:
    """Quintic Newton-Schulz orthogonalisation of a 2-D matrix in fp32 (no transpose for tall inputs)."""
    a, b, c = NS_COEFFS
    x = g.float()
    x = x / (x.norm() + eps)
    for _ in range(steps):
        gram = x @ x.T
        poly = b * gram + c * (gram @ gram)
        x = a * x + poly @ x
    return x


# --------------------------------------------------------------------------- moe
def grouped_swiglu_experts(
    x_sorted: torch.Tensor,
    counts: torch.Tensor,
    gate_w: torch.Tensor,
    up_w: torch.Tensor,
    down_w: torch.Tensor,
) -> torch.Tensor:
    """Ragged expert SwiGLU.  x_sorted rows are grouped by expert; counts[e] rows go to expert e.

    gate_w/up_w: (E, D, H); down_w: (E, H, D).
    """
    out = torch.empty_like(x_sorted)
    start = 0
    for e, n in enumerate(counts.tolist()):
        if n == 0:
            continue
        seg = x_sorted[start : start + n]
        hid = F.silu(seg @ gate_w[e]) * (seg @ up_w[e])
        out[start : start + n] = hid @ down_w[e]
        start += n
    return out
