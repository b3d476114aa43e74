"""Mixture of modality-aware experts (MoMa): shared attention, per-modality expert-choice feed-forward.

Tokens are split by ``modality_ids``; inside a modality every expert *chooses* its top ``ceil(c * N)`` tokens by
an independent sigmoid score (with Gumbel noise on the logits while training), computes its MLP on them and adds
the score-weighted result back.  Tokens that no expert picks pass through with a zero FFN contribution.
Padded positions (``key_padding_mask`` false) are not routed.

Parity: kempnerforge/model/moma.py:71-468 (router / ``experts.{modality}.experts.{j}`` parameter names, default
capacity 1 / num_experts, ``expert_counts`` per modality, zero-token modalities pass through).
"""

from __future__ import annotations

import math

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from kempnerforge_b200.models.attention import Attention
from kempnerforge_b200.models.mlp import build_mlp
from kempnerforge_b200.models.norm import build_norm
from kempnerforge_b200.models.recompute import checkpoint_contexts


def _gumbel_like(t: torch.Tensor) -> torch.Tensor:
    u = torch.rand_like(t, dtype=torch.float32).clamp_(1e-9, 1.0 - 1e-9)
    return (-torch.log(-torch.log(u))).to(t.dtype)


class ExpertChoiceSigmoidRouter(nn.Module):
    def __init__(self, dim: int, num_experts: int, capacity_factor: float, gumbel_noise: bool = True) -> None:
        super().__init__()
        if num_experts <= 0:
            raise ValueError(f"ExpertChoiceSigmoidRouter: num_experts must be positive (got {num_experts})")
        if capacity_factor <= 0:
            raise ValueError(f"ExpertChoiceSigmoidRouter: capacity_factor must be positive (got {capacity_factor})")
        self.gate = nn.Linear(dim, num_experts, bias=False)
        self.num_experts, self.capacity_factor, self.gumbel_noise = num_experts, capacity_factor, gumbel_noise
        self.expert_counts = torch.zeros(num_experts)

    def forward(self, x: torch.Tensor):
        """x (N, D) -> (scores (E, k_e), token indices (E, k_e))."""
        if x.dim() != 2:
            raise ValueError(f"ExpertChoiceSigmoidRouter.forward expects (N, D); got shape {tuple(x.shape)}")
        n = x.shape[0]
        if n == 0:
            return x.new_zeros(self.num_experts, 0), torch.zeros(self.num_experts, 0, dtype=torch.long, device=x.device)
        logits = self.gate(x)
        if self.training and self.gumbel_noise:
            logits = logits + _gumbel_like(logits) - _gumbel_like(logits)
        scores = torch.sigmoid(logits)
        k_e = min(n, max(1, math.ceil(self.capacity_factor * n)))
        top_scores, top_idx = torch.topk(scores.t(), k=k_e, dim=1)
        self.expert_counts = torch.full((self.num_experts,), float(k_e), device=x.device)
        return top_scores, top_idx


class ExpertChoiceMoE(nn.Module):
    def __init__(self, dim: int, hidden_dim: int, num_experts: int, capacity_factor: float, activation: str = "silu",
                 gumbel_noise: bool = True) -> None:
        super().__init__()
        self.dim, self.num_experts = dim, num_experts
        self.router = ExpertChoiceSigmoidRouter(dim, num_experts, capacity_factor, gumbel_noise)
        self.experts = nn.ModuleList(build_mlp(dim, hidden_dim, activation) for _ in range(num_experts))

    @property
    def expert_counts(self) -> torch.Tensor:
        return self.router.expert_counts

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if x.dim() != 2:
            raise ValueError(f"ExpertChoiceMoE.forward expects (N, D); got shape {tuple(x.shape)}")
        if x.shape[0] == 0:
            return x
        scores, idx = self.router(x)
        out = torch.zeros_like(x)
        for e, expert in enumerate(self.experts):
            picked = x.index_select(0, idx[e])
            out = out.index_add(0, idx[e], scores[e].unsqueeze(-1).to(x.dtype) * expert(picked))
        return out


class MoMaFFN(nn.Module):
    def __init__(self, config, modalities, experts_per_modality: dict[str, int],
                 capacity_factor_per_modality: dict[str, float], gumbel_noise: bool = True) -> None:
        super().__init__()
        if not modalities:
            raise ValueError("MoMaFFN requires at least one modality")
        for label, table in (("experts_per_modality", experts_per_modality),
                             ("capacity_factor_per_modality", capacity_factor_per_modality)):
            missing = set(modalities) - set(table)
            if missing:
                raise ValueError(f"MoMaFFN: {label} missing entries for {sorted(missing)}")
        self.modalities = tuple(modalities)
        self.experts = nn.ModuleDict({
            m: ExpertChoiceMoE(config.dim, config.computed_expert_ffn_hidden_dim, experts_per_modality[m],
                               capacity_factor_per_modality[m], config.activation, gumbel_noise)
            for m in self.modalities})
        self.aux_loss = torch.tensor(0.0)
        self.z_loss = torch.tensor(0.0)

    def forward(self, x: torch.Tensor, modality_ids: torch.Tensor, key_padding_mask: torch.Tensor | None = None):
        if x.dim() != 3:
            raise ValueError(f"MoMaFFN.forward expects (B, S, D); got shape {tuple(x.shape)}")
        if modality_ids.shape != x.shape[:2]:
            raise ValueError(f"MoMaFFN.forward: modality_ids shape {tuple(modality_ids.shape)} does not match {tuple(x.shape[:2])}")
        if modality_ids.dtype != torch.long:
            raise ValueError(f"MoMaFFN.forward: modality_ids dtype must be torch.long (got {modality_ids.dtype})")
        b, s, d = x.shape
        flat = x.reshape(b * s, d)
        mod = modality_ids.reshape(-1)
        valid = key_padding_mask.reshape(-1) if key_padding_mask is not None else None
        out = torch.zeros_like(flat)
        routed = 0
        for i, m in enumerate(self.modalities):
            sel = mod == i
            routed += int(sel.sum())
            if valid is not None:
                sel = sel & valid
            idx = sel.nonzero(as_tuple=False).squeeze(-1)
            if idx.numel() == 0:
                continue
            out = out.index_copy(0, idx, self.experts[m](flat.index_select(0, idx)))
        if routed != b * s:
            raise ValueError(
                f"MoMaFFN.forward: modality_ids contains out-of-range values; {b * s - routed} of {b * s} positions "
                f"did not match any modality (allowed: 0..{len(self.modalities) - 1})")
        return out.view(b, s, d)


class MoMaBlock(nn.Module):
    def __init__(self, config, modalities, experts_per_modality=None, capacity_factor_per_modality=None,
                 gumbel_noise: bool | None = None, layer_idx: int | None = None) -> None:
        """Either ``MoMaBlock(config, vlm_config, layer_idx)`` (everything from the VLM section) or the reference's
        explicit form ``MoMaBlock(config, modalities, experts_per_modality, capacity_factor_per_modality, gumbel_noise,
        layer_idx)``."""
        super().__init__()
        if hasattr(modalities, "moma_modalities"):
            vlm_config = modalities
            if layer_idx is None:
                layer_idx = experts_per_modality        # third positional argument of the short form
        else:
            from types import SimpleNamespace

            caps_in = dict(capacity_factor_per_modality or {})
            vlm_config = SimpleNamespace(moma_modalities=tuple(modalities),
                                         moma_experts_per_modality=dict(experts_per_modality or {}),
                                         moma_gumbel_noise=bool(gumbel_noise),
                                         effective_capacity_factor=lambda m: caps_in.get(m, 0.0))
        self.layer_idx = layer_idx
        self.ac_mode = "none"
        self.modalities = tuple(vlm_config.moma_modalities)
        self.attention_norm = build_norm(config.norm_type, config.dim, config.norm_eps)
        self.attention = Attention(config.dim, config.n_heads, config.n_kv_heads, config.head_dim, config.qk_norm,
                                   config.sdpa_backend)
        self.mlp_norm = build_norm(config.norm_type, config.dim, config.norm_eps)
        caps = {m: vlm_config.effective_capacity_factor(m) for m in self.modalities}
        self.mlp = MoMaFFN(config, self.modalities, dict(vlm_config.moma_experts_per_modality), caps,
                           vlm_config.moma_gumbel_noise)

    def _attn_branch(self, x, rope_cos, rope_sin, doc_ids, key_padding_mask):
        return self.attention(self.attention_norm(x), rope_cos, rope_sin, doc_ids=doc_ids, key_padding_mask=key_padding_mask)

    def _body(self, x, rope_cos, rope_sin, modality_ids, doc_ids, key_padding_mask, selective):
        if selective:
            attn = checkpoint(self._attn_branch, x, rope_cos, rope_sin, doc_ids, key_padding_mask, use_reentrant=False,
                              context_fn=checkpoint_contexts)
        else:
            attn = self._attn_branch(x, rope_cos, rope_sin, doc_ids, key_padding_mask)
        x = x + attn
        return x + self.mlp(self.mlp_norm(x), modality_ids=modality_ids, key_padding_mask=key_padding_mask)

    def forward(self, x, rope_cos, rope_sin, modality_ids, *, doc_ids=None, key_padding_mask=None):
        """``ac_mode`` (set by ``apply_ac``): "full" recomputes the whole block in the backward pass (the random state is
        restored, so Gumbel routing noise repeats), "selective" only its attention branch.  (In the reference whole-block
        checkpointing does not reach this block type.)"""
        recompute = self.training and torch.is_grad_enabled()
        if recompute and self.ac_mode == "full":
            return checkpoint(self._body, x, rope_cos, rope_sin, modality_ids, doc_ids, key_padding_mask, False,
                              use_reentrant=False, context_fn=checkpoint_contexts)
        return self._body(x, rope_cos, rope_sin, modality_ids, doc_ids, key_padding_mask,
                          recompute and self.ac_mode == "selective")
