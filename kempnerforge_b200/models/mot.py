"""Mixture-of-Transformers blocks: every modality has its own norms, q/k/v/o projections and feed-forward,
while attention itself runs once over the concatenated (image, then text) sequence.

Each modality's positions restart at zero for the rotary embedding.  Output projections and (dense) down
projections start at zero so a warm-started model reproduces the text-only network at step 0;
``mot_warm_start_from_text_stack`` copies a text-only / joint-decoder state dict into every modality's copy.

Parity: kempnerforge/model/mot.py:35-461 (parameter names ``attn.q_proj.{modality}.weight`` etc.,
``attn_norm.{modality}``, ``mlp.{modality}``, equal head counts across modalities, causal mask over the joint
sequence combined with an optional key-padding mask).
"""

from __future__ import annotations

import logging

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from kempnerforge_b200.models.mlp import build_mlp
from kempnerforge_b200.models.moe import MoEMLP, build_moe
from kempnerforge_b200.models.norm import RMSNorm, build_norm
from kempnerforge_b200.models.recompute import checkpoint_contexts
from kempnerforge_b200.ops import functional as F

log = logging.getLogger(__name__)


class MoTAttention(nn.Module):
    def __init__(self, dim: int, n_heads: int, n_kv_heads: int, modalities: tuple[str, ...],
                 head_dim: int | None = None, qk_norm: bool = False) -> None:
        super().__init__()
        if not modalities:
            raise ValueError("MoTAttention requires at least one modality")
        if n_kv_heads <= 0 or n_heads % n_kv_heads:
            raise ValueError(f"MoTAttention: n_heads={n_heads} must be a positive multiple of n_kv_heads={n_kv_heads}")
        self.modalities = tuple(modalities)
        self.n_heads, self.n_kv_heads = n_heads, n_kv_heads
        self.head_dim = head_dim or dim // n_heads
        hd = self.head_dim
        per = lambda i, o: nn.ModuleDict({m: nn.Linear(i, o, bias=False) for m in self.modalities})  # noqa: E731
        self.q_proj = per(dim, n_heads * hd)
        self.k_proj = per(dim, n_kv_heads * hd)
        self.v_proj = per(dim, n_kv_heads * hd)
        self.o_proj = per(n_heads * hd, dim)
        for m in self.modalities:
            self.o_proj[m].weight._kf_zero_init = True
            nn.init.zeros_(self.o_proj[m].weight)
        self.q_norm = nn.ModuleDict({m: RMSNorm(hd) for m in self.modalities}) if qk_norm else None
        self.k_norm = nn.ModuleDict({m: RMSNorm(hd) for m in self.modalities}) if qk_norm else None

    def forward(self, streams: dict[str, torch.Tensor], rope: dict, is_causal: bool = True,
                key_padding_mask: torch.Tensor | None = None) -> dict[str, torch.Tensor]:
        if set(streams) != set(self.modalities):
            raise ValueError(f"MoTAttention.forward: streams keys {sorted(streams)} != modalities {sorted(self.modalities)}")
        hd, h, hkv = self.head_dim, self.n_heads, self.n_kv_heads
        qs, ks, vs, lengths = [], [], [], {}
        for m in self.modalities:
            x = streams[m]
            b, t, _ = x.shape
            lengths[m] = t
            qkv = F.fused_linear(x, [self.q_proj[m].weight, self.k_proj[m].weight, self.v_proj[m].weight])
            qkv = qkv.view(b, t, h + 2 * hkv, hd)
            if self.q_norm is not None:
                qkv = torch.cat([self.q_norm[m](qkv[:, :, :h]), self.k_norm[m](qkv[:, :, h : h + hkv]),
                                 qkv[:, :, h + hkv :]], dim=2)
            cos, sin = rope[m]
            qkv = F.rope(qkv, cos, sin, n_rot_heads=h + hkv)
            qs.append(qkv[:, :, :h])
            ks.append(qkv[:, :, h : h + hkv])
            vs.append(qkv[:, :, h + hkv :])
        q, k, v = torch.cat(qs, dim=1), torch.cat(ks, dim=1), torch.cat(vs, dim=1)
        out = F.attention(q, k, v, causal=is_causal, key_padding_mask=key_padding_mask)
        result, off = {}, 0
        for m in self.modalities:
            t = lengths[m]
            o = out[:, off : off + t].reshape(out.shape[0], t, h * hd)
            result[m] = F.linear(o, self.o_proj[m].weight)
            off += t
        return result


class MoTBlock(nn.Module):
    def __init__(self, config, modalities, layer_idx: int) -> None:
        """``modalities``: a tuple of stream names, or a VLM config that carries ``mot_modalities``."""
        super().__init__()
        mods = getattr(modalities, "mot_modalities", modalities)
        if not mods:
            raise ValueError("MoTBlock requires at least one modality")
        self.layer_idx = layer_idx
        self.modalities = tuple(mods)
        self.ac_mode = "none"
        norm = lambda: build_norm(config.norm_type, config.dim, config.norm_eps)  # noqa: E731
        self.attn_norm = nn.ModuleDict({m: norm() for m in self.modalities})
        self.attn = MoTAttention(config.dim, config.n_heads, config.n_kv_heads, self.modalities, config.head_dim, config.qk_norm)
        self.mlp_norm = nn.ModuleDict({m: norm() for m in self.modalities})
        if config.is_moe_layer(layer_idx):
            self.mlp = nn.ModuleDict({
                m: build_moe(config.dim, config.computed_expert_ffn_hidden_dim, config.num_experts, config.moe_top_k,
                             config.activation, config.moe_router, config.moe_shared_experts, config.moe_capacity_factor,
                             config.moe_gradient_scale, config.moe_sequence_aux_loss_weight, config.moe_bias_schedule,
                             config.moe_packed_experts)
                for m in self.modalities})
        else:
            self.mlp = nn.ModuleDict({m: build_mlp(config.dim, config.computed_ffn_hidden_dim, config.activation)
                                      for m in self.modalities})
        for m in self.modalities:
            sub = self.mlp[m]
            if not isinstance(sub, MoEMLP) and hasattr(sub, "down_proj"):
                sub.down_proj.weight._kf_zero_init = True
                nn.init.zeros_(sub.down_proj.weight)

    def _attn_branch(self, streams, rope, key_padding_mask):
        return self.attn({m: self.attn_norm[m](streams[m]) for m in self.modalities}, rope, True, key_padding_mask)

    def _body(self, streams, rope, key_padding_mask, selective):
        if selective:
            attn = checkpoint(self._attn_branch, streams, rope, key_padding_mask, use_reentrant=False,
                              context_fn=checkpoint_contexts)
        else:
            attn = self._attn_branch(streams, rope, key_padding_mask)
        mid = {m: streams[m] + attn[m] for m in self.modalities}
        return {m: mid[m] + self.mlp[m](self.mlp_norm[m](mid[m])) for m in self.modalities}

    def forward(self, streams: dict[str, torch.Tensor], rope: dict, key_padding_mask: torch.Tensor | None = None):
        """``ac_mode`` (set by ``apply_ac``): "full" recomputes the whole block in the backward pass, "selective" only
        the joint attention over the streams."""
        if set(streams) != set(self.modalities):
            raise ValueError(f"MoTBlock.forward: streams keys {sorted(streams)} != modalities {sorted(self.modalities)}")
        recompute = self.training and torch.is_grad_enabled()
        if recompute and self.ac_mode == "full":
            return checkpoint(self._body, streams, rope, key_padding_mask, False, use_reentrant=False,
                              context_fn=checkpoint_contexts)
        return self._body(streams, rope, key_padding_mask, recompute and self.ac_mode == "selective")


_PER_MODALITY = ("attention_norm", "attention.q_proj", "attention.k_proj", "attention.v_proj", "attention.o_proj",
                 "attention.q_norm", "attention.k_norm", "mlp_norm", "mlp")
_RENAME = {"attention_norm": "attn_norm", "attention": "attn"}


def text_key_to_mot_keys(key: str, modalities: tuple[str, ...]) -> list[str]:
    """Names under which a text-stack parameter lives in a MoT model (one per modality), or [key] if shared."""
    parts = key.split(".")
    if parts[0] == "norm":
        return [".".join(["mot_norms", m, *parts[1:]]) for m in modalities] + [key]
    if parts[0] != "layers" or len(parts) < 4:
        return [key]
    rest = ".".join(parts[2:])
    for stem in sorted(_PER_MODALITY, key=len, reverse=True):
        if rest == stem or rest.startswith(stem + "."):
            tail = rest[len(stem):]
            new_stem = ".".join(_RENAME.get(p, p) for p in stem.split("."))
            return [f"layers.{parts[1]}.{new_stem}.{m}{tail}" for m in modalities]
    return [key]


@torch.no_grad()
def mot_warm_start_from_text_stack(model: nn.Module, text_state: dict[str, torch.Tensor], strict: bool = False) -> int:
    """Copy a text-only (or joint-decoder) state dict into every modality's parameters of a MoT transformer."""
    mods = tuple(getattr(model, "_mot_modalities", ())) or ("image", "text")
    target = dict(model.state_dict())
    copied = 0
    for key, value in text_state.items():
        key = key.removeprefix("transformer.")
        for name in text_key_to_mot_keys(key, mods):
            dst = target.get(name)
            if dst is None:
                if strict and name != key:
                    raise KeyError(f"{name} (from {key}) not found in the MoT model")
                continue
            local = dst.to_local() if hasattr(dst, "to_local") else dst
            if local.shape != value.shape:        # never skipped silently: the source is the wrong architecture
                raise ValueError(f"shape mismatch for {name}: {tuple(local.shape)} vs {tuple(value.shape)}")
            local.copy_(value.to(local.dtype))
            copied += 1
    log.info("MoT warm start: copied %d tensors", copied)
    return copied
