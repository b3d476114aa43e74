"""Decoder-only transformer.

Module and parameter names fix the checkpoint keys (``token_embedding.embedding``,
``layers.{i}.attention.{q,k,v,o}_proj``, ``layers.{i}.mlp...``, ``norm``,
``output_head.proj``); ``layers`` is a ``ModuleDict`` keyed by the global layer
index so a pipeline stage that owns layers 16..31 keeps the same keys.

Activation checkpointing is a property of the block (``ac_mode``) rather than a
wrapper module, so it never changes parameter names.  ``compute_loss`` runs the
output head fused with the cross entropy so (tokens, vocab) logits are never
materialised during training.

Parity: kempnerforge/model/transformer.py:35-528 (pre-norm block, MoE placement,
RoPE tables kept in fp32 outside the state dict, meta-device init hook, MoE
accessors, ``forward(tokens, modality=, kv_caches=, doc_ids=)`` and its argument
rules, cross-attention cadence, MoT / MoMa dispatch).
"""

from __future__ import annotations

import os

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from kempnerforge_b200.models.recompute import checkpoint_contexts

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.config.sections import ModelConfig
from kempnerforge_b200.models.attention import Attention, KVCache
from kempnerforge_b200.models.embedding import OutputHead, TokenEmbedding
from kempnerforge_b200.models.init import init_weights
from kempnerforge_b200.models.mlp import build_mlp
from kempnerforge_b200.models.modality import ModalityContext
from kempnerforge_b200.models.moe import MoEMLP, build_moe
from kempnerforge_b200.models.norm import build_norm
from kempnerforge_b200.models.position import precompute_rope_frequencies
from kempnerforge_b200.ops import functional as F


_FUSED_BLOCK_OFF = bool(os.environ.get("KF_DISABLE_FUSED_BLOCK"))


class TransformerBlock(nn.Module):
    """x + Attn(Norm(x)) followed by x + FFN(Norm(x))."""

    def __init__(self, config: ModelConfig, layer_idx: int) -> None:
        super().__init__()
        self.layer_idx = layer_idx
        self.ac_mode = "none"  # "none" | "full" | "selective", set by apply_ac
        self.attention_norm = build_norm(config.norm_type, config.dim, config.norm_eps)
        self.attention = Attention(
            config.dim, config.n_heads, config.n_kv_heads, config.head_dim, config.qk_norm, config.sdpa_backend
        )
        self.mlp_norm = build_norm(config.norm_type, config.dim, config.norm_eps)
        if config.is_moe_layer(layer_idx):
            self.mlp = build_moe(
                dim=config.dim,
                hidden_dim=config.computed_expert_ffn_hidden_dim,
                num_experts=config.num_experts,
                top_k=config.moe_top_k,
                activation=config.activation,
                router_type=config.moe_router,
                shared_experts=config.moe_shared_experts,
                capacity_factor=config.moe_capacity_factor,
                gradient_scale=config.moe_gradient_scale,
                sequence_aux_loss_weight=config.moe_sequence_aux_loss_weight,
                bias_schedule=config.moe_bias_schedule,
                packed_experts=config.moe_packed_experts,
                shared_expert_widen=config.moe_shared_expert_widen,
            )
        else:
            self.mlp = build_mlp(config.dim, config.computed_ffn_hidden_dim, config.activation)

    def _attn_branch(self, x, cos, sin, kv_cache, doc_ids, key_padding_mask):
        return self.attention(
            self.attention_norm(x), cos, sin, kv_cache=kv_cache, doc_ids=doc_ids, key_padding_mask=key_padding_mask
        )

    def _body(self, x, cos, sin, kv_cache, doc_ids, key_padding_mask):
        if self.ac_mode == "selective" and self.training and torch.is_grad_enabled() and kv_cache is None:
            attn = checkpoint(
                self._attn_branch, x, cos, sin, None, doc_ids, key_padding_mask, use_reentrant=False,
                context_fn=checkpoint_contexts,
            )
        else:
            if x.is_cuda and not _FUSED_BLOCK_OFF and F.use_native(x):
                from kempnerforge_b200.ops import fused_block

                if fused_block.attn_half_supported(self, x, kv_cache, doc_ids, key_padding_mask):
                    # blocks the whole-block node does not cover (mixture-of-experts layers): the attention
                    # sub-layer as one node, residual included
                    x = fused_block.attn_half(self, x, cos, sin)
                    return x + self.mlp(self.mlp_norm(x))
            attn = self._attn_branch(x, cos, sin, kv_cache, doc_ids, key_padding_mask)
        x = x + attn
        return x + self.mlp(self.mlp_norm(x))

    def forward(self, x, rope_cos, rope_sin, *, kv_cache: KVCache | None = None, doc_ids=None, key_padding_mask=None):
        if (x.is_cuda and self.ac_mode in ("none", "full") and not _FUSED_BLOCK_OFF
                and not getattr(self, "_kf_fp8_block", False)):
            from kempnerforge_b200.ops import fused_block

            if F.use_native(x) and fused_block.dense_block_supported(self, x, kv_cache, doc_ids, key_padding_mask):
                return fused_block.dense_block(self, x, rope_cos, rope_sin)
        unit = getattr(self.attention.q_proj.weight, "_kf_flat", None)
        if unit is not None and getattr(unit, "sharded", False) and unit.engine.shared_staging:
            if torch.is_grad_enabled() and x.requires_grad:
                raise RuntimeError("sharded parameters (ZeRO-3) train through the fused dense block only; this call "
                                   "(masks, caches, hooks or an unsupported dtype) needs the resident engine")
            unit.engine.acquire(unit, everything=True)  # gradient-free paths read whole parameters
        if self.ac_mode == "full" and self.training and torch.is_grad_enabled() and kv_cache is None:
            return checkpoint(
                self._body, x, rope_cos, rope_sin, None, doc_ids, key_padding_mask, use_reentrant=False,
                context_fn=checkpoint_contexts,
            )
        return self._body(x, rope_cos, rope_sin, kv_cache, doc_ids, key_padding_mask)


class Transformer(nn.Module):
    def __init__(self, config: ModelConfig, *, vlm_config=None, num_image_tokens: int = 0,
                 layer_ids: list[int] | None = None, with_embedding: bool = True, with_head: bool = True) -> None:
        """``layer_ids`` / ``with_embedding`` / ``with_head`` build only a slice of the network (a pipeline
        stage); the layer keys stay the global indices so checkpoint names do not depend on the split."""
        super().__init__()
        self.config = config
        self.is_pipeline_stage = layer_ids is not None
        self.token_embedding: TokenEmbedding | None = (
            TokenEmbedding(config.vocab_size, config.dim) if with_embedding else None
        )
        self._mot_modalities: tuple[str, ...] = ()
        self._moma_modalities: tuple[str, ...] = ()
        self._mot_n_image = 0
        self._ca_cadence = 0
        arch = getattr(vlm_config, "arch", None)
        blocks: dict[str, nn.Module] = {}
        if arch == "mot":
            from kempnerforge_b200.models.mot import MoTBlock

            text_kv = config.n_kv_heads if config.n_kv_heads is not None else config.n_heads
            if hasattr(vlm_config, "resolved_image_heads"):
                img_heads, img_kv = vlm_config.resolved_image_heads(config.n_heads, text_kv)
                if img_heads != config.n_heads or img_kv != text_kv:
                    raise ValueError("MoT requires equal head counts across modalities (one global attention): image "
                                     f"{img_heads}/{img_kv} vs text {config.n_heads}/{text_kv}")
            self._mot_modalities = tuple(vlm_config.mot_modalities)
            self._mot_n_image = num_image_tokens
            for i in range(config.n_layers):
                blocks[str(i)] = MoTBlock(config, vlm_config, i)
        elif arch == "moma":
            from kempnerforge_b200.models.moma import MoMaBlock

            self._moma_modalities = tuple(vlm_config.moma_modalities)
            for i in range(config.n_layers):
                blocks[str(i)] = MoMaBlock(config, vlm_config, i)
        else:
            for i in (range(config.n_layers) if layer_ids is None else layer_ids):
                blocks[str(i)] = TransformerBlock(config, i)
        self.layers = nn.ModuleDict(blocks)
        self.cross_attention_layers = nn.ModuleDict()
        if arch == "cross_attention":
            from kempnerforge_b200.models.cross_attention import CrossAttentionBlock

            self._ca_cadence = vlm_config.cross_attention_every_n_layers
            heads, kv_heads = vlm_config.resolved_heads(config.n_heads)
            for j in range(config.n_layers // self._ca_cadence):
                self.cross_attention_layers[str(j)] = CrossAttentionBlock(config, heads, kv_heads)
        self.norm: nn.Module | None = build_norm(config.norm_type, config.dim, config.norm_eps) if with_head else None
        self.mot_norms = nn.ModuleDict()
        if self._mot_modalities:
            self.mot_norms = nn.ModuleDict(
                {m: build_norm(config.norm_type, config.dim, config.norm_eps) for m in self._mot_modalities}
            )
        self.output_head: OutputHead | None = OutputHead(config.dim, config.vocab_size) if with_head else None
        if config.tie_embeddings and with_head and with_embedding:
            self.output_head.tie_weights(self.token_embedding)
        self._rope_cos: torch.Tensor | None = None
        self._rope_sin: torch.Tensor | None = None
        self.tp = None  # TPContext set by apply_tensor_parallel
        if not any(p.is_meta for p in self.parameters()):
            self.init_weights_and_freqs()

    # ------------------------------------------------------------------ init
    def init_weights_and_freqs(self, device=None) -> None:
        """(Re)draw all weights and rebuild the RoPE tables; call after ``to_empty`` on meta builds."""
        init_weights(self, self.config.n_layers, self.config.init_std)
        for m in self.modules():
            if isinstance(m, nn.modules.normalization.LayerNorm) or type(m).__name__ == "RMSNorm":
                with torch.no_grad():
                    m.weight.fill_(1.0)
                    if getattr(m, "bias", None) is not None:
                        m.bias.zero_()
        if device is None:
            device = next(self.parameters()).device
        self._rope_cos, self._rope_sin = precompute_rope_frequencies(
            self.config.head_dim, self.config.max_seq_len, self.config.rope_theta, device=device
        )

    def rope_tables(self, device, start: int, length: int):
        if self._rope_cos is None:
            self._rope_cos, self._rope_sin = precompute_rope_frequencies(
                self.config.head_dim, self.config.max_seq_len, self.config.rope_theta, device=device
            )
        if self._rope_cos.device != device:
            self._rope_cos = self._rope_cos.to(device)
            self._rope_sin = self._rope_sin.to(device)
        if start + length > self._rope_cos.shape[0]:
            raise ValueError(f"sequence position {start + length} exceeds max_seq_len {self._rope_cos.shape[0]}")
        return self._rope_cos[start : start + length], self._rope_sin[start : start + length]

    # ------------------------------------------------------------------ MoE accessors
    def _moe_layers(self):
        for name, layer in self.layers.items():
            mlp = getattr(layer, "mlp", None)
            if isinstance(mlp, MoEMLP):
                yield int(name), mlp

    def set_moe_step(self, step: int, max_steps: int) -> None:
        for _, mlp in self._moe_layers():
            if hasattr(mlp.router, "set_step"):
                mlp.router.set_step(step, max_steps)

    def _sum_moe(self, attr: str) -> torch.Tensor:
        dev = next(self.parameters()).device
        total = torch.zeros((), device=dev)
        for _, mlp in self._moe_layers():
            total = total + getattr(mlp, attr).to(dev)
        for layer in self.layers.values():  # MoMa layers expose the same scalars
            if type(getattr(layer, "mlp", None)).__name__ == "MoMaFFN":
                total = total + getattr(layer.mlp, attr).to(dev)
        return total

    def get_moe_aux_loss(self) -> torch.Tensor:
        return self._sum_moe("aux_loss")

    def get_moe_router_z_loss(self) -> torch.Tensor:
        return self._sum_moe("z_loss")

    def get_expert_counts(self) -> dict[int, torch.Tensor]:
        return {i: mlp.expert_counts for i, mlp in self._moe_layers()}

    def get_moma_expert_counts(self) -> dict[int, dict[str, torch.Tensor]]:
        out = {}
        for name, layer in self.layers.items():
            mlp = getattr(layer, "mlp", None)
            if type(mlp).__name__ == "MoMaFFN":
                out[int(name)] = {m: mlp.experts[m].expert_counts for m in mlp.modalities}
        return out

    # ------------------------------------------------------------------ forward
    def forward_hidden(
        self,
        tokens: torch.Tensor | None = None,
        *,
        modality: ModalityContext | None = None,
        kv_caches: list[KVCache] | None = None,
        doc_ids: torch.Tensor | None = None,
    ) -> torch.Tensor:
        """Everything up to (and including) the final norm and ``output_slice``; no output head."""
        ctx = modality if modality is not None else ModalityContext()
        if (tokens is None) == (ctx.inputs_embeds is None):
            raise ValueError("Transformer.forward requires exactly one of tokens or modality.inputs_embeds")
        if kv_caches is not None:
            for field in ("output_slice", "prefix_embeds", "image_features", "modality_ids"):
                if getattr(ctx, field) is not None:
                    raise ValueError(f"modality.{field} is training-only; cannot be combined with kv_caches")
        if ctx.modality_ids is not None and ctx.modality_ids.dtype != torch.long:
            raise ValueError(f"modality.modality_ids.dtype must be torch.long, got {ctx.modality_ids.dtype}")

        h = self.token_embedding(tokens) if tokens is not None else ctx.inputs_embeds
        if ctx.prefix_embeds is not None:
            h = torch.cat([ctx.prefix_embeds.to(h.dtype), h], dim=1)
        seq_len = h.shape[1]
        start = kv_caches[0].seq_len if kv_caches is not None else 0
        cos, sin = self.rope_tables(h.device, start, seq_len)
        kpm = ctx.key_padding_mask
        tp = self.tp
        if tp is not None and tp.sequence_parallel:
            if seq_len % tp.size:
                raise ValueError(f"sequence length {seq_len} is not divisible by tp={tp.size}")
            h = tp.scatter_sequence(h)

        if self._moma_modalities or self._mot_modalities:
            kind = "MoMa" if self._moma_modalities else "MoT"
            if ctx.modality_ids is None:
                raise ValueError(f"{kind} model requires modality.modality_ids (got None)")
            if ctx.modality_ids.shape != h.shape[:2]:
                raise ValueError(
                    f"modality.modality_ids shape {tuple(ctx.modality_ids.shape)} does not match "
                    f"residual shape {tuple(h.shape[:2])}"
                )
        if self._moma_modalities:
            for layer in self.layers.values():
                h = layer(h, cos, sin, ctx.modality_ids, doc_ids=doc_ids, key_padding_mask=kpm)
            h = self.norm(h)
        elif self._mot_modalities:
            n_img = self._mot_n_image
            n_txt = seq_len - n_img
            streams = {"image": h[:, :n_img], "text": h[:, n_img:]}
            rope = {"image": (cos[:n_img], sin[:n_img]), "text": (cos[:n_txt], sin[:n_txt])}
            for layer in self.layers.values():
                streams = layer(streams, rope, key_padding_mask=kpm)
            h = torch.cat([self.mot_norms[m](streams[m]) for m in ("image", "text")], dim=1)
        else:
            ca_blocks = list(self.cross_attention_layers.values()) if self._ca_cadence else []
            image_features = ctx.image_features
            for pos, (key, layer) in enumerate(self.layers.items()):
                i = int(key)
                cache = kv_caches[pos] if kv_caches is not None else None
                h = layer(h, cos, sin, kv_cache=cache, doc_ids=doc_ids, key_padding_mask=kpm)
                if ca_blocks and (i + 1) % self._ca_cadence == 0:
                    j = (i + 1) // self._ca_cadence - 1
                    if j < len(ca_blocks):
                        if image_features is None:
                            raise ValueError(
                                "Cross-Attention block fired but modality.image_features is None."
                            )
                        h = ca_blocks[j](h, image_features.to(h.dtype), ctx.image_mask)
            if self.norm is not None:
                h = self.norm(h)
        if tp is not None and tp.sequence_parallel:
            h = tp.gather_sequence(h)
        if ctx.output_slice is not None:
            h = h[:, ctx.output_slice, :]
        return h

    def forward(self, tokens=None, *, modality=None, kv_caches=None, doc_ids=None) -> torch.Tensor:
        h = self.forward_hidden(tokens, modality=modality, kv_caches=kv_caches, doc_ids=doc_ids)
        if self.output_head is None:
            return h
        head_tp = getattr(self.output_head, "tp", None)
        if head_tp is None:
            return self.output_head(h)
        # vocabulary-parallel head: assemble the full vocabulary for callers that want logits
        return head_tp.gather_vocab(self.output_head(head_tp.head_input(h)))

    def compute_loss(
        self,
        tokens: torch.Tensor | None,
        labels: torch.Tensor,
        *,
        modality: ModalityContext | None = None,
        doc_ids: torch.Tensor | None = None,
        z_loss_weight: float = 0.0,
        chunk_tokens: int = 4096,
    ) -> torch.Tensor:
        """Mean next-token cross entropy (+ z-loss) with the head GEMM fused into the loss."""
        h = self.forward_hidden(tokens, modality=modality, doc_ids=doc_ids)
        head_tp = getattr(self.output_head, "tp", None)
        if head_tp is not None:
            from kempnerforge_b200.parallel.tensor_parallel import vocab_parallel_cross_entropy

            logits = self.output_head(head_tp.head_input(h))
            return vocab_parallel_cross_entropy(
                logits.reshape(-1, logits.shape[-1]), labels.reshape(-1), head_tp, z_loss_weight)
        return F.linear_cross_entropy(
            h, self.output_head.proj.weight, labels, z_loss_weight, chunk_tokens or 4096
        )


registry.register("model", "transformer", lambda model_config, **kw: Transformer(model_config, **kw))
