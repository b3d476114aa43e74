"""Vision-language wrapper: vision encoder -> adapter -> decoder, composed by an architecture strategy.

A strategy turns (pixel values, token ids, frame mask) into the ``ModalityContext`` the decoder understands:
  joint_decoder    image embeddings are prepended to the text embeddings; logits are returned for text positions
  cross_attention  image embeddings feed the cross-attention side channel; the residual stream is text only
  mot / moma       like joint_decoder plus per-position modality ids (0 = image, 1 = text)
Video clips (B, F, 3, H, W) are encoded frame by frame (frames folded into the batch) and their tokens
concatenated in frame order; ``frame_mask`` (B, F) marks real frames and expands to a per-token key mask.
Strategies hold no parameters and are not sub-modules, so they appear in no state dict.

Label convention: by default the logits of position t are scored against token t+1 (``shift_labels=True``);
the reference scores position t against token t (kempnerforge/data/vlm_dataset.py:70-115), which is available
as ``shift_labels=False``.

Parity: kempnerforge/model/vlm.py:56-470.
"""

from __future__ import annotations

from typing import Protocol, runtime_checkable

import torch
from torch import nn

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.models.adapter import build_adapter
from kempnerforge_b200.models.modality import ModalityContext
from kempnerforge_b200.models.transformer import Transformer
from kempnerforge_b200.models.vision import build_vision_encoder


def project_visual_features(wrapper: "VLMWrapper", pixel_values: torch.Tensor) -> torch.Tensor:
    is_video = pixel_values.dim() == 5
    frames = pixel_values.shape[1] if is_video else 1
    if frames != wrapper.frames_per_clip:
        raise ValueError(
            f"frames-per-clip mismatch: received {frames} frame(s) but the wrapper was built with "
            f"frames_per_clip={wrapper.frames_per_clip}")
    b = pixel_values.shape[0]
    x = pixel_values.reshape(b * frames, *pixel_values.shape[2:]) if is_video else pixel_values
    feats = wrapper.vision_encoder(x)
    feats = feats.to(next(wrapper.adapter.parameters()).dtype)
    emb = wrapper.adapter(feats)
    return emb.reshape(b, frames * emb.shape[1], emb.shape[2]) if is_video else emb


def visual_token_mask(frame_mask: torch.Tensor | None, num_visual_tokens: int) -> torch.Tensor | None:
    if frame_mask is None:
        return None
    frames = frame_mask.shape[1]
    if num_visual_tokens % frames:
        raise ValueError(f"num_visual_tokens ({num_visual_tokens}) must be a multiple of num_frames ({frames})")
    return frame_mask.bool().repeat_interleave(num_visual_tokens // frames, dim=1)


def prefix_key_padding_mask(frame_mask, num_visual_tokens: int, input_ids: torch.Tensor):
    vmask = visual_token_mask(frame_mask, num_visual_tokens)
    if vmask is None:
        return None
    text = torch.ones(input_ids.shape, dtype=torch.bool, device=vmask.device)
    return torch.cat([vmask, text], dim=1)


@runtime_checkable
class ModalityStrategy(Protocol):
    """What a registered modality strategy provides.  Strategies hold no parameters and are not sub-modules of
    the wrapper, so they are neither sharded nor checkpointed.  Parity: kempnerforge/model/vlm.py:56-74."""

    def prepare(self, wrapper, pixel_values: torch.Tensor, input_ids: torch.Tensor,
                frame_mask: torch.Tensor | None = None) -> ModalityContext: ...

    def num_image_tokens(self, wrapper) -> int: ...


class _PrefixStrategy:
    with_modality_ids = False

    def prepare(self, wrapper, pixel_values, input_ids, frame_mask=None) -> ModalityContext:
        emb = project_visual_features(wrapper, pixel_values)
        n = emb.shape[1]
        ids = None
        if self.with_modality_ids:
            b, t = input_ids.shape
            ids = torch.zeros(b, n + t, dtype=torch.long, device=input_ids.device)
            ids[:, n:] = 1
        return ModalityContext(prefix_embeds=emb, output_slice=slice(n, None), modality_ids=ids,
                               key_padding_mask=prefix_key_padding_mask(frame_mask, n, input_ids))

    def num_image_tokens(self, wrapper) -> int:
        return wrapper.frames_per_clip * wrapper.adapter.output_num_tokens(wrapper.vision_encoder.num_tokens)


@registry.register("modality_strategy", "joint_decoder")
class JointDecoderStrategy(_PrefixStrategy):
    pass


@registry.register("modality_strategy", "mot")
class MoTStrategy(_PrefixStrategy):
    with_modality_ids = True


@registry.register("modality_strategy", "moma")
class MoMaStrategy(_PrefixStrategy):
    with_modality_ids = True


@registry.register("modality_strategy", "cross_attention")
class CrossAttentionStrategy:
    def prepare(self, wrapper, pixel_values, input_ids, frame_mask=None) -> ModalityContext:
        emb = project_visual_features(wrapper, pixel_values)
        return ModalityContext(image_features=emb, image_mask=visual_token_mask(frame_mask, emb.shape[1]))

    def num_image_tokens(self, wrapper) -> int:
        return 0


def build_modality_strategy(vlm):
    return registry.get("modality_strategy", vlm.arch)()


class VLMWrapper(nn.Module):
    def __init__(self, vision_encoder, adapter, transformer: Transformer, strategy, frames_per_clip: int = 1) -> None:
        super().__init__()
        self.vision_encoder = vision_encoder
        self.adapter = adapter
        self.transformer = transformer
        self.frames_per_clip = frames_per_clip
        self.strategy = strategy  # plain object: no parameters, not a sub-module
        self.config = transformer.config

    @property
    def num_image_tokens(self) -> int:
        return self.strategy.num_image_tokens(self)

    def forward(self, pixel_values, input_ids, labels=None, frame_mask=None):
        ctx = self.strategy.prepare(self, pixel_values, input_ids, frame_mask=frame_mask)
        return self.transformer(tokens=input_ids, modality=ctx), labels

    def compute_loss(self, pixel_values, input_ids, labels, frame_mask=None, z_loss_weight: float = 0.0,
                     shift_labels: bool = True, **_) -> torch.Tensor:
        ctx = self.strategy.prepare(self, pixel_values, input_ids, frame_mask=frame_mask)
        if shift_labels:
            pad = torch.full_like(labels[:, :1], -100)
            labels = torch.cat([labels[:, 1:], pad], dim=1)
        return self.transformer.compute_loss(input_ids, labels, modality=ctx, z_loss_weight=z_loss_weight)


def inner_transformer(model: nn.Module) -> nn.Module:
    model = getattr(model, "_orig_mod", model)
    return model.transformer if isinstance(model, VLMWrapper) else model


def is_encoder_frozen(specs) -> bool:
    relevant = [s for s in specs if s.module == "vision_encoder" or s.module.startswith("vision_encoder.")]
    return bool(relevant) and all(s.frozen for s in relevant)


def build_vlm_wrapper(model_config, vision_config, adapter_config, vlm_config, frames_per_clip: int = 1) -> VLMWrapper:
    encoder = build_vision_encoder(vision_config)
    in_dim = vision_config.feature_dim or encoder.feature_dim
    adapter = build_adapter(adapter_config, in_dim=in_dim, out_dim=model_config.dim)
    visual = frames_per_clip * adapter.output_num_tokens(encoder.num_tokens)
    need = vlm_config.residual_stream_image_tokens(visual) + vlm_config.max_text_len
    if model_config.max_seq_len < need:
        raise ValueError(
            f"max_seq_len ({model_config.max_seq_len}) insufficient for VLM at build time: visual tokens {visual} "
            f"(frames_per_clip {frames_per_clip} x adapter output of encoder.num_tokens {encoder.num_tokens}) "
            f"+ vlm.max_text_len ({vlm_config.max_text_len}) = {need}")
    transformer = Transformer(model_config, vlm_config=vlm_config, num_image_tokens=visual)
    return VLMWrapper(encoder, adapter, transformer, build_modality_strategy(vlm_config), frames_per_clip)


_is_encoder_frozen = is_encoder_frozen   # underscore spellings used by code written against the reference
_visual_token_mask = visual_token_mask
