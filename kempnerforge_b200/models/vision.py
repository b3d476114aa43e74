"""Vision encoders: a deterministic random stub and HuggingFace SigLIP2 / CLIP towers.

Every encoder maps pixel values (B, 3, H, W) to patch features (B, num_tokens, feature_dim) and exposes
``num_tokens`` and ``feature_dim``.  The random encoder has no weights worth training: it produces, for a
given image content, always the same pseudo-random features, which is all the plumbing tests need.

Parity: kempnerforge/model/vision.py:43-200 (registry keys ``random`` / ``siglip2`` / ``clip``; defaults of the
stub 16 tokens x 768; HF towers via ``AutoModel(...).vision_model``; CLIP's class token is dropped; the token
count of an HF tower is (image_size // patch_size)^2).
"""

from __future__ import annotations

import torch
from torch import nn

from kempnerforge_b200.config.registry import registry


class VisionEncoder(nn.Module):
    num_tokens: int
    feature_dim: int


class RandomVisionEncoder(VisionEncoder):
    def __init__(self, num_tokens: int = 16, feature_dim: int = 768, seed: int = 0) -> None:
        super().__init__()
        self.num_tokens, self.feature_dim = num_tokens, feature_dim
        # a fixed random projection of coarse image statistics: deterministic per image, different across images
        gen = torch.Generator().manual_seed(1234 + seed)
        # drawn on the CPU whatever device context the module is built under (the generator lives there), so the basis
        # is the same on every device; ``.to(device)`` moves it with the module
        basis = torch.randn(3 * 16, num_tokens * feature_dim, generator=gen, device="cpu") / 7.0
        self.register_buffer("basis", basis.to(torch.empty(0).device if torch.empty(0).device.type != "meta" else "cpu"),
                             persistent=False)
        # no parameters and nothing in the state dict (like the reference's stub): a non-persistent buffer carries
        # the module's device and dtype
        self.register_buffer("_anchor", torch.zeros(1), persistent=False)

    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        b = pixel_values.shape[0]
        coarse = torch.nn.functional.adaptive_avg_pool2d(pixel_values.float(), 4).reshape(b, -1)
        feats = torch.tanh(coarse @ self.basis.float()).reshape(b, self.num_tokens, self.feature_dim)
        return feats.to(self._anchor.dtype)


class HFVisionEncoder(VisionEncoder):
    def __init__(self, path: str, drop_cls: bool | None = None, num_tokens: int | None = None,
                 feature_dim: int | None = None, *, has_cls_token: bool | None = None, strip_cls: bool | None = None) -> None:
        """``drop_cls`` (``strip_cls`` in the reference's spelling) removes position 0 of the tower's output;
        ``has_cls_token`` says whether the tower emits a class token at all (default: it does exactly when it is
        dropped).  ``num_tokens`` is what ``forward`` returns per image: the patch grid, plus one for a class token
        that is kept."""
        super().__init__()
        if strip_cls is not None:
            drop_cls = strip_cls
        drop_cls = bool(drop_cls)
        if has_cls_token is None:
            has_cls_token = drop_cls
        if drop_cls and not has_cls_token:
            raise ValueError("strip_cls=True is meaningless when has_cls_token=False: the tower emits no class token")
        from transformers import AutoModel

        full = AutoModel.from_pretrained(path)
        self.model = getattr(full, "vision_model", full)
        cfg = self.model.config
        self.drop_cls, self.has_cls_token = drop_cls, has_cls_token
        self.num_tokens = num_tokens or (cfg.image_size // cfg.patch_size) ** 2 + int(has_cls_token and not drop_cls)
        self.feature_dim = feature_dim or cfg.hidden_size

    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        first = next(self.model.parameters(), None)
        if first is not None:
            pixel_values = pixel_values.to(first.dtype)
        hidden = self.model(pixel_values=pixel_values).last_hidden_state
        return hidden[:, 1:] if self.drop_cls else hidden


@registry.register("vision_encoder", "random")
def _build_random(path: str = "", num_tokens: int | None = None, feature_dim: int | None = None):
    return RandomVisionEncoder(num_tokens or 16, feature_dim or 768)


def _require_path(path: str, kind: str) -> None:
    if not path:
        raise ValueError(f"vision_encoder_path must be set for the {kind} encoder (a Hugging Face model id or directory)")


@registry.register("vision_encoder", "siglip2")
def _build_siglip2(path: str, num_tokens: int | None = None, feature_dim: int | None = None):
    _require_path(path, "siglip2")
    return HFVisionEncoder(path, drop_cls=False, num_tokens=num_tokens, feature_dim=feature_dim)


@registry.register("vision_encoder", "clip")
def _build_clip(path: str, num_tokens: int | None = None, feature_dim: int | None = None):
    _require_path(path, "clip")
    return HFVisionEncoder(path, drop_cls=True, num_tokens=num_tokens, feature_dim=feature_dim, has_cls_token=True)


_HFVisionEncoder = HFVisionEncoder   # underscore spelling used by code written against the reference


def build_vision_encoder(config) -> VisionEncoder:
    return registry.get("vision_encoder", config.type)(
        config.path, num_tokens=config.num_tokens or None, feature_dim=config.feature_dim or None)
