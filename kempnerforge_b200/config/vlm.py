"""Vision-language sections: ``[vision_encoder]``, ``[adapter]``, ``[vlm]``, ``[video]``.

``[vlm]`` is a discriminated union on ``arch``: each architecture registers its
own dataclass under the ``vlm_config`` registry category and the loader picks
the subclass from the ``arch`` key.

Parity: kempnerforge/config/vlm.py:54-479 (FreezeSpec/FreezeStage, VLMConfig and
the four arch configs), adapter.py:21-108, vision.py:31-59, video.py:24-87.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.config.sections import _require

BASE_MODULE_PATTERNS: dict[str, list[str]] = {
    "transformer": ["transformer", "transformer.*"],
    "vision_encoder": ["vision_encoder", "vision_encoder.*"],
    "adapter": ["adapter", "adapter.*"],
}

_RESERVED_ARCHS: tuple[str, ...] = ()   # architecture names that are reserved but not built (none)
DEFAULT_MODULE_PATTERNS = BASE_MODULE_PATTERNS   # the name this table has in the reference (kempnerforge/config/vlm.py)

# adapter families that shrink the visual token grid
POOLING_ADAPTER_TYPES: tuple[str, ...] = ("avgpool", "attentional_pool")
DIVISIBLE_ONLY_POOL_TYPES: tuple[str, ...] = ("attentional_pool",)
ADAPTER_TYPES: tuple[str, ...] = ("mlp_2layer", "linear") + POOLING_ADAPTER_TYPES
VISION_ENCODER_TYPES: tuple[str, ...] = ("random", "siglip2", "clip")
VIDEO_DATASET_TYPES: tuple[str, ...] = ("webvid",)
SAMPLING_POLICIES: tuple[str, ...] = ("uniform",)


def _patterns(**extra: list[str]) -> dict[str, list[str]]:
    out = {k: list(v) for k, v in BASE_MODULE_PATTERNS.items()}
    out.update({k: list(v) for k, v in extra.items()})
    return out


def pooled_token_count(num_input_tokens: int, window: int, require_divisible: bool = False) -> int:
    """Tokens left after pooling a square grid of ``num_input_tokens`` with a ``window``² kernel."""
    _require(window > 0, f"pool window must be positive (got {window})")
    _require(num_input_tokens > 0, f"the number of input tokens must be positive (got {num_input_tokens})")
    side = math.isqrt(num_input_tokens)
    _require(side * side == num_input_tokens, f"pooling adapters need a square patch grid (got {num_input_tokens} tokens)")
    if require_divisible:
        _require(side % window == 0, f"ragged grid: token grid side {side} is not divisible by pool_window {window}")
    out_side = -(-side // window)
    return out_side * out_side


@dataclass(frozen=True)
class FreezeSpec:
    """Freeze (or thaw) every parameter matched by the module alias ``module``."""

    module: str
    frozen: bool = True


@dataclass(frozen=True)
class FreezeStage:
    """From ``start_step`` on, apply ``specs`` on top of the current freeze state."""

    start_step: int
    specs: tuple[FreezeSpec, ...]


def _check_modalities(key: str, names: tuple[str, ...]) -> None:
    _require(len(names) >= 2, f"vlm.{key} must have at least 2 entries (got {names!r})")
    for needed in ("text", "image"):
        _require(needed in names, f"vlm.{key} must include '{needed}' (got {names!r})")
    _require(len(set(names)) == len(names), f"vlm.{key} must not contain duplicates (got {names!r})")


@dataclass
class VLMConfig:
    arch: str = "joint_decoder"
    max_text_len: int = 512
    freeze: list[FreezeSpec] = field(default_factory=lambda: [FreezeSpec("vision_encoder", True)])
    freeze_schedule: list[FreezeStage] = field(default_factory=list)
    module_patterns: dict[str, list[str]] = field(default_factory=_patterns)

    def __post_init__(self) -> None:
        known = registry.list("vlm_config")
        _require(self.arch in known, f"Unknown vlm.arch: {self.arch!r}. Registered: {sorted(known)}.")
        _require(self.max_text_len > 0, "vlm.max_text_len must be positive")
        starts = [s.start_step for s in self.freeze_schedule]
        _require(
            all(a < b for a, b in zip(starts, starts[1:])),
            "vlm.freeze_schedule start_steps must be strictly monotonic",
        )

    def residual_stream_image_tokens(self, num_tokens: int) -> int:
        """Image tokens that occupy positions of the decoder's residual stream."""
        return num_tokens

    @classmethod
    def for_arch(cls, arch: str, **kwargs: Any) -> "VLMConfig":
        if not registry.has("vlm_config", arch):
            raise ValueError(
                f"Unknown vlm.arch: {arch!r}. Registered: {sorted(registry.list('vlm_config'))}."
            )
        return registry.get("vlm_config", arch)(**kwargs)


@registry.register("vlm_config", "joint_decoder")
@dataclass
class JointDecoderConfig(VLMConfig):
    arch: str = "joint_decoder"


@registry.register("vlm_config", "cross_attention")
@dataclass
class CrossAttentionConfig(VLMConfig):
    arch: str = "cross_attention"
    cross_attention_every_n_layers: int = 4
    cross_attention_n_heads: int = 0
    cross_attention_n_kv_heads: int = 0
    module_patterns: dict[str, list[str]] = field(
        default_factory=lambda: _patterns(
            cross_attention=[
                "transformer.cross_attention_layers",
                "transformer.cross_attention_layers.*",
            ]
        )
    )

    def __post_init__(self) -> None:
        super().__post_init__()
        _require(
            self.cross_attention_every_n_layers > 0,
            f"vlm.cross_attention_every_n_layers must be positive (got {self.cross_attention_every_n_layers})",
        )
        _require(
            self.cross_attention_n_heads >= 0 and self.cross_attention_n_kv_heads >= 0,
            "vlm.cross_attention_n_heads and cross_attention_n_kv_heads must be non-negative",
        )

    def residual_stream_image_tokens(self, num_tokens: int) -> int:
        return 0  # image features enter through the cross-attention side channel

    def resolved_heads(self, model_n_heads: int) -> tuple[int, int]:
        _require(model_n_heads > 0, f"model_n_heads must be positive (got {model_n_heads})")
        heads = self.cross_attention_n_heads or model_n_heads
        return heads, (self.cross_attention_n_kv_heads or heads)


@registry.register("vlm_config", "mot")
@dataclass
class MoTConfig(VLMConfig):
    arch: str = "mot"
    mot_modalities: tuple[str, ...] = ("image", "text")
    mot_image_n_heads: int = 0
    mot_image_n_kv_heads: int = 0
    mot_warm_start_from_text: bool = False
    mot_warm_start_path: str = ""
    module_patterns: dict[str, list[str]] = field(
        default_factory=lambda: _patterns(mot=["transformer.layers", "transformer.layers.*"])
    )

    def __post_init__(self) -> None:
        super().__post_init__()
        _check_modalities("mot_modalities", self.mot_modalities)
        _require(
            self.mot_image_n_heads >= 0 and self.mot_image_n_kv_heads >= 0,
            "vlm.mot_image_n_heads and mot_image_n_kv_heads must be non-negative",
        )
        _require(
            not self.mot_warm_start_from_text or bool(self.mot_warm_start_path),
            "vlm.mot_warm_start_from_text=True requires vlm.mot_warm_start_path",
        )

    def resolved_image_heads(self, model_n_heads: int, model_n_kv_heads: int = 0) -> tuple[int, int]:
        _require(model_n_heads > 0, f"model_n_heads must be positive (got {model_n_heads})")
        heads = self.mot_image_n_heads or model_n_heads
        return heads, (self.mot_image_n_kv_heads or model_n_kv_heads or heads)


@registry.register("vlm_config", "moma")
@dataclass
class MoMaConfig(VLMConfig):
    arch: str = "moma"
    moma_modalities: tuple[str, ...] = ("image", "text")
    moma_experts_per_modality: dict[str, int] = field(default_factory=lambda: {"image": 4, "text": 4})
    moma_capacity_factor: float = 0.0
    moma_gumbel_noise: bool = True
    module_patterns: dict[str, list[str]] = field(
        default_factory=lambda: _patterns(moma=["transformer.layers", "transformer.layers.*"])
    )

    def __post_init__(self) -> None:
        super().__post_init__()
        _check_modalities("moma_modalities", self.moma_modalities)
        have, want = set(self.moma_experts_per_modality), set(self.moma_modalities)
        _require(
            not (want - have),
            f"vlm.moma_experts_per_modality missing entries for {sorted(want - have)}",
        )
        _require(
            not (have - want),
            f"vlm.moma_experts_per_modality has unknown modality keys {sorted(have - want)}",
        )
        for name, n in self.moma_experts_per_modality.items():
            _require(n > 0, f"vlm.moma_experts_per_modality[{name!r}] must be positive (got {n})")
        _require(
            self.moma_capacity_factor >= 0,
            f"vlm.moma_capacity_factor must be >= 0 (got {self.moma_capacity_factor})",
        )

    def effective_capacity_factor(self, modality: str) -> float:
        if self.moma_capacity_factor > 0:
            return self.moma_capacity_factor
        return 1.0 / self.moma_experts_per_modality[modality]


# --------------------------------------------------------------------------- adapter / encoder / video
@dataclass
class AdapterConfig:
    type: str = "mlp_2layer"
    hidden_dim: int = 0
    activation: str = "gelu"
    pool_window: int = 2
    pool_heads: int = 16

    def __post_init__(self) -> None:
        known = set(ADAPTER_TYPES) | set(registry.list("adapter"))
        _require(self.type in known, f"Unknown adapter.type: {self.type!r}. Registered: {sorted(known)}.")
        _require(self.hidden_dim >= 0, f"adapter.hidden_dim must be non-negative (got {self.hidden_dim})")
        _require(
            self.activation in ("gelu", "silu", "relu"),
            f"Unknown adapter.activation: {self.activation!r}. Options: 'gelu', 'silu', 'relu'.",
        )
        _require(self.pool_window > 0, f"adapter.pool_window must be positive (got {self.pool_window})")
        _require(self.pool_heads > 0, f"adapter.pool_heads must be positive (got {self.pool_heads})")

    def extra_kwargs(self) -> dict[str, Any]:
        return {
            "hidden_dim": self.hidden_dim or None,
            "activation": self.activation,
            "pool_window": self.pool_window,
            "pool_heads": self.pool_heads,
        }

    def output_num_tokens(self, num_input_tokens: int) -> int:
        if num_input_tokens <= 0 or self.type not in POOLING_ADAPTER_TYPES:
            return num_input_tokens
        return pooled_token_count(
            num_input_tokens, self.pool_window, self.type in DIVISIBLE_ONLY_POOL_TYPES
        )


@dataclass
class VisionEncoderConfig:
    type: str = "random"
    path: str = ""
    feature_dim: int = 0
    num_tokens: int = 0

    def __post_init__(self) -> None:
        known = set(VISION_ENCODER_TYPES) | set(registry.list("vision_encoder"))
        _require(
            self.type in known, f"Unknown vision_encoder.type: {self.type!r}. Registered: {sorted(known)}."
        )
        _require(self.feature_dim >= 0, f"vision_encoder.feature_dim must be non-negative (got {self.feature_dim})")
        _require(self.num_tokens >= 0, f"vision_encoder.num_tokens must be non-negative (got {self.num_tokens})")


@dataclass
class VideoConfig:
    data_root: str = ""
    dataset_type: str = "webvid"
    dataset_name: str = "webvid-10M"
    sampling_policy: str = "uniform"
    split: str = "train"
    max_samples: int = 0
    max_frames: int = 16
    min_frames: int = 4
    fps: float = 2.0
    frame_size: int = 224
    prompt: str = ""

    def __post_init__(self) -> None:
        datasets = set(VIDEO_DATASET_TYPES) | set(registry.list("video_dataset"))
        policies = set(SAMPLING_POLICIES) | set(registry.list("sampling_policy"))
        _require(
            self.dataset_type in datasets,
            f"video.dataset_type must be one of {sorted(datasets)} (got {self.dataset_type!r})",
        )
        _require(
            self.sampling_policy in policies,
            f"video.sampling_policy must be one of {sorted(policies)} (got {self.sampling_policy!r})",
        )
        _require(
            self.split in ("train", "validation"),
            f"video.split must be one of ('train', 'validation') (got {self.split!r})",
        )
        _require(self.max_samples >= 0, f"video.max_samples must be non-negative (got {self.max_samples})")
        _require(self.min_frames >= 1, f"video.min_frames must be >= 1 (got {self.min_frames})")
        _require(self.max_frames >= 1, f"video.max_frames must be >= 1 (got {self.max_frames})")
        _require(
            self.min_frames <= self.max_frames,
            f"video.min_frames ({self.min_frames}) must be <= video.max_frames ({self.max_frames})",
        )
        _require(self.fps > 0, f"video.fps must be positive (got {self.fps})")
        _require(self.frame_size > 0, f"video.frame_size must be positive (got {self.frame_size})")
