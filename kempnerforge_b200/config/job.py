"""``JobConfig``: the aggregate of every section plus the cross-section rules.

Rules that only need the config run at construction; rules that need the world
size run in ``validate(world_size)`` which the trainer calls once the process
group exists.

Parity: kempnerforge/config/job.py:30-283 (same sections, same rejected
combinations: seq_len > max_seq_len, tied embeddings + PP, eval without a
source, TP divisibility, FP8 + TP, MoE + PP, EP without MoE / indivisible,
VLM + PP, MoMa + num_experts / EP).
"""

from __future__ import annotations

import logging
from dataclasses import dataclass, field

from kempnerforge_b200.config.sections import (
    CheckpointConfig,
    DataConfig,
    DistributedConfig,
    EvalConfig,
    MetricsConfig,
    ModelConfig,
    OptimizerConfig,
    ProfilingConfig,
    SchedulerConfig,
    TrainConfig,
    _require,
)
from kempnerforge_b200.config.vlm import (
    AdapterConfig,
    MoMaConfig,
    VideoConfig,
    VisionEncoderConfig,
    VLMConfig,
)

_log = logging.getLogger(__name__)
_HF_ENCODERS = frozenset({"siglip2", "clip"})


@dataclass
class JobConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    train: TrainConfig = field(default_factory=TrainConfig)
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    scheduler: SchedulerConfig = field(default_factory=SchedulerConfig)
    data: DataConfig = field(default_factory=DataConfig)
    eval: EvalConfig = field(default_factory=EvalConfig)
    distributed: DistributedConfig = field(default_factory=DistributedConfig)
    checkpoint: CheckpointConfig = field(default_factory=CheckpointConfig)
    metrics: MetricsConfig = field(default_factory=MetricsConfig)
    profiling: ProfilingConfig = field(default_factory=ProfilingConfig)
    vision_encoder: VisionEncoderConfig | None = None
    adapter: AdapterConfig | None = None
    vlm: VLMConfig | None = None
    video: VideoConfig | None = None

    # -- construction-time rules -------------------------------------------
    def __post_init__(self) -> None:
        _require(
            self.video is None or self.vlm is not None,
            "[video] is set but [vlm] is missing; video training runs through the VLM wrapper",
        )
        if self.vlm is None:
            return
        _require(
            self.vision_encoder is not None,
            "[vlm] is set but [vision_encoder] is missing; a VLM run requires a vision encoder section.",
        )
        if self.adapter is None:
            self.adapter = AdapterConfig()
        enc = self.vision_encoder
        if enc.type in _HF_ENCODERS and (enc.feature_dim > 0 or enc.num_tokens > 0):
            given = ", ".join(f"{k}={getattr(enc, k)}" for k in ("feature_dim", "num_tokens") if getattr(enc, k) > 0)
            _log.warning(
                "vision_encoder.type=%r probes its own dims; the explicit %s overrides the probe and may disagree with "
                "the loaded model",
                enc.type, given,
            )
        need = self._vlm_required_positions()
        if need is not None:
            _require(
                self.model.max_seq_len >= need,
                f"model.max_seq_len ({self.model.max_seq_len}) insufficient for VLM: needs {need} "
                f"(image tokens in the residual stream + vlm.max_text_len ({self.vlm.max_text_len}))",
            )

    def _vlm_required_positions(self) -> int | None:
        """Residual-stream length a VLM sample needs, or None when the encoder probes it later."""
        if self.vlm is None or self.vision_encoder is None or self.vision_encoder.num_tokens <= 0:
            return None
        per_frame = self.adapter.output_num_tokens(self.vision_encoder.num_tokens)
        frames = self.video.max_frames if self.video is not None else 1
        return self.vlm.residual_stream_image_tokens(frames * per_frame) + self.vlm.max_text_len

    @property
    def is_vlm(self) -> bool:
        return self.vlm is not None

    @property
    def is_video(self) -> bool:
        return self.video is not None

    # -- world-size dependent rules ------------------------------------------
    def validate(self, world_size: int = 1) -> None:
        dist, model, train = self.distributed, self.model, self.train
        dist.validate_world_size(world_size)
        _require(
            train.seq_len <= model.max_seq_len,
            f"train.seq_len ({train.seq_len}) exceeds model.max_seq_len ({model.max_seq_len})",
        )
        _require(
            not (model.tie_embeddings and dist.pp > 1),
            "Tied embeddings are not supported with pipeline parallelism "
            "(embedding and output head must be on different stages)",
        )
        _require(
            not self.eval.enabled or bool(self.eval.dataset_path or self.eval.hf_dataset_name),
            "eval.enabled is True but no eval data source is configured. "
            "Set eval.dataset_path or eval.hf_dataset_name.",
        )
        if dist.tp > 1:
            _require(
                model.n_heads % dist.tp == 0,
                f"n_heads ({model.n_heads}) must be divisible by tp ({dist.tp})",
            )
            _require(
                model.n_kv_heads % dist.tp == 0,
                f"n_kv_heads ({model.n_kv_heads}) must be divisible by tp ({dist.tp})",
            )
        _require(
            not (train.is_fp8 and dist.tp > 1),
            "FP8 + Tensor Parallelism is not yet supported. Use FP8 with FSDP only, or TP without FP8.",
        )
        _require(
            not (model.is_moe and dist.pp > 1),
            "MoE + Pipeline Parallelism is not supported. Use FSDP, TP, or EP instead.",
        )
        if dist.ep > 1:
            _require(model.is_moe, "ep > 1 requires an MoE model (num_experts > 0)")
            _require(
                model.num_experts % dist.ep == 0,
                f"num_experts ({model.num_experts}) must be divisible by ep ({dist.ep})",
            )
        if self.vlm is not None:
            need = self._vlm_required_positions()
            if need is not None:
                _require(
                    train.seq_len >= need,
                    f"train.seq_len ({train.seq_len}) insufficient for VLM: needs {need}",
                )
            _require(dist.pp == 1, "VLM + Pipeline Parallelism is not supported.")
            if isinstance(self.vlm, MoMaConfig):
                _require(
                    model.num_experts == 0,
                    "MoMa + model.num_experts > 0 is rejected; MoMa takes its expert counts from "
                    "vlm.moma_experts_per_modality",
                )
                _require(dist.ep == 1, "MoMa + Expert Parallelism is not supported.")
