"""Typed configuration sections of a training job.

Every section is a dataclass whose field names and defaults match the TOML
keys of the reference presets, so a reference preset loads unchanged.  The
validation of a single section lives in ``__post_init__``; rules that span
sections or need the world size live in ``JobConfig.validate``.

Parity (field names / defaults / checks):
  kempnerforge/config/model.py:22-171, training.py:20-82, optimizer.py:9-37,
  scheduler.py:9-42, distributed.py:16-78, checkpoint.py:12-103, data.py:9-101,
  eval.py:9-27, metrics.py:9-22, profiling.py:9-19.

Additions that the reference cannot express (all default to the reference
behaviour): ``ModelConfig.moe_first_k_dense`` (dense FFN in the first k
layers), ``ModelConfig.moe_shared_expert_widen`` (one shared MLP whose hidden
size is multiplied by ``moe_shared_experts``), ``DistributedConfig.ep_in_dp``
(expert-parallel ranks are also data-parallel ranks), ``TrainConfig.hooks``
(import paths of ``TrainingHook`` classes).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field, fields, replace
from enum import StrEnum
from typing import Literal

from kempnerforge_b200.config.registry import registry


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


# --------------------------------------------------------------------------- model
class NormType(StrEnum):
    rmsnorm = "rmsnorm"
    layernorm = "layernorm"


class Activation(StrEnum):
    silu = "silu"
    gelu = "gelu"
    relu = "relu"


_ATTN_BACKENDS = ("auto", "flash", "efficient", "cudnn", "math")
_BIAS_SCHEDULES = ("constant", "cosine_decay", "linear_warmup")


@dataclass
class ModelConfig:
    dim: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int | None = None
    vocab_size: int = 32000
    ffn_dim_multiplier: float = 1.0
    ffn_hidden_dim: int | None = None
    norm_type: NormType = NormType.rmsnorm
    norm_eps: float = 1e-5
    activation: Activation = Activation.silu
    max_seq_len: int = 2048
    rope_theta: float = 10000.0
    tie_embeddings: bool = False
    qk_norm: bool = False
    init_std: float = 0.02
    model_type: str = "transformer"
    sdpa_backend: str = "auto"
    # mixture of experts; num_experts == 0 keeps the model dense
    num_experts: int = 0
    moe_top_k: int = 2
    moe_frequency: int = 1
    moe_router: str = "softmax_topk"
    moe_shared_experts: int = 0
    moe_aux_loss_weight: float = 0.01
    moe_capacity_factor: float = 0.0
    moe_sequence_aux_loss_weight: float = 0.0
    moe_gradient_scale: bool = False
    moe_bias_schedule: str = "constant"
    moe_packed_experts: bool = False
    moe_expert_ffn_multiplier: float = 1.0
    moe_router_z_loss_weight: float = 0.0
    # extensions (see module docstring)
    moe_first_k_dense: int = 0
    moe_shared_expert_widen: bool = False

    def __post_init__(self) -> None:
        if self.n_kv_heads is None:
            self.n_kv_heads = self.n_heads
        _require(
            self.dim > 0 and self.n_layers > 0 and self.n_heads > 0,
            "dim, n_layers, and n_heads must be positive",
        )
        _require(self.vocab_size > 0, "vocab_size must be positive")
        _require(self.n_kv_heads > 0, "n_kv_heads must be positive")
        _require(
            self.dim % self.n_heads == 0,
            f"dim ({self.dim}) must be divisible by n_heads ({self.n_heads})",
        )
        _require(
            self.n_heads % self.n_kv_heads == 0,
            f"n_heads ({self.n_heads}) must be divisible by n_kv_heads ({self.n_kv_heads})",
        )
        _require(
            self.sdpa_backend in _ATTN_BACKENDS,
            f"Unknown sdpa_backend: '{self.sdpa_backend}'. Options: {_ATTN_BACKENDS}",
        )
        _require(self.moe_first_k_dense >= 0, "moe_first_k_dense must be non-negative")
        if self.num_experts > 0:
            _require(self.moe_top_k > 0, "moe_top_k must be positive when num_experts > 0")
            _require(
                self.moe_top_k <= self.num_experts,
                f"moe_top_k ({self.moe_top_k}) must be <= num_experts ({self.num_experts})",
            )
            _require(self.moe_frequency > 0, "moe_frequency must be positive")
            _require(
                self.moe_sequence_aux_loss_weight >= 0,
                "moe_sequence_aux_loss_weight must be non-negative",
            )
            _require(
                self.moe_bias_schedule in _BIAS_SCHEDULES,
                f"Unknown moe_bias_schedule: '{self.moe_bias_schedule}'. Options: {_BIAS_SCHEDULES}",
            )
            _require(self.moe_expert_ffn_multiplier > 0, "moe_expert_ffn_multiplier must be positive")
            _require(
                self.moe_router_z_loss_weight >= 0, "moe_router_z_loss_weight must be non-negative"
            )

    # -- derived quantities ------------------------------------------------
    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads

    @property
    def computed_ffn_hidden_dim(self) -> int:
        """SwiGLU width: explicit override, else 4*dim*2/3*mult rounded up to 256."""
        if self.ffn_hidden_dim is not None:
            return self.ffn_hidden_dim
        unrounded = int(4 * self.dim * (2 / 3) * self.ffn_dim_multiplier)
        return 256 * math.ceil(unrounded / 256)

    @property
    def computed_expert_ffn_hidden_dim(self) -> int:
        """Width of one routed/shared expert, a multiple of 16 (at least 16)."""
        scaled = int(self.computed_ffn_hidden_dim * self.moe_expert_ffn_multiplier)
        return max(16, 16 * round(scaled / 16))

    def is_moe_layer(self, layer_idx: int) -> bool:
        """True when block ``layer_idx`` carries an MoE feed-forward."""
        if not self.is_moe or layer_idx < self.moe_first_k_dense:
            return False
        return (layer_idx + 1) % self.moe_frequency == 0

    @property
    def num_moe_layers(self) -> int:
        return sum(self.is_moe_layer(i) for i in range(self.n_layers))

    @property
    def num_params_estimate(self) -> int:
        """Total parameter count (all experts counted; tied head counted once)."""
        d, hd = self.dim, self.head_dim
        attn = 2 * d * self.n_heads * hd + 2 * d * self.n_kv_heads * hd
        norms = 2 * d
        dense_ffn = 3 * d * self.computed_ffn_hidden_dim
        total = 0
        for i in range(self.n_layers):
            if self.is_moe_layer(i):
                one = 3 * d * self.computed_expert_ffn_hidden_dim
                total += attn + norms + d * self.num_experts
                total += (self.num_experts + self.moe_shared_experts) * one
            else:
                total += attn + norms + dense_ffn
        total += self.vocab_size * d + d
        if not self.tie_embeddings:
            total += self.vocab_size * d
        return total


# --------------------------------------------------------------------------- train
class ActivationCheckpointing(StrEnum):
    none = "none"
    full = "full"
    selective = "selective"


_PRECISIONS = ("bf16", "fp16", "fp32", "fp8")


@dataclass
class TrainConfig:
    batch_size: int = 8  # per-device micro-batch
    seq_len: int = 2048
    max_steps: int = 100000
    grad_accum_steps: int = 1
    grad_clip_norm: float = 1.0
    seed: int = 42
    data_seed: int | None = None
    compile_model: bool = True  # accepted for preset compatibility; no tracing compiler here
    mixed_precision: Literal["bf16", "fp16", "fp32", "fp8"] = "bf16"
    activation_checkpointing: ActivationCheckpointing = ActivationCheckpointing.none
    loss_fn: str = "cross_entropy"
    z_loss_weight: float = 0.0
    ce_chunk_size: int = 0
    shutdown_timeout_sec: float = 600.0
    nccl_health_check_interval: int = 0
    hooks: list[str] = field(default_factory=list)  # "package.module:ClassName"

    def __post_init__(self) -> None:
        for name in ("batch_size", "seq_len", "max_steps", "grad_accum_steps", "grad_clip_norm"):
            _require(getattr(self, name) > 0, f"{name} must be positive")
        _require(self.mixed_precision in _PRECISIONS, f"mixed_precision must be one of {_PRECISIONS}")

    @property
    def param_dtype(self):
        """Storage dtype of parameters (fp8 computes in fp8 but stores bf16)."""
        import torch

        return {
            "bf16": torch.bfloat16,
            "fp16": torch.float16,
            "fp32": torch.float32,
            "fp8": torch.bfloat16,
        }[self.mixed_precision]

    @property
    def is_fp8(self) -> bool:
        return self.mixed_precision == "fp8"

    @property
    def effective_data_seed(self) -> int:
        return self.seed if self.data_seed is None else self.data_seed


# --------------------------------------------------------------------------- optimizer / scheduler
@dataclass
class OptimizerConfig:
    name: str = "adamw"
    lr: float = 3e-4
    weight_decay: float = 0.1
    betas: tuple[float, float] = (0.9, 0.95)
    eps: float = 1e-8
    fused: bool = True
    muon_momentum: float = 0.95
    muon_ns_steps: int = 5
    muon_adam_lr: float | None = None
    schedule_free_warmup_steps: int = 0

    def __post_init__(self) -> None:
        _require(self.lr > 0, "lr must be positive")
        _require(self.weight_decay >= 0, "weight_decay must be non-negative")
        _require(all(0 <= b < 1 for b in self.betas), "betas must be in [0, 1)")
        _require(0 < self.muon_momentum < 1, "muon_momentum must be in (0, 1)")
        _require(self.muon_ns_steps > 0, "muon_ns_steps must be positive")
        _require(
            self.schedule_free_warmup_steps >= 0, "schedule_free_warmup_steps must be non-negative"
        )


class SchedulerType(StrEnum):
    cosine = "cosine"
    linear = "linear"
    wsd = "wsd"
    constant = "constant"
    rex = "rex"
    none = "none"


@dataclass
class SchedulerConfig:
    name: SchedulerType = SchedulerType.cosine
    warmup_steps: int = 2000
    decay_steps: int | None = None
    min_lr_ratio: float = 0.1
    stable_steps: int | None = None
    wsd_decay_type: str = "cosine"
    rex_alpha: float = 1.0

    def __post_init__(self) -> None:
        _require(self.warmup_steps >= 0, "warmup_steps must be non-negative")
        _require(0 <= self.min_lr_ratio <= 1, "min_lr_ratio must be in [0, 1]")
        _require(
            self.wsd_decay_type in ("cosine", "linear", "sqrt"),
            f"wsd_decay_type must be 'cosine', 'linear', or 'sqrt', got '{self.wsd_decay_type}'",
        )
        _require(self.rex_alpha > 0, "rex_alpha must be positive")


# --------------------------------------------------------------------------- distributed
class PipelineSchedule(StrEnum):
    schedule_1f1b = "1f1b"
    gpipe = "gpipe"
    interleaved_1f1b = "interleaved_1f1b"


@dataclass
class DistributedConfig:
    dp_shard: int = -1  # -1: whatever is left of the world
    dp_replicate: int = 1
    tp: int = 1
    pp: int = 1
    pp_schedule: PipelineSchedule = PipelineSchedule.schedule_1f1b
    cp: int = 1
    ep: int = 1
    nccl_timeout_sec: int = 1800
    backend: str = "cpu:gloo,cuda:nccl"
    # extension: EP ranks live inside the data-parallel dimension (each EP rank
    # routes its own tokens) instead of multiplying the world size.
    ep_in_dp: bool = False
    # extension: memory plan of the data-parallel engine.  "resident" keeps whole parameters and gradients on every
    # rank (optimizer state sharded); "sharded" is ZeRO-3 (1/N of parameters, gradients and state per rank, weights
    # gathered inside the GEMMs that read them); "auto" picks "sharded" only when "resident" would not fit.
    param_sharding: str = "auto"

    def __post_init__(self) -> None:
        _require(self.dp_shard == -1 or self.dp_shard > 0, "dp_shard must be -1 (auto) or positive")
        for name in ("dp_replicate", "tp", "pp", "cp", "ep"):
            _require(getattr(self, name) >= 1, f"{name} must be >= 1")

    def _fixed_product(self) -> int:
        ep = 1 if self.ep_in_dp else self.ep
        return self.dp_replicate * self.tp * self.pp * self.cp * ep

    def _resolve_dp_shard(self, world_size: int) -> int:
        if self.dp_shard > 0:
            return self.dp_shard
        rest = self._fixed_product()
        _require(
            world_size % rest == 0,
            f"world_size ({world_size}) not divisible by dp_replicate*tp*pp*cp*ep ({rest})",
        )
        return world_size // rest

    def validate_world_size(self, world_size: int) -> None:
        shard = self._resolve_dp_shard(world_size)
        got = shard * self._fixed_product()
        _require(
            got == world_size,
            f"Parallelism dimensions ({self.dp_replicate} x {shard} x {self.tp} x {self.pp} x "
            f"{self.cp} x {self.ep}{' (inside dp)' if self.ep_in_dp else ''} = {got}) "
            f"do not match world_size ({world_size})",
        )
        if self.ep_in_dp and self.ep > 1:
            _require(
                (shard * self.dp_replicate) % self.ep == 0,
                f"ep ({self.ep}) must divide the data-parallel size ({shard * self.dp_replicate})",
            )

    def resolve(self, world_size: int) -> "DistributedConfig":
        out = replace(self, dp_shard=self._resolve_dp_shard(world_size))
        out.validate_world_size(world_size)
        return out


# --------------------------------------------------------------------------- checkpoint
class AsyncCheckpointMode(StrEnum):
    disabled = "disabled"
    async_ = "async"
    async_pinned = "async_with_pinned_mem"


@dataclass
class DynamicCheckpointWindow:
    """Step range ``[start, stop]`` inside which a named strategy picks the save steps."""

    start: int = 0
    stop: int = 512
    strategy: str = "power2"

    def __post_init__(self) -> None:
        _require(self.start >= 0, "dyn_ckpt_window.start must be >= 0")
        _require(self.stop >= self.start, "dyn_ckpt_window.stop must be >= start")
        known = registry.list("dyn_ckpt_strategy")
        _require(
            self.strategy in known,
            f"unknown dyn_ckpt_window.strategy {self.strategy!r}; registered: {known}",
        )

    def is_milestone(self, step: int) -> bool:
        return bool(registry.get("dyn_ckpt_strategy", self.strategy)(self, step))


def _power_of_two_offsets(window: DynamicCheckpointWindow, step: int) -> bool:
    """start, start+1, start+2, start+4, ... up to stop."""
    if not (window.start <= step <= window.stop):
        return False
    delta = step - window.start
    return delta & (delta - 1) == 0  # true for 0 and for powers of two


registry.register("dyn_ckpt_strategy", "power2", _power_of_two_offsets)


@dataclass
class CheckpointConfig:
    dir: str = "checkpoints"
    interval: int = 1000
    dyn_ckpt_window: DynamicCheckpointWindow | None = None
    async_mode: AsyncCheckpointMode = AsyncCheckpointMode.disabled
    keep_last_n: int = 3
    load_path: str | None = None
    export_dtype: Literal["float32", "bfloat16"] = "bfloat16"
    exclude_from_loading: list[str] = field(default_factory=list)
    ignore_freeze_mismatch: bool = False

    def __post_init__(self) -> None:
        _require(self.interval > 0, "interval must be positive")

    def should_save(self, step: int) -> bool:
        win = self.dyn_ckpt_window
        if win is not None and win.start <= step <= win.stop:
            return win.is_milestone(step)
        return step % self.interval == 0

    def is_dynamic_milestone(self, step: int) -> bool:
        return self.dyn_ckpt_window is not None and self.dyn_ckpt_window.is_milestone(step)


# --------------------------------------------------------------------------- data
@dataclass
class DatasetSource:
    path: str = ""
    weight: float = 1.0
    name: str = ""
    hf_name: str = ""
    hf_config: str = ""

    def __post_init__(self) -> None:
        _require(self.weight > 0, f"Dataset weight must be positive, got {self.weight}")


@dataclass
class TrainingPhase:
    start_step: int = 0
    dataset_weights: dict[str, float] = field(default_factory=dict)
    lr_scale: float = 1.0

    def __post_init__(self) -> None:
        _require(self.start_step >= 0, "TrainingPhase.start_step must be non-negative")
        _require(self.lr_scale > 0, "TrainingPhase.lr_scale must be positive")
        for key, w in self.dataset_weights.items():
            _require(w >= 0, f"TrainingPhase.dataset_weights['{key}'] must be non-negative")


@dataclass
class DataConfig:
    dataset_path: str = ""
    file_pattern: str = "*.npy"
    tokenizer_path: str = ""
    num_workers: int = 4
    pin_memory: bool = True
    prefetch_factor: int = 2
    hf_dataset_name: str | None = None
    hf_dataset_config: str | None = None
    hf_dataset_split: str = "train"
    hf_dataset_text_field: str = "text"
    hf_dataset_image_field: str = "image"
    hf_dataset_prompt_field: str = ""
    hf_image_size: int = 224
    hf_streaming: bool = False
    pack_sequences: bool = False
    datasets: list[DatasetSource] = field(default_factory=list)
    mix_temperature: float = 1.0
    phases: list[TrainingPhase] = field(default_factory=list)
    anneal_start_step: int = 0
    anneal_weights: dict[str, float] = field(default_factory=dict)

    def __post_init__(self) -> None:
        _require(self.num_workers >= 0, "num_workers must be non-negative")
        _require(self.prefetch_factor >= 1, "prefetch_factor must be >= 1")
        _require(self.mix_temperature > 0, "mix_temperature must be positive")
        for src in self.datasets:
            _require(
                bool(src.path or src.hf_name),
                f"DatasetSource '{src.name}' must have either path or hf_name",
            )
        starts = [p.start_step for p in self.phases]
        _require(
            all(a < b for a, b in zip(starts, starts[1:])),
            "data.phases start_steps must be strictly monotonically increasing",
        )
        _require(self.anneal_start_step >= 0, "anneal_start_step must be non-negative")
        _require(
            not (self.phases and self.anneal_start_step > 0),
            "Cannot use both data.phases and data.anneal_start_step",
        )

    def effective_phases(self) -> list[TrainingPhase]:
        """Explicit phases, or the single phase implied by the annealing shortcut."""
        if self.phases:
            return list(self.phases)
        if self.anneal_start_step > 0 and self.anneal_weights:
            return [
                TrainingPhase(
                    start_step=self.anneal_start_step, dataset_weights=dict(self.anneal_weights)
                )
            ]
        return []


# --------------------------------------------------------------------------- eval / metrics / profiling
@dataclass
class EvalConfig:
    enabled: bool = False
    interval: int = 1000
    steps: int = 50
    dataset_path: str = ""
    file_pattern: str = "*.npy"
    hf_dataset_name: str | None = None
    hf_dataset_config: str | None = None
    hf_dataset_split: str = "validation"

    def __post_init__(self) -> None:
        _require(self.interval > 0, "eval interval must be positive")
        _require(self.steps > 0, "eval steps must be positive")


@dataclass
class MetricsConfig:
    log_interval: int = 10
    enable_wandb: bool = False
    enable_tensorboard: bool = False
    wandb_project: str = "kempnerforge"
    wandb_run_name: str | None = None
    wandb_run_id: str = ""
    tensorboard_dir: str = "tb_logs"

    def __post_init__(self) -> None:
        _require(self.log_interval > 0, "log_interval must be positive")


@dataclass
class ProfilingConfig:
    enable: bool = False
    start_step: int = 5
    end_step: int = 8
    trace_dir: str = "profiler_traces"

    def __post_init__(self) -> None:
        _require(self.end_step > self.start_step, "end_step must be greater than start_step")


def section_field_names(cls) -> list[str]:
    return [f.name for f in fields(cls)]
