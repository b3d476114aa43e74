"""Configuration: typed sections, TOML + CLI loader, component registry."""

from kempnerforge_b200.config.job import JobConfig
from kempnerforge_b200.config.loader import (
    ConfigError,
    config_from_dict,
    config_to_dict,
    load_config,
    parse_cli_overrides,
)
from kempnerforge_b200.config.registry import Registry, registry
from kempnerforge_b200.config.sections import (
    Activation,
    ActivationCheckpointing,
    AsyncCheckpointMode,
    CheckpointConfig,
    DataConfig,
    DatasetSource,
    DistributedConfig,
    DynamicCheckpointWindow,
    EvalConfig,
    MetricsConfig,
    ModelConfig,
    NormType,
    OptimizerConfig,
    PipelineSchedule,
    ProfilingConfig,
    SchedulerConfig,
    SchedulerType,
    TrainConfig,
    TrainingPhase,
)
from kempnerforge_b200.config.vlm import (
    AdapterConfig,
    CrossAttentionConfig,
    FreezeSpec,
    FreezeStage,
    JointDecoderConfig,
    MoMaConfig,
    MoTConfig,
    VideoConfig,
    VisionEncoderConfig,
    VLMConfig,
)

__all__ = [n for n in dir() if not n.startswith("_")]
