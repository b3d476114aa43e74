"""Config sections, loader, CLI overrides, registry and cross-section validation."""

import pytest

from kempnerforge_b200.config import (
    CheckpointConfig,
    ConfigError,
    DataConfig,
    DatasetSource,
    DistributedConfig,
    DynamicCheckpointWindow,
    JobConfig,
    ModelConfig,
    OptimizerConfig,
    SchedulerConfig,
    TrainConfig,
    TrainingPhase,
    config_from_dict,
    config_to_dict,
    load_config,
    parse_cli_overrides,
    registry,
)


def test_model_derived_dims():
    c = ModelConfig(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, vocab_size=128256, ffn_dim_multiplier=1.3)
    assert c.head_dim == 128
    assert c.computed_ffn_hidden_dim == 14336
    c13 = ModelConfig(dim=5120, n_layers=40, n_heads=40, n_kv_heads=8, ffn_dim_multiplier=1.3)
    assert c13.computed_ffn_hidden_dim == 17920
    assert ModelConfig(dim=2048, n_heads=16, ffn_hidden_dim=10944, num_experts=64, moe_top_k=6,
                       moe_expert_ffn_multiplier=0.12865497).computed_expert_ffn_hidden_dim == 1408


def test_model_param_estimate_matches_llama3_8b():
    c = ModelConfig(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, vocab_size=128256, ffn_hidden_dim=14336)
    assert abs(c.num_params_estimate - 8.03e9) < 0.01e9


@pytest.mark.parametrize("kwargs", [
    dict(dim=0), dict(dim=100, n_heads=3), dict(n_heads=8, n_kv_heads=3), dict(vocab_size=0),
    dict(sdpa_backend="bogus"), dict(num_experts=4, moe_top_k=5), dict(num_experts=4, moe_bias_schedule="x"),
])
def test_model_rejects(kwargs):
    with pytest.raises(ValueError):
        ModelConfig(**kwargs)


def test_moe_layer_placement():
    c = ModelConfig(dim=64, n_layers=6, n_heads=4, num_experts=4, moe_frequency=2)
    assert [c.is_moe_layer(i) for i in range(6)] == [False, True, False, True, False, True]
    c = ModelConfig(dim=64, n_layers=4, n_heads=4, num_experts=4, moe_first_k_dense=1)
    assert [c.is_moe_layer(i) for i in range(4)] == [False, True, True, True]


def test_train_config_dtypes():
    import torch

    assert TrainConfig(mixed_precision="fp8").param_dtype == torch.bfloat16
    assert TrainConfig(mixed_precision="fp8").is_fp8
    assert TrainConfig(seed=7).effective_data_seed == 7
    assert TrainConfig(seed=7, data_seed=9).effective_data_seed == 9
    with pytest.raises(ValueError):
        TrainConfig(batch_size=0)


def test_distributed_resolution():
    d = DistributedConfig(tp=2)
    assert d.resolve(8).dp_shard == 4
    with pytest.raises(ValueError):
        DistributedConfig(dp_shard=3, tp=2).validate_world_size(8)
    with pytest.raises(ValueError):
        DistributedConfig(tp=3).resolve(8)
    # EP multiplies the world size unless it is folded into DP
    assert DistributedConfig(ep=8).resolve(8).dp_shard == 1
    assert DistributedConfig(ep=8, ep_in_dp=True).resolve(8).dp_shard == 8


def test_checkpoint_cadence_and_dynamic_window():
    c = CheckpointConfig(interval=100, dyn_ckpt_window=DynamicCheckpointWindow(start=0, stop=16))
    saves = [s for s in range(0, 40) if c.should_save(s)]
    assert saves == [0, 1, 2, 4, 8, 16]
    assert c.should_save(100) and not c.should_save(150)
    assert c.is_dynamic_milestone(8) and not c.is_dynamic_milestone(9)
    with pytest.raises(ValueError):
        DynamicCheckpointWindow(strategy="nope")


def test_data_config_rules():
    with pytest.raises(ValueError):
        DataConfig(datasets=[DatasetSource(name="x")])
    with pytest.raises(ValueError):
        DataConfig(phases=[TrainingPhase(start_step=5), TrainingPhase(start_step=5)])
    with pytest.raises(ValueError):
        DataConfig(phases=[TrainingPhase(start_step=5)], anneal_start_step=3)
    d = DataConfig(anneal_start_step=10, anneal_weights={"a": 1.0})
    assert d.effective_phases()[0].start_step == 10


def test_cli_overrides_grammar():
    t = parse_cli_overrides(["--train.seq_len=128", "--optimizer.fused", "--model.rope_theta=5e5",
                             "--optimizer.betas=(0.9,0.99)", "--data.dataset_path=/a/b", "--checkpoint.load_path=none"])
    assert t["train"]["seq_len"] == 128 and t["optimizer"]["fused"] is True
    assert t["model"]["rope_theta"] == 5e5 and t["optimizer"]["betas"] == (0.9, 0.99)
    assert t["data"]["dataset_path"] == "/a/b" and t["checkpoint"]["load_path"] is None
    with pytest.raises(ConfigError):
        parse_cli_overrides(["train.seq_len=1"])
    assert parse_cli_overrides(["configs/train/debug.toml", "--train.seq_len=4"]) == {"train": {"seq_len": 4}}   # a preset path is skipped
    with pytest.raises(ConfigError):
        parse_cli_overrides(["--seq_len=1"])


def test_load_config_layers(tmp_path):
    f = tmp_path / "c.toml"
    f.write_text("""
[model]
dim = 256
n_heads = 4
n_layers = 2
[train]
seq_len = 64
activation_checkpointing = "full"
[scheduler]
name = "wsd"
[[data.datasets]]
path = "/x"
weight = 2.0
[[data.phases]]
start_step = 10
lr_scale = 0.5
[data.phases.dataset_weights]
x = 1.0
[checkpoint.dyn_ckpt_window]
stop = 8
""")
    c = load_config(f, ["--train.seq_len=32", "--model.n_kv_heads=2"])
    assert c.model.dim == 256 and c.model.n_kv_heads == 2 and c.train.seq_len == 32
    assert str(c.train.activation_checkpointing) == "full" and str(c.scheduler.name) == "wsd"
    assert c.data.datasets[0].weight == 2.0 and c.data.phases[0].dataset_weights == {"x": 1.0}
    assert c.checkpoint.dyn_ckpt_window.stop == 8
    round_trip = config_from_dict(config_to_dict(c))
    assert round_trip.model == c.model and round_trip.data.phases == c.data.phases


def test_unknown_keys_and_bad_types():
    with pytest.raises(ConfigError):
        load_config(None, ["--model.bogus=1"])
    with pytest.raises(ConfigError):
        load_config(None, ["--nosuch.key=1"])
    with pytest.raises(ConfigError):
        load_config(None, ["--train.seq_len=abc"])
    with pytest.raises(ConfigError):
        load_config(None, ["--train.mixed_precision=fp4"])
    with pytest.raises(FileNotFoundError):
        load_config("/nonexistent.toml")


def test_vlm_union_dispatch():
    c = load_config(None, ["--vlm.arch=cross_attention", "--vlm.cross_attention_every_n_layers=2",
                           "--vision_encoder.type=random", "--vision_encoder.num_tokens=16", "--vision_encoder.feature_dim=32"])
    assert type(c.vlm).__name__ == "CrossAttentionConfig" and c.adapter is not None
    assert c.vlm.residual_stream_image_tokens(16) == 0
    with pytest.raises(ValueError):
        load_config(None, ["--vlm.arch=mot"])  # needs [vision_encoder]
    with pytest.raises(ConfigError):
        load_config(None, ["--vlm.arch=nonsense", "--vision_encoder.type=random"])
    with pytest.raises(ValueError):
        load_config(None, ["--video.max_frames=4"])


@pytest.mark.parametrize("overrides,world", [
    (["--train.seq_len=4096", "--model.max_seq_len=2048"], 1),
    (["--model.tie_embeddings=true", "--distributed.pp=2"], 2),
    (["--eval.enabled=true"], 1),
    (["--distributed.tp=3", "--model.n_heads=32"], 3),
    (["--distributed.tp=2", "--train.mixed_precision=fp8"], 2),
    (["--model.num_experts=4", "--distributed.pp=2"], 2),
    (["--distributed.ep=2"], 2),
    (["--model.num_experts=3", "--model.moe_top_k=1", "--distributed.ep=2"], 2),
    (["--distributed.dp_shard=3"], 4),
])
def test_job_validate_rejections(overrides, world):
    cfg = load_config(None, overrides)
    with pytest.raises(ValueError):
        cfg.validate(world)


def test_registry_surface():
    registry.register("loss", "tmp_test_loss", lambda a, b: 0)
    assert "tmp_test_loss" in registry.list_losses()
    with pytest.raises(ValueError):
        registry.register("loss", "tmp_test_loss", lambda a, b: 0)
    with pytest.raises(KeyError):
        registry.get_loss("definitely_missing")
    registry.unregister("loss", "tmp_test_loss")

    @registry.register_scheduler("tmp_sched")
    def _s(cfg, max_steps):
        return lambda step: 1.0

    assert registry.get_scheduler("tmp_sched") is _s
    registry.unregister("scheduler", "tmp_sched")


def test_reference_presets_load():
    import glob
    import os
    from pathlib import Path

    # the reference checkout: KF_REFERENCE_ROOT, else a "reference" directory beside this repository
    ref = os.environ.get("KF_REFERENCE_ROOT") or str(Path(__file__).resolve().parents[2] / "reference")
    files = glob.glob(os.path.join(ref, "configs", "train", "*.toml"))
    if not files:
        pytest.skip("reference presets not available")
    for f in files:
        cfg = load_config(f)
        assert isinstance(cfg, JobConfig), os.path.basename(f)


def test_optimizer_scheduler_validation():
    with pytest.raises(ValueError):
        OptimizerConfig(lr=0)
    with pytest.raises(ValueError):
        OptimizerConfig(betas=(1.0, 0.9))
    with pytest.raises(ValueError):
        SchedulerConfig(min_lr_ratio=2)
    with pytest.raises(ValueError):
        SchedulerConfig(wsd_decay_type="exp")


def test_reference_import_paths_resolve():
    """Code written against the reference's module layout finds the same objects here."""
    from kempnerforge_b200.config.checkpoint import AsyncCheckpointMode, CheckpointConfig  # noqa: F401
    from kempnerforge_b200.config.model import ModelConfig as M2
    from kempnerforge_b200.config.schema import JobConfig, ModelConfig  # noqa: F401
    from kempnerforge_b200.distributed import clip_grad_norm_, get_dp_info, init_distributed  # noqa: F401
    from kempnerforge_b200.distributed.parallel import build_parallel_model  # noqa: F401
    from kempnerforge_b200.distributed.utils import clip_grad_norm_ as c2
    from kempnerforge_b200.model.attention import Attention, KVCache  # noqa: F401
    from kempnerforge_b200.model.transformer import Transformer
    from kempnerforge_b200.models.transformer import Transformer as T2

    assert M2 is ModelConfig and Transformer is T2 and c2 is clip_grad_norm_


def test_cli_none_reaches_enum_members_and_optional_fields():
    cfg = load_config(None, ["--scheduler.name=none", "--checkpoint.load_path=None", "--scheduler.decay_steps=null"])
    assert str(cfg.scheduler.name) == "none" and cfg.scheduler.decay_steps is None
