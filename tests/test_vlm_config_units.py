"""Vision-language configuration: architecture union, head resolution, modality lists, adapter / encoder /
video sections.  Mirrors tests/unit/test_vlm_config.py, test_vision_config.py, test_video_config.py of the reference."""

from __future__ import annotations

import pytest

from kempnerforge_b200.config import load_config
from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.config.vlm import (AdapterConfig, CrossAttentionConfig, FreezeSpec, FreezeStage,
                                          JointDecoderConfig, MoMaConfig, MoTConfig, VideoConfig, VisionEncoderConfig,
                                          VLMConfig, pooled_token_count)


# --------------------------------------------------------------------------- architecture union
def test_defaults_and_registered_archs():
    c = VLMConfig()
    assert c.arch == "joint_decoder" and c.max_text_len == 512
    assert c.freeze == [FreezeSpec("vision_encoder", True)] and c.freeze_schedule == []
    assert {"joint_decoder", "cross_attention", "mot", "moma"} <= set(registry.list("vlm_config"))


@pytest.mark.parametrize("arch,cls", [("joint_decoder", JointDecoderConfig), ("cross_attention", CrossAttentionConfig),
                                      ("mot", MoTConfig), ("moma", MoMaConfig)])
def test_for_arch_returns_the_subclass(arch, cls):
    c = VLMConfig.for_arch(arch, max_text_len=64)
    assert type(c) is cls and c.arch == arch and c.max_text_len == 64


def test_for_arch_unknown_lists_the_registered_names():
    with pytest.raises(ValueError) as err:
        VLMConfig.for_arch("perceiver")
    assert "joint_decoder" in str(err.value) and "mot" in str(err.value)
    with pytest.raises(ValueError):
        VLMConfig(arch="perceiver")


def test_base_rules():
    with pytest.raises(ValueError):
        VLMConfig(max_text_len=0)
    ok = VLMConfig(freeze_schedule=[FreezeStage(10, (FreezeSpec("adapter", False),)),
                                    FreezeStage(20, (FreezeSpec("vision_encoder", False),))])
    assert [s.start_step for s in ok.freeze_schedule] == [10, 20]
    with pytest.raises(ValueError):
        VLMConfig(freeze_schedule=[FreezeStage(20, ()), FreezeStage(10, ())])
    with pytest.raises(ValueError):
        VLMConfig(freeze_schedule=[FreezeStage(10, ()), FreezeStage(10, ())])


def test_residual_stream_image_tokens_per_arch():
    assert JointDecoderConfig().residual_stream_image_tokens(49) == 49
    assert MoTConfig().residual_stream_image_tokens(49) == 49
    assert CrossAttentionConfig().residual_stream_image_tokens(49) == 0


# --------------------------------------------------------------------------- cross attention
def test_cross_attention_rules_and_head_resolution():
    c = CrossAttentionConfig()
    assert c.cross_attention_every_n_layers == 4 and "cross_attention" in c.module_patterns
    for bad in (dict(cross_attention_every_n_layers=0), dict(cross_attention_n_heads=-1), dict(cross_attention_n_kv_heads=-2)):
        with pytest.raises(ValueError):
            CrossAttentionConfig(**bad)
    assert c.resolved_heads(16) == (16, 16)                                               # both inherit: MHA
    assert CrossAttentionConfig(cross_attention_n_kv_heads=4).resolved_heads(16) == (16, 4)   # GQA
    assert CrossAttentionConfig(cross_attention_n_heads=8).resolved_heads(16) == (8, 8)
    assert CrossAttentionConfig(cross_attention_n_heads=8, cross_attention_n_kv_heads=2).resolved_heads(16) == (8, 2)
    with pytest.raises(ValueError):
        c.resolved_heads(0)


# --------------------------------------------------------------------------- MoT / MoMa
def test_mot_rules():
    c = MoTConfig()
    assert c.mot_modalities == ("image", "text") and c.mot_warm_start_path == "" and "mot" in c.module_patterns
    for bad in (("image",), ("image", "audio"), ("text", "audio"), ("image", "text", "text")):
        with pytest.raises(ValueError):
            MoTConfig(mot_modalities=bad)
    for bad in (dict(mot_image_n_heads=-1), dict(mot_image_n_kv_heads=-1), dict(mot_warm_start_from_text=True)):
        with pytest.raises(ValueError):
            MoTConfig(**bad)
    ok = MoTConfig(mot_warm_start_from_text=True, mot_warm_start_path="/ckpt")
    assert ok.mot_warm_start_path == "/ckpt"
    assert MoTConfig(mot_warm_start_path="/ckpt").mot_warm_start_from_text is False


def test_mot_image_head_resolution():
    assert MoTConfig().resolved_image_heads(16) == (16, 16)
    assert MoTConfig().resolved_image_heads(16, 4) == (16, 4)                # inherits the model's GQA
    assert MoTConfig(mot_image_n_kv_heads=2).resolved_image_heads(16, 4) == (16, 2)
    assert MoTConfig(mot_image_n_heads=8).resolved_image_heads(16) == (8, 8)
    with pytest.raises(ValueError):
        MoTConfig().resolved_image_heads(0)


def test_moma_rules_and_capacity():
    c = MoMaConfig()
    assert c.moma_experts_per_modality == {"image": 4, "text": 4} and c.moma_gumbel_noise is True
    assert c.effective_capacity_factor("image") == 0.25
    assert MoMaConfig(moma_capacity_factor=1.5).effective_capacity_factor("text") == 1.5
    assert MoMaConfig(moma_experts_per_modality={"image": 2, "text": 8}).effective_capacity_factor("text") == 0.125
    for bad in (dict(moma_experts_per_modality={"image": 4}), dict(moma_experts_per_modality={"image": 4, "text": 4, "audio": 1}),
                dict(moma_experts_per_modality={"image": 0, "text": 4}), dict(moma_capacity_factor=-0.1),
                dict(moma_modalities=("image",))):
        with pytest.raises(ValueError):
            MoMaConfig(**bad)


# --------------------------------------------------------------------------- adapter / encoder
def test_adapter_rules_and_token_counts():
    a = AdapterConfig()
    assert a.type == "mlp_2layer" and a.output_num_tokens(196) == 196 and a.extra_kwargs()["hidden_dim"] is None
    for bad in (dict(type="nope"), dict(hidden_dim=-1), dict(activation="tanh"), dict(pool_window=0), dict(pool_heads=0)):
        with pytest.raises(ValueError):
            AdapterConfig(**bad)
    assert AdapterConfig(hidden_dim=64).extra_kwargs()["hidden_dim"] == 64
    assert pooled_token_count(196, 2) == 49
    assert pooled_token_count(196, 1) == 196


def test_vision_encoder_rules():
    v = VisionEncoderConfig()
    assert (v.type, v.path, v.feature_dim, v.num_tokens) == ("random", "", 0, 0)   # zeros: inferred from the encoder
    e = VisionEncoderConfig(type="siglip2", path="/models/s", feature_dim=768, num_tokens=196)
    assert e.path == "/models/s" and e.feature_dim == 768
    for bad in (dict(type="resnet"), dict(feature_dim=-1), dict(num_tokens=-1)):
        with pytest.raises(ValueError):
            VisionEncoderConfig(**bad)
    for name in ("random", "siglip2", "clip"):
        VisionEncoderConfig(type=name)


# --------------------------------------------------------------------------- video
def test_video_defaults_and_rules():
    v = VideoConfig()
    assert (v.dataset_type, v.sampling_policy, v.split, v.max_frames, v.min_frames) == ("webvid", "uniform", "train", 16, 4)
    for bad in (dict(split="test"), dict(min_frames=8, max_frames=4), dict(fps=0.0), dict(fps=-1.0), dict(frame_size=0),
                dict(max_samples=-1), dict(min_frames=0), dict(max_frames=0), dict(dataset_type="kinetics"),
                dict(sampling_policy="random_walk")):
        with pytest.raises(ValueError):
            VideoConfig(**bad)
    assert VideoConfig(split="validation", max_samples=10).max_samples == 10


def test_video_section_needs_a_vlm_section(tmp_path):
    p = tmp_path / "v.toml"
    p.write_text('[video]\ndata_root = "/data/webvid"\n')
    with pytest.raises(ValueError):
        load_config(str(p))
    p.write_text('[vlm]\narch = "joint_decoder"\n[vision_encoder]\ntype = "random"\nfeature_dim = 32\nnum_tokens = 4\n'
                 '[video]\ndata_root = "/data/webvid"\nmax_frames = 8\n')
    cfg = load_config(str(p))
    assert cfg.is_video and cfg.is_vlm and cfg.video.max_frames == 8
    p.write_text('[vlm]\narch = "mot"\n[vision_encoder]\ntype = "random"\nfeature_dim = 32\nnum_tokens = 4\n')
    cfg = load_config(str(p))
    assert cfg.is_vlm and not cfg.is_video and type(cfg.vlm) is MoTConfig
    p.write_text('[train]\nbatch_size = 2\n')
    cfg = load_config(str(p))
    assert not cfg.is_vlm and not cfg.is_video
