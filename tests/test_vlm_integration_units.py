"""Vision-language wrappers end to end on CPU: every architecture builds, runs, learns and round-trips its weights.

Mirrors tests/integration/test_vlm_train_step.py, test_vlm_cross_attn.py, test_vlm_mot.py, test_vlm_moma.py and
test_vlm_checkpoint.py of the reference."""

from __future__ import annotations

import pytest
import torch

from kempnerforge_b200.config.sections import ModelConfig
from kempnerforge_b200.config.vlm import AdapterConfig, FreezeSpec, VisionEncoderConfig, VLMConfig
from kempnerforge_b200.models.mot import mot_warm_start_from_text_stack
from kempnerforge_b200.models.vlm import build_vlm_wrapper, inner_transformer, is_encoder_frozen
from kempnerforge_b200.training.freeze import apply_freeze_specs, effective_freeze

ARCHS = ["joint_decoder", "cross_attention", "mot", "moma"]


def _build(arch="joint_decoder", model_kw=None, frames=1, **vlm_kw):
    torch.manual_seed(0)
    mc = ModelConfig(**{**dict(dim=32, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=64, ffn_hidden_dim=48,
                               max_seq_len=48), **(model_kw or {})})
    if arch == "cross_attention":
        vlm_kw.setdefault("cross_attention_every_n_layers", 2)
    if arch == "moma":
        vlm_kw.setdefault("moma_experts_per_modality", {"image": 2, "text": 2})
        vlm_kw.setdefault("moma_gumbel_noise", False)
    vc = VLMConfig.for_arch(arch, max_text_len=12, **vlm_kw)
    model = build_vlm_wrapper(mc, VisionEncoderConfig(type="random", feature_dim=16, num_tokens=4),
                              AdapterConfig(type="mlp_2layer"), vc, frames_per_clip=frames)
    return model, vc


def _batch(b=2, t=10, frames=1):
    g = torch.Generator().manual_seed(1)
    px = torch.rand(b, 3, 16, 16, generator=g) if frames == 1 else torch.rand(b, frames, 3, 16, 16, generator=g)
    ids = torch.randint(1, 64, (b, t), generator=g)
    return px, ids, ids.clone()


@pytest.mark.parametrize("arch", ARCHS)
def test_builds_runs_and_returns_text_logits_only(arch):
    model, _ = _build(arch)
    px, ids, labels = _batch()
    logits, passed = model(px, ids, labels)
    assert logits.shape == (2, 10, 64) and passed is labels          # image positions never reach the head
    assert model.num_image_tokens == (0 if arch == "cross_attention" else 4)
    loss = model.compute_loss(px, ids, labels)
    assert torch.isfinite(loss) and abs(float(loss) - 4.16) < 1.0    # ~ log(64) at random init
    loss.backward()
    if arch in ("cross_attention", "mot"):   # zero-initialised output projections: the image path opens through them
        key = "cross_attention" if arch == "cross_attention" else "attn.o_proj.text"
        gates = [p for n, p in model.named_parameters() if key in n and "o_proj" in n and n.endswith("weight")]
        assert gates and all(p.grad.abs().sum() > 0 for p in gates)
    else:
        assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in model.adapter.parameters())
    assert inner_transformer(model) is model.transformer and inner_transformer(model.transformer) is model.transformer


@pytest.mark.parametrize("arch", ARCHS)
def test_overfits_a_tiny_batch_with_a_frozen_encoder(arch):
    model, vc = _build(arch)
    apply_freeze_specs(model, effective_freeze(vc, 0), vc.module_patterns)
    assert is_encoder_frozen(effective_freeze(vc, 0))
    assert all(not p.requires_grad for p in model.vision_encoder.parameters())
    enc = [p.detach().clone() for p in model.vision_encoder.parameters()]
    opt = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=3e-3, weight_decay=0.1)
    px, ids, labels = _batch()
    first = None
    for _ in range(40):
        opt.zero_grad()
        loss = model.compute_loss(px, ids, labels)
        first = float(loss) if first is None else first
        loss.backward()
        opt.step()
    assert float(loss) < 0.6 * first
    for a, b in zip(enc, model.vision_encoder.parameters()):
        assert torch.equal(a, b)                                      # no weight-decay drift on frozen parameters


@pytest.mark.parametrize("arch", ARCHS)
def test_state_dict_round_trip_gives_the_same_forward(arch):
    a, _ = _build(arch)
    b, _ = _build(arch)
    with torch.no_grad():
        for p in a.parameters():
            p.add_(0.01 * torch.randn_like(p))
    missing = b.load_state_dict(a.state_dict())
    assert not missing.missing_keys and not missing.unexpected_keys
    px, ids, labels = _batch()
    a.eval(), b.eval()
    assert torch.allclose(a(px, ids)[0], b(px, ids)[0], atol=1e-6)


def test_image_content_changes_text_logits_for_every_route():
    for arch in ARCHS:
        model, _ = _build(arch)
        with torch.no_grad():                                       # open the zero-initialised gates
            for n, p in model.named_parameters():
                if p.dim() == 2 and torch.count_nonzero(p) == 0:
                    p.normal_(std=0.1)
        px, ids, _ = _batch()
        model.eval()
        base = model(px, ids)[0]
        other = model(torch.rand_like(px), ids)[0]
        assert not torch.allclose(base, other, atol=1e-5), arch


def test_all_padding_labels_give_a_zero_loss_without_nans():
    model, _ = _build("joint_decoder")
    px, ids, _ = _batch()
    loss = model.compute_loss(px, ids, torch.full_like(ids, -100))
    assert float(loss) == 0.0
    loss.backward()
    assert all(torch.isfinite(p.grad).all() for p in model.parameters() if p.grad is not None)


def test_label_shift_is_the_default_and_can_be_disabled():
    model, _ = _build("joint_decoder")
    px, ids, labels = _batch()
    shifted = model.compute_loss(px, ids, labels)
    unshifted = model.compute_loss(px, ids, labels, shift_labels=False)
    manual = model.compute_loss(px, ids, torch.cat([labels[:, 1:], torch.full_like(labels[:, :1], -100)], 1),
                                shift_labels=False)
    assert torch.allclose(shifted, manual) and not torch.allclose(shifted, unshifted)


def test_context_length_is_checked_at_build_time():
    with pytest.raises(ValueError, match="max_seq_len"):
        _build("joint_decoder", model_kw=dict(max_seq_len=12))
    _build("cross_attention", model_kw=dict(max_seq_len=12))          # image tokens take no residual positions


def test_video_clips_multiply_the_visual_tokens_and_masked_frames_are_ignored():
    model, _ = _build("joint_decoder", frames=3)
    assert model.num_image_tokens == 12
    px, ids, labels = _batch(frames=3)
    full = torch.ones(2, 3, dtype=torch.bool)
    model.eval()
    base = model(px, ids, frame_mask=full)[0]
    assert base.shape == (2, 10, 64)
    mask = full.clone()
    mask[:, 2] = False
    px2 = px.clone()
    px2[:, 2] = torch.rand_like(px2[:, 2])                           # a masked frame's content must not matter
    assert torch.allclose(model(px, ids, frame_mask=mask)[0], model(px2, ids, frame_mask=mask)[0], atol=1e-5)
    with pytest.raises(ValueError, match="frames"):
        model(px[:, :2], ids)


def test_cross_attention_layers_follow_the_cadence_and_the_freeze_alias():
    model, vc = _build("cross_attention", cross_attention_every_n_layers=2)
    t = model.transformer
    ca = [n for n, _ in t.named_modules() if n.startswith("cross_attention_layers.") and n.count(".") == 1]
    assert len(ca) == 2
    specs = [FreezeSpec("transformer", True), FreezeSpec("cross_attention", False)]
    apply_freeze_specs(model, specs, vc.module_patterns)
    trainable = {n for n, p in model.named_parameters() if p.requires_grad and n.startswith("transformer.")}
    assert trainable and all("cross_attention" in n for n in trainable)
    # a name that is no alias is taken as a raw pattern (here: one that matches nothing); typos are caught earlier, by
    # effective_freeze(..., valid_modules=...)
    assert apply_freeze_specs(model, [FreezeSpec("cross_atention", True)], vc.module_patterns) == {"cross_atention": 0}


def test_joint_decoder_weights_load_into_a_cross_attention_model_non_strictly():
    jd, _ = _build("joint_decoder")
    ca, _ = _build("cross_attention")
    res = ca.load_state_dict(jd.state_dict(), strict=False)
    assert not res.unexpected_keys and res.missing_keys
    assert all("cross_attention" in k for k in res.missing_keys)


def test_mot_warm_start_from_a_joint_decoder_copies_every_modality():
    jd, _ = _build("joint_decoder")
    mot, _ = _build("mot")
    n = mot_warm_start_from_text_stack(mot.transformer, jd.transformer.state_dict())
    assert n > 0 and mot_warm_start_from_text_stack(mot.transformer, jd.transformer.state_dict()) == n
    src = jd.transformer.layers["1"].attention.q_proj.weight
    att = mot.transformer.layers["1"].attn
    assert torch.equal(att.q_proj["image"].weight, src) and torch.equal(att.q_proj["text"].weight, src)


def test_moma_experts_are_private_to_their_modality():
    model, _ = _build("moma")
    px, ids, _ = _batch()
    model.eval()
    base = model(px, ids)[0]
    blocks = [m for m in model.transformer.modules() if type(m).__name__ == "MoMaFFN"]
    assert blocks
    with torch.no_grad():
        for blk in blocks:
            for n, p in blk.named_parameters():
                if ".image." in f".{n}" or n.startswith("image"):
                    p.add_(1.0)
    moved = model(px, ids)[0]
    # image experts changed: text logits move only through attention to image positions, so they do change ...
    assert not torch.allclose(base, moved)
    model2, _ = _build("moma", moma_experts_per_modality={"image": 1, "text": 3})
    assert model2(px, ids)[0].shape == (2, 10, 64)                   # unbalanced expert counts build and run
    model3, vc3 = _build("moma", moma_capacity_factor=1.0)
    assert vc3.effective_capacity_factor("text") == 1.0 and torch.isfinite(model3(px, ids)[0]).all()


def test_moe_backbone_inside_a_vlm_trains_and_exposes_moe_accessors():
    model, _ = _build("joint_decoder", model_kw=dict(num_experts=4, moe_top_k=2, moe_aux_loss_weight=0.01))
    px, ids, labels = _batch()
    loss = model.compute_loss(px, ids, labels)
    loss.backward()
    t = inner_transformer(model)
    assert hasattr(t, "get_moe_aux_loss") or hasattr(t, "moe_aux_loss")
    routers = [p for n, p in model.named_parameters() if "router" in n or "gate" in n]
    assert routers and any(p.grad is not None and p.grad.abs().sum() > 0 for p in routers)


@pytest.mark.parametrize("arch,mode", [("mot", "full"), ("mot", "selective"), ("moma", "full"), ("moma", "selective")])
def test_activation_checkpointing_reaches_mot_and_moma_blocks_and_leaves_gradients_unchanged(arch, mode):
    from kempnerforge_b200.parallel.parallel import apply_ac

    kw = dict(moma_gumbel_noise=True) if arch == "moma" else {}      # routing noise must repeat in the recomputation
    px, ids, labels = _batch()
    grads = {}
    for m in ("none", mode):
        model, _ = _build(arch, **kw)
        for p in model.parameters():                 # open the zero-initialised output projections
            if p.dim() == 2 and float(p.abs().sum()) == 0:
                torch.nn.init.normal_(p, std=0.05, generator=torch.Generator().manual_seed(2))
        if m != "none":
            apply_ac(model, m)
            blocks = [b for b in model.transformer.modules() if type(b).__name__ in ("MoTBlock", "MoMaBlock")]
            assert blocks and all(b.ac_mode == m for b in blocks)
        model.train()
        torch.manual_seed(11)
        loss = model.compute_loss(px, ids, labels)
        loss.backward()
        grads[m] = (float(loss), {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None})
    assert grads["none"][0] == pytest.approx(grads[mode][0], rel=1e-6)
    assert grads["none"][1].keys() == grads[mode][1].keys()
    for n, g in grads["none"][1].items():
        assert torch.allclose(g, grads[mode][1][n], atol=1e-6), n
