"""Mixture-of-experts layers on CPU, one behaviour per test: the MoE MLP and its statistics, placement inside the
transformer, shared experts, capacity, gradient scaling, packed expert storage and the expert-parallel config rules.

Behaviours of kempnerforge/model/moe.py, kempnerforge/model/router.py, kempnerforge/model/transformer.py (MoE
accessors) and kempnerforge/config/{model,distributed,job}.py (MoE / EP validation)."""

import pytest
import torch

from kempnerforge_b200.config import DistributedConfig, ModelConfig, config_from_dict
from kempnerforge_b200.models import Transformer
from kempnerforge_b200.models.moe import MoEMLP, apply_capacity, build_moe

DIM, HID, E, K = 32, 48, 4, 2


def _tokens(n=24, seed=0):
    return torch.randn(1, n, DIM, generator=torch.Generator().manual_seed(seed))


def _cfg(**kw):
    base = dict(dim=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=32, ffn_hidden_dim=48,
                num_experts=4, moe_top_k=2)
    base.update(kw)
    return ModelConfig(**base)


# --------------------------------------------------------------------------- the MoE MLP
def test_output_has_the_input_shape_and_every_parameter_gets_a_gradient():
    torch.manual_seed(0)
    moe = build_moe(DIM, HID, E, K)
    x = _tokens().requires_grad_(True)
    y = moe(x)
    assert y.shape == x.shape
    (y.pow(2).mean() + moe.aux_loss).backward()
    assert x.grad is not None
    missing = [n for n, p in moe.named_parameters() if p.grad is None]
    assert missing == []          # 24 tokens x top-2 over 4 experts: every expert saw tokens


def test_statistics_are_available_after_a_forward():
    moe = build_moe(DIM, HID, E, K)
    moe(_tokens())
    assert moe.aux_loss.dim() == 0 and float(moe.aux_loss) > 0
    assert moe.expert_counts.shape == (E,) and int(moe.expert_counts.sum()) == 24 * K


def test_z_loss_is_the_mean_squared_logsumexp_of_the_gate_logits():
    moe = build_moe(DIM, HID, E, K)
    x = _tokens()
    moe(x)
    logits = moe.router.gate(x.reshape(-1, DIM)).float()
    assert torch.allclose(moe.z_loss, torch.logsumexp(logits, dim=-1).pow(2).mean(), atol=1e-6)


def test_experts_do_not_share_weights_and_come_from_the_mlp_registry():
    moe = build_moe(DIM, HID, E, K)
    mods = moe.expert_modules()
    assert len(mods) == E and type(mods[0]).__name__ == "SwiGLUMLP"
    assert not torch.equal(mods[0].up_proj.weight, mods[1].up_proj.weight)
    gelu = build_moe(DIM, HID, E, K, activation="gelu")
    assert type(gelu.expert_modules()[0]).__name__ == "StandardMLP" and gelu(_tokens()).shape == (1, 24, DIM)


def test_one_expert_with_top_one_is_the_dense_mlp():
    torch.manual_seed(1)
    moe = build_moe(DIM, HID, 1, 1)
    x = _tokens()
    assert torch.allclose(moe(x), moe.expert_modules()[0](x), atol=1e-6)


# --------------------------------------------------------------------------- inside the transformer
def test_moe_frequency_and_first_dense_layers_place_the_moe_blocks():
    every = Transformer(_cfg(n_layers=4))
    assert [isinstance(b.mlp, MoEMLP) for b in every.layers.values()] == [True] * 4
    alternate = Transformer(_cfg(n_layers=4, moe_frequency=2))
    kinds = [isinstance(b.mlp, MoEMLP) for b in alternate.layers.values()]
    assert sum(kinds) == 2 and kinds != [True] * 4
    dense_first = Transformer(_cfg(n_layers=4, moe_first_k_dense=1))
    assert not isinstance(dense_first.layers["0"].mlp, MoEMLP) and isinstance(dense_first.layers["1"].mlp, MoEMLP)


def test_a_dense_model_reports_zero_losses_and_no_counts():
    dense = Transformer(_cfg(num_experts=0))
    dense(torch.randint(0, 64, (1, 8)))
    assert float(dense.get_moe_aux_loss()) == 0.0 and float(dense.get_moe_router_z_loss()) == 0.0
    assert dense.get_expert_counts() == {}
    dense.set_moe_step(3, 10)     # nothing to propagate to: must not raise


def test_model_level_accessors_sum_over_the_moe_layers():
    model = Transformer(_cfg())
    model(torch.randint(0, 64, (2, 8)))
    per_layer = [b.mlp.aux_loss for b in model.layers.values()]
    assert torch.allclose(model.get_moe_aux_loss(), sum(per_layer))
    counts = model.get_expert_counts()
    assert sorted(counts) == [0, 1] and all(int(c.sum()) == 2 * 8 * 2 for c in counts.values())
    assert float(model.get_moe_router_z_loss()) > 0


def test_router_statistics_are_not_part_of_the_state_dict():
    keys = Transformer(_cfg()).state_dict().keys()
    assert not any("aux_loss" in k or "z_loss" in k or "expert_counts" in k for k in keys)


def test_fine_grained_experts_are_narrower_and_the_estimate_counts_them():
    fine = _cfg(moe_expert_ffn_multiplier=0.5)
    assert fine.computed_expert_ffn_hidden_dim < fine.computed_ffn_hidden_dim
    model = Transformer(fine)
    up = model.layers["0"].mlp.expert_modules()[0].up_proj.weight
    assert up.shape[0] == fine.computed_expert_ffn_hidden_dim
    assert abs(fine.num_params_estimate - sum(p.numel() for p in model.parameters())) / fine.num_params_estimate < 0.05


def test_set_moe_step_reaches_sigmoid_routers_only():
    sig = Transformer(_cfg(moe_router="sigmoid_topk", moe_bias_schedule="cosine_decay"))
    sig.set_moe_step(7, 20)
    assert all(b.mlp.router._step == 7 and b.mlp.router._max_steps == 20 for b in sig.layers.values())
    soft = Transformer(_cfg())
    soft.set_moe_step(7, 20)
    assert not hasattr(soft.layers["0"].mlp.router, "_step")


# --------------------------------------------------------------------------- shared experts
def test_the_shared_expert_is_added_for_every_token():
    torch.manual_seed(2)
    moe = build_moe(DIM, HID, E, K, shared_experts=1)
    x = _tokens()
    full = moe(x)
    shared = moe.shared_expert
    moe.shared_expert = None
    assert torch.allclose(full, moe(x) + shared(x.reshape(-1, DIM)).view_as(x), atol=1e-6)


def test_shared_expert_width_and_parameter_count():
    base = build_moe(DIM, HID, E, K)
    one = build_moe(DIM, HID, E, K, shared_experts=2)
    wide = build_moe(DIM, HID, E, K, shared_experts=2, shared_expert_widen=True)
    n = lambda m: sum(p.numel() for p in m.parameters())  # noqa: E731
    assert n(one) - n(base) == 3 * DIM * HID                 # one shared MLP of the experts' width, however many are asked for
    assert n(wide) - n(base) == 3 * DIM * HID * 2             # widened: one MLP of shared_experts x the width


# --------------------------------------------------------------------------- capacity
def test_capacity_zeroes_the_weights_of_late_arrivals_only():
    idx = torch.tensor([[0], [0], [0], [1]])
    w = torch.ones(4, 1)
    new_w, new_idx = apply_capacity(w, idx, num_experts=2, capacity_factor=1.0)   # capacity = ceil(4 * 1 / 2) = 2 per slot
    assert new_w.squeeze(1).tolist() == [1.0, 1.0, 0.0, 1.0] and torch.equal(new_idx, idx)


def test_capacity_factor_zero_keeps_everything_and_training_still_works():
    torch.manual_seed(3)
    free = build_moe(DIM, HID, E, K, capacity_factor=0.0)
    tight = build_moe(DIM, HID, E, K, capacity_factor=0.5)
    tight.load_state_dict(free.state_dict())
    x = _tokens(64)
    assert not torch.allclose(free(x), tight(x))       # some assignments were dropped
    tight(x).sum().backward()
    assert all(torch.isfinite(p.grad).all() for p in tight.parameters() if p.grad is not None)


# --------------------------------------------------------------------------- gradient scaling
def test_gradient_scale_is_off_by_default_and_acts_in_training_only():
    assert build_moe(DIM, HID, E, K).gradient_scale is False
    torch.manual_seed(4)
    plain = build_moe(DIM, HID, E, K)
    scaled = build_moe(DIM, HID, E, K, gradient_scale=True)
    scaled.load_state_dict(plain.state_dict())
    x = _tokens(40)
    assert torch.allclose(plain.eval()(x), scaled.eval()(x), atol=1e-6)
    y = scaled.train()(x)
    assert y.shape == x.shape and torch.isfinite(y).all()
    y.sum().backward()
    assert all(torch.isfinite(p.grad).all() for p in scaled.parameters() if p.grad is not None)


# --------------------------------------------------------------------------- packed experts
def test_packed_storage_is_three_stacked_tensors_without_an_expert_list():
    packed = build_moe(DIM, HID, E, K, packed_experts=True)
    names = dict(packed.named_parameters())
    assert packed.up_w.shape == (E, DIM, HID) and packed.gate_w.shape == (E, DIM, HID) and packed.down_w.shape == (E, HID, DIM)
    assert not any(n.startswith("experts.") for n in names) and not hasattr(packed, "experts")
    assert {"up_w", "gate_w", "down_w"} <= set(names)
    assert len(names) == 3 + 1                      # + the router's gate: the count does not grow with the experts
    more = build_moe(DIM, HID, 16, K, packed_experts=True)
    assert len(dict(more.named_parameters())) == len(names)


def test_non_gated_packed_experts_store_no_gate():
    packed = build_moe(DIM, HID, E, K, activation="gelu", packed_experts=True)
    assert not hasattr(packed, "gate_w") and packed.up_w.shape == (E, DIM, HID)


@pytest.mark.parametrize("activation", ["silu", "gelu"])
def test_packed_and_unpacked_experts_compute_the_same_function(activation):
    torch.manual_seed(5)
    plain = build_moe(DIM, HID, E, K, activation=activation)
    packed = build_moe(DIM, HID, E, K, activation=activation, packed_experts=True)
    packed.router.load_state_dict(plain.router.state_dict())
    with torch.no_grad():
        for e, mod in enumerate(plain.expert_modules()):
            packed.up_w[e].copy_(mod.up_proj.weight.t())
            packed.down_w[e].copy_(mod.down_proj.weight.t())
            if activation == "silu":
                packed.gate_w[e].copy_(mod.gate_proj.weight.t())
    x = _tokens(30)
    assert torch.allclose(plain(x), packed(x), atol=1e-5)
    packed(x).sum().backward()
    assert packed.up_w.grad is not None and float(packed.up_w.grad.abs().sum()) > 0


def test_the_transformer_passes_the_packed_flag_down():
    assert Transformer(_cfg(moe_packed_experts=True)).layers["0"].mlp.packed_experts is True
    assert _cfg().moe_packed_experts is False


# --------------------------------------------------------------------------- config rules
def test_sigmoid_router_options_are_validated():
    with pytest.raises(ValueError):
        _cfg(moe_sequence_aux_loss_weight=-0.1)
    with pytest.raises(ValueError):
        _cfg(moe_bias_schedule="exponential")
    for name in ("constant", "cosine_decay", "linear_warmup"):
        assert str(_cfg(moe_bias_schedule=name).moe_bias_schedule) == name
    d = _cfg()
    assert d.moe_sequence_aux_loss_weight == 0.0 and str(d.moe_bias_schedule) == "constant" and d.moe_gradient_scale is False


def test_expert_parallel_degree_defaults_to_one_and_joins_the_world_size_product():
    d = DistributedConfig()
    assert d.ep == 1
    cfg = config_from_dict({"model": dict(num_experts=8, moe_top_k=2), "distributed": dict(ep=2, dp_shard=2)})
    cfg.validate(world_size=4)
    with pytest.raises(ValueError):
        cfg.validate(world_size=6)


def test_expert_parallelism_needs_experts_it_can_divide():
    with pytest.raises(ValueError):
        config_from_dict({"model": dict(num_experts=0), "distributed": dict(ep=2)}).validate(world_size=2)
    with pytest.raises(ValueError):
        config_from_dict({"model": dict(num_experts=6, moe_top_k=2), "distributed": dict(ep=4)}).validate(world_size=4)
    with pytest.raises(ValueError):
        DistributedConfig(ep=0)
