"""Activation capture, training hooks and the optimizer zoo on CPU.

Mirrors tests/unit/test_hooks.py, test_training_hooks.py, test_additional_optimizers.py and test_optimizer.py of
the reference."""

from __future__ import annotations

import copy
import sys
import types

import numpy as np
import pytest
import torch
from torch import nn

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.config.sections import ModelConfig, OptimizerConfig
from kempnerforge_b200.models.hooks import ActivationStore, extract_representations, save_activations
from kempnerforge_b200.models.transformer import Transformer
from kempnerforge_b200.training.hooks import HookRunner, StepContext, TrainingHook, load_hooks
from kempnerforge_b200.training.optimizer import (FusedAdamW, Lion, Muon, ScheduleFreeAdamW, build_optimizer,
                                                  build_param_groups, is_muon_eligible, newton_schulz, should_decay)


def _model():
    torch.manual_seed(0)
    return Transformer(ModelConfig(dim=32, n_layers=3, n_heads=4, n_kv_heads=2, vocab_size=40, ffn_hidden_dim=48,
                                   max_seq_len=16))


# --------------------------------------------------------------------------- activation capture
def test_activation_store_captures_named_modules_detached():
    m = _model()
    ids = torch.randint(0, 40, (2, 7))
    with ActivationStore(m, ["layers.0", "layers.2.mlp", "norm"]) as store:
        assert store.layer_names == ["layers.0", "layers.2.mlp", "norm"]
        m(ids)
        for name in store.layer_names:
            act = store.get(name)
            assert act.shape == (2, 7, 32) and not act.requires_grad and act.device.type == "cpu"
            assert act.abs().sum() > 0
        first = store.get("norm").clone()
        m(torch.randint(0, 40, (2, 7)))
        assert store.get("norm").shape == (2, 7, 32) and not torch.equal(store.get("norm"), first)   # the latest pass only
        store.clear()
        assert store.get("norm") is None and store.activations == {}
    with ActivationStore(m, ["norm"], keep_history=True) as hist:
        m(ids)
        m(ids)
        assert len(hist.history("norm")) == 2 and torch.equal(hist.history("norm")[1], hist.get("norm"))
    assert not any(mod._forward_hooks for mod in m.modules())          # no hook outlives the context
    m(ids)                                                            # and the model still runs


def test_activation_store_rejects_unknown_modules_and_does_not_touch_weights():
    m = _model()
    with pytest.raises(KeyError):
        ActivationStore(m, ["layers.99"]).enable()          # unknown names surface when the hooks are installed
    before = copy.deepcopy(m.state_dict())
    with ActivationStore(m, ["layers.1"]) as store:
        m(torch.randint(0, 40, (1, 5)))
        assert set(store.activations) == {"layers.1"}
    after = m.state_dict()
    assert all(torch.equal(before[k], after[k]) for k in before)


def test_captured_block_output_matches_a_manual_forward():
    m = _model().eval()
    ids = torch.randint(0, 40, (1, 6))
    with ActivationStore(m, ["layers.0", "layers.1"]) as store:
        m(ids)
        first, second = store.get("layers.0"), store.get("layers.1")
    with torch.no_grad():
        h = m.forward_hidden(ids)                                     # final hidden states (after the last norm)
    assert first.shape == second.shape == h.shape and not torch.allclose(first, second)


def test_extract_representations_pooling_modes_and_save(tmp_path):
    m = _model()
    m.train()
    batches = [{"input_ids": torch.randint(0, 40, (2, 6))} for _ in range(3)]
    full = extract_representations(m, batches, ["layers.1", "norm"])
    assert full["layers.1"].shape == (6, 6, 32) and m.training
    mean = extract_representations(m, batches, ["norm"], pool="mean")["norm"]
    last = extract_representations(m, batches, ["norm"], pool="last")["norm"]
    assert mean.shape == last.shape == (6, 32)
    assert torch.allclose(mean, full["norm"].mean(1), atol=1e-6) and torch.allclose(last, full["norm"][:, -1], atol=1e-6)
    raw = extract_representations(m, [b["input_ids"] for b in batches[:1]], ["norm"])   # plain tensors work too
    assert raw["norm"].shape == (2, 6, 32)
    path = tmp_path / "nested" / "acts"
    path.parent.mkdir()
    save_activations(full, str(path))
    loaded = np.load(str(path) + ".npz")
    assert set(loaded.files) == {"layers.1", "norm"} and loaded["norm"].shape == (6, 6, 32)


# --------------------------------------------------------------------------- training hooks
class _Recorder(TrainingHook):
    def __init__(self, log, tag):
        self.log, self.tag = log, tag

    def on_train_begin(self, config):
        self.log.append((self.tag, "begin", config))

    def on_step_end(self, ctx):
        self.log.append((self.tag, "step", ctx.step))

    def on_eval_end(self, eval_metrics, step):
        self.log.append((self.tag, "eval", step))

    def on_checkpoint_save(self, step, path):
        self.log.append((self.tag, "ckpt", path))

    def on_train_end(self, step, tokens_seen):
        self.log.append((self.tag, "end", tokens_seen))


def test_hook_runner_dispatches_every_event_in_registration_order():
    log = []
    runner = HookRunner([_Recorder(log, "a")])
    runner.add(_Recorder(log, "b"))
    ctx = StepContext(step=3, loss=1.0, grad_norm=0.5, lr=1e-3, tokens_seen=99, model="m", optimizer="o")
    runner.on_train_begin("cfg")
    runner.on_step_end(ctx)
    runner.on_eval_end({"eval/loss": 1.0}, 3)
    runner.on_checkpoint_save(3, "/ckpt/step_3")
    runner.on_train_end(3, 99)
    assert [e[:2] for e in log] == [(t, ev) for ev in ("begin", "step", "eval", "ckpt", "end") for t in ("a", "b")]
    assert ctx.model == "m" and ctx.metrics == {}


def test_hook_base_class_is_a_noop_and_partial_overrides_work():
    HookRunner().on_step_end(StepContext(1, 0.0, 0.0, 0.0, 0))          # empty runner
    HookRunner(None).on_train_end(1, 1)
    base = TrainingHook()
    for call in (lambda: base.on_train_begin(None), lambda: base.on_step_end(None), lambda: base.on_eval_end({}, 0),
                 lambda: base.on_checkpoint_save(0, ""), lambda: base.on_train_end(0, 0)):
        assert call() is None

    class OnlySteps(TrainingHook):
        seen = 0

        def on_step_end(self, ctx):
            OnlySteps.seen += 1

    r = HookRunner([OnlySteps()])
    r.on_train_begin(None)
    r.on_step_end(StepContext(1, 0.0, 0.0, 0.0, 0))
    r.on_train_end(1, 1)
    assert OnlySteps.seen == 1


def test_hooks_load_from_module_colon_class_specs():
    mod = types.ModuleType("kf_test_hook_module")

    class Mine(TrainingHook):
        pass

    mod.Mine = Mine
    sys.modules["kf_test_hook_module"] = mod
    try:
        (hook,) = load_hooks(["kf_test_hook_module:Mine"])
        assert isinstance(hook, Mine) and load_hooks([]) == []
        with pytest.raises(ValueError):
            load_hooks(["kf_test_hook_module.Mine"])
        with pytest.raises(AttributeError):
            load_hooks(["kf_test_hook_module:Missing"])
    finally:
        del sys.modules["kf_test_hook_module"]


# --------------------------------------------------------------------------- optimizers
def _quadratic():
    torch.manual_seed(1)
    net = nn.Sequential(nn.Linear(8, 16), nn.Tanh(), nn.Linear(16, 4))
    x, y = torch.randn(64, 8), torch.randn(64, 4)
    return net, lambda: (net(x) - y).square().mean()


@pytest.mark.parametrize("name,lr", [("adamw", 1e-2), ("lion", 1e-3), ("schedule_free_adamw", 1e-2), ("muon", 2e-2)])
def test_every_registered_optimizer_reduces_the_loss_with_finite_updates(name, lr):
    net, loss_fn = _quadratic()
    opt = build_optimizer(net, OptimizerConfig(name=name, lr=lr, weight_decay=0.01))
    assert name in registry.list("optimizer")
    first = float(loss_fn())
    for _ in range(60):
        opt.zero_grad()
        loss = loss_fn()
        loss.backward()
        opt.step()
    assert float(loss_fn()) < first
    assert all(torch.isfinite(p).all() for p in net.parameters())


def test_param_groups_split_by_the_decay_rule():
    net = nn.Sequential(nn.Linear(4, 4), nn.LayerNorm(4))
    groups = build_param_groups(net, weight_decay=0.1)
    assert [g["weight_decay"] for g in groups] == [0.1, 0.0]
    assert len(groups[0]["params"]) == 1 and len(groups[1]["params"]) == 3       # only the 2-D weight decays
    assert should_decay("embed.weight", torch.zeros(10, 4)) and not should_decay("fc.bias", torch.zeros(4))
    assert not should_decay("norm.weight", torch.zeros(4)) and not should_decay("attn.bias_table", torch.zeros(4, 4))
    frozen = nn.Linear(4, 4)
    frozen.weight.requires_grad_(False)
    assert sum(len(g["params"]) for g in build_param_groups(frozen, 0.1)) == 1


def test_lion_keeps_one_buffer_and_moves_by_the_sign():
    p = nn.Parameter(torch.tensor([1.0, -2.0, 3.0]))
    opt = Lion([p], lr=0.1, betas=(0.9, 0.99), weight_decay=0.0)
    p.grad = torch.tensor([0.5, -0.25, 0.0])
    opt.step()
    assert torch.allclose(p.data, torch.tensor([0.9, -1.9, 3.0]))
    (state,) = opt.state.values()
    assert [k for k, v in state.items() if torch.is_tensor(v) and v.shape == p.shape] == ["exp_avg"]
    assert torch.allclose(state["exp_avg"], 0.01 * p.grad)
    decayed = nn.Parameter(torch.tensor([1.0]))
    opt2 = Lion([decayed], lr=0.1, weight_decay=0.5)
    decayed.grad = torch.tensor([0.0])
    opt2.step()
    assert torch.allclose(decayed.data, torch.tensor([0.95]))                      # decoupled decay only


@pytest.mark.parametrize("cls,kw", [(Lion, dict(lr=1e-3)), (ScheduleFreeAdamW, dict(lr=1e-2, warmup_steps=3)),
                                    (FusedAdamW, dict(lr=1e-2))])
def test_optimizer_state_round_trip_continues_identically(cls, kw):
    def run(resume_at=None):
        torch.manual_seed(2)
        net = nn.Linear(6, 3)
        opt = cls(net.parameters(), **kw)
        x = torch.randn(10, 6)
        for step in range(6):
            if step == resume_at:
                state, weights = copy.deepcopy(opt.state_dict()), copy.deepcopy(net.state_dict())
                net = nn.Linear(6, 3)
                net.load_state_dict(weights)
                opt = cls(net.parameters(), **kw)
                opt.load_state_dict(state)
            opt.zero_grad()
            net(x).square().mean().backward()
            opt.step()
        return [p.detach().clone() for p in net.parameters()]

    for a, b in zip(run(), run(resume_at=3)):
        assert torch.allclose(a, b, atol=1e-7)


def test_schedule_free_warmup_and_parameter_views():
    p = nn.Parameter(torch.ones(4))
    opt = ScheduleFreeAdamW([p], lr=0.1, warmup_steps=4)
    moves = []
    for _ in range(5):
        before = p.detach().clone()
        p.grad = torch.ones(4)
        opt.step()
        moves.append(float((p.detach() - before).abs().max()))
    assert moves[0] < moves[3]                                       # the step size ramps up during warm-up
    train_view = p.detach().clone()
    opt.eval_params()
    eval_view = p.detach().clone()
    opt.eval_params()                                                # idempotent
    assert torch.equal(p.detach(), eval_view) and not torch.equal(train_view, eval_view)
    opt.train_params()
    assert torch.allclose(p.detach(), train_view, atol=1e-6)
    assert OptimizerConfig().schedule_free_warmup_steps == 0
    with pytest.raises(ValueError):
        OptimizerConfig(schedule_free_warmup_steps=-1)


def test_newton_schulz_and_muon_partition():
    torch.manual_seed(3)
    g = torch.randn(16, 32)
    o = newton_schulz(g, steps=5).float()
    sv = torch.linalg.svdvals(o)
    assert sv.max() < 1.3 and sv.min() > 0.3                          # roughly orthonormal rows
    assert is_muon_eligible(torch.zeros(64, 64)) and is_muon_eligible(torch.zeros(8, 4, 16))
    assert not is_muon_eligible(torch.zeros(64)) and not is_muon_eligible(torch.zeros(1000, 8))
    net = nn.Sequential(nn.Linear(16, 16), nn.LayerNorm(16))
    opt = build_optimizer(net, OptimizerConfig(name="muon", lr=0.02, muon_adam_lr=1e-3))
    assert isinstance(opt, Muon)
    muon_params = [p for g_ in opt.param_groups for p in g_["params"]]
    assert any(p is net[0].weight for p in muon_params)
    adam_params = [p for g_ in opt.inner_adam.param_groups for p in g_["params"]]
    assert any(p is net[1].weight for p in adam_params) and all(g_["lr"] == 1e-3 for g_ in opt.inner_adam.param_groups)
    state = opt.state_dict()
    opt.load_state_dict(state)


def test_optimizer_config_rules():
    for bad in (dict(lr=0.0), dict(weight_decay=-1.0), dict(betas=(0.9, 1.0)), dict(muon_momentum=1.0), dict(muon_ns_steps=0)):
        with pytest.raises(ValueError):
            OptimizerConfig(**bad)
    with pytest.raises((KeyError, ValueError)):
        build_optimizer(nn.Linear(2, 2), OptimizerConfig(name="sgd_with_hats"))
    opt = build_optimizer(nn.Linear(2, 2), OptimizerConfig(name="adamw", betas=(0.8, 0.9), eps=1e-6))
    assert opt.param_groups[0]["betas"] == (0.8, 0.9) and opt.param_groups[0]["eps"] == 1e-6


def test_activation_store_enable_disable_and_dataset_extraction(tmp_path):
    m = _model()
    store = ActivationStore(m, layers=["norm"])
    assert not store.enabled and store.layer_names == ["norm"]      # hooks are installed by enable(), not at construction
    tokens = torch.randint(0, 40, (2, 5))
    m(tokens)
    assert store.get("norm") is None          # nothing captured while disabled
    store.enable()
    store.enable()                            # idempotent
    assert store.enabled and sum(len(mod._forward_hooks) for mod in m.modules()) == 1
    m(tokens)
    assert store.get("norm").shape[0] == 2
    store.disable()
    assert not store.enabled
    with pytest.raises(ValueError, match="not found"):
        ActivationStore(m, layers=["nope"]).enable()

    class Samples(torch.utils.data.Dataset):
        def __len__(self):
            return 7

        def __getitem__(self, i):
            return {"input_ids": torch.full((5,), i % 40, dtype=torch.long)}

    reps = extract_representations(m, Samples(), ["norm"], torch.device("cpu"), batch_size=3, max_samples=5)
    assert reps["norm"].shape[0] == 5
    everything = extract_representations(m, Samples(), ["norm"], batch_size=4)
    assert everything["norm"].shape[0] == 7 and torch.equal(everything["norm"][:5], reps["norm"])
