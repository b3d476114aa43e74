"""Optimizers, schedulers, losses, hooks, freezing, flat parameter groups and the trainer step (CPU)."""

import math

import pytest
import torch

from kempnerforge_b200.config import ModelConfig, OptimizerConfig, SchedulerConfig, config_from_dict
from kempnerforge_b200.models import Transformer
from kempnerforge_b200.ops import ref
from kempnerforge_b200.parallel.flat import flatten_model
from kempnerforge_b200.training import (
    HookRunner,
    Lion,
    ScheduleFreeAdamW,
    StepContext,
    TrainingHook,
    build_loss_fn,
    build_optimizer,
    chunked_cross_entropy,
    cross_entropy,
    is_muon_eligible,
    lr_factor_fn,
    maybe_no_sync,
    newton_schulz,
    z_loss,
)
from kempnerforge_b200.training.freeze import apply_freeze_specs, canonical_freeze_meta, effective_freeze, freeze_params

TINY = dict(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=256, max_seq_len=64)


# ------------------------------------------------------------------ schedulers
def test_warmup_and_first_step_lr_is_zero():
    f = lr_factor_fn(SchedulerConfig(name="cosine", warmup_steps=4), 20)
    assert [f(i) for i in range(5)] == [0.0, 0.25, 0.5, 0.75, 1.0]


@pytest.mark.parametrize("name", ["cosine", "linear", "wsd", "constant", "rex", "none"])
def test_schedule_endpoints(name):
    cfg = SchedulerConfig(name=name, warmup_steps=2, min_lr_ratio=0.1, stable_steps=3)
    f = lr_factor_fn(cfg, 12)
    end = f(12)
    if name in ("constant", "none"):
        assert end == 1.0
    else:
        assert abs(end - 0.1) < 1e-9
    assert all(0.0 <= f(s) <= 1.0 + 1e-12 for s in range(0, 30))
    if name == "none":
        assert f(0) == 1.0


def test_cosine_midpoint_and_rex_alpha():
    f = lr_factor_fn(SchedulerConfig(name="cosine", warmup_steps=0, min_lr_ratio=0.0), 10)
    assert abs(f(5) - 0.5) < 1e-9
    r = lr_factor_fn(SchedulerConfig(name="rex", warmup_steps=0, min_lr_ratio=0.0, rex_alpha=2.0), 10)
    assert abs(r(5) - 0.25) < 1e-9
    w = lr_factor_fn(SchedulerConfig(name="wsd", warmup_steps=0, stable_steps=4, min_lr_ratio=0.0, wsd_decay_type="linear"), 8)
    assert w(3) == 1.0 and abs(w(6) - 0.5) < 1e-9


# ------------------------------------------------------------------ losses
def test_cross_entropy_variants_agree():
    torch.manual_seed(0)
    logits, labels = torch.randn(3, 7, 11), torch.randint(0, 11, (3, 7))
    labels[0, :3] = -100
    want = torch.nn.functional.cross_entropy(logits.reshape(-1, 11), labels.reshape(-1), ignore_index=-100)
    assert torch.allclose(cross_entropy(logits, labels), want, atol=1e-6)
    assert torch.allclose(chunked_cross_entropy(logits, labels, chunk_size=4), want, atol=1e-6)
    all_ignored = torch.full((3, 7), -100)
    assert cross_entropy(logits, all_ignored).item() == 0.0
    assert torch.allclose(z_loss(logits, 0.5), 0.5 * torch.logsumexp(logits, -1).pow(2).mean())
    cfg = config_from_dict({"train": {"loss_fn": "chunked_cross_entropy", "z_loss_weight": 0.1, "ce_chunk_size": 5}})
    assert torch.allclose(build_loss_fn(cfg.train)(logits, labels), want + z_loss(logits, 0.1), atol=1e-6)


# ------------------------------------------------------------------ optimizers
def _quadratic_descends(opt_name, **kw):
    torch.manual_seed(0)
    lin = torch.nn.Linear(8, 8, bias=True)
    opt = build_optimizer(lin, OptimizerConfig(name=opt_name, **kw))
    x, y = torch.randn(64, 8), torch.randn(64, 8)
    losses = []
    for _ in range(60):
        loss = (lin(x) - y).pow(2).mean()
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses


@pytest.mark.parametrize("name,kw", [("adamw", dict(lr=1e-2)), ("lion", dict(lr=1e-3)),
                                     ("schedule_free_adamw", dict(lr=1e-2)), ("muon", dict(lr=1e-2))])
def test_optimizers_reduce_loss(name, kw):
    losses = _quadratic_descends(name, **kw)
    assert losses[-1] < losses[0] * 0.9


def test_param_groups_decay_rule():
    m = Transformer(ModelConfig(**TINY))
    opt = build_optimizer(m, OptimizerConfig(weight_decay=0.1))
    decay, no_decay = opt.param_groups
    assert decay["weight_decay"] == 0.1 and no_decay["weight_decay"] == 0.0
    assert all(p.dim() > 1 for p in decay["params"]) and all(p.dim() <= 1 for p in no_decay["params"])
    emb = m.token_embedding.embedding.weight
    assert any(p is emb for p in decay["params"])  # embeddings are decayed, like the reference


def test_lion_update_rule():
    p = torch.nn.Parameter(torch.tensor([1.0, -2.0]))
    opt = Lion([p], lr=0.1, betas=(0.9, 0.99), weight_decay=0.5)
    p.grad = torch.tensor([0.3, -0.1])
    opt.step()
    want = torch.tensor([1.0, -2.0]) * (1 - 0.1 * 0.5) - 0.1 * torch.sign(torch.tensor([0.03, -0.01]))
    assert torch.allclose(p.detach(), want, atol=1e-6)
    assert torch.allclose(opt.state[p]["exp_avg"], torch.tensor([0.003, -0.001]), atol=1e-7)


def test_schedule_free_eval_train_roundtrip_and_state():
    p = torch.nn.Parameter(torch.randn(4))
    opt = ScheduleFreeAdamW([p], lr=0.1, warmup_steps=2)
    for _ in range(3):
        p.grad = torch.randn(4)
        opt.step()
    y = p.detach().clone()
    opt.eval_params()
    assert torch.allclose(p.detach(), opt.state[p]["x"])
    opt.train_params()
    assert torch.allclose(p.detach(), y, atol=1e-6)
    sd = opt.state_dict()
    assert sd["_k"] == 3 and sd["_warmup_steps"] == 2
    opt2 = ScheduleFreeAdamW([p], lr=0.1)
    opt2.load_state_dict(sd)
    assert opt2._k == 3 and opt2.warmup_steps == 2


def test_newton_schulz_orthogonalises_and_muon_eligibility():
    torch.manual_seed(0)
    g = torch.randn(32, 48)
    x = newton_schulz(g, 5)
    sv = torch.linalg.svdvals(x)
    assert sv.max() < 1.3 and sv.min() > 0.5  # the quintic pushes singular values into a band around one
    a, b, c = ref.NS_COEFFS
    y = g / (g.norm() + 1e-7)
    for _ in range(5):
        A = y @ y.T
        y = a * y + (b * A + c * A @ A) @ y
    assert torch.allclose(x, y, atol=1e-5)
    assert is_muon_eligible(torch.empty(64, 64)) and not is_muon_eligible(torch.empty(64))
    assert not is_muon_eligible(torch.empty(4, 2048)) and is_muon_eligible(torch.empty(8, 4, 16))


def test_muon_splits_params_and_ties_adam_lr():
    m = Transformer(ModelConfig(**TINY))
    opt = build_optimizer(m, OptimizerConfig(name="muon", lr=0.02, muon_adam_lr=0.001))
    assert opt.inner_adam is not None
    muon_ids = {id(p) for g in opt.param_groups for p in g["params"]}
    assert id(m.layers["0"].attention.q_proj.weight) in muon_ids
    assert id(m.norm.weight) not in muon_ids
    for g in opt.param_groups:
        g["lr"] = 0.01
    tok = torch.randint(0, 256, (2, 9))
    m.compute_loss(tok[:, :-1], tok[:, 1:]).backward()
    opt.step()
    assert abs(opt.inner_adam.param_groups[0]["lr"] - 0.0005) < 1e-12
    sd = opt.state_dict()
    assert "_adam_state" in sd and sd["_initial_lr"] == 0.02


# ------------------------------------------------------------------ flat groups
def test_flat_groups_match_unflattened_adamw_with_accumulation():
    torch.manual_seed(0)
    cfg = ModelConfig(**TINY)
    a, b = Transformer(cfg), Transformer(cfg)
    b.load_state_dict(a.state_dict())
    groups = flatten_model(a)
    assert [g.name for g in groups] == ["layers.0", "layers.1", "root"]
    q, k = a.layers["0"].attention.q_proj.weight, a.layers["0"].attention.k_proj.weight
    assert k.data_ptr() == q.data_ptr() + q.numel() * 4  # q|k|v are adjacent: one GEMM operand
    oa = build_optimizer(a, OptimizerConfig(lr=1e-2))
    ob = build_optimizer(b, OptimizerConfig(lr=1e-2, fused=False))
    tok = torch.randint(0, 256, (4, 17))
    for _ in range(3):
        for model, opt in ((a, oa), (b, ob)):
            for micro in range(2):
                sl = tok[2 * micro : 2 * micro + 2]
                (model.compute_loss(sl[:, :-1], sl[:, 1:]) / 2).backward()
            for g in getattr(model, "_kf_flat_groups", []):
                g.finalize_grads()
            opt.step()
            for g in getattr(model, "_kf_flat_groups", []):
                g.zero_grad()
            opt.zero_grad()
    for (n, pa), (_, pb) in zip(a.named_parameters(), b.named_parameters()):
        assert torch.allclose(pa, pb, atol=1e-6), n
    st = oa.state[q]
    assert set(st) == {"step", "exp_avg", "exp_avg_sq"} and float(st["step"]) == 3.0


# ------------------------------------------------------------------ hooks / grad / freeze
def test_hook_runner_order_and_context():
    calls = []

    class H(TrainingHook):
        def __init__(self, tag):
            self.tag = tag

        def on_step_end(self, ctx):
            calls.append((self.tag, ctx.step, ctx.loss))

        def on_train_end(self, step, tokens_seen):
            calls.append((self.tag, "end", tokens_seen))

    r = HookRunner([H("a"), H("b")])
    r.on_train_begin(None)
    r.on_step_end(StepContext(step=3, loss=1.5, grad_norm=0.1, lr=1e-3, tokens_seen=10))
    r.on_train_end(3, 10)
    assert calls == [("a", 3, 1.5), ("b", 3, 1.5), ("a", "end", 10), ("b", "end", 10)]


def test_maybe_no_sync_toggles_engine_flag():
    class M:
        def __init__(self):
            self.flags = []

        def set_requires_gradient_sync(self, f):
            self.flags.append(f)

    m = M()
    with maybe_no_sync(m, 0, 3):
        pass
    with maybe_no_sync(m, 2, 3):
        pass
    assert m.flags == [False, True, True, True]
    with maybe_no_sync(object(), 0, 2):
        pass


def test_freeze_helpers():
    from kempnerforge_b200.config import FreezeSpec, FreezeStage, JointDecoderConfig

    m = torch.nn.ModuleDict({"transformer": torch.nn.Linear(2, 2), "adapter": torch.nn.Linear(2, 2)})
    assert freeze_params(m, ["adapter", "adapter.*"]) == 6          # elements flipped: a 2 x 2 weight and a bias of 2
    assert not m["adapter"].weight.requires_grad and m["transformer"].weight.requires_grad
    pats = {"transformer": ["transformer", "transformer.*"], "adapter": ["adapter", "adapter.*"]}
    apply_freeze_specs(m, [FreezeSpec("adapter", False), FreezeSpec("transformer", True)], pats)
    assert m["adapter"].weight.requires_grad and not m["transformer"].weight.requires_grad
    assert apply_freeze_specs(m, [FreezeSpec("nope")], pats) == {"nope": 0}   # not an alias: a raw pattern that matches nothing
    meta = canonical_freeze_meta([FreezeSpec("b", True), FreezeSpec("a", False), FreezeSpec("b", False), FreezeSpec("b", True)])
    assert meta == [{"module": "a", "frozen": False}, {"module": "b", "frozen": False}, {"module": "b", "frozen": True}]
    vc = JointDecoderConfig(freeze=[FreezeSpec("vision_encoder", True)],
                            freeze_schedule=[FreezeStage(10, (FreezeSpec("vision_encoder", False),))])
    assert effective_freeze(vc, 5)[0].frozen and not effective_freeze(vc, 10)[0].frozen


# ------------------------------------------------------------------ trainer
def _tiny_job(**train):
    return config_from_dict({
        "model": TINY,
        "train": {"batch_size": 2, "seq_len": 32, "max_steps": 6, "mixed_precision": "fp32", "seed": 0, **train},
        "scheduler": {"warmup_steps": 2},
        "metrics": {"log_interval": 100},
    })


def test_trainer_step_and_nan_skip():
    from kempnerforge_b200.training.trainer import Trainer

    t = Trainer(_tiny_job(grad_accum_steps=2, activation_checkpointing="full"), init_dist=False)
    out = t.train_step()
    assert out["lr"] == 0.0 and math.isfinite(out["loss"]) and out["grad_norm"] > 0
    before = [p.detach().clone() for p in t.model.parameters()]
    with torch.no_grad():
        t.model.norm.weight.fill_(float("nan"))
    bad = t.train_step()
    assert bad["skipped"] == 1.0 and t.nan_detector.state.consecutive_nans == 1
    with torch.no_grad():
        t.model.norm.weight.fill_(1.0)
    after = [p.detach().clone() for p in t.model.parameters()]
    for (n, _), x, y in zip(t.model.named_parameters(), before, after):
        if n != "norm.weight":
            assert torch.equal(x, y), n  # a skipped step leaves the weights alone


def test_trainer_learns_repeating_pattern():
    from kempnerforge_b200.training.trainer import Trainer

    cfg = _tiny_job(max_steps=40)
    cfg.optimizer.lr = 3e-3
    t = Trainer(cfg, init_dist=False)
    pattern = torch.arange(33).repeat(2, 1) % 7
    batch = {"input_ids": pattern[:, :-1], "labels": pattern[:, 1:]}
    losses = [t.train_step([batch])["loss"] for _ in range(40)]
    assert losses[-1] < 0.5 * losses[0]


def test_fit_stops_when_the_native_kernel_status_word_is_set(monkeypatch):
    """A non-zero status word (a device-side wait that ran out) ends the run at the next logging step with its own
    stop reason instead of training on with a missing result."""
    from kempnerforge_b200.training.trainer import Trainer

    t = Trainer(_tiny_job(max_steps=6), init_dist=False)
    assert t._native_status() == 0                       # CPU: nothing to read
    words = iter([0, 6])
    monkeypatch.setattr(Trainer, "_native_status", lambda self: next(words))
    t.config.metrics.log_interval = 2
    out = t.fit()
    assert out["stop_reason"] == "kernel_status" and out["step"] == 2   # checked at step 1 (clean) and step 2 (set)
