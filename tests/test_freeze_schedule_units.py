"""Parameter freezing (patterns, aliases, canonical metadata, staged schedules) and the constant / WSD / REX
learning-rate schedules, one behaviour per test (CPU).

Behaviours of kempnerforge/training/freeze.py and kempnerforge/training/scheduler.py (schedule extensions)."""

import math

import pytest
import torch
from torch import nn

from kempnerforge_b200.config import SchedulerConfig, load_config
from kempnerforge_b200.config.vlm import FreezeSpec, FreezeStage
from kempnerforge_b200.training import lr_factor_fn
from kempnerforge_b200.training.freeze import apply_freeze_specs, canonical_freeze_meta, effective_freeze, freeze_params


# --------------------------------------------------------------------------- freezing
class _Toy(nn.Module):
    def __init__(self):
        super().__init__()
        self.vision_encoder = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4))
        self.adapter = nn.Linear(4, 4)
        self.transformer = nn.ModuleDict({"layers": nn.ModuleList([nn.Linear(4, 4), nn.Linear(4, 4)])})


PATTERNS = {"vision_encoder": ["vision_encoder.*"], "adapter": ["adapter.*"], "transformer": ["transformer.*"]}


def _trainable(model):
    return {n for n, p in model.named_parameters() if p.requires_grad}


def test_matching_parameters_are_frozen_and_counted():
    m = _Toy()
    assert freeze_params(m, ["vision_encoder.*"]) == 2 * (16 + 4)        # the number of ELEMENTS whose flag changed
    assert not any(n.startswith("vision_encoder") for n in _trainable(m)) and "adapter.weight" in _trainable(m)


def test_no_patterns_change_nothing_and_freezing_twice_is_the_same_as_once():
    m = _Toy()
    before = _trainable(m)
    assert freeze_params(m, []) == 0 and _trainable(m) == before
    assert freeze_params(m, ["adapter.*"]) == 20
    once = _trainable(m)
    assert freeze_params(m, ["adapter.*"]) == 0 and _trainable(m) == once      # nothing left to flip


def test_thawing_is_freezing_with_the_flag_off():
    m = _Toy()
    freeze_params(m, ["*"])
    assert _trainable(m) == set()
    freeze_params(m, ["adapter.*"], frozen=False)
    assert _trainable(m) == {"adapter.weight", "adapter.bias"}


def test_patterns_match_fully_qualified_parameter_names_and_add_up():
    m = _Toy()
    assert freeze_params(m, ["transformer.layers.1.weight"]) == 16
    assert freeze_params(m, ["vision_encoder.0"]) == 0            # a module name alone is not a parameter name
    assert freeze_params(m, ["vision_encoder.0.*"]) == 20
    m2 = _Toy()
    assert freeze_params(m2, ["adapter.*", "transformer.layers.0.*"]) == 40


def test_specs_resolve_aliases_and_later_specs_override_earlier_ones():
    m = _Toy()
    counts = apply_freeze_specs(m, [FreezeSpec("vision_encoder"), FreezeSpec("adapter"), FreezeSpec("adapter", frozen=False)],
                                PATTERNS)
    assert counts == {"vision_encoder": 40, "adapter": 20}       # per alias: elements flipped by its LAST spec
    assert "adapter.weight" in _trainable(m) and "vision_encoder.0.weight" not in _trainable(m)


def test_a_name_that_is_no_alias_is_used_as_a_raw_pattern():
    m = _Toy()
    assert apply_freeze_specs(m, [FreezeSpec("transformer.layers.0.*")], PATTERNS) == {"transformer.layers.0.*": 20}
    assert "transformer.layers.0.weight" not in _trainable(m) and "transformer.layers.1.weight" in _trainable(m)
    assert apply_freeze_specs(_Toy(), [FreezeSpec("vison_encoder")], PATTERNS) == {"vison_encoder": 0}   # a typo matches nothing


def test_canonical_metadata_ignores_order_and_duplicates():
    a = canonical_freeze_meta([FreezeSpec("adapter", False), FreezeSpec("vision_encoder")])
    b = canonical_freeze_meta([FreezeSpec("vision_encoder"), FreezeSpec("adapter", False), FreezeSpec("vision_encoder")])
    assert a == b == [{"module": "adapter", "frozen": False}, {"module": "vision_encoder", "frozen": True}]
    # the same module with both flags keeps both pairs (the set of pairs is what gets compared at resume)
    assert len(canonical_freeze_meta([FreezeSpec("adapter"), FreezeSpec("adapter", False)])) == 2
    assert canonical_freeze_meta([]) == []


def test_a_schedule_applies_only_the_stages_that_have_started():
    base = [FreezeSpec("vision_encoder"), FreezeSpec("adapter", False)]
    stages = [FreezeStage(100, (FreezeSpec("vision_encoder", False),)), FreezeStage(50, (FreezeSpec("adapter"),))]
    view = lambda step: {s.module: s.frozen for s in effective_freeze(step, base, stages)}  # noqa: E731
    assert view(0) == {"vision_encoder": True, "adapter": False}
    assert view(50) == {"vision_encoder": True, "adapter": True}
    assert view(100) == {"vision_encoder": False, "adapter": True}
    assert effective_freeze(10, base, []) == base          # one spec per module, in order of first appearance


def test_later_stages_win_whatever_order_they_are_listed_in():
    stages = [FreezeStage(20, (FreezeSpec("adapter", False),)), FreezeStage(10, (FreezeSpec("adapter"),))]
    assert [s.frozen for s in effective_freeze(30, [], stages)] == [False]
    assert [s.frozen for s in effective_freeze(30, [], list(reversed(stages)))] == [False]
    assert [s.frozen for s in effective_freeze(15, [], stages)] == [True]


def test_module_keys_are_checked_against_the_valid_set_when_one_is_given():
    valid = {"vision_encoder", "adapter"}
    with pytest.raises(ValueError, match="base"):
        effective_freeze(0, [FreezeSpec("adaptr")], [], valid_modules=valid)
    with pytest.raises(ValueError, match="step 5"):
        effective_freeze(9, [], [FreezeStage(5, (FreezeSpec("encoder"),))], valid_modules=valid)
    assert effective_freeze(9, [FreezeSpec("anything")], [])[0].module == "anything"     # no set, no check


# --------------------------------------------------------------------------- schedules
def _f(name, max_steps=100, **kw):
    return lr_factor_fn(SchedulerConfig(name=name, **kw), max_steps)


def test_constant_ramps_then_stays_at_one():
    f = _f("constant", warmup_steps=10)
    assert f(0) == 0.0 and f(5) == 0.5 and f(10) == 1.0 and f(55) == 1.0 and f(99) == 1.0
    assert _f("constant", warmup_steps=0)(0) == 1.0


@pytest.mark.parametrize("shape", ["cosine", "linear", "sqrt"])
def test_wsd_holds_then_cools_down_to_the_floor(shape):
    f = _f("wsd", warmup_steps=10, stable_steps=40, wsd_decay_type=shape, min_lr_ratio=0.1)
    assert f(10) == 1.0 and f(49) == 1.0 and f(50) == pytest.approx(1.0)
    assert f(100) == pytest.approx(0.1) and f(500) == pytest.approx(0.1)
    mid = f(75)
    assert 0.1 < mid < 1.0
    assert all(f(s + 1) <= f(s) + 1e-12 for s in range(50, 100))


def test_wsd_shapes_differ_in_the_middle_and_sqrt_stays_above_linear():
    mk = lambda shape: _f("wsd", warmup_steps=0, stable_steps=20, wsd_decay_type=shape, min_lr_ratio=0.0)  # noqa: E731
    lin, sq, cos = mk("linear"), mk("sqrt"), mk("cosine")
    assert lin(60) == pytest.approx(0.5) and sq(60) == pytest.approx(math.sqrt(0.5)) and cos(60) == pytest.approx(0.5)
    assert sq(80) > lin(80) and cos(40) > lin(40) and cos(90) < lin(90)
    with pytest.raises(ValueError):
        SchedulerConfig(name="wsd", wsd_decay_type="exp")


def test_rex_is_linear_for_alpha_one_convex_above_and_concave_below():
    lin = _f("rex", warmup_steps=0, rex_alpha=1.0, min_lr_ratio=0.0)
    assert [lin(s) for s in (0, 25, 50, 100)] == pytest.approx([1.0, 0.75, 0.5, 0.0])
    fast = _f("rex", warmup_steps=0, rex_alpha=2.0, min_lr_ratio=0.0)
    slow = _f("rex", warmup_steps=0, rex_alpha=0.5, min_lr_ratio=0.0)
    assert fast(50) == pytest.approx(0.25) and slow(50) == pytest.approx(math.sqrt(0.5))
    assert fast(50) < lin(50) < slow(50)


def test_rex_respects_warmup_the_floor_and_rejects_a_non_positive_exponent():
    f = _f("rex", warmup_steps=10, rex_alpha=1.0, min_lr_ratio=0.2)
    assert f(0) == 0.0 and f(10) == 1.0 and f(100) == pytest.approx(0.2) and f(95) == pytest.approx(0.2)
    with pytest.raises(ValueError):
        SchedulerConfig(name="rex", rex_alpha=0.0)


def test_schedule_options_come_through_toml_and_the_command_line(tmp_path):
    p = tmp_path / "s.toml"
    p.write_text('[scheduler]\nname = "wsd"\nwsd_decay_type = "sqrt"\nstable_steps = 30\n')
    cfg = load_config(str(p))
    assert str(cfg.scheduler.name) == "wsd" and cfg.scheduler.wsd_decay_type == "sqrt" and cfg.scheduler.stable_steps == 30
    cfg = load_config(str(p), ["--scheduler.name=rex", "--scheduler.rex_alpha=2.5"])
    assert str(cfg.scheduler.name) == "rex" and cfg.scheduler.rex_alpha == 2.5
    d = SchedulerConfig()
    assert d.wsd_decay_type == "cosine" and d.rex_alpha == 1.0 and str(d.name) == "cosine"


def test_the_scheduler_drives_a_real_optimizer():
    from kempnerforge_b200.training import build_scheduler

    opt = torch.optim.SGD([nn.Parameter(torch.zeros(1))], lr=2.0)
    sched = build_scheduler(opt, SchedulerConfig(name="rex", warmup_steps=2, rex_alpha=1.0, min_lr_ratio=0.0), max_steps=6)
    seen = []
    for _ in range(6):
        seen.append(opt.param_groups[0]["lr"])
        opt.step()
        sched.step()
    assert seen == pytest.approx([0.0, 1.0, 2.0, 1.5, 1.0, 0.5])
