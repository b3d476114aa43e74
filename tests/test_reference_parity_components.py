"""Component-level parity with the unmodified reference (``baseline/_ref``) on CPU: routers, Newton-Schulz
orthogonalisation, evaluation, activation extraction, freeze helpers and the NaN detector, each fed the same inputs on
both sides.  Skipped when the reference is not installed."""

from __future__ import annotations

import math
import sys
from pathlib import Path

import pytest
import torch
from torch import nn

ROOT = Path(__file__).resolve().parents[1]
REF = ROOT / "baseline" / "_ref"
pytestmark = pytest.mark.skipif(not (REF / "kempnerforge").is_dir(), reason="reference package not installed")


def _ref_path():
    if str(REF) not in sys.path:
        sys.path.insert(0, str(REF))


# --------------------------------------------------------------------------- routers
def test_softmax_router_weights_indices_and_auxiliary_loss_match():
    _ref_path()
    from kempnerforge.model.router import SoftmaxTopKRouter as Ref

    from kempnerforge_b200.models.router import SoftmaxTopKRouter as Mine

    torch.manual_seed(0)
    a, b = Ref(32, 8, 2), Mine(32, 8, 2)
    b.load_state_dict(a.state_dict())
    x = torch.randn(40, 32)
    (wa, ia), (wb, ib) = a(x), b(x)
    assert torch.equal(ia, ib) and torch.allclose(wa, wb, atol=1e-6)
    assert torch.allclose(a.aux_loss, b.aux_loss, atol=1e-6)
    assert torch.equal(a.expert_counts.float(), b.expert_counts.float())


@pytest.mark.parametrize("schedule", ["constant", "cosine_decay", "linear_warmup"])
def test_sigmoid_router_follows_the_reference_through_bias_updates(schedule):
    """Three training steps: the balancing bias and the utilisation average move between steps, so parity of step 3
    checks the update rule and its schedule, not just the forward pass."""
    _ref_path()
    from kempnerforge.model.router import SigmoidTopKRouter as Ref

    from kempnerforge_b200.models.router import SigmoidTopKRouter as Mine

    torch.manual_seed(1)
    kw = dict(bias_update_rate=0.05, ema_decay=0.9, sequence_aux_loss_weight=0.01, bias_schedule=schedule)
    a, b = Ref(16, 6, 2, **kw), Mine(16, 6, 2, **kw)
    b.load_state_dict(a.state_dict())
    a.train(), b.train()
    for step in range(3):
        a.set_step(step, 10), b.set_step(step, 10)
        x = torch.randn(24, 16) + 0.3 * step
        (wa, ia), (wb, ib) = a(x), b(x)
        assert torch.equal(ia, ib), step
        assert torch.allclose(wa, wb, atol=1e-6), step
        assert torch.allclose(a.aux_loss, b.aux_loss, atol=1e-6), step
        assert torch.allclose(a.expert_bias, b.expert_bias, atol=1e-7), step
        assert torch.allclose(a.expert_ema, b.expert_ema, atol=1e-7), step


# --------------------------------------------------------------------------- Newton-Schulz
@pytest.mark.parametrize("shape", [(48, 48), (32, 96), (96, 32)])
def test_newton_schulz_matches_for_square_wide_and_tall_matrices(shape):
    _ref_path()
    from kempnerforge.training.optimizer import _newton_schulz as ref_ns

    from kempnerforge_b200.training.optimizer import newton_schulz

    g = torch.randn(*shape, generator=torch.Generator().manual_seed(2))
    want, got = ref_ns(g.clone(), steps=5), newton_schulz(g.clone(), steps=5)
    assert got.shape == want.shape
    assert torch.allclose(got.float(), want.float(), atol=2e-2), float((got.float() - want.float()).abs().max())


# --------------------------------------------------------------------------- evaluation
def test_evaluation_returns_the_reference_loss_and_perplexity():
    _ref_path()
    from kempnerforge.training.eval import run_eval as ref_eval
    from kempnerforge.training.loss import cross_entropy_loss as ref_ce

    from kempnerforge_b200.config import ModelConfig
    from kempnerforge_b200.models import Transformer
    from kempnerforge_b200.training.eval import run_eval
    from kempnerforge_b200.training.loss import cross_entropy_loss

    torch.manual_seed(3)
    model = Transformer(ModelConfig(dim=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=50, max_seq_len=32))
    g = torch.Generator().manual_seed(4)
    batches = []
    for _ in range(3):        # fewer batches than eval steps: both sides restart the loader
        tok = torch.randint(0, 50, (2, 17), generator=g)
        labels = tok[:, 1:].clone()
        labels[0, :3] = -100
        batches.append({"input_ids": tok[:, :-1].contiguous(), "labels": labels})
    want = ref_eval(model, batches, ref_ce, torch.device("cpu"), 5)
    got = run_eval(model, batches, cross_entropy_loss, torch.device("cpu"), 5)
    assert set(want) <= set(got)
    assert got["eval/loss"] == pytest.approx(want["eval/loss"], rel=1e-6)
    assert got["eval/perplexity"] == pytest.approx(want["eval/perplexity"], rel=1e-6)
    assert got["eval/perplexity"] == pytest.approx(math.exp(got["eval/loss"]), rel=1e-6)


# --------------------------------------------------------------------------- activation capture
def test_activation_store_and_extraction_return_the_reference_tensors():
    _ref_path()
    from kempnerforge.model.hooks import ActivationStore as RefStore
    from kempnerforge.model.hooks import extract_representations as ref_extract

    from kempnerforge_b200.config import ModelConfig
    from kempnerforge_b200.models import Transformer
    from kempnerforge_b200.models.hooks import ActivationStore, extract_representations

    torch.manual_seed(5)
    model = Transformer(ModelConfig(dim=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=50, max_seq_len=16)).eval()
    layers = ["layers.0.attention", "layers.1.mlp", "norm"]
    ids = torch.randint(0, 50, (3, 8), generator=torch.Generator().manual_seed(6))
    ra, mine = RefStore(model, layers=layers), ActivationStore(model, layers=layers)
    for store in (ra, mine):
        store.enable()
        with torch.no_grad():
            model(ids)
        store.disable()
    assert sorted(ra.layer_names) == sorted(mine.layer_names)
    for name in layers:
        assert torch.equal(ra.get(name), mine.get(name)), name
    assert mine.get("no.such.layer") is None and ra.get("no.such.layer") is None

    class Data(torch.utils.data.Dataset):
        def __len__(self):
            return 7

        def __getitem__(self, i):
            return {"input_ids": torch.randint(0, 50, (8,), generator=torch.Generator().manual_seed(100 + i))}

    want = ref_extract(model, Data(), layers, torch.device("cpu"), batch_size=3, max_samples=5)
    got = extract_representations(model, Data(), layers, torch.device("cpu"), batch_size=3, max_samples=5)
    assert want.keys() == got.keys()
    for name in layers:
        assert got[name].shape == want[name].shape == (5, 8, 32) and torch.equal(got[name], want[name]), name


# --------------------------------------------------------------------------- freezing
class _Toy(nn.Module):
    def __init__(self):
        super().__init__()
        self.vision_encoder = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 4))
        self.adapter = nn.Linear(4, 6)
        self.transformer = nn.ModuleDict({"layers": nn.ModuleList([nn.Linear(6, 6), nn.Linear(6, 6)])})


def test_freeze_helpers_agree_with_the_reference():
    _ref_path()
    from kempnerforge.config.vlm import FreezeSpec as RSpec
    from kempnerforge.config.vlm import FreezeStage as RStage
    from kempnerforge.training import freeze as rf

    from kempnerforge_b200.config.vlm import FreezeSpec, FreezeStage
    from kempnerforge_b200.training import freeze as mf

    patterns = {"vision_encoder": ["vision_encoder.*"], "adapter": ["adapter.*"], "transformer": ["transformer.*"]}
    for pats in (["vision_encoder.*"], ["adapter.weight", "transformer.layers.1.*"], [], ["*"], ["adapter"]):
        a, b = _Toy(), _Toy()
        assert rf.freeze_params(a, pats) == mf.freeze_params(b, pats), pats
        assert [p.requires_grad for p in a.parameters()] == [p.requires_grad for p in b.parameters()], pats
    triples = [("vision_encoder", True), ("adapter", True), ("adapter", False), ("transformer", True)]
    a, b = _Toy(), _Toy()
    want = rf.apply_freeze_specs(a, [RSpec(m, f) for m, f in triples], patterns)
    got = mf.apply_freeze_specs(b, [FreezeSpec(m, f) for m, f in triples], patterns)
    assert dict(want) == dict(got)
    assert [p.requires_grad for p in a.parameters()] == [p.requires_grad for p in b.parameters()]
    assert rf.canonical_freeze_meta([RSpec(m, f) for m, f in triples]) == mf.canonical_freeze_meta(
        [FreezeSpec(m, f) for m, f in triples])
    base = [("vision_encoder", True), ("adapter", False)]
    stages = [(100, [("vision_encoder", False)]), (50, [("adapter", True), ("transformer", True)])]
    for step in (0, 49, 50, 99, 100, 1000):
        want = rf.effective_freeze(step, [RSpec(m, f) for m, f in base],
                                   [RStage(s, tuple(RSpec(m, f) for m, f in specs)) for s, specs in stages])
        got = mf.effective_freeze(step, [FreezeSpec(m, f) for m, f in base],
                                  [FreezeStage(s, tuple(FreezeSpec(m, f) for m, f in specs)) for s, specs in stages])
        assert [(s.module, s.frozen) for s in want] == [(s.module, s.frozen) for s in got], step


# --------------------------------------------------------------------------- NaN detector
@pytest.mark.parametrize("action", ["warn", "skip"])
def test_nan_detector_counts_and_recommends_rollback_like_the_reference(action):
    _ref_path()
    from kempnerforge.resilience.health import NaNDetector as Ref

    from kempnerforge_b200.resilience import NaNDetector

    a, b = Ref(action=action, max_consecutive=3, max_history=4), NaNDetector(action=action, max_consecutive=3, max_history=4)
    losses = [2.0, float("nan"), 1.9, float("inf"), float("nan"), float("-inf"), 1.5, float("nan")]
    for step, loss in enumerate(losses):
        assert a.check_loss(loss, step) == b.check_loss(loss, step), step
        assert a.should_rollback == b.should_rollback, step
        assert a.state.consecutive_nans == b.state.consecutive_nans and a.state.total_nans == b.state.total_nans, step
        assert list(a.state.nan_steps) == list(b.state.nan_steps), step
    a.reset(), b.reset()
    assert a.state.consecutive_nans == b.state.consecutive_nans == 0 and a.state.total_nans == b.state.total_nans


def test_nan_detector_raises_in_raise_mode_on_both_sides():
    _ref_path()
    from kempnerforge.resilience.health import NaNDetector as Ref

    from kempnerforge_b200.resilience import NaNDetector

    for cls in (Ref, NaNDetector):
        det = cls(action="raise")
        assert det.check_loss(1.0, 0) is True
        with pytest.raises(RuntimeError, match="NaN/Inf"):
            det.check_loss(float("nan"), 1)
        with pytest.raises(ValueError):
            cls(action="explode")


# --------------------------------------------------------------------------- sampling
@pytest.mark.parametrize("kw", [dict(temperature=0.0), dict(temperature=0.7), dict(top_k=5), dict(top_p=0.6),
                                dict(temperature=1.3, top_k=12, top_p=0.9), dict(top_k=1000), dict(top_p=0.5)])
def test_sampling_draws_the_reference_tokens_from_the_same_random_state(kw):
    _ref_path()
    from kempnerforge.model.generate import sample as ref_sample

    from kempnerforge_b200.models.generate import sample

    logits = torch.randn(6, 40, generator=torch.Generator().manual_seed(7)) * 2.0
    logits[0, :4] = torch.log(torch.tensor([0.5, 0.3, 0.15, 0.05]))      # a row whose mass hits top_p = 0.5 exactly
    logits[0, 4:] = float("-inf")
    for seed in range(5):
        torch.manual_seed(seed)
        want = ref_sample(logits.clone(), **kw)
        torch.manual_seed(seed)
        got = sample(logits.clone(), **kw)
        assert torch.equal(want, got), (kw, seed)


# --------------------------------------------------------------------------- layouts, cadence, job environment
def test_pipeline_layer_assignment_matches():
    _ref_path()
    from kempnerforge.distributed.pipeline_parallel import compute_layer_assignment as ref_assign

    from kempnerforge_b200.parallel.pipeline_parallel import compute_layer_assignment

    for n_layers in (1, 4, 7, 32, 40):
        for pp in (1, 2, 3, 4, 8):
            if pp <= n_layers:
                assert [tuple(x) for x in compute_layer_assignment(n_layers, pp)] == [tuple(x) for x in ref_assign(n_layers, pp)]


def test_parallel_layout_resolution_and_its_rejections_match():
    _ref_path()
    from kempnerforge.config.distributed import DistributedConfig as Ref

    from kempnerforge_b200.config import DistributedConfig

    fields = ("dp_replicate", "dp_shard", "tp", "pp", "cp", "ep")
    cases = [dict(), dict(tp=2), dict(tp=4, pp=2), dict(dp_replicate=2), dict(dp_shard=4, tp=2), dict(ep=2),
             dict(ep=8), dict(tp=3), dict(dp_shard=3, tp=2), dict(pp=2, ep=2, tp=2), dict(dp_replicate=2, dp_shard=2, tp=2)]
    for world in (1, 2, 8, 16):
        for kw in cases:
            outcomes = []
            for cls in (Ref, DistributedConfig):
                try:
                    r = cls(**kw).resolve(world)
                    outcomes.append(tuple(getattr(r, f) for f in fields))
                except ValueError:
                    outcomes.append("rejected")
            assert outcomes[0] == outcomes[1], (world, kw, outcomes)


def test_checkpoint_cadence_with_a_dynamic_window_matches():
    _ref_path()
    from kempnerforge.config.checkpoint import CheckpointConfig as Ref
    from kempnerforge.config.checkpoint import DynamicCheckpointWindow as RefWin

    from kempnerforge_b200.config import CheckpointConfig, DynamicCheckpointWindow

    for win_kw in (None, dict(start=0, stop=64), dict(start=10, stop=200), dict(start=5, stop=5)):
        for interval in (7, 50):
            a = Ref(interval=interval, dyn_ckpt_window=RefWin(**win_kw) if win_kw else None)
            b = CheckpointConfig(interval=interval, dyn_ckpt_window=DynamicCheckpointWindow(**win_kw) if win_kw else None)
            for step in range(0, 260):
                assert a.should_save(step) == b.should_save(step), (win_kw, interval, step)
                assert a.is_dynamic_milestone(step) == b.is_dynamic_milestone(step), (win_kw, interval, step)


def test_slurm_environment_and_resume_path_are_read_the_same_way(tmp_path, monkeypatch):
    _ref_path()
    from kempnerforge.resilience import elastic as ref

    from kempnerforge_b200.resilience import elastic as mine

    for key in list(__import__("os").environ):
        if key.startswith("SLURM_"):
            monkeypatch.delenv(key)
    assert ref.get_slurm_info() is None and mine.get_slurm_info() is None
    assert ref.is_slurm_job() == mine.is_slurm_job() is False and ref.is_slurm_requeue() == mine.is_slurm_requeue() is False
    env = {"SLURM_JOB_ID": "4242", "SLURM_JOB_NAME": "forge", "SLURM_NNODES": "4", "SLURM_NTASKS_PER_NODE": "8",
           "SLURM_JOB_PARTITION": "gpu", "SLURM_RESTART_COUNT": "2", "SLURM_ARRAY_TASK_ID": "3", "SLURM_NODELIST": "n[1-4]"}
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    a, b = ref.get_slurm_info(), mine.get_slurm_info()
    for field in a.__dataclass_fields__:
        assert getattr(a, field) == getattr(b, field), field
    assert ref.is_slurm_requeue() and mine.is_slurm_requeue()
    # resume path: nothing, then step directories only, then a "latest" link
    assert ref.resolve_resume_path(str(tmp_path / "none")) is None and mine.resolve_resume_path(str(tmp_path / "none")) is None
    for s in (5, 20, 100):
        (tmp_path / f"step_{s}").mkdir()
    assert ref.resolve_resume_path(str(tmp_path)).resolve() == mine.resolve_resume_path(str(tmp_path)).resolve() == (tmp_path / "step_100").resolve()
    (tmp_path / "latest").symlink_to("step_20")
    assert ref.resolve_resume_path(str(tmp_path)).resolve() == mine.resolve_resume_path(str(tmp_path)).resolve() == (tmp_path / "step_20").resolve()
