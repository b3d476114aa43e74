"""Checkpoint manager (layout, retention, async protocol, trust check, resume) and resilience helpers."""

import json
import os
import signal
import time

import pytest
import torch

from kempnerforge_b200.checkpoint import CheckpointManager, UntrustedCheckpointError, check_trusted_file
from kempnerforge_b200.config import CheckpointConfig, DynamicCheckpointWindow, ModelConfig, OptimizerConfig, SchedulerConfig
from kempnerforge_b200.models import Transformer
from kempnerforge_b200.parallel.flat import flatten_model
from kempnerforge_b200.resilience import NaNDetector, ShutdownHandler, check_nccl_health, resolve_resume_path
from kempnerforge_b200.training import build_optimizer, build_scheduler

TINY = dict(dim=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=16)


def _setup(opt_name="adamw", flat=True, seed=0):
    torch.manual_seed(seed)
    model = Transformer(ModelConfig(**TINY))
    if flat:
        flatten_model(model)
    opt = build_optimizer(model, OptimizerConfig(name=opt_name, lr=1e-2))
    sched = build_scheduler(opt, SchedulerConfig(warmup_steps=2), 20)
    return model, opt, sched


def _step(model, opt, sched, seed):
    g = torch.Generator().manual_seed(seed)
    tok = torch.randint(0, 64, (2, 9), generator=g)
    model.compute_loss(tok[:, :-1], tok[:, 1:]).backward()
    for fg in getattr(model, "_kf_flat_groups", []):
        fg.finalize_grads()
    opt.step()
    sched.step()
    for fg in getattr(model, "_kf_flat_groups", []):
        fg.zero_grad()
    opt.zero_grad()


@pytest.mark.parametrize("opt_name,flat", [("adamw", True), ("adamw", False), ("lion", True), ("muon", True),
                                           ("schedule_free_adamw", True)])
def test_save_load_resumes_bit_exact(tmp_path, opt_name, flat):
    cfg = CheckpointConfig(dir=str(tmp_path), interval=1)
    model, opt, sched = _setup(opt_name, flat)
    for s in range(3):
        _step(model, opt, sched, s)
    CheckpointManager(cfg, model, opt).save(3, tokens_seen=48, scheduler=sched, extra={"phase_idx": 1})
    for s in range(3, 6):
        _step(model, opt, sched, s)
    want = {n: p.detach().clone() for n, p in model.named_parameters()}

    model2, opt2, sched2 = _setup(opt_name, flat, seed=123)  # different init: everything must come from the file
    step, tokens, extra = CheckpointManager(cfg, model2, opt2).load(scheduler=sched2)
    assert (step, tokens, extra["phase_idx"]) == (3, 48, 1)
    assert sched2.last_epoch == 3
    for s in range(3, 6):
        _step(model2, opt2, sched2, s)
    for n, p in model2.named_parameters():
        assert torch.equal(p.detach(), want[n]), n


def test_layout_latest_and_metadata(tmp_path):
    cfg = CheckpointConfig(dir=str(tmp_path))
    model, opt, sched = _setup()
    _step(model, opt, sched, 0)
    mgr = CheckpointManager(cfg, model, opt)
    d = mgr.save(7, 100, scheduler=sched)
    assert d.name == "step_7" and (d / ".metadata").exists() and (d / "train_state.pt").exists()
    assert json.loads((d / "metadata.json").read_text()) == {"step": 7, "tokens_seen": 100}
    assert os.readlink(tmp_path / "latest") == "step_7"
    assert mgr.peek_saved_step() == 7
    assert resolve_resume_path(tmp_path) == d.resolve()
    import torch.distributed.checkpoint as dcp

    # the tensor keys are the reference's: "model.<fqn>" and "optimizer.state.<fqn>.exp_avg"
    keys = set(dcp.FileSystemReader(str(d)).read_metadata().state_dict_metadata)
    assert "model.layers.0.attention.q_proj.weight" in keys
    assert "optimizer.state.layers.0.attention.q_proj.weight.exp_avg" in keys
    assert "optimizer.state.norm.weight.step" in keys


def test_retention_keeps_latest_and_milestones(tmp_path):
    cfg = CheckpointConfig(dir=str(tmp_path), keep_last_n=2, dyn_ckpt_window=DynamicCheckpointWindow(start=0, stop=4))
    model, opt, sched = _setup()
    _step(model, opt, sched, 0)
    mgr = CheckpointManager(cfg, model, opt)
    for s in (1, 2, 3, 5, 6, 7):
        mgr.save(s)
    names = sorted(p.name for p in tmp_path.iterdir() if p.name.startswith("step_"))
    assert names == ["step_1", "step_2", "step_6", "step_7"]  # 1, 2 are window milestones; 3 and 5 were pruned


def test_async_commits_latest_late(tmp_path):
    cfg = CheckpointConfig(dir=str(tmp_path), async_mode="async")
    model, opt, sched = _setup()
    _step(model, opt, sched, 0)
    mgr = CheckpointManager(cfg, model, opt)
    mgr.save(1)
    assert not (tmp_path / "latest").exists()  # flush in flight: nothing is committed yet
    mgr.save(2)
    assert os.readlink(tmp_path / "latest") == "step_1"  # the previous save was committed first
    mgr.wait()
    assert os.readlink(tmp_path / "latest") == "step_2"
    step, _, _ = CheckpointManager(cfg, *_setup()[:2]).load()
    assert step == 2


def test_incomplete_checkpoint_falls_back(tmp_path):
    cfg = CheckpointConfig(dir=str(tmp_path))
    model, opt, sched = _setup()
    _step(model, opt, sched, 0)
    mgr = CheckpointManager(cfg, model, opt)
    mgr.save(1)
    broken = tmp_path / "step_2"
    broken.mkdir()  # a directory without .metadata, as an interrupted flush would leave it
    (tmp_path / "latest").unlink()
    (tmp_path / "latest").symlink_to("step_2")
    step, _, _ = CheckpointManager(cfg, *_setup()[:2]).load()
    assert step == 1
    empty = CheckpointManager(CheckpointConfig(dir=str(tmp_path / "none")), *_setup()[:2]).load()
    assert empty == (0, 0, {})


def test_explicit_path_is_honoured_and_train_state_only_load_needs_no_tensors(tmp_path):
    """Fallback to an older checkpoint is for auto-resume only; an explicit path fails loudly.  A load that wants
    only the train state does not look at the tensor data."""
    cfg = CheckpointConfig(dir=str(tmp_path))
    model, opt, sched = _setup()
    _step(model, opt, sched, 0)
    CheckpointManager(cfg, model, opt).save(1, tokens_seen=7, scheduler=sched)
    broken = tmp_path / "step_2"
    broken.mkdir()
    with pytest.raises(BaseException):   # torch's CheckpointException derives from BaseException
        CheckpointManager(cfg, *_setup()[:2]).load(path=str(broken))
    for f in (tmp_path / "step_1").glob("*.distcp"):
        f.unlink()
    (tmp_path / "step_1" / ".metadata").unlink()
    step, tokens, _ = CheckpointManager(cfg, *_setup()[:2]).load(path=str(tmp_path / "step_1"),
                                                                exclude_keys=["model", "optimizer"])
    assert (step, tokens) == (1, 7)


def test_pipeline_stage_reads_the_step_level_train_state(tmp_path):
    """With pipeline parallelism rank 0 writes ``step_N/train_state.pt`` (the reference's layout) beside the per-stage
    copies, and a stage without its own copy falls back to it."""
    cfg = CheckpointConfig(dir=str(tmp_path))
    model, opt, sched = _setup()
    _step(model, opt, sched, 0)
    CheckpointManager(cfg, model, opt, pp_rank=0).save(1, tokens_seen=11, scheduler=sched, extra={"wandb_run_id": "abc"})
    assert (tmp_path / "step_1" / "train_state.pt").exists() and (tmp_path / "step_1" / "pp0" / "train_state.pt").exists()
    (tmp_path / "step_1" / "pp0" / "train_state.pt").unlink()          # what a reference-written checkpoint looks like
    model2, opt2, sched2 = _setup(seed=5)
    step, tokens, extra = CheckpointManager(cfg, model2, opt2, pp_rank=0).load(scheduler=sched2)
    assert (step, tokens, extra.get("wandb_run_id")) == (1, 11, "abc") and sched2.last_epoch == sched.last_epoch


def test_exclude_optimizer_and_dataloader_stash(tmp_path):
    cfg = CheckpointConfig(dir=str(tmp_path))
    model, opt, sched = _setup()
    _step(model, opt, sched, 0)

    class Loader:
        def __init__(self):
            self.state = {"epoch": 0}

        def state_dict(self):
            return {"epoch": 4}

        def load_state_dict(self, s):
            self.state = s

    CheckpointManager(cfg, model, opt).save(1, dataloader=Loader())
    model2, opt2, _ = _setup(seed=5)
    mgr = CheckpointManager(cfg, model2, opt2)
    mgr.load(exclude_keys=["optimizer"])
    assert torch.equal(model2.norm.weight, model.norm.weight)
    assert float(opt2._flat_groups[0].step_count) == 0
    late = Loader()
    mgr.apply_dataloader_state(late)
    assert late.state == {"epoch": 4}


def test_untrusted_train_state_is_refused(tmp_path):
    f = tmp_path / "train_state.pt"
    torch.save({"step": 1}, f)
    check_trusted_file(f)
    os.chmod(f, 0o666)
    check_trusted_file(f)                       # writable by others: a warning, not a refusal
    real = os.getuid
    os.getuid = lambda: real() + 1
    try:
        with pytest.raises(UntrustedCheckpointError):
            check_trusted_file(f)
    finally:
        os.getuid = real


def test_freeze_metadata_mismatch(tmp_path):
    cfg = CheckpointConfig(dir=str(tmp_path))
    model, opt, sched = _setup()
    _step(model, opt, sched, 0)
    CheckpointManager(cfg, model, opt).save(1, extra={"vlm_freeze": [{"module": "vision_encoder", "frozen": True}]})
    mgr = CheckpointManager(cfg, *_setup()[:2])
    with pytest.raises(ValueError):
        mgr.load(vlm_freeze_expected=[{"module": "vision_encoder", "frozen": False}])
    cfg.ignore_freeze_mismatch = True
    assert CheckpointManager(cfg, *_setup()[:2]).load(vlm_freeze_expected=[{"module": "vision_encoder", "frozen": False}])[0] == 1


# ------------------------------------------------------------------ resilience
def test_nan_detector_state_machine():
    d = NaNDetector(action="warn", max_consecutive=2)
    assert d.check_loss(1.0, 1)
    assert not d.check_loss(float("nan"), 2) and not d.should_rollback
    assert not d.check_loss(float("inf"), 3) and d.should_rollback
    assert d.check_loss(0.5, 4) and not d.should_rollback and d.state.total_nans == 2
    assert d.state.nan_steps == [2, 3] and d.state.last_good_step == 4
    with pytest.raises(RuntimeError):
        NaNDetector(action="raise").check_loss(float("nan"), 1)
    with pytest.raises(ValueError):
        NaNDetector(action="explode")
    assert not d.check_values(1.0, 2.0, all_ranks_finite=False, step=5)  # another rank saw a NaN


def test_shutdown_handler_flag_and_timer():
    h = ShutdownHandler(timeout_sec=30)
    h.register()
    try:
        assert not h.should_shutdown()
        os.kill(os.getpid(), signal.SIGUSR1)
        time.sleep(0.05)
        assert h.should_shutdown() and h.signal_received == signal.SIGUSR1 and h._timer is not None
    finally:
        h.unregister()
    assert h._timer is None


def test_health_checks_without_process_group():
    assert check_nccl_health(timeout_sec=0.1) is True


def test_collective_timeout_is_reported(monkeypatch):
    import torch.distributed as dist

    class _Work:
        def wait(self, timeout=None):
            return False

    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: 2)
    monkeypatch.setattr(dist, "get_backend", lambda group=None: "gloo")
    monkeypatch.setattr(dist, "all_reduce", lambda *a, **k: _Work())
    assert check_nccl_health(timeout_sec=0.01) is False


def test_resume_path_resolution(tmp_path):
    assert resolve_resume_path(tmp_path) is None
    (tmp_path / "step_5").mkdir()
    (tmp_path / "step_20").mkdir()
    (tmp_path / "junk").mkdir()
    assert resolve_resume_path(tmp_path).name == "step_20"
    (tmp_path / "latest").symlink_to("step_5")
    assert resolve_resume_path(tmp_path).name == "step_5"
