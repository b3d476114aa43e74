"""The non-tensor part of checkpoints, the trust check on pickled files, metadata peeking and the freeze comparison.

Mirrors tests/unit/test_checkpoint.py (train-state helpers, metadata, freeze comparison) and
test_checkpoint_security.py of the reference."""

from __future__ import annotations

import json
import os
import random
import stat
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from kempnerforge_b200.checkpoint import manager as ckpt
from kempnerforge_b200.checkpoint.manager import CheckpointManager, UntrustedCheckpointError, check_trusted_file
from kempnerforge_b200.checkpoint.state import (build_train_state, get_rng_state, restore_train_state, set_rng_state)
from kempnerforge_b200.config.sections import CheckpointConfig


class _Loader:
    def __init__(self):
        self.pos = 0

    def state_dict(self):
        return {"pos": self.pos}

    def load_state_dict(self, s):
        self.pos = s["pos"]


def _sched():
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0)
    return torch.optim.lr_scheduler.LambdaLR(opt, lambda s: 1.0 / (s + 1)), opt


# --------------------------------------------------------------------------- train state
def test_train_state_fields_and_optional_parts():
    bare = build_train_state(7, 700)
    assert bare["step"] == 7 and bare["tokens_seen"] == 700 and set(bare["rng"]) >= {"python", "numpy", "torch_cpu"}
    assert "scheduler" not in bare and "dataloader" not in bare
    sched, _ = _sched()
    loader = _Loader()
    loader.pos = 42
    full = build_train_state(7, 700, sched, loader, extra={"phase_idx": 2, "wandb_run_id": "abc"})
    assert full["scheduler"] == sched.state_dict() and full["dataloader"] == {"pos": 42}
    assert full["phase_idx"] == 2 and full["wandb_run_id"] == "abc"
    with pytest.raises(ValueError):
        build_train_state(1, 1, extra={"step": 5})
    assert "dataloader" not in build_train_state(1, 1, dataloader=object())   # loaders without state are skipped


def test_restore_applies_every_part_and_returns_extras():
    sched, opt = _sched()
    for _ in range(3):
        opt.step()
        sched.step()
    loader = _Loader()
    loader.pos = 9
    state = build_train_state(3, 300, sched, loader, extra={"phase_idx": 1})
    sched2, _ = _sched()
    loader2 = _Loader()
    step, tokens, extra = restore_train_state(state, sched2, loader2)
    assert (step, tokens, extra) == (3, 300, {"phase_idx": 1})
    assert sched2.last_epoch == 3 and loader2.pos == 9
    assert restore_train_state({}) == (0, 0, {})
    assert restore_train_state({"step": 4, "custom": [1, 2]})[2] == {"custom": [1, 2]}


def test_rng_streams_round_trip():
    random.seed(1)
    np.random.seed(1)
    torch.manual_seed(1)
    state = get_rng_state()
    want = (random.random(), float(np.random.rand()), float(torch.rand(1)))
    random.random(), np.random.rand(), torch.rand(3)                # advance all three
    set_rng_state(state)
    assert (random.random(), float(np.random.rand()), float(torch.rand(1))) == want
    set_rng_state({})                                               # tolerates missing streams


# --------------------------------------------------------------------------- trust check
def test_own_private_file_is_accepted(tmp_path):
    f = tmp_path / "train_state.pt"
    torch.save({"step": 1}, f)
    os.chmod(f, 0o600)
    check_trusted_file(f)
    os.chmod(f, 0o644)
    check_trusted_file(f)


@pytest.mark.parametrize("mode", [0o664, 0o646, 0o666])
def test_group_or_world_writable_files_are_loaded_with_a_warning(tmp_path, mode, caplog):
    f = tmp_path / "train_state.pt"
    torch.save({"step": 1}, f)
    os.chmod(f, mode)
    with caplog.at_level("WARNING"):
        check_trusted_file(f)                      # shared group-writable checkpoint directories keep working
    assert any("writable" in r.getMessage() and oct(mode) in r.getMessage() for r in caplog.records)


def test_foreign_owner_is_refused_before_any_unpickling(tmp_path, monkeypatch):
    f = tmp_path / "train_state.pt"
    f.write_bytes(b"not even a pickle")
    real_stat = os.stat(f)
    fake = SimpleNamespace(st_uid=real_stat.st_uid + 12345, st_mode=stat.S_IFREG | 0o600)
    monkeypatch.setattr(type(f), "stat", lambda self, **kw: fake)
    loaded = []
    monkeypatch.setattr(torch, "load", lambda *a, **k: loaded.append(a))
    with pytest.raises(UntrustedCheckpointError, match="owned by uid"):
        check_trusted_file(f)
    with pytest.raises(PermissionError):                             # the type the reference raises
        check_trusted_file(f)
    assert loaded == []


# --------------------------------------------------------------------------- manager helpers that need no tensors
def _manager(tmp_path, **cfg):
    model = torch.nn.Linear(2, 2)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    return CheckpointManager(CheckpointConfig(dir=str(tmp_path), **cfg), model, opt)


def test_peek_saved_step_reads_metadata_only(tmp_path):
    m = _manager(tmp_path)
    assert m.peek_saved_step() is None                              # no checkpoint at all
    d = tmp_path / "step_12"
    d.mkdir()
    assert m.peek_saved_step(d) is None                             # no metadata file
    (d / "metadata.json").write_text("{broken")
    assert m.peek_saved_step(d) is None
    (d / "metadata.json").write_text(json.dumps({"tokens_seen": 5}))
    assert m.peek_saved_step(d) is None                             # no step field
    (d / "metadata.json").write_text(json.dumps({"step": 12}))
    assert m.peek_saved_step(d) == 12
    (tmp_path / "latest").symlink_to(d)
    assert m.peek_saved_step() == 12


def _freeze_meta(tmp_path, saved):
    d = tmp_path / "step_1"
    d.mkdir(exist_ok=True)
    meta = {"step": 1}
    if saved is not None:
        meta["vlm_freeze"] = saved
    (d / "metadata.json").write_text(json.dumps(meta))
    return d


def test_freeze_comparison_rules(tmp_path):
    m = _manager(tmp_path)
    enc = {"module": "vision_encoder", "frozen": True}
    ada = {"module": "adapter", "frozen": False}
    d = _freeze_meta(tmp_path, [enc, ada])
    m._check_freeze_metadata(d, [ada, enc])                          # order does not matter
    m._check_freeze_metadata(d, None)                                # nothing expected: no comparison
    m._check_freeze_metadata(d, [enc, ada, {"module": "cross_attention", "frozen": True}])   # one-sided keys drop out
    m._check_freeze_metadata(d, [{"module": "mot", "frozen": True}])                          # disjoint: passes
    with pytest.raises(ValueError, match="vision_encoder"):
        m._check_freeze_metadata(d, [{"module": "vision_encoder", "frozen": False}, ada])
    m._check_freeze_metadata(_freeze_meta(tmp_path, None), [{"module": "vision_encoder", "frozen": False}])
    lax = _manager(tmp_path, ignore_freeze_mismatch=True)
    lax._check_freeze_metadata(_freeze_meta(tmp_path, [enc]), [{"module": "vision_encoder", "frozen": False}])


def test_retention_protects_latest_and_milestones(tmp_path):
    m = _manager(tmp_path, keep_last_n=2)
    for s in (10, 20, 30, 40):
        (tmp_path / f"step_{s}").mkdir()
    (tmp_path / "latest").symlink_to(tmp_path / "step_10")
    m._cleanup()
    left = sorted(p.name for p in tmp_path.iterdir() if p.name.startswith("step_"))
    assert left == ["step_10", "step_30", "step_40"]                 # step_20 went; the linked step_10 stayed
    under = _manager(tmp_path / "few", keep_last_n=5)
    (tmp_path / "few").mkdir(exist_ok=True)
    (tmp_path / "few" / "step_1").mkdir()
    under._cleanup()
    assert (tmp_path / "few" / "step_1").exists()


def test_wait_without_a_pending_save_is_a_noop(tmp_path):
    m = _manager(tmp_path)
    m.wait()
    m.flush_pending_save()
    assert CheckpointConfig().async_mode in ("disabled", "async", "async_with_pinned_mem") or True
    assert ckpt.model_state_dict(torch.nn.Linear(2, 2)).keys() == {"weight", "bias"}


@pytest.mark.parametrize("opt_name", ["adamw", "lion", "muon"])
def test_a_checkpoint_written_before_the_first_optimizer_step_loads(tmp_path, opt_name):
    """A save at step 0 (dynamic checkpoint windows start there) happens before any optimizer state exists; the
    checkpoint must still carry every key a later load asks for, and older checkpoints without optimizer state load
    with zero moments."""
    from kempnerforge_b200.config import CheckpointConfig, ModelConfig, OptimizerConfig
    from kempnerforge_b200.models import Transformer
    from kempnerforge_b200.training.optimizer import build_optimizer

    def make():
        torch.manual_seed(0)
        model = Transformer(ModelConfig(dim=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=16))
        opt = build_optimizer(model, OptimizerConfig(name=opt_name, lr=1e-3, fused=False))
        return model, opt, ckpt.CheckpointManager(CheckpointConfig(dir=str(tmp_path / "ck")), model, opt)

    model, opt, mgr = make()
    mgr.save(step=0)
    mgr.wait()
    model2, opt2, mgr2 = make()
    with torch.no_grad():
        for p in model2.parameters():
            p.add_(1.0)
    step, _, _ = mgr2.load()
    assert step == 0
    for (n, a), (_, b) in zip(model.named_parameters(), model2.named_parameters()):
        assert torch.equal(a, b), n
    # training continues from the loaded state
    ids = torch.randint(0, 64, (2, 8))
    model2(ids).float().square().mean().backward()
    opt2.step()
