"""Host-side failure detection, seeding and checkpoint trust rules, one behaviour per test (CPU; failures are injected
with fakes of the failing call, never on a device).

Behaviours of kempnerforge/resilience/health.py (collective health check with a deadline),
kempnerforge/distributed/setup.py (seeding) and the ownership / permission check before ``train_state.pt`` is
unpickled (kempnerforge/checkpoint/manager.py)."""

import os
import pickle
import random
import stat
from datetime import timedelta

import numpy as np
import pytest
import torch
import torch.distributed as dist

from kempnerforge_b200.checkpoint import UntrustedCheckpointError, check_trusted_file
from kempnerforge_b200.parallel.setup import set_seed
from kempnerforge_b200.resilience import check_gpu_health, check_native_kernel_status, check_nccl_health


# --------------------------------------------------------------------------- collective health check
class _Work:
    def __init__(self, result=True, raises=None, value=None, tensor=None):
        self.result, self.raises, self.value, self.tensor, self.timeouts = result, raises, value, tensor, []

    def wait(self, timeout=None):
        self.timeouts.append(timeout)
        if self.raises is not None:
            raise self.raises
        if self.value is not None:
            self.tensor.fill_(self.value)
        return self.result


def _fake_group(monkeypatch, make_work, world=4):
    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: world)
    monkeypatch.setattr(dist, "get_backend", lambda group=None: "gloo")
    works = []

    def all_reduce(t, group=None, async_op=False):
        assert async_op, "the health check must not block without a deadline"
        works.append(make_work(t))
        return works[-1]

    monkeypatch.setattr(dist, "all_reduce", all_reduce)
    return works


def test_health_check_passes_without_a_process_group():
    assert check_nccl_health(timeout_sec=0.01) is True


def test_the_deadline_reaches_the_wait_as_a_timedelta(monkeypatch):
    works = _fake_group(monkeypatch, lambda t: _Work(value=4.0, tensor=t))
    assert check_nccl_health(timeout_sec=2.5) is True
    assert works[0].timeouts == [timedelta(seconds=2.5)]


def test_a_wait_that_returns_false_is_a_failed_check(monkeypatch):
    _fake_group(monkeypatch, lambda t: _Work(result=False))
    assert check_nccl_health(timeout_sec=0.01) is False


def test_a_wait_that_raises_is_a_failed_check_not_an_exception(monkeypatch):
    _fake_group(monkeypatch, lambda t: _Work(raises=RuntimeError("watchdog: collective timed out")))
    assert check_nccl_health(timeout_sec=0.01) is False


def test_a_wrong_sum_is_a_failed_check(monkeypatch):
    _fake_group(monkeypatch, lambda t: _Work(value=3.0, tensor=t), world=4)   # one rank did not contribute
    assert check_nccl_health(timeout_sec=0.01) is False


def test_gpu_probe_never_raises_and_says_why_it_is_unhealthy(monkeypatch):
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    out = check_gpu_health()
    assert out["healthy"] is False and out["cuda_available"] is False and "not available" in out["error"]
    assert check_native_kernel_status() == 0


# --------------------------------------------------------------------------- seeding
def test_set_seed_seeds_every_generator_the_run_uses():
    set_seed(123)
    first = (random.random(), float(np.random.rand()), float(torch.rand(())))
    set_seed(123)
    assert (random.random(), float(np.random.rand()), float(torch.rand(()))) == first
    set_seed(124)
    assert (random.random(), float(np.random.rand()), float(torch.rand(()))) != first


def test_pipeline_stages_get_different_streams_and_other_ranks_the_same():
    set_seed(7, pp_rank=0)
    a = torch.rand(4)
    set_seed(7, pp_rank=1)
    b = torch.rand(4)
    set_seed(7, pp_rank=0)          # what any data- or tensor-parallel peer of stage 0 calls
    assert not torch.equal(a, b) and torch.equal(torch.rand(4), a)


def test_seeds_larger_than_32_bits_do_not_break_numpy():
    set_seed(2**40 + 5)
    assert 0.0 <= float(np.random.rand()) < 1.0


# --------------------------------------------------------------------------- trust check before unpickling
def _private_file(tmp_path, name="train_state.pt"):
    p = tmp_path / name
    p.write_bytes(pickle.dumps({"step": 3}))
    p.chmod(0o600)
    return p


def test_own_private_file_is_accepted(tmp_path):
    check_trusted_file(_private_file(tmp_path))


def test_read_permission_for_others_is_fine(tmp_path):
    p = _private_file(tmp_path)
    p.chmod(0o644)
    check_trusted_file(p)


@pytest.mark.parametrize("bit", [stat.S_IWGRP, stat.S_IWOTH])
def test_files_that_others_may_write_load_with_a_warning(tmp_path, bit, caplog):
    p = _private_file(tmp_path)
    p.chmod(0o600 | bit)
    with caplog.at_level("WARNING"):
        check_trusted_file(p)
    assert any("writable" in r.getMessage() for r in caplog.records)


def test_files_of_another_user_are_refused_with_a_permission_error(tmp_path, monkeypatch):
    p = _private_file(tmp_path)
    owner = p.stat().st_uid
    monkeypatch.setattr(os, "getuid", lambda: owner + 1000)
    with pytest.raises(PermissionError, match="owned by uid"):
        check_trusted_file(p)
    with pytest.raises(UntrustedCheckpointError):
        check_trusted_file(p)


def test_an_untrusted_train_state_is_refused_before_its_pickle_runs(tmp_path):
    """The payload would raise on load: the refusal must come first."""
    from kempnerforge_b200.checkpoint import CheckpointManager
    from kempnerforge_b200.config import CheckpointConfig

    class Bomb:
        def __reduce__(self):
            return (exec, ("raise SystemExit('pickle payload executed')",))

    step = tmp_path / "step_1"
    step.mkdir()
    f = step / "train_state.pt"
    f.write_bytes(pickle.dumps(Bomb()))
    mgr = CheckpointManager(CheckpointConfig(dir=str(tmp_path)), torch.nn.Linear(2, 2), None)
    real = os.getuid
    os.getuid = lambda: real() + 1            # the file now belongs to "somebody else"
    try:
        with pytest.raises(UntrustedCheckpointError):
            mgr.load(path=str(step), exclude_keys=["model", "optimizer"])
    finally:
        os.getuid = real
