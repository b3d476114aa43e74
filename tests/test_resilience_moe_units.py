"""Shutdown handling, NaN policy, SLURM discovery, resume-path resolution; routers and MoE layers.

Mirrors tests/unit/test_resilience.py, test_router.py and test_moe.py of the reference."""

from __future__ import annotations

import os
import signal

import pytest
import torch
from torch import nn

from kempnerforge_b200.config.sections import DistributedConfig, ModelConfig
from kempnerforge_b200.models.moe import MoEMLP, apply_capacity, build_moe
from kempnerforge_b200.models.router import SigmoidTopKRouter, SoftmaxTopKRouter, build_router
from kempnerforge_b200.models.transformer import Transformer
from kempnerforge_b200.resilience.elastic import (get_slurm_info, is_slurm_job, is_slurm_requeue, list_step_dirs,
                                                  log_job_info, resolve_resume_path)
from kempnerforge_b200.resilience.health import NaNDetector
from kempnerforge_b200.resilience.signal_handler import ShutdownHandler


# --------------------------------------------------------------------------- shutdown handler
def test_shutdown_handler_flags_signals_and_restores_handlers():
    h = ShutdownHandler(timeout_sec=0)
    assert not h.should_shutdown() and h.signal_received is None
    before = signal.getsignal(signal.SIGUSR1)
    h.register()
    h.register()                                   # idempotent
    try:
        os.kill(os.getpid(), signal.SIGUSR1)
        assert h.should_shutdown() and h.signal_received == signal.SIGUSR1
        os.kill(os.getpid(), signal.SIGTERM)       # a second signal does not change the record
        assert h.signal_received == signal.SIGUSR1 and h._timer is None   # timeout 0: no force-exit timer
    finally:
        h.unregister()
    assert signal.getsignal(signal.SIGUSR1) == before


def test_shutdown_timer_is_a_daemon_and_finish_cancels_it():
    h = ShutdownHandler(timeout_sec=3600)
    h.request()
    assert h.should_shutdown() and h._timer is not None and h._timer.daemon
    h.finish()
    assert h._timer is None
    h.finish()


# --------------------------------------------------------------------------- NaN policy
def test_nan_detector_bookkeeping():
    d = NaNDetector(action="warn", max_consecutive=3, max_history=4)
    assert d.check_loss(2.5, 1) and d.state.last_good_loss == 2.5 and d.state.last_good_step == 1
    for step, bad in enumerate([float("nan"), float("inf"), float("-inf")], start=2):
        assert not d.check_loss(bad, step)
    assert d.state.consecutive_nans == 3 and d.state.total_nans == 3 and d.should_rollback and d.should_stop
    assert d.check_loss(2.0, 5) and d.state.consecutive_nans == 0 and d.state.total_nans == 3 and not d.should_rollback
    for step in range(6, 12):
        d.check_loss(float("nan"), step)
    assert len(d.state.nan_steps) == 4             # history is capped
    d.reset()
    assert d.state.total_nans == 0 and d.state.nan_steps == [] and d.state.last_good_loss == float("inf")


def test_nan_detector_actions():
    with pytest.raises(ValueError):
        NaNDetector(action="explode")
    with pytest.raises(RuntimeError, match="step 7"):
        NaNDetector(action="raise").check_loss(float("nan"), 7)
    skip = NaNDetector(action="skip")
    assert not skip.check_loss(float("nan"), 1) and skip.check_loss(1.0, 2)
    assert not skip.check_values(1.0, float("inf"), True, 3) and not skip.check_values(1.0, 1.0, False, 4)
    assert skip.check_values(1.0, 1.0, True, 5)


def test_nan_detector_gradient_scan():
    m = nn.Linear(3, 3)
    m(torch.ones(1, 3)).sum().backward()
    d = NaNDetector()
    assert d.check_gradients(m, 1)
    m.weight.grad[0, 0] = float("nan")
    assert not d.check_gradients(m, 2)
    with pytest.raises(RuntimeError, match="weight"):
        NaNDetector(action="raise").check_gradients(m, 3)


# --------------------------------------------------------------------------- SLURM discovery / resume path
_SLURM = ("SLURM_JOB_ID", "SLURM_JOB_NAME", "SLURM_JOB_NODELIST", "SLURM_JOB_NUM_NODES", "SLURM_NTASKS_PER_NODE",
          "SLURM_TASKS_PER_NODE", "SLURM_RESTART_COUNT", "SLURM_ARRAY_TASK_ID", "SLURM_JOB_PARTITION")


def test_slurm_discovery(monkeypatch, caplog):
    for k in _SLURM:
        monkeypatch.delenv(k, raising=False)
    assert get_slurm_info() is None and not is_slurm_job() and not is_slurm_requeue()
    log_job_info()
    monkeypatch.setenv("SLURM_JOB_ID", "123")
    info = get_slurm_info()
    assert is_slurm_job() and info.job_id == "123" and info.num_nodes == 1 and info.restart_count == 0
    monkeypatch.setenv("SLURM_JOB_NUM_NODES", "4")
    monkeypatch.setenv("SLURM_TASKS_PER_NODE", "8(x4)")
    monkeypatch.setenv("SLURM_RESTART_COUNT", "2")
    monkeypatch.setenv("SLURM_ARRAY_TASK_ID", "7")
    monkeypatch.setenv("SLURM_JOB_PARTITION", "gpu")
    info = get_slurm_info()
    assert (info.num_nodes, info.tasks_per_node, info.restart_count, info.array_task_id, info.partition) == (4, 8, 2, "7", "gpu")
    assert is_slurm_requeue()
    log_job_info()
    monkeypatch.setenv("SLURM_RESTART_COUNT", "0")
    assert not is_slurm_requeue()
    monkeypatch.setenv("SLURM_RESTART_COUNT", "junk")
    assert not is_slurm_requeue() and get_slurm_info().restart_count == 0


def test_resume_path_prefers_latest_then_the_highest_step(tmp_path):
    assert resolve_resume_path(tmp_path / "missing") is None and resolve_resume_path(tmp_path) is None
    for name in ("step_5", "step_100", "step_20", "notes", "step_x"):
        (tmp_path / name).mkdir()
    (tmp_path / "step_7").write_text("a file, not a checkpoint")
    assert [s for s, _ in list_step_dirs(tmp_path)] == [5, 20, 100]
    assert resolve_resume_path(tmp_path).name == "step_100"
    (tmp_path / "latest").symlink_to(tmp_path / "step_20")
    assert resolve_resume_path(tmp_path).name == "step_20"      # the link wins over a higher step
    (tmp_path / "latest").unlink()
    (tmp_path / "latest").symlink_to(tmp_path / "step_999")     # dangling link: fall back
    assert resolve_resume_path(tmp_path).name == "step_100"
    big = tmp_path / "step_12345678901"
    big.mkdir()
    assert resolve_resume_path(tmp_path) == big


# --------------------------------------------------------------------------- routers
def test_softmax_router_contract():
    torch.manual_seed(0)
    r = SoftmaxTopKRouter(16, 8, 2)
    x = torch.randn(64, 16, requires_grad=True)
    w, idx = r(x)
    assert w.shape == idx.shape == (64, 2) and int(idx.min()) >= 0 and int(idx.max()) < 8
    assert torch.allclose(w.sum(-1), torch.ones(64), atol=1e-6) and (idx[:, 0] != idx[:, 1]).all()
    assert float(r.expert_counts.sum()) == 128 and r.expert_counts.shape == (8,)
    assert float(r.aux_loss) >= 1.0 - 1e-4                       # switch-style loss: 1 at perfect balance
    (w.sum() + r.aux_loss + r.z_loss).backward()
    assert r.gate.weight.grad.abs().sum() > 0 and x.grad is not None
    want_z = torch.logsumexp(r.gate(x).float(), -1).pow(2).mean()
    assert torch.allclose(r.z_loss, want_z, atol=1e-6)
    uniform = SoftmaxTopKRouter(16, 4, 4)
    nn.init.zeros_(uniform.gate.weight)
    uniform(torch.randn(32, 16))
    assert float(uniform.aux_loss) == pytest.approx(1.0, abs=1e-5)


def test_sigmoid_router_balances_through_its_bias_and_freezes_in_eval():
    torch.manual_seed(1)
    r = SigmoidTopKRouter(16, 4, 1, bias_update_rate=0.05)
    with torch.no_grad():
        r.gate.weight.zero_()
        r.gate.weight[0] = 1.0                                    # expert 0 wins for x with a positive sum
    x = torch.rand(256, 16)
    w, idx = r(x)
    assert torch.allclose(w.sum(-1), torch.ones(256)) and float(r.aux_loss) == 0.0
    first_share = float(r.expert_counts[0]) / 256
    for _ in range(300):
        r(x)
    assert float(r.expert_counts[0]) / 256 < first_share           # the bias pushed load off the hot expert
    assert float(r.expert_bias[0]) < 0 < float(r.expert_bias[1:].max())
    r.eval()
    bias, ema = r.expert_bias.detach().clone(), r.expert_ema.clone()
    r(x)
    assert torch.equal(bias, r.expert_bias) and torch.equal(ema, r.expert_ema)


@pytest.mark.parametrize("schedule,rates", [("constant", (1.0, 1.0, 1.0)), ("cosine_decay", (1.0, 0.5, 0.0)),
                                            ("linear_warmup", (0.0, 1.0, 1.0))])
def test_bias_rate_schedules(schedule, rates):
    r = SigmoidTopKRouter(8, 4, 2, bias_update_rate=0.1, bias_schedule=schedule)
    for step, want in zip((0, 50, 100), rates):
        r.set_step(step, 100)
        assert r._effective_bias_rate() == pytest.approx(0.1 * want, abs=1e-9)


def test_sequence_aux_loss_and_router_registry():
    r = build_router("sigmoid_topk", 8, 4, 2, sequence_aux_loss_weight=0.5)
    r(torch.randn(32, 8))
    assert isinstance(r, SigmoidTopKRouter) and float(r.aux_loss) > 0
    r.aux_loss.backward()
    assert r.gate.weight.grad.abs().sum() > 0
    assert isinstance(build_router("softmax_topk", 8, 4, 2), SoftmaxTopKRouter)
    with pytest.raises((KeyError, ValueError)):
        build_router("hash", 8, 4, 2)


# --------------------------------------------------------------------------- MoE layers
def test_single_expert_moe_equals_its_dense_mlp():
    torch.manual_seed(2)
    moe = build_moe(16, 32, 1, 1)
    x = torch.randn(3, 5, 16)
    assert torch.allclose(moe(x), moe.expert_modules()[0](x), atol=1e-6)


def test_shared_expert_is_added_for_every_token():
    torch.manual_seed(3)
    moe = build_moe(16, 32, 4, 2, shared_experts=1)
    base = build_moe(16, 32, 4, 2)
    base.load_state_dict({k: v for k, v in moe.state_dict().items() if not k.startswith("shared_expert")})
    x = torch.randn(2, 6, 16)
    assert torch.allclose(moe(x), base(x) + moe.shared_expert(x), atol=1e-6)
    wide = build_moe(16, 32, 4, 2, shared_experts=2, shared_expert_widen=True)
    assert wide.shared_expert.up_proj.weight.shape[0] == 64
    moe(x).sum().backward()
    assert all(p.grad is not None for p in moe.shared_expert.parameters())


def test_capacity_keeps_the_first_arrivals_per_expert_slot():
    idx = torch.tensor([[0], [0], [0], [1], [0]])
    w = torch.ones(5, 1)
    kept, same = apply_capacity(w, idx, num_experts=2, capacity_factor=0.8)   # cap = ceil(5/2*0.8) = 2
    assert same is idx and kept.flatten().tolist() == [1, 1, 0, 1, 0]
    moe = build_moe(16, 32, 4, 2, capacity_factor=0.25)
    out = moe(torch.randn(1, 64, 16))
    out.sum().backward()
    assert torch.isfinite(out).all()
    free = build_moe(16, 32, 4, 2, capacity_factor=0.0)
    assert free.capacity_factor == 0.0


def test_load_scaling_applies_in_training_only():
    """Expert outputs are scaled by (average load / expert load) while training; evaluation is unchanged."""
    torch.manual_seed(4)
    a = build_moe(16, 32, 4, 2, gradient_scale=False)
    b = build_moe(16, 32, 4, 2, gradient_scale=True)
    b.load_state_dict(a.state_dict())
    x = torch.randn(2, 16, 16)
    out = b(x)
    assert out.shape == x.shape and not torch.allclose(a(x), out, atol=1e-6)
    out.square().sum().backward()
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in b.parameters())
    a.eval(), b.eval()
    assert torch.allclose(a(x), b(x), atol=1e-6)
    assert build_moe(16, 32, 4, 2).gradient_scale is False


def _moe_cfg(**kw):
    base = dict(dim=32, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=64, ffn_hidden_dim=48, max_seq_len=16,
                num_experts=4, moe_top_k=2)
    base.update(kw)
    return ModelConfig(**base)


def test_transformer_moe_accessors_and_placement():
    torch.manual_seed(5)
    m = Transformer(_moe_cfg(moe_frequency=2, moe_aux_loss_weight=0.01, moe_router_z_loss_weight=0.001))
    kinds = [isinstance(m.layers[str(i)].mlp, MoEMLP) for i in range(4)]
    assert kinds == [False, True, False, True]
    ids = torch.randint(0, 64, (2, 8))
    m(ids)
    assert float(m.get_moe_aux_loss()) > 0 and float(m.get_moe_router_z_loss()) > 0
    counts = m.get_expert_counts()
    assert sorted(counts) == [1, 3] and all(float(c.sum()) == 2 * 8 * 2 for c in counts.values())
    assert not any("aux_loss" in k or "z_loss" in k or "expert_counts" in k for k in m.state_dict())
    dense = Transformer(ModelConfig(dim=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, ffn_hidden_dim=48,
                                    max_seq_len=16))
    dense(ids)
    assert float(dense.get_moe_aux_loss()) == 0.0 and float(dense.get_moe_router_z_loss()) == 0.0
    assert dense.get_expert_counts() == {}
    dense.set_moe_step(3, 10)                                      # no-op without sigmoid routers


def test_sigmoid_transformer_propagates_the_step_and_trains():
    m = Transformer(_moe_cfg(moe_router="sigmoid_topk", moe_bias_schedule="cosine_decay", moe_shared_experts=1))
    m.set_moe_step(5, 10)
    routers = [mod for mod in m.modules() if isinstance(mod, SigmoidTopKRouter)]
    assert len(routers) == 4 and all(r._step == 5 and r._max_steps == 10 for r in routers)
    ids = torch.randint(0, 64, (2, 8))
    loss = m.compute_loss(ids, ids)
    loss.backward()
    assert float(m.get_moe_aux_loss()) == 0.0
    assert all(p.grad is not None for n, p in m.named_parameters() if "experts" in n or "gate" in n)


def test_fine_grained_experts_are_narrower():
    fine = _moe_cfg(num_experts=8, moe_expert_ffn_multiplier=0.25)
    want = fine.computed_expert_ffn_hidden_dim
    assert 0 < want < fine.computed_ffn_hidden_dim
    m = Transformer(fine)
    assert m.layers["0"].mlp.expert_modules()[0].up_proj.weight.shape == (want, 32)
    with pytest.raises(ValueError):
        _moe_cfg(moe_expert_ffn_multiplier=0.0)


def test_expert_parallel_config_rules():
    assert DistributedConfig().ep == 1
    cfg = DistributedConfig(ep=2).resolve(8)
    assert cfg.ep == 2 and cfg.dp_shard == 4
    with pytest.raises(ValueError):
        DistributedConfig(ep=3).resolve(8)
    with pytest.raises(ValueError):
        DistributedConfig(ep=0)


@pytest.mark.parametrize("accum", [1, 3])
def test_sigmoid_router_is_consistent_under_activation_checkpointing(accum):
    """The balancing bias moves in every forward pass; the recomputation of a checkpointed block must route with
    the bias its first pass used, update nothing, and give the gradients of an un-checkpointed run."""
    from kempnerforge_b200.parallel.parallel import apply_ac

    def run(mode):
        torch.manual_seed(11)
        m = Transformer(_moe_cfg(moe_router="sigmoid_topk", num_experts=8, moe_top_k=2, n_layers=3))
        for r in (mod for mod in m.modules() if isinstance(mod, SigmoidTopKRouter)):
            r.bias_update_rate = 0.5          # large nudges: a second update would visibly change the routing
        apply_ac(m, mode)
        m.train()
        g = torch.Generator().manual_seed(3)
        m.set_moe_step(0, 10)
        losses = []
        for _ in range(accum):               # forward/backward pairs, as in gradient accumulation
            ids = torch.randint(0, 64, (2, 16), generator=g)
            loss = m.compute_loss(ids, ids)
            loss.backward()
            losses.append(float(loss))
        grads = {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None}
        state = {n: b.clone() for n, b in m.named_buffers() if "expert_ema" in n}
        bias = {n: p.detach().clone() for n, p in m.named_parameters() if n.endswith("expert_bias")}
        return losses, grads, state, bias

    plain, ckpt = run("none"), run("full")
    assert plain[0] == pytest.approx(ckpt[0], rel=1e-6)
    for n in plain[1]:
        assert torch.allclose(plain[1][n], ckpt[1][n], atol=1e-5, rtol=1e-4), n
    for part in (2, 3):                       # moving averages and biases were updated once per forward, not twice
        for n in plain[part]:
            assert torch.allclose(plain[part][n], ckpt[part][n], atol=1e-7), n
