"""The alternative spellings of small API members (properties, aliases, functional forms) behave like the primary ones."""

from __future__ import annotations

import pytest
import torch
from torch import nn

from kempnerforge_b200.config import ModelConfig


def test_loss_aliases_and_toml_loader(tmp_path):
    from kempnerforge_b200.config.loader import load_config, load_toml
    from kempnerforge_b200.training import loss as L

    logits, labels = torch.randn(2, 5, 11), torch.randint(0, 11, (2, 5))
    labels[0, 0] = -100
    assert torch.equal(L.cross_entropy_loss(logits, labels), L.cross_entropy(logits, labels))
    torch.testing.assert_close(L.chunked_cross_entropy_loss(logits, labels, chunk_size=3), L.cross_entropy(logits, labels))
    path = tmp_path / "c.toml"
    path.write_text("[train]\nseq_len = 64\n")
    assert load_toml(path) == {"train": {"seq_len": 64}} and load_config(path).train.seq_len == 64
    with pytest.raises(FileNotFoundError):
        load_toml(tmp_path / "absent.toml")


def test_rank_requeue_shutdown_and_pending_properties(monkeypatch):
    from kempnerforge_b200.checkpoint.async_save import AsyncCheckpointer
    from kempnerforge_b200.parallel.setup import is_rank_zero
    from kempnerforge_b200.resilience.elastic import SLURMInfo
    from kempnerforge_b200.resilience.signal_handler import ShutdownHandler

    monkeypatch.setenv("RANK", "3")
    assert not is_rank_zero()
    monkeypatch.setenv("RANK", "0")
    assert is_rank_zero()
    assert SLURMInfo(restart_count=2).is_requeued and not SLURMInfo().is_requeued
    h = ShutdownHandler(timeout_sec=600)
    assert not h.shutdown_requested and not h.should_shutdown()
    h.request()
    try:
        assert h.shutdown_requested and h.should_shutdown()
    finally:
        h.finish()
    saver = AsyncCheckpointer("disabled")
    assert saver.is_pending is False and saver.pending is False


def test_mixed_precision_policy_feeds_build_parallel_model():
    from kempnerforge_b200.parallel.parallel import MixedPrecisionPolicy, build_parallel_model, default_mp_policy

    pol = default_mp_policy()
    assert pol == MixedPrecisionPolicy(torch.bfloat16, torch.float32, True)
    cfg = ModelConfig(dim=32, n_layers=1, n_heads=4, n_kv_heads=2, vocab_size=64, ffn_hidden_dim=48, max_seq_len=16)
    model = build_parallel_model(cfg, torch.device("cpu"), None, mp_policy=default_mp_policy(torch.float32))
    assert next(model.parameters()).dtype == torch.float32
    with pytest.raises(ValueError):
        build_parallel_model(cfg, torch.device("cpu"), None, mp_policy=MixedPrecisionPolicy(reduce_dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        build_parallel_model(cfg, torch.device("cpu"), None, vision_config=object())


def test_functional_grouped_expert_forward_matches_a_loop():
    from kempnerforge_b200.models.mlp import build_mlp
    from kempnerforge_b200.models.moe import grouped_expert_forward, grouped_expert_forward_packed

    torch.manual_seed(0)
    for act in ("silu", "gelu"):
        experts = nn.ModuleList([build_mlp(16, 24, act) for _ in range(3)])
        counts = [4, 0, 3]
        x = torch.randn(sum(counts), 16)
        want = torch.cat([experts[e](x[lo:lo + n]) for e, (lo, n) in enumerate(zip([0, 4, 4], counts))])
        got = grouped_expert_forward(x, counts, experts)
        torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
        swiglu = hasattr(experts[0], "gate_proj")
        up = torch.stack([e.up_proj.weight.t() for e in experts])
        down = torch.stack([e.down_proj.weight.t() for e in experts])
        gate = torch.stack([e.gate_proj.weight.t() for e in experts]) if swiglu else None
        packed = grouped_expert_forward_packed(x, torch.tensor(counts), up, down, gate, None if swiglu else experts[0].act)
        torch.testing.assert_close(packed, want, rtol=1e-4, atol=1e-5)
    assert grouped_expert_forward(x[:0], [0, 0, 0], experts).shape == (0, 16)


def test_strategies_satisfy_the_protocol_and_adapters_reset():
    from kempnerforge_b200.config.registry import registry
    from kempnerforge_b200.models import adapter as A
    from kempnerforge_b200.models.vlm import ModalityStrategy

    for name in registry.list_modality_strategies():
        strat = registry.get_modality_strategy(name)
        strat = strat() if isinstance(strat, type) else strat
        assert isinstance(strat, ModalityStrategy), name
    torch.manual_seed(0)
    for ad in (A.MLP2LayerAdapter(8, 12), A.LinearAdapter(8, 12), A.AvgPoolAdapter(8, 12, pool_window=2),
               A.AttentionalPoolAdapter(8, 12, pool_window=2, pool_heads=2)):
        before = [p.clone() for p in ad.parameters()]
        ad.reset_parameters()
        assert any(not torch.equal(a, b) for a, b in zip(before, ad.parameters()))
    x = torch.randn(2, 36, 8)
    avg = A.AvgPoolAdapter(8, 12, pool_window=2)
    assert avg(x).shape == (2, 9, 12) and avg(x, pool_window=3).shape == (2, 4, 12)
    att = A.AttentionalPoolAdapter(8, 12, pool_window=2, pool_heads=2)
    assert att(x).shape == (2, 9, 12) and att(x, pool_window=3).shape == (2, 4, 12) and att.head_dim == 4
    with pytest.raises(ValueError):
        att(x, pool_window=4)
    with pytest.raises(ValueError):
        avg(x, pool_window=0)


def test_stage_module_reinitialises_and_init_weights_accepts_a_config():
    from kempnerforge_b200.models.init import init_weights
    from kempnerforge_b200.parallel.pipeline_parallel import build_stage_module

    cfg = ModelConfig(dim=32, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=64, ffn_hidden_dim=48, max_seq_len=16)
    torch.manual_seed(0)
    stage = build_stage_module(cfg, 1, 2)
    before = stage.layers["2"].attention.q_proj.weight.clone() if hasattr(stage.layers, "keys") else None
    stage.init_weights_and_freqs()
    assert stage._rope_cos is not None and stage._rope_cos.shape[0] == 16
    if before is not None:
        assert not torch.equal(before, stage.layers["2"].attention.q_proj.weight)
    lin = nn.Sequential(nn.Linear(8, 8))
    torch.manual_seed(1)
    init_weights(lin, cfg)
    a = lin[0].weight.clone()
    torch.manual_seed(1)
    init_weights(lin, cfg.n_layers, cfg.init_std)
    assert torch.equal(a, lin[0].weight)


def test_positional_orders_shared_with_other_callers():
    from kempnerforge_b200.config import JobConfig
    from kempnerforge_b200.data.sampler import DistributedSampler
    from kempnerforge_b200.metrics.mfu import compute_mfu, estimate_model_flops_per_token
    from kempnerforge_b200.metrics.tracker import MetricsTracker

    cfg = ModelConfig(dim=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, ffn_hidden_dim=48, max_seq_len=16)
    # (config, tokens/s, gpus, peak TFLOP/s per GPU, sequence length)
    a = compute_mfu(cfg, 1e6, 2, 100.0, 8)
    assert a == pytest.approx(estimate_model_flops_per_token(cfg, 8) * 1e6 / (2 * 100e12))
    assert compute_mfu(cfg, 1e6, 2, 100.0) == pytest.approx(estimate_model_flops_per_token(cfg) * 1e6 / 200e12)
    assert compute_mfu(cfg, 1e6, 0, 100.0) == 0.0 and compute_mfu(cfg, 1e6, 1, 0.0) == 0.0
    data = list(range(10))
    s1, s2 = DistributedSampler(data, 2, 0, shuffle=False), DistributedSampler(dataset=data, num_replicas=2, rank=0, shuffle=False)
    assert list(s1) == list(s2) == list(DistributedSampler(10, 2, 0, shuffle=False))
    with pytest.raises(TypeError):
        DistributedSampler()
    job = JobConfig()
    job.model = cfg
    t = MetricsTracker(job, 4, 123.0)
    assert (t.num_gpus, t.peak_tflops, t.seq_len, t.model_config) == (4, 123.0, job.train.seq_len, cfg)
    t2 = MetricsTracker(job.metrics, cfg, 4, 64, 0, 123.0)
    assert (t2.num_gpus, t2.peak_tflops, t2.seq_len) == (4, 123.0, 64)
    assert MetricsTracker(job, num_gpus=2, gpu_peak_tflops=50.0).peak_tflops == 50.0


def test_freeze_and_eval_helpers_accept_explicit_lists_and_flags():
    from kempnerforge_b200.config.vlm import FreezeSpec, FreezeStage
    from kempnerforge_b200.training.eval import run_eval, should_build_eval_dataloader
    from kempnerforge_b200.training.freeze import effective_freeze

    base = [FreezeSpec("vision_encoder", True), FreezeSpec("adapter", False)]
    sched = [FreezeStage(start_step=10, specs=(FreezeSpec("vision_encoder", False),)),
             FreezeStage(start_step=5, specs=(FreezeSpec("adapter", True),))]
    at = lambda step: {s.module: s.frozen for s in effective_freeze(step, base, sched)}  # noqa: E731
    assert at(0) == {"vision_encoder": True, "adapter": False}
    assert at(7) == {"vision_encoder": True, "adapter": True}
    assert at(10) == {"vision_encoder": False, "adapter": True}
    with pytest.raises(ValueError):
        effective_freeze(0, base, sched, valid_modules={"adapter"})
    assert should_build_eval_dataloader(True, True) == (False, True)
    assert should_build_eval_dataloader(True, False) == (True, False)
    assert should_build_eval_dataloader(False, True) == (False, False)

    torch.manual_seed(0)
    model = nn.Sequential(nn.Embedding(16, 8), nn.Linear(8, 16))
    batches = [{"input_ids": torch.randint(0, 16, (2, 4)), "labels": torch.randint(0, 16, (2, 4))} for _ in range(2)]
    loss_fn = lambda logits, labels: nn.functional.cross_entropy(logits.flatten(0, 1), labels.flatten())  # noqa: E731
    out = run_eval(model, batches, loss_fn, torch.device("cpu"), 3)
    want = sum(float(loss_fn(model(b["input_ids"]), b["labels"])) for b in (batches[0], batches[1], batches[0])) / 3
    assert out["eval/loss"] == pytest.approx(want, rel=1e-5) and out["eval/perplexity"] > 1.0
    assert run_eval(model, batches, loss_fn, torch.device("cpu"), eval_steps=3) == out
    with pytest.raises(TypeError):
        run_eval(model, batches, loss_fn, torch.device("cpu"))


def test_pipeline_stage_spellings():
    from kempnerforge_b200.parallel.pipeline_parallel import PipelineStageModule, compute_layer_assignment

    cfg = ModelConfig(dim=32, n_layers=6, n_heads=4, n_kv_heads=2, vocab_size=64, ffn_hidden_dim=48, max_seq_len=16)
    a = PipelineStageModule(cfg, 1, 3)
    b = PipelineStageModule(cfg, stage_id=1, num_stages=3)
    assert list(a.layers.keys()) == list(b.layers.keys()) == [str(i) for i in range(*compute_layer_assignment(6, 3)[1])]
    c = PipelineStageModule(cfg, 0, 2, (0, 5))
    assert list(c.layers.keys()) == ["0", "1", "2", "3", "4"] and c.is_first and not c.is_last
    with pytest.raises(TypeError):
        PipelineStageModule(cfg)


def test_reference_module_paths_resolve_to_the_same_module_objects():
    """One import finder serves the reference's layout (kempnerforge/config/<section>.py, kempnerforge/model/*,
    kempnerforge/distributed/*): an alias is the target module itself, never a second execution of its file."""
    import importlib
    import sys

    from kempnerforge_b200 import _reference_paths as rp

    for alias, real in [("config.model", "config.sections"), ("config.optimizer", "config.sections"),
                        ("config.vision", "config.vlm"), ("config.schema", "config"), ("model", "models"),
                        ("model.moe", "models.moe"), ("distributed", "parallel"),
                        ("distributed.tensor_parallel", "parallel.tensor_parallel"), ("distributed.utils", "parallel")]:
        assert rp.resolve(f"kempnerforge_b200.{alias}") == f"kempnerforge_b200.{real}"
        assert importlib.import_module(f"kempnerforge_b200.{alias}") is importlib.import_module(f"kempnerforge_b200.{real}")
    assert rp.resolve("kempnerforge_b200.models.moe") is None and rp.resolve("torch.distributed") is None
    assert sum(isinstance(f, rp.ReferencePathFinder) for f in sys.meta_path) == 1
    rp.install()                                   # installing twice adds nothing
    assert sum(isinstance(f, rp.ReferencePathFinder) for f in sys.meta_path) == 1
    from kempnerforge_b200.config.schema import JobConfig, ModelConfig, MoMaConfig, SchedulerType  # noqa: F401
    from kempnerforge_b200.distributed import (apply_ac, apply_fsdp2, apply_tensor_parallel, build_pipeline_schedule,  # noqa: F401
                                               build_stage_module, clip_grad_norm_, default_mp_policy, get_dp_mesh,
                                               get_pp_rank, get_tp_mesh, is_rank_zero)
    from kempnerforge_b200.models.moe import MoEMLP

    assert sys.modules["kempnerforge_b200.model.moe"].MoEMLP is MoEMLP
    try:
        importlib.import_module("kempnerforge_b200.model.no_such_module")
    except ModuleNotFoundError:
        pass
    else:
        raise AssertionError("an alias of a missing module must not import")
