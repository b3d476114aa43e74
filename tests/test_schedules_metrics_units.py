"""Learning-rate schedule shapes, modality-context rules, MFU arithmetic, metrics tracker and logging helpers.

Mirrors tests/unit/test_scheduler_extensions.py, test_modality_context.py, test_performance.py and
test_observability.py of the reference.
"""

from __future__ import annotations

import json
import logging
import math

import pytest
import torch

from kempnerforge_b200.config import load_config
from kempnerforge_b200.config.sections import MetricsConfig, ModelConfig, SchedulerConfig
from kempnerforge_b200.metrics import logger as kf_logger
from kempnerforge_b200.metrics.memory import DeviceMemoryMonitor, format_memory, get_memory_stats
from kempnerforge_b200.metrics.mfu import (active_params, compute_mfu, estimate_model_flops_per_token,
                                          get_gpu_peak_tflops)
from kempnerforge_b200.metrics.tracker import MetricsTracker
from kempnerforge_b200.models.modality import ModalityContext
from kempnerforge_b200.training.scheduler import build_scheduler, lr_factor_fn


def _f(name, max_steps=1000, **kw):
    return lr_factor_fn(SchedulerConfig(name=name, **kw), max_steps)


# --------------------------------------------------------------------------- schedules
@pytest.mark.parametrize("name", ["cosine", "linear", "wsd", "constant", "rex"])
def test_warmup_is_linear_from_zero(name):
    f = _f(name, warmup_steps=100)
    assert f(0) == 0.0 and f(50) == pytest.approx(0.5) and f(100) == pytest.approx(1.0)


def test_constant_is_flat_after_warmup_and_without_warmup():
    f = _f("constant", warmup_steps=10)
    assert f(10) == f(500) == f(999) == 1.0
    assert _f("constant", warmup_steps=0)(0) == 1.0


def test_cosine_and_linear_endpoints():
    c = _f("cosine", warmup_steps=100, min_lr_ratio=0.1)
    assert c(550) == pytest.approx(0.55) and c(1000) == pytest.approx(0.1) and c(5000) == pytest.approx(0.1)
    lin = _f("linear", warmup_steps=100, min_lr_ratio=0.0)
    assert lin(550) == pytest.approx(0.5) and lin(1000) == pytest.approx(0.0)


@pytest.mark.parametrize("shape", ["cosine", "linear", "sqrt"])
def test_wsd_phases(shape):
    f = _f("wsd", warmup_steps=100, stable_steps=400, min_lr_ratio=0.1, wsd_decay_type=shape)
    assert f(100) == f(300) == f(499) == 1.0           # stable
    assert f(500) == pytest.approx(1.0)                 # decay starts at the peak
    assert f(1000) == pytest.approx(0.1)                # and ends at the floor
    mid = f(750)
    want = {"cosine": 0.55, "linear": 0.55, "sqrt": 0.1 + 0.9 * math.sqrt(0.5)}[shape]
    assert mid == pytest.approx(want)


def test_wsd_sqrt_stays_above_linear_and_curves_differ():
    kw = dict(warmup_steps=0, stable_steps=0, min_lr_ratio=0.0)
    lin, sq, co = (_f("wsd", wsd_decay_type=s, **kw) for s in ("linear", "sqrt", "cosine"))
    for s in (100, 500, 900):
        assert sq(s) > lin(s)
    assert len({round(fn(300), 6) for fn in (lin, sq, co)}) == 3
    assert lin(0) == sq(0) == co(0) == 1.0 and lin(1000) == sq(1000) == pytest.approx(co(1000)) == 0.0


def test_invalid_schedule_options_are_rejected():
    with pytest.raises(ValueError):
        SchedulerConfig(wsd_decay_type="exp")
    with pytest.raises(ValueError):
        SchedulerConfig(rex_alpha=0.0)
    with pytest.raises(ValueError):
        SchedulerConfig(min_lr_ratio=1.5)
    with pytest.raises(ValueError):
        SchedulerConfig(warmup_steps=-1)


def test_rex_shapes():
    lin = _f("rex", warmup_steps=0, min_lr_ratio=0.0, rex_alpha=1.0)
    assert lin(250) == pytest.approx(0.75) and lin(1000) == 0.0
    convex = _f("rex", warmup_steps=0, min_lr_ratio=0.0, rex_alpha=2.0)
    high = _f("rex", warmup_steps=0, min_lr_ratio=0.0, rex_alpha=0.5)
    assert convex(500) == pytest.approx(0.25) and high(500) == pytest.approx(math.sqrt(0.5))
    floor = _f("rex", warmup_steps=0, min_lr_ratio=0.2, rex_alpha=1.0)
    assert floor(900) == pytest.approx(0.2) and floor(1000) == pytest.approx(0.2)


def test_scheduler_options_from_toml_and_cli(tmp_path):
    p = tmp_path / "s.toml"
    p.write_text('[scheduler]\nname = "wsd"\nwsd_decay_type = "sqrt"\nstable_steps = 5\n')
    cfg = load_config(str(p), ["--scheduler.rex_alpha=2.5"])
    assert str(cfg.scheduler.name) == "wsd" and cfg.scheduler.wsd_decay_type == "sqrt" and cfg.scheduler.rex_alpha == 2.5
    p.write_text('[scheduler]\nname = "rex"\n')
    assert str(load_config(str(p)).scheduler.name) == "rex"
    p.write_text('[scheduler]\nname = "constant"\n')
    assert str(load_config(str(p)).scheduler.name) == "constant"
    assert SchedulerConfig().wsd_decay_type == "cosine" and SchedulerConfig().rex_alpha == 1.0


def test_build_scheduler_drives_optimizer_lr():
    p = torch.nn.Parameter(torch.zeros(1))
    opt = torch.optim.SGD([p], lr=2.0)
    sched = build_scheduler(opt, SchedulerConfig(name="linear", warmup_steps=2, min_lr_ratio=0.0), 6)
    seen = []
    for _ in range(6):
        seen.append(opt.param_groups[0]["lr"])
        opt.step()
        sched.step()
    assert seen == pytest.approx([0.0, 1.0, 2.0, 1.5, 1.0, 0.5])


# --------------------------------------------------------------------------- modality context
def _t(*shape):
    return torch.zeros(*shape)


@pytest.mark.parametrize("kw", [
    {}, dict(output_slice=slice(1, None)), dict(inputs_embeds=_t(1, 2, 4)), dict(prefix_embeds=_t(1, 2, 4)),
    dict(image_features=_t(1, 2, 4)), dict(image_features=_t(1, 2, 4), image_mask=_t(1, 2)),
    dict(prefix_embeds=_t(1, 2, 4), key_padding_mask=_t(1, 6)), dict(prefix_embeds=_t(1, 2, 4), modality_ids=_t(1, 6)),
    dict(inputs_embeds=_t(1, 2, 4), modality_ids=_t(1, 2)),
])
def test_modality_context_accepts(kw):
    ModalityContext(**kw)


@pytest.mark.parametrize("kw", [
    dict(inputs_embeds=_t(1, 2, 4), prefix_embeds=_t(1, 2, 4)), dict(inputs_embeds=_t(1, 2, 4), image_features=_t(1, 2, 4)),
    dict(prefix_embeds=_t(1, 2, 4), image_features=_t(1, 2, 4)),
    dict(inputs_embeds=_t(1, 2, 4), prefix_embeds=_t(1, 2, 4), image_features=_t(1, 2, 4)),
    dict(image_mask=_t(1, 2)), dict(key_padding_mask=_t(1, 2)), dict(modality_ids=_t(1, 2)),
    dict(modality_ids=_t(1, 2), output_slice=slice(0, 1)), dict(image_features=_t(1, 2, 4), key_padding_mask=_t(1, 2)),
])
def test_modality_context_rejects(kw):
    with pytest.raises(ValueError):
        ModalityContext(**kw)


def test_modality_context_is_frozen():
    ctx = ModalityContext()
    with pytest.raises(Exception):
        ctx.output_slice = slice(0, 1)


# --------------------------------------------------------------------------- MFU arithmetic
def _dense(**kw):
    base = dict(dim=256, n_layers=4, n_heads=8, n_kv_heads=4, vocab_size=1000, ffn_hidden_dim=512, max_seq_len=128)
    base.update(kw)
    return ModelConfig(**base)


def test_flops_per_token_formula_and_scaling():
    c = _dense()
    want = 6.0 * active_params(c) + 12.0 * c.n_layers * c.dim * 128
    assert estimate_model_flops_per_token(c, 128) == want > 0
    assert estimate_model_flops_per_token(_dense(n_layers=8), 128) > want
    assert estimate_model_flops_per_token(c, 256) - want == 12.0 * c.n_layers * c.dim * 128


def test_llama_7b_flops_are_about_six_times_its_parameters():
    c = ModelConfig(dim=4096, n_layers=32, n_heads=32, n_kv_heads=32, vocab_size=32000, ffn_hidden_dim=11008,
                    max_seq_len=4096)
    f = estimate_model_flops_per_token(c, 4096)
    assert 6.0 * 6.5e9 < f < 6.0 * 6.5e9 + 12.0 * 32 * 4096 * 4096 + 1e9


def test_compute_mfu_arithmetic():
    c = _dense()
    per_tok = estimate_model_flops_per_token(c, 128)
    assert compute_mfu(c, 0.0, 1, seq_len=128, peak_tflops=100.0) == 0.0
    one = compute_mfu(c, 1e6, 1, seq_len=128, peak_tflops=100.0)
    assert one == pytest.approx(per_tok * 1e6 / 100e12)
    assert compute_mfu(c, 1e6, 4, seq_len=128, peak_tflops=100.0) == pytest.approx(one / 4)
    assert compute_mfu(c, 1e6, 1, seq_len=128, peak_tflops=200.0) == pytest.approx(one / 2)


def test_moe_counts_active_parameters_only():
    dense = _dense()
    moe2 = _dense(num_experts=8, moe_top_k=2)
    moe4 = _dense(num_experts=8, moe_top_k=4)
    more_experts = _dense(num_experts=16, moe_top_k=2)
    assert active_params(moe4) > active_params(moe2) > active_params(dense)
    # doubling the number of experts does not change the per-token work (the router GEMM is not counted)
    assert active_params(more_experts) == active_params(moe2)
    shared = _dense(num_experts=8, moe_top_k=2, moe_shared_experts=1)
    assert active_params(shared) > active_params(moe2)
    sparse = _dense(num_experts=8, moe_top_k=2, moe_frequency=2)
    assert active_params(dense) < active_params(sparse) < active_params(moe2)


def test_peak_lookup_prefers_a_measurement_file(tmp_path, monkeypatch):
    p = tmp_path / "peaks.json"
    p.write_text(json.dumps({"bf16_tflops": 1234.5}))
    assert get_gpu_peak_tflops(measured_peaks_path=str(p)) == 1234.5
    monkeypatch.setenv("KF_MEASURED_PEAKS", str(p))
    assert get_gpu_peak_tflops() == 1234.5
    p.write_text("not json")
    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert get_gpu_peak_tflops() == 1.0


@pytest.mark.parametrize("name,cap,expect_key", [("NVIDIA B200", (10, 0), "B200"), ("NVIDIA H100 80GB HBM3", (9, 0), "H100"),
                                                 ("Mystery Blackwell", (10, 0), "B200"), ("Mystery Hopper", (9, 0), "H100"),
                                                 ("Mystery Ampere", (8, 0), "A100"), ("Old Card", (7, 0), None)])
def test_peak_lookup_by_name_then_capability(monkeypatch, name, cap, expect_key):
    from kempnerforge_b200.metrics import mfu

    monkeypatch.delenv("KF_MEASURED_PEAKS", raising=False)
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "current_device", lambda: 0)
    monkeypatch.setattr(torch.cuda, "get_device_name", lambda d=None: name)
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda d=None: cap)
    want = mfu.GPU_PEAK_TFLOPS[expect_key] if expect_key else 100.0
    assert get_gpu_peak_tflops() == want


# --------------------------------------------------------------------------- memory helpers
def test_memory_stats_on_cpu():
    stats = get_memory_stats()
    assert {"peak_gb", "total_gb"} <= set(stats) and all(v >= 0 for v in stats.values())
    assert isinstance(format_memory(stats), str)
    mon = DeviceMemoryMonitor()
    mon.reset_peak()
    assert set(mon.stats()) == set(stats)
    mon.start_recording()
    assert mon.capture_snapshot("t") is None or isinstance(mon.capture_snapshot("t"), str)
    mon.stop_recording()


# --------------------------------------------------------------------------- tracker
class _Backend:
    def __init__(self):
        self.logged, self.closed = [], False

    def log(self, metrics, step):
        self.logged.append((step, dict(metrics)))

    def close(self):
        self.closed = True


def _tracker(**kw):
    cfg = MetricsConfig(log_interval=5)
    return MetricsTracker(cfg, model_config=kw.pop("model_config", None), peak_tflops=100.0, **kw)


def test_tracker_logs_on_interval_and_on_step_one():
    tr = _tracker()
    out = {}
    for step in range(1, 12):
        tr.start_step()
        out[step] = tr.end_step(step, loss=2.0, grad_norm=1.0, lr=1e-3, tokens_in_step=1000)
    assert [s for s, m in out.items() if m is not None] == [1, 5, 10]
    m = out[5]
    assert m.step == 5 and m.loss == 2.0 and m.grad_norm == 1.0 and m.lr == 1e-3 and m.tokens_per_sec > 0 and m.mfu == 0.0


def test_tracker_mfu_and_smoothing():
    tr = _tracker(model_config=_dense(), seq_len=128)
    tr.start_step()
    m1 = tr.end_step(1, 4.0, 1.0, 1e-3, 1000)
    assert m1.mfu > 0 and m1.smoothed_loss == 4.0
    for step in range(2, 6):
        tr.start_step()
        m = tr.end_step(step, 2.0, 1.0, 1e-3, 1000)
    assert 2.0 < m.smoothed_loss < 4.0


def test_tracker_dispatches_to_backends_and_closes():
    tr = _tracker()
    be = _Backend()
    tr.backends.append(be)
    tr.start_step()
    tr.end_step(1, 2.0, 1.0, 1e-3, 100, extra={"aux": 0.5, "note": "text"})
    step, payload = be.logged[0]
    assert step == 1 and payload["train/loss"] == 2.0 and payload["aux"] == 0.5 and "note" not in payload
    tr.log_eval({"eval/loss": 1.5}, 1)
    tr.log_extra({"x": 1.0}, 1)
    assert be.logged[1] == (1, {"eval/loss": 1.5}) and be.logged[2] == (1, {"x": 1.0})
    tr.close()
    assert be.closed and tr.backends == []
    tr.close()  # idempotent


def test_tracker_backends_only_on_rank_zero_and_survive_missing_packages(tmp_path, monkeypatch):
    cfg = MetricsConfig(enable_wandb=True, enable_tensorboard=True, tensorboard_dir=str(tmp_path / "tb"))
    other = MetricsTracker(cfg, rank=1, peak_tflops=1.0)
    other.init_backends()
    assert other.backends == []
    import builtins

    real_import = builtins.__import__

    def fake_import(name, *a, **k):
        if name.startswith("wandb") or name.startswith("torch.utils.tensorboard") or name.startswith("tensorboard"):
            raise ImportError(name)
        return real_import(name, *a, **k)

    monkeypatch.setattr(builtins, "__import__", fake_import)
    zero = MetricsTracker(cfg, rank=0, peak_tflops=1.0)
    zero.init_backends()   # both optional packages missing: warns, does not raise
    assert zero.backends == []
    zero.close()


# --------------------------------------------------------------------------- logging helpers
def test_rank_filter_and_formatter(monkeypatch):
    rec = logging.LogRecord("kempnerforge_b200.x", logging.INFO, __file__, 1, "hello %s", ("world",), None)
    err = logging.LogRecord("kempnerforge_b200.x", logging.ERROR, __file__, 1, "bad", (), None)
    monkeypatch.setenv("RANK", "0")
    assert kf_logger.RankFilter().filter(rec)
    monkeypatch.setenv("RANK", "3")
    assert not kf_logger.RankFilter().filter(rec) and kf_logger.RankFilter(all_ranks=True).filter(rec)
    assert kf_logger.RankFilter().filter(err)  # errors are shown from every rank
    plain = kf_logger.RankFormatter(use_color=False).format(rec)
    assert "[rank 3]" in plain and "hello world" in plain and "\x1b[" not in plain
    monkeypatch.setattr(kf_logger, "_supports_color", lambda: True)      # an interactive terminal
    assert "\x1b[" in kf_logger.RankFormatter(use_color=True).format(rec)
    monkeypatch.undo()
    monkeypatch.setenv("NO_COLOR", "1")
    assert kf_logger.RankFormatter().use_color is False and kf_logger.RankFormatter(use_color=True).use_color is False
    monkeypatch.setenv("RANK", "3")
    assert kf_logger.RankFilter(rank=3).filter(rec) and not kf_logger.RankFilter(rank=1).filter(rec)


def test_get_logger_namespaces_and_format_metrics():
    lg = kf_logger.get_logger("mymodule")
    assert lg.name == "kempnerforge_b200.mymodule" and kf_logger.get_logger().name == "kempnerforge_b200"
    line = kf_logger.format_metrics(12, {"loss": 2.34567, "lr": 3e-4, "grad_norm": 0.8123, "tok/s": 12345.6, "mfu": 41.23,
                                         "mem": "10.1/180GB", "step_time": 0.531, "count": 7, "ratio": 0.125, "tag": "x"})
    assert line.startswith("[step 12]")
    for piece in ("loss=2.3457", "lr=3.00e-04", "grad_norm=0.812", "tok/s=12,346", "mfu=41.2%", "mem=10.1/180GB",
                  "step_time=0.53s", "count=7", "tag=x"):
        assert piece in line, piece


# --------------------------------------------------------------------------- region timers / interval memory reports
def test_timer_collection_region_calls_and_disabled_mode():
    from kempnerforge_b200.profiling.cuda_timer import CUDATimerCollection

    timers = CUDATimerCollection(["forward", "backward", "never"], enabled=True)
    timers.start("forward")
    sum(range(1000))
    timers.stop("forward")
    timers.start("backward")
    timers.stop("backward")
    all_ms = timers.elapsed_all()
    assert list(all_ms) == ["forward", "backward", "never"] and all_ms["never"] == 0.0
    assert all_ms["forward"] >= 0.0 and timers.elapsed_ms("forward") == all_ms["forward"]
    with timers.timer("extra"):
        pass
    assert "extra" in timers.elapsed_all() and timers.summary()["forward"]["count"] == 1
    off = CUDATimerCollection(["forward"], enabled=False)
    off.start("forward")
    off.stop("forward")
    assert off.elapsed_ms("forward") == 0.0 and off.elapsed_all() == {"forward": 0.0} and not off.enabled
    assert CUDATimerCollection(False).enabled is False and CUDATimerCollection().enabled is True


def test_memory_monitor_interval_report_without_a_gpu(caplog):
    import logging

    from kempnerforge_b200.metrics.memory import (DeviceMemoryMonitor, format_memory_stats, get_memory_utilization,
                                                  reset_peak_memory)

    assert get_memory_utilization() == 0.0 or 0.0 < get_memory_utilization() <= 1.0
    text = format_memory_stats()
    assert text.startswith("GPU mem: ") and "GB total (" in text
    reset_peak_memory()
    mon = DeviceMemoryMonitor(snapshot_step=3, snapshot_dir="unused_dir")
    with caplog.at_level(logging.INFO):
        stats = mon.report(3)
    assert {"allocated_gb", "peak_gb", "reserved_gb", "total_gb", "mem_utilization"} <= set(stats)
    assert "[step 3] GPU mem:" in caplog.text and mon._snapshot_taken
    assert DeviceMemoryMonitor(None, "somewhere").snapshot_dir == "somewhere"


# --------------------------------------------------------------------------- record fields, back-end keys, lazy back-ends
def test_step_record_and_backend_keys_are_the_reference_ones():
    """Dashboards and scripts written against kempnerforge/metrics/tracker.py read these names."""
    tr = _tracker(model_config=_dense(), seq_len=128)
    be = _Backend()
    tr.backends.append(be)
    tr.start_step()
    m = tr.end_step(1, 3.0, 0.5, 1e-3, 1000)
    for field in ("loss", "grad_norm", "lr", "tokens_per_sec", "mfu", "step_time_sec", "allocated_gb", "peak_gb",
                  "reserved_gb", "total_gb", "mem_utilization"):
        assert hasattr(m, field), field
    assert m.step_time == m.step_time_sec and m.peak_memory_gb == m.peak_gb and m.total_memory_gb == m.total_gb
    assert type(m)() .loss == 0.0                                      # every field has a default
    _, payload = be.logged[0]
    assert {"train/loss", "train/grad_norm", "train/lr", "train/tokens_per_sec", "train/mfu", "train/step_time_sec",
            "gpu/allocated_gb", "gpu/peak_gb", "gpu/reserved_gb", "gpu/mem_utilization", "smoothed/loss",
            "smoothed/tokens_per_sec", "smoothed/mfu", "smoothed/step_time"} <= payload.keys()
    assert payload["smoothed/loss"] == 3.0 and tr._smoothed["loss"] == 3.0


def test_backends_start_lazily_and_a_failed_start_only_disables_them(monkeypatch, tmp_path):
    import sys
    import types

    from kempnerforge_b200.metrics.tracker import TensorBoardBackend, WandBBackend

    cfg = MetricsConfig(enable_wandb=True, wandb_project="p", wandb_run_name="r")
    calls = []
    fake = types.ModuleType("wandb")
    fake.init = lambda **kw: calls.append(kw) or types.SimpleNamespace(id="abc123", url="http://x")
    fake.log = lambda metrics, step: calls.append(("log", step, dict(metrics)))
    fake.finish = lambda: calls.append("finish")
    monkeypatch.setitem(sys.modules, "wandb", fake)
    be = WandBBackend(cfg)
    assert calls == [] and be.active                                   # nothing happens at construction
    be.log({"train/loss": 1.0}, step=3)
    assert calls[0]["project"] == "p" and calls[0]["resume"] == "allow" and "id" not in calls[0]
    assert calls[1] == ("log", 3, {"train/loss": 1.0}) and cfg.wandb_run_id == "abc123" and be.run_id == "abc123"
    be.close()
    assert calls[-1] == "finish"
    resumed = WandBBackend(cfg)                                        # the stored id resumes the same run
    resumed._ensure_init()
    assert calls[-1]["id"] == "abc123"

    def boom(**kw):
        raise RuntimeError("no API key")

    fake.init = boom
    bad = WandBBackend(MetricsConfig(enable_wandb=True))
    bad.log({"x": 1.0}, step=1)                                        # warns, does not raise
    assert not bad.active
    bad.close()

    tb = TensorBoardBackend(MetricsConfig(tensorboard_dir=str(tmp_path / "tb")))
    assert tb._writer is None and not (tmp_path / "tb").exists()
    monkeypatch.setitem(sys.modules, "torch.utils.tensorboard", None)  # the import fails
    tb.log({"a": 1.0}, step=1)
    assert tb._writer is False and not tb.active
    tb.close()


def test_init_backends_runs_once(monkeypatch):
    from kempnerforge_b200.metrics import tracker as tracker_mod

    made = []

    class FakeTB(_Backend):
        def __init__(self, cfg):
            super().__init__()
            made.append(self)

        def _ensure_init(self):
            pass

    monkeypatch.setattr(tracker_mod, "TensorBoardBackend", FakeTB)
    tr = MetricsTracker(MetricsConfig(enable_tensorboard=True), rank=0, peak_tflops=1.0)
    tr.init_backends()
    tr.init_backends()
    assert len(made) == 1 and tr.backends == made


def test_memory_snapshot_never_raises(monkeypatch, tmp_path):
    from kempnerforge_b200.metrics.memory import DeviceMemoryMonitor

    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    assert DeviceMemoryMonitor(snapshot_dir=str(tmp_path)).capture_snapshot(step=10) is None
    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)

    def boom(*a, **k):
        raise RuntimeError("allocator history unavailable")

    monkeypatch.setattr(torch.cuda.memory, "_record_memory_history", boom)
    assert DeviceMemoryMonitor(device=0, snapshot_dir=str(tmp_path)).capture_snapshot(step=1) is None
