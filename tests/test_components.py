"""Smaller components on CPU: activation extraction, sampling, MFU / memory / timers / profiler helpers, the MoMa
architecture, adapters' token counts, checkpoint conversion."""

import json
import os

import numpy as np
import pytest
import torch

from kempnerforge_b200.config import ModelConfig, config_from_dict


def _tiny_model(**over):
    from kempnerforge_b200.models.transformer import Transformer

    cfg = ModelConfig(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=128, max_seq_len=32, **over)
    torch.manual_seed(0)
    return Transformer(cfg), cfg


# ------------------------------------------------------------------ activation hooks
def test_activation_store_and_extract_representations(tmp_path):
    from kempnerforge_b200.models.hooks import ActivationStore, extract_representations, save_activations

    model, cfg = _tiny_model()
    tokens = torch.randint(0, 128, (3, 16))
    names = ["layers.0.attention", "layers.1.mlp", "norm"]
    with ActivationStore(model, names, keep_history=True) as store:
        model(tokens)
        model(tokens)
        got = store.get("layers.1.mlp")
        assert got.shape == (3, 16, 64) and got.device.type == "cpu"       # the latest pass
        assert len(store.history("norm")) == 2 and store.history("norm")[0].shape == (3, 16, 64)
    kept = store.get("norm").clone()
    model(torch.randint(0, 128, (3, 16)))  # hooks are gone: nothing new is recorded
    assert torch.equal(store.get("norm"), kept)
    with pytest.raises(KeyError):
        ActivationStore(model, ["layers.9.mlp"]).enable()
    reps = extract_representations(model, [{"input_ids": tokens}, tokens[:1]], names, pool="mean")
    assert reps["norm"].shape == (4, 64) and model.training
    last = extract_representations(model, [tokens], ["norm"], pool="last")["norm"]
    assert last.shape == (3, 64)
    path = str(tmp_path / "acts.npz")
    save_activations(reps, path)
    loaded = np.load(path)
    assert set(loaded.files) == {"layers.0.attention", "layers.1.mlp", "norm"}


# ------------------------------------------------------------------ sampling
def test_sample_temperature_top_k_top_p():
    from kempnerforge_b200.models.generate import sample

    logits = torch.tensor([[0.0, 5.0, 1.0, 4.0], [3.0, 0.0, 0.0, 0.0]])
    assert sample(logits, temperature=0.0).squeeze(-1).tolist() == [1, 0]
    g = torch.Generator().manual_seed(0)
    picks = torch.stack([sample(logits, temperature=1.0, top_k=2, generator=g) for _ in range(200)], dim=1)
    assert set(picks[0].tolist()) <= {1, 3} and set(picks[1].tolist()) <= {0, 1, 2, 3}
    nucleus = torch.stack([sample(logits, temperature=1.0, top_p=0.5, generator=g) for _ in range(200)], dim=1)
    assert set(nucleus[0].tolist()) == {1}       # the top token alone carries > 0.5 of the mass
    assert set(nucleus[1].tolist()) == {0}


# ------------------------------------------------------------------ metrics / profiling helpers
def test_mfu_formula_and_moe_active_parameters(tmp_path):
    from kempnerforge_b200.metrics.mfu import active_params, compute_mfu, estimate_model_flops_per_token, get_gpu_peak_tflops

    dense = ModelConfig(dim=256, n_layers=4, n_heads=8, n_kv_heads=8, vocab_size=1000, max_seq_len=128)
    flops = estimate_model_flops_per_token(dense, 128)
    assert flops == pytest.approx(6 * active_params(dense) + 12 * 4 * 256 * 128)
    assert compute_mfu(dense, tokens_per_sec=1e6, num_gpus=2, seq_len=128, peak_tflops=100.0) == pytest.approx(
        flops * 1e6 / (2 * 100e12))
    moe = ModelConfig(dim=256, n_layers=4, n_heads=8, n_kv_heads=8, vocab_size=1000, max_seq_len=128, num_experts=8,
                      moe_top_k=2)
    assert active_params(moe) < moe.num_params_estimate       # only top-k of the experts count
    peaks = tmp_path / "peaks.json"
    peaks.write_text(json.dumps({"bf16_tflops": 1234.0}))
    assert get_gpu_peak_tflops(measured_peaks_path=str(peaks)) == 1234.0


def test_memory_stats_timers_and_kernel_buckets():
    from kempnerforge_b200.metrics.memory import DeviceMemoryMonitor, format_memory, get_memory_stats
    from kempnerforge_b200.profiling.cuda_timer import CUDATimerCollection
    from kempnerforge_b200.profiling.profiler import build_profiler, categorize_kernel

    stats = get_memory_stats()
    assert {"peak_gb", "total_gb"} <= set(stats) and "GB" in format_memory(stats)
    mon = DeviceMemoryMonitor()
    mon.reset_peak()
    assert isinstance(mon.stats(), dict) and mon.capture_snapshot("x") is None   # no GPU: nothing to record
    timers = CUDATimerCollection(enabled=True)
    for _ in range(3):
        with timers.timer("step"):
            torch.ones(1000).sum()
    summary = timers.summary()
    assert summary["step"]["count"] == 3 and summary["step"]["mean_ms"] >= 0
    timers.reset()
    assert timers.summary() == {}
    assert categorize_kernel("kf2::kf_gemm_bf16_tcgen05_2cta<false, true>") == "matmul"
    assert categorize_kernel("ncclDevKernel_ReduceScatter_Sum_bf16_RING_LL") == "comm"
    assert categorize_kernel("kf::kf_symm_rs_norm_bf16") == "fused_comm"
    assert categorize_kernel("kf::rs::kf_gemm_rs_tcgen05") == "fused_comm"
    assert categorize_kernel("kf_attn_fwd_tcgen05") == "attention"
    cfg = config_from_dict({"profiling": {"enable": False}})
    assert build_profiler(cfg.profiling) is None


# ------------------------------------------------------------------ MoMa architecture and adapters
def test_moma_wrapper_trains_on_cpu():
    from kempnerforge_b200.models.vlm import build_vlm_wrapper

    cfg = config_from_dict({
        "model": dict(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=128, ffn_hidden_dim=128, max_seq_len=64),
        "train": dict(batch_size=2, seq_len=16, mixed_precision="fp32"),
        "vision_encoder": dict(type="random", feature_dim=32, num_tokens=4),
        "vlm": dict(arch="moma", max_text_len=12),
    })
    torch.manual_seed(0)
    model = build_vlm_wrapper(cfg.model, cfg.vision_encoder, cfg.adapter, cfg.vlm)
    pixels = torch.randn(2, 3, 8, 8)
    ids = torch.randint(0, 128, (2, 12))
    loss = model.compute_loss(pixels, ids, ids.clone())
    loss.backward()
    assert torch.isfinite(loss) and loss.item() > 0
    counts = model.transformer.get_moma_expert_counts()
    assert counts and all(set(v) <= {"text", "image"} for v in counts.values())
    trained = [n for n, p in model.named_parameters() if p.grad is not None and p.grad.abs().sum() > 0]
    assert any("adapter" in n for n in trained) and any("layers.0" in n for n in trained)


def test_adapter_output_token_counts():
    from kempnerforge_b200.config.vlm import AdapterConfig

    assert AdapterConfig(type="mlp_2layer").output_num_tokens(196) == 196
    assert AdapterConfig(type="avgpool", pool_window=2).output_num_tokens(196) == 49       # 14x14 grid -> 7x7
    assert AdapterConfig(type="avgpool", pool_window=4).output_num_tokens(196) == 16       # ragged edge: ceil(14/4)^2
    assert AdapterConfig(type="attentional_pool", pool_window=2).output_num_tokens(196) == 49


# ------------------------------------------------------------------ checkpoint conversion
def test_convert_checkpoint_round_trip(tmp_path):
    import importlib.util

    from kempnerforge_b200.checkpoint import CheckpointManager
    from kempnerforge_b200.training.trainer import Trainer

    spec = importlib.util.spec_from_file_location(
        "convert_checkpoint", os.path.join(os.path.dirname(os.path.dirname(__file__)), "scripts", "convert_checkpoint.py"))
    conv = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(conv)
    assert conv.hf_to_kf_key(conv.kf_to_hf_key("layers.3.attention.q_proj.weight")) == "layers.3.attention.q_proj.weight"
    cfg = config_from_dict({
        "model": dict(dim=64, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=128, max_seq_len=32),
        "train": dict(batch_size=2, seq_len=16, mixed_precision="fp32", max_steps=2),
        "checkpoint": dict(dir=str(tmp_path / "ckpt")),
    })
    t = Trainer(cfg, init_dist=False)
    mgr = CheckpointManager(cfg.checkpoint, t.model, t.optimizer)
    step_dir = mgr.save(1, tokens_seen=32, scheduler=t.scheduler)
    mgr.wait()
    hf_dir, back_dir = str(tmp_path / "hf"), str(tmp_path / "back")
    conv.dcp_to_hf(str(step_dir), hf_dir, cfg.model, dtype="float32")
    hf_cfg = json.load(open(os.path.join(hf_dir, "config.json")))
    assert hf_cfg["hidden_size"] == 64 and hf_cfg["num_key_value_heads"] == 2
    conv.hf_to_dcp(hf_dir, back_dir, cfg.model)
    want = {n: p.detach().clone() for n, p in t.model.named_parameters()}
    for p in t.model.parameters():
        torch.nn.init.zeros_(p)
    CheckpointManager(cfg.checkpoint, t.model, t.optimizer).load(path=back_dir, exclude_keys=["optimizer"])
    for n, p in t.model.named_parameters():
        assert torch.allclose(p, want[n]), n


def test_profile_analysis_counts_each_kernel_once_and_writes_a_summary(tmp_path):
    """Self times are summed (inclusive times would count a kernel under every caller), every bucket is present
    (attention kernels included), and the reference's flat keys are filled (kempnerforge/profiling/profiler.py:71-127)."""
    from types import SimpleNamespace

    from kempnerforge_b200.profiling.profiler import analyze_profiler, print_profiler_summary, save_profiler_summary

    def evt(key, self_us, flops=0, count=1):
        return SimpleNamespace(key=key, self_device_time_total=self_us, device_time_total=10 * self_us, flops=flops, count=count)

    events = [evt("ProfilerStep#3", 99999), evt("kf::kf_gemm_bf16_tcgen05_2cta", 5000, int(1e12), 8),
              evt("kf_attn_fwd_tcgen05", 1000), evt("ncclDevKernel_AllReduce", 1500), evt("kf::kf_gemm_rs_tcgen05", 500),
              evt("Memcpy DtoD", 250), evt("elementwise_kernel", 750), evt("aten::linear", 0)]
    prof = SimpleNamespace(key_averages=lambda: events)
    st = analyze_profiler(prof)
    assert st["total_cuda_time_us"] == 9000 and st["totals_us"]["attention"] == 1000
    assert st["matmul_time_us"] == 6000 and st["comm_time_us"] == 2000 and st["memory_time_us"] == 250 and st["other_time_us"] == 750
    assert abs(st["matmul_pct"] + st["comm_pct"] + st["memory_pct"] + st["other_pct"] - 100.0) < 1e-9
    assert st["total_flops"] == int(1e12) and abs(st["achieved_tflops"] - 1e12 / 9e-3 / 1e12) < 1e-9
    assert st["top_kernels"][0][0] == "kf::kf_gemm_bf16_tcgen05_2cta" and st["peak_tflops"] > 0
    path = save_profiler_summary(st, prof, str(tmp_path / "t"))
    text = open(path).read()
    assert "attention" in text and "kf_gemm_bf16_tcgen05_2cta" in text and "TFLOP/s" in text
    assert analyze_profiler(SimpleNamespace(key_averages=lambda: []))["total_cuda_time_us"] == 0
    # a real (CPU-only) profile goes through without device events
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU]) as real:
        torch.ones(64, 64) @ torch.ones(64, 64)
    out = print_profiler_summary(real, str(tmp_path / "real"))
    assert out["total_cuda_time_us"] == 0 and (tmp_path / "real" / "summary.md").exists()
