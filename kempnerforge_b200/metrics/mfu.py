"""Model-FLOPs utilisation.

FLOPs per token = 6 * P_active + 12 * L * D * S, where P_active excludes the token embedding
(a lookup) but includes the output head, and for MoE layers counts only the routed top-k experts
plus the shared expert that actually runs.  The peak is looked up by GPU name; Blackwell parts are
listed with their dense (non-sparse) bf16 rates, and a measured peak can be supplied instead.

Parity: kempnerforge/metrics/mfu.py:25-180 (formula and public functions).  Difference: the
reference has no Blackwell entry and would fall back to the Hopper number on a B200.
"""

from __future__ import annotations

import json
import os

import torch

# dense bf16 tensor-core TFLOP/s
GPU_PEAK_TFLOPS: dict[str, float] = {
    "B200": 2250.0,
    "GB200": 2500.0,
    "B100": 1800.0,
    "H200": 989.0,
    "H100 PCIe": 756.0,
    "H100": 989.0,
    "A100": 312.0,
    "L40S": 362.0,
    "A10G": 125.0,
    "RTX 4090": 330.0,
    "RTX 3090": 142.0,
}
_GPU_PEAK_TFLOPS = GPU_PEAK_TFLOPS


def get_gpu_peak_tflops(device: int | None = None, measured_peaks_path: str | None = None) -> float:
    """Peak bf16 TFLOP/s: an explicit measurement file wins, then the name table, then a capability guess."""
    path = measured_peaks_path or os.environ.get("KF_MEASURED_PEAKS")
    if path and os.path.exists(path):
        try:
            with open(path) as fh:
                return float(json.load(fh)["bf16_tflops"])
        except (OSError, KeyError, ValueError):
            pass
    if not torch.cuda.is_available():
        return 1.0
    if device is None:
        try:
            device = torch.cuda.current_device()
        except Exception:  # noqa: BLE001  no usable context yet
            device = 0
    name = torch.cuda.get_device_name(device)
    for key in sorted(GPU_PEAK_TFLOPS, key=len, reverse=True):
        if key.lower() in name.lower():
            return GPU_PEAK_TFLOPS[key]
    major, _ = torch.cuda.get_device_capability(device)
    if major >= 10:
        return GPU_PEAK_TFLOPS["B200"]
    if major >= 9:
        return GPU_PEAK_TFLOPS["H100"]
    if major >= 8:
        return GPU_PEAK_TFLOPS["A100"]
    return 100.0


def active_params(model_config) -> int:
    """Parameters that take part in one token's forward pass, without the embedding table."""
    c = model_config
    d, hd = c.dim, c.head_dim
    attn = 2 * d * c.n_heads * hd + 2 * d * c.n_kv_heads * hd
    total = 0
    for i in range(c.n_layers):
        if c.is_moe_layer(i):
            he = c.computed_expert_ffn_hidden_dim
            shared = 0
            if c.moe_shared_experts > 0:  # one shared MLP runs (optionally widened)
                shared = 3 * d * he * (c.moe_shared_experts if c.moe_shared_expert_widen else 1)
            total += attn + c.moe_top_k * 3 * d * he + shared  # the router GEMM is left out, as in the reference's formula
        else:
            total += attn + 3 * d * c.computed_ffn_hidden_dim
    return total + c.vocab_size * d  # output head


def estimate_model_flops_per_token(config, seq_len: int | None = None) -> float:
    seq_len = config.max_seq_len if seq_len is None else seq_len
    return 6.0 * active_params(config) + 12.0 * config.n_layers * config.dim * seq_len


def compute_mfu(config, tokens_per_sec: float, num_gpus: int = 1, gpu_peak_tflops: float | None = None,
                seq_len: int | None = None, *, peak_tflops: float | None = None) -> float:
    """Utilisation in [0, 1] of ``num_gpus`` GPUs at ``tokens_per_sec`` (whole job).  ``gpu_peak_tflops`` (also
    spelled ``peak_tflops``) is per GPU and detected when omitted; ``seq_len`` defaults to the model's maximum.
    Parity: kempnerforge/metrics/mfu.py:150-180."""
    peak = gpu_peak_tflops if gpu_peak_tflops is not None else peak_tflops
    if peak is None:
        peak = get_gpu_peak_tflops()
    if not peak or not num_gpus:
        return 0.0
    seq = seq_len if seq_len is not None else config.max_seq_len
    return estimate_model_flops_per_token(config, seq) * tokens_per_sec / (peak * 1e12 * num_gpus)
