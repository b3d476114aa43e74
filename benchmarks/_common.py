"""Shared shapes for the micro-benchmarks: the 125 M-parameter model the reference benches
(benchmarks/bench_forward.py: dim 768, 12 layers, 12 heads, vocab 32000, batch 4 x seq 512),
shrunk automatically on a CPU so the suites stay runnable anywhere."""

from __future__ import annotations

import torch

from kempnerforge_b200.config import ModelConfig


def dtype_for(device: torch.device) -> torch.dtype:
    return torch.bfloat16 if device.type == "cuda" else torch.float32


def bench_model_config(device: torch.device, **over) -> ModelConfig:
    if device.type == "cuda":
        base = dict(dim=768, n_layers=12, n_heads=12, n_kv_heads=12, vocab_size=32000, max_seq_len=2048)
    else:
        base = dict(dim=128, n_layers=2, n_heads=4, n_kv_heads=4, vocab_size=1024, max_seq_len=512)
    base.update(over)
    return ModelConfig(**base)


def batch_shape(device: torch.device) -> tuple[int, int]:
    return (4, 512) if device.type == "cuda" else (2, 64)
