"""The non-tensor part of a checkpoint (``train_state.pt``): counters, RNG streams, scheduler and
data-loader positions, plus free-form extras (phase index, experiment-tracker run id, freeze metadata).

Parity: kempnerforge/checkpoint/state.py:21-119 (keys: step, tokens_seen, rng{python, numpy,
torch_cpu, torch_cuda}, scheduler, dataloader, extras merged at top level).
"""

from __future__ import annotations

import random
from typing import Any

import numpy as np
import torch


def get_rng_state() -> dict[str, Any]:
    state = {"python": random.getstate(), "numpy": np.random.get_state(), "torch_cpu": torch.get_rng_state()}
    if torch.cuda.is_available():
        state["torch_cuda"] = torch.cuda.get_rng_state()
    return state


def set_rng_state(state: dict[str, Any]) -> None:
    if "python" in state:
        random.setstate(state["python"])
    if "numpy" in state:
        np.random.set_state(state["numpy"])
    if "torch_cpu" in state:
        torch.set_rng_state(state["torch_cpu"].cpu() if torch.is_tensor(state["torch_cpu"]) else state["torch_cpu"])
    if "torch_cuda" in state and torch.cuda.is_available():
        torch.cuda.set_rng_state(state["torch_cuda"].cpu())


def build_train_state(step: int, tokens_seen: int, scheduler=None, dataloader=None, extra: dict | None = None) -> dict:
    state: dict[str, Any] = {"step": step, "tokens_seen": tokens_seen, "rng": get_rng_state()}
    if scheduler is not None:
        state["scheduler"] = scheduler.state_dict()
    if dataloader is not None and hasattr(dataloader, "state_dict"):
        state["dataloader"] = dataloader.state_dict()
    if extra:
        for k, v in extra.items():
            if k in state:
                raise ValueError(f"extra key {k!r} collides with a reserved train-state key")
            state[k] = v
    return state


_RESERVED = ("step", "tokens_seen", "rng", "scheduler", "dataloader")


def restore_train_state(state: dict, scheduler=None, dataloader=None) -> tuple[int, int, dict]:
    """Apply RNG / scheduler / data-loader state; returns (step, tokens_seen, extras)."""
    if "rng" in state:
        set_rng_state(state["rng"])
    if scheduler is not None and "scheduler" in state:
        scheduler.load_state_dict(state["scheduler"])
    if dataloader is not None and "dataloader" in state and hasattr(dataloader, "load_state_dict"):
        dataloader.load_state_dict(state["dataloader"])
    extra = {k: v for k, v in state.items() if k not in _RESERVED}
    return int(state.get("step", 0)), int(state.get("tokens_seen", 0)), extra
