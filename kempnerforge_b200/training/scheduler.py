"""Learning-rate schedules as multiplicative factors of the base LR (``LambdaLR``).

All schedules ramp linearly over ``warmup_steps`` first (factor step/warmup, so the very
first optimizer step runs with LR 0, like the reference).  After warm-up, with
s = step - warmup, D = decay length and m = min_lr_ratio:
  cosine   m + (1-m)/2 * (1 + cos(pi * min(1, s/D)))
  linear   1 - (1-m) * min(1, s/D)
  wsd      1.0 for ``stable_steps`` (default 0), then a cosine / linear / sqrt cool-down to m
  constant 1.0
  rex      max(m, (1 - s/D)^alpha)
  none     1.0 from step 0 (for schedule-free optimizers)

Parity: kempnerforge/training/scheduler.py:24-184.
"""

from __future__ import annotations

import math
from collections.abc import Callable

import torch
from torch.optim.lr_scheduler import LambdaLR

from kempnerforge_b200.config.registry import registry
from kempnerforge_b200.config.sections import SchedulerConfig


def _with_warmup(warmup: int, after: Callable[[int], float]) -> Callable[[int], float]:
    def factor(step: int) -> float:
        if warmup > 0 and step < warmup:
            return step / warmup
        return after(step - warmup)

    return factor


def _decay_len(cfg: SchedulerConfig, max_steps: int, used: int) -> int:
    return max(1, cfg.decay_steps if cfg.decay_steps is not None else max_steps - used)


def _cosine(cfg: SchedulerConfig, max_steps: int):
    d, m = _decay_len(cfg, max_steps, cfg.warmup_steps), cfg.min_lr_ratio
    return _with_warmup(cfg.warmup_steps, lambda s: m + 0.5 * (1 - m) * (1 + math.cos(math.pi * min(1.0, s / d))))


def _linear(cfg: SchedulerConfig, max_steps: int):
    d, m = _decay_len(cfg, max_steps, cfg.warmup_steps), cfg.min_lr_ratio
    return _with_warmup(cfg.warmup_steps, lambda s: 1.0 - (1 - m) * min(1.0, s / d))


def _wsd(cfg: SchedulerConfig, max_steps: int):
    m = cfg.min_lr_ratio
    stable = cfg.stable_steps or 0
    d = _decay_len(cfg, max_steps, cfg.warmup_steps + stable)
    shape = cfg.wsd_decay_type

    def after(s: int) -> float:
        if s < stable:
            return 1.0
        p = min(1.0, (s - stable) / d)
        if shape == "linear":
            return 1.0 - (1 - m) * p
        if shape == "sqrt":
            return m + (1 - m) * math.sqrt(1.0 - p)
        return m + 0.5 * (1 - m) * (1 + math.cos(math.pi * p))

    return _with_warmup(cfg.warmup_steps, after)


def _constant(cfg: SchedulerConfig, max_steps: int):
    return _with_warmup(cfg.warmup_steps, lambda s: 1.0)


def _rex(cfg: SchedulerConfig, max_steps: int):
    d, m, alpha = _decay_len(cfg, max_steps, cfg.warmup_steps), cfg.min_lr_ratio, cfg.rex_alpha
    return _with_warmup(cfg.warmup_steps, lambda s: max(m, (1.0 - min(1.0, s / d)) ** alpha))


def _none(cfg: SchedulerConfig, max_steps: int):
    return lambda step: 1.0


for _name, _fn in (("cosine", _cosine), ("linear", _linear), ("wsd", _wsd), ("constant", _constant),
                   ("rex", _rex), ("none", _none)):
    registry.register("scheduler", _name, _fn)


def lr_factor_fn(config: SchedulerConfig, max_steps: int) -> Callable[[int], float]:
    return registry.get("scheduler", str(config.name))(config, max_steps)


def build_scheduler(optimizer: torch.optim.Optimizer, config: SchedulerConfig, max_steps: int) -> LambdaLR:
    return LambdaLR(optimizer, lr_factor_fn(config, max_steps))
