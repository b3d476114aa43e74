"""Training-loop extension points.

A hook subclasses ``TrainingHook`` and overrides any of the five callbacks; the
``HookRunner`` calls every registered hook in order.  Hooks can be listed in the
config (``[train] hooks = ["package.module:Class"]``) or passed to the ``Trainer``.

Parity: kempnerforge/training/hooks.py:31-97 (``StepContext`` fields, callback names).
"""

from __future__ import annotations

import importlib
from dataclasses import dataclass, field
from typing import Any


@dataclass
class StepContext:
    step: int
    loss: float
    grad_norm: float
    lr: float
    tokens_seen: int
    model: Any = None
    optimizer: Any = None
    metrics: dict[str, float] = field(default_factory=dict)


class TrainingHook:
    def on_train_begin(self, config: Any) -> None: ...

    def on_step_end(self, ctx: StepContext) -> None: ...

    def on_eval_end(self, metrics: dict[str, float], step: int) -> None: ...

    def on_checkpoint_save(self, step: int, path: str) -> None: ...

    def on_train_end(self, step: int, tokens_seen: int) -> None: ...


class HookRunner:
    def __init__(self, hooks: list[TrainingHook] | None = None) -> None:
        self.hooks: list[TrainingHook] = list(hooks or [])

    def add(self, hook: TrainingHook) -> None:
        self.hooks.append(hook)

    def _each(self, name: str, *args: Any) -> None:
        for h in self.hooks:
            getattr(h, name)(*args)

    def on_train_begin(self, config: Any) -> None:
        self._each("on_train_begin", config)

    def on_step_end(self, ctx: StepContext) -> None:
        self._each("on_step_end", ctx)

    def on_eval_end(self, metrics: dict[str, float], step: int) -> None:
        self._each("on_eval_end", metrics, step)

    def on_checkpoint_save(self, step: int, path: str) -> None:
        self._each("on_checkpoint_save", step, path)

    def on_train_end(self, step: int, tokens_seen: int) -> None:
        self._each("on_train_end", step, tokens_seen)


def load_hooks(specs: list[str]) -> list[TrainingHook]:
    """Instantiate hooks from ``"package.module:ClassName"`` strings."""
    out = []
    for spec in specs:
        mod_name, _, cls_name = spec.partition(":")
        if not cls_name:
            raise ValueError(f"hook spec {spec!r} must look like 'package.module:ClassName'")
        cls = getattr(importlib.import_module(mod_name), cls_name)
        out.append(cls())
    return out
