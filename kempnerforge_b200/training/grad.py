"""Gradient-accumulation helper: skip gradient synchronisation on all but the last micro-step.

Parity: kempnerforge/training/grad.py:15-39.  Works with our sharded engine (``set_requires_gradient_sync``)
and with PyTorch FSDP2 modules, which expose the same method.
"""

from __future__ import annotations

import contextlib


@contextlib.contextmanager
def maybe_no_sync(model, micro_step: int, grad_accum_steps: int):
    last = micro_step == grad_accum_steps - 1
    setter = getattr(model, "set_requires_gradient_sync", None)
    if setter is None or grad_accum_steps == 1:
        yield
        return
    setter(last)
    try:
        yield
    finally:
        setter(True)
