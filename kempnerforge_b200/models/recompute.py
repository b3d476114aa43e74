"""Which pass of an activation-checkpointed region is running on this thread.

``torch.utils.checkpoint`` runs a region twice: once in the forward pass and once more, during backward, to
rebuild the activations.  Modules whose forward has side effects (a router that nudges its balancing bias) must
apply them once and must reproduce the first pass's decisions in the second.  The checkpoint calls of this package
pass :func:`checkpoint_contexts` as ``context_fn``; such modules ask :func:`phase`.
"""

from __future__ import annotations

import threading
from contextlib import contextmanager

_state = threading.local()


def phase() -> str | None:
    """``"forward"`` inside a checkpointed region's first pass, ``"recompute"`` inside its second, else None."""
    return getattr(_state, "phase", None)


@contextmanager
def _phase(name: str):
    prev = phase()
    _state.phase = name
    try:
        yield
    finally:
        _state.phase = prev


def checkpoint_contexts():
    """``context_fn`` for ``torch.utils.checkpoint.checkpoint(..., use_reentrant=False)``."""
    return _phase("forward"), _phase("recompute")
