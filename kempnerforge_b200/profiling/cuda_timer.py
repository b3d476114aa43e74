"""CUDA-event timers for named regions of the training step.

``CUDATimerCollection(enabled=False)`` costs nothing, so call sites can stay in place.  Events are
resolved lazily in ``elapsed_ms`` / ``summary`` so timing adds no synchronisation to the region.

Parity: kempnerforge/profiling/cuda_timer.py:27-115.
"""

from __future__ import annotations

import contextlib
import time
from collections import defaultdict

import torch


class CUDATimer:
    def __init__(self, name: str = "") -> None:
        self.name = name
        self._cuda = torch.cuda.is_available()
        self._pairs: list[tuple] = []
        self._start = None
        self._host_ms: list[float] = []

    def start(self) -> None:
        if self._cuda:
            self._start = torch.cuda.Event(enable_timing=True)
            self._start.record()
        else:
            self._start = time.perf_counter()

    def stop(self) -> None:
        if self._start is None:
            return
        if self._cuda:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self._pairs.append((self._start, end))
        else:
            self._host_ms.append((time.perf_counter() - self._start) * 1e3)
        self._start = None

    def __enter__(self):
        self.start()
        return self

    def __exit__(self, *exc):
        self.stop()

    def elapsed_ms(self) -> list[float]:
        if self._cuda and self._pairs:
            torch.cuda.synchronize()
            self._host_ms.extend(s.elapsed_time(e) for s, e in self._pairs)
            self._pairs = []
        return list(self._host_ms)

    def reset(self) -> None:
        self._pairs, self._host_ms, self._start = [], [], None


class CUDATimerCollection:
    """Named timers.  ``CUDATimerCollection(["forward", "backward"], enabled=...)`` pre-declares regions for the
    ``start(region)`` / ``stop(region)`` / ``elapsed_ms(region)`` / ``elapsed_all()`` calls (latest interval of each
    region, 0.0 when it never ran); ``timer(name)`` context managers and ``summary()`` accumulate every interval."""

    def __init__(self, regions: list[str] | bool | None = None, enabled: bool = True) -> None:
        if isinstance(regions, bool):          # CUDATimerCollection(False)
            regions, enabled = None, regions
        self.enabled = enabled
        self.regions = list(regions or [])
        self._timers: dict[str, CUDATimer] = defaultdict(CUDATimer)
        if enabled:
            for name in self.regions:
                self._timers[name].name = name

    def start(self, region: str) -> None:
        if self.enabled:
            self._timers[region].start()

    def stop(self, region: str) -> None:
        if self.enabled:
            self._timers[region].stop()

    def elapsed_ms(self, region: str) -> float:
        """Milliseconds of the region's most recent start/stop interval (synchronises); 0.0 if disabled or never run."""
        if not self.enabled or region not in self._timers:
            return 0.0
        ms = self._timers[region].elapsed_ms()
        return ms[-1] if ms else 0.0

    def elapsed_all(self) -> dict[str, float]:
        names = list(dict.fromkeys([*self.regions, *self._timers]))
        return {name: self.elapsed_ms(name) for name in names}

    def timer(self, name: str):
        if not self.enabled:
            return contextlib.nullcontext()
        t = self._timers[name]
        t.name = name
        return t

    def summary(self) -> dict[str, dict[str, float]]:
        out = {}
        for name, t in self._timers.items():
            ms = t.elapsed_ms()
            if ms:
                out[name] = {"count": len(ms), "total_ms": sum(ms), "mean_ms": sum(ms) / len(ms), "max_ms": max(ms)}
        return out

    def reset(self) -> None:
        for t in self._timers.values():
            t.reset()
