"""Device-memory statistics for the *current* device and optional allocation-history snapshots.

Parity: kempnerforge/metrics/memory.py:18-167.  Difference: the statistics default to the calling
process's current device instead of device index 0.
"""

from __future__ import annotations

import os
import pickle

import torch

GB = 1024**3


def get_memory_stats(device: int | None = None) -> dict[str, float]:
    if not torch.cuda.is_available():
        return {"allocated_gb": 0.0, "peak_gb": 0.0, "reserved_gb": 0.0, "total_gb": 0.0}
    dev = torch.cuda.current_device() if device is None else device
    return {
        "allocated_gb": torch.cuda.memory_allocated(dev) / GB,
        "peak_gb": torch.cuda.max_memory_allocated(dev) / GB,
        "reserved_gb": torch.cuda.memory_reserved(dev) / GB,
        "total_gb": torch.cuda.get_device_properties(dev).total_memory / GB,
    }


def format_memory(stats: dict[str, float]) -> str:
    return f"{stats['peak_gb']:.1f}/{stats['total_gb']:.0f}GB"


class DeviceMemoryMonitor:
    def __init__(self, device: int | None = None, snapshot_dir: str | None = None) -> None:
        self.device = device
        self.snapshot_dir = snapshot_dir
        self._recording = False

    def reset_peak(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.reset_peak_memory_stats(self.device)

    def stats(self) -> dict[str, float]:
        return get_memory_stats(self.device)

    def start_recording(self, max_entries: int = 100000) -> None:
        if torch.cuda.is_available() and hasattr(torch.cuda.memory, "_record_memory_history"):
            torch.cuda.memory._record_memory_history(max_entries=max_entries)
            self._recording = True

    def capture_snapshot(self, tag: str = "snapshot") -> str | None:
        if not (self._recording and self.snapshot_dir):
            return None
        os.makedirs(self.snapshot_dir, exist_ok=True)
        path = os.path.join(self.snapshot_dir, f"{tag}.pickle")
        with open(path, "wb") as fh:
            pickle.dump(torch.cuda.memory._snapshot(), fh)
        return path

    def stop_recording(self) -> None:
        if self._recording:
            torch.cuda.memory._record_memory_history(enabled=None)
            self._recording = False
