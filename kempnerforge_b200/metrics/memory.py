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


def get_memory_utilization(device: int | None = None) -> float:
    """Peak allocated bytes as a fraction of the device's memory (0.0 without a GPU)."""
    stats = get_memory_stats(device)
    return stats["peak_gb"] / stats["total_gb"] if stats["total_gb"] else 0.0


def format_memory_stats(device: int | None = None) -> str:
    s = get_memory_stats(device)
    return (f"GPU mem: {s['allocated_gb']:.1f}GB allocated, {s['peak_gb']:.1f}GB peak, {s['reserved_gb']:.1f}GB reserved / "
            f"{s['total_gb']:.1f}GB total ({get_memory_utilization(device):.0%})")


def reset_peak_memory(device: int | None = None) -> None:
    if torch.cuda.is_available():
        torch.cuda.reset_peak_memory_stats(device)


class DeviceMemoryMonitor:
    """Per-interval memory statistics: ``report(step)`` returns the statistics plus ``mem_utilization``, logs one
    line, captures an allocation snapshot when ``step == snapshot_step`` (once) and resets the peak counter so the
    next report covers only its own interval."""

    def __init__(self, device: int | None = None, snapshot_step: int | str | None = None,
                 snapshot_dir: str | None = None) -> None:
        if isinstance(snapshot_step, str):     # DeviceMemoryMonitor(device, "dir")
            snapshot_step, snapshot_dir = None, snapshot_step
        self.device = device
        self.snapshot_step = snapshot_step
        self.snapshot_dir = snapshot_dir if snapshot_dir is not None else ("memory_snapshots" if snapshot_step is not None else None)
        self._recording = False
        self._snapshot_taken = False

    def report(self, step: int) -> dict[str, float]:
        import logging

        stats = get_memory_stats(self.device)
        stats["mem_utilization"] = get_memory_utilization(self.device)
        logging.getLogger(__name__).info(f"[step {step}] {format_memory_stats(self.device)}")
        if self.snapshot_step is not None and step == self.snapshot_step and not self._snapshot_taken:
            self._snapshot_taken = True
            self.start_recording()
            self.capture_snapshot(step)
            self.stop_recording()
        self.reset_peak()
        return stats

    def reset_peak(self) -> None:
        if torch.cuda.is_available():
            torch.cuda.reset_peak_memory_stats(self.device)

    def stats(self) -> dict[str, float]:
        return get_memory_stats(self.device)

    def start_recording(self, max_entries: int = 100000) -> None:
        if torch.cuda.is_available() and hasattr(torch.cuda.memory, "_record_memory_history"):
            torch.cuda.memory._record_memory_history(max_entries=max_entries)
            self._recording = True

    def capture_snapshot(self, tag: str | int = "snapshot", *, step: int | None = None) -> str | None:
        """Writes ``<snapshot_dir>/<tag>.pickle`` (``snapshot_step_<n>_device_<d>.pickle`` for an integer step) and
        returns its path.  Without a GPU, a snapshot directory or a working allocator history it returns None: a
        diagnostic must never end a run.  When no recording is active, one is started and stopped around the capture."""
        import logging

        if step is not None:
            tag = int(step)
        if not torch.cuda.is_available() or not self.snapshot_dir:
            return None
        own_recording = not self._recording
        try:
            if own_recording:
                self.start_recording()
                torch.cuda.synchronize(self.device)
            os.makedirs(self.snapshot_dir, exist_ok=True)
            if isinstance(tag, int):
                dev = self.device if self.device is not None else torch.cuda.current_device()
                tag = f"snapshot_step_{tag}_device_{dev}"
            path = os.path.join(self.snapshot_dir, f"{tag}.pickle")
            with open(path, "wb") as fh:
                pickle.dump(torch.cuda.memory._snapshot(), fh)
            return path
        except Exception as e:  # noqa: BLE001
            logging.getLogger(__name__).warning("memory snapshot failed: %s", e)
            return None
        finally:
            if own_recording:
                try:
                    self.stop_recording()
                except Exception:  # noqa: BLE001
                    self._recording = False

    def stop_recording(self) -> None:
        if self._recording:
            torch.cuda.memory._record_memory_history(enabled=None)
            self._recording = False
