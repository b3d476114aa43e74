"""Observability: logger, MFU, memory statistics, step metrics tracker."""

from kempnerforge_b200.metrics.logger import format_metrics, get_logger, setup_logging
from kempnerforge_b200.metrics.memory import (DeviceMemoryMonitor, format_memory, format_memory_stats, get_memory_stats,
                                              get_memory_utilization, reset_peak_memory)
from kempnerforge_b200.metrics.mfu import (
    GPU_PEAK_TFLOPS,
    active_params,
    compute_mfu,
    estimate_model_flops_per_token,
    get_gpu_peak_tflops,
)
from kempnerforge_b200.metrics.tracker import MetricsTracker, StepMetrics, TensorBoardBackend, WandBBackend

__all__ = [n for n in dir() if not n.startswith("_")]
