"""Profiling: torch.profiler wrapper and CUDA-event timers."""

from kempnerforge_b200.profiling.cuda_timer import CUDATimer, CUDATimerCollection
from kempnerforge_b200.profiling.profiler import analyze_profiler, build_profiler, categorize_kernel, print_profiler_summary

__all__ = [n for n in dir() if not n.startswith("_")]
