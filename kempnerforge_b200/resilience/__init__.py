"""Fault tolerance: signals, NaN tracking, health probes, resume discovery."""

from kempnerforge_b200.resilience.elastic import (
    SLURMInfo,
    get_slurm_info,
    is_slurm_job,
    is_slurm_requeue,
    list_step_dirs,
    log_job_info,
    resolve_resume_path,
)
from kempnerforge_b200.resilience.health import (
    NaNDetector,
    NaNState,
    check_gpu_health,
    check_native_kernel_status,
    check_nccl_health,
)
from kempnerforge_b200.resilience.signal_handler import ShutdownHandler

__all__ = [n for n in dir() if not n.startswith("_")]
