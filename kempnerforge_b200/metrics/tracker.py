"""Per-step metrics: timing, throughput, MFU, memory, smoothing, stdout line and optional backends.

Step time is measured on the device with CUDA events when a GPU is present (the events are read
one step late, so no synchronisation is added to the step), otherwise with the host clock.
Logging happens when ``step % log_interval == 0`` or ``step == 1``.  W&B and TensorBoard
back-ends exist only on rank 0.

Parity: kempnerforge/metrics/tracker.py:22-309 (``StepMetrics`` fields, ``start_step/end_step/
log_eval/close``, EMA 0.1 smoothing, back-end classes).  Difference: device timing instead of an
unsynchronised host clock.
"""

from __future__ import annotations

import os
import time
from dataclasses import dataclass

import torch

from kempnerforge_b200.metrics.logger import format_metrics, get_logger
from kempnerforge_b200.metrics.memory import format_memory, get_memory_stats
from kempnerforge_b200.metrics.mfu import compute_mfu, get_gpu_peak_tflops

log = get_logger("metrics")


@dataclass
class StepMetrics:
    step: int
    loss: float
    grad_norm: float
    lr: float
    tokens_per_sec: float
    mfu: float
    step_time: float
    peak_memory_gb: float = 0.0
    total_memory_gb: float = 0.0
    smoothed_loss: float = 0.0
    smoothed_tokens_per_sec: float = 0.0


class WandBBackend:
    def __init__(self, project, run_name: str | None = None, run_id: str = "", config: dict | None = None) -> None:
        """``project`` is a project name, or a metrics config carrying ``wandb_project / wandb_run_name / wandb_run_id``."""
        if hasattr(project, "wandb_project"):
            project, run_name, run_id = project.wandb_project, project.wandb_run_name, project.wandb_run_id
        import wandb

        self._wandb = wandb
        self.run = wandb.init(project=project, name=run_name, id=run_id or None, resume="allow", config=config)
        self.run_id = self.run.id

    def log(self, metrics: dict, step: int) -> None:
        self._wandb.log(metrics, step=step)

    def close(self) -> None:
        self._wandb.finish()


class TensorBoardBackend:
    def __init__(self, log_dir) -> None:
        """``log_dir`` is a directory, or a metrics config carrying ``tensorboard_dir``."""
        log_dir = getattr(log_dir, "tensorboard_dir", log_dir)
        from torch.utils.tensorboard import SummaryWriter

        self.writer = SummaryWriter(log_dir)

    def log(self, metrics: dict, step: int) -> None:
        for k, v in metrics.items():
            if isinstance(v, (int, float)):
                self.writer.add_scalar(k, v, step)

    def close(self) -> None:
        self.writer.close()


class MetricsTracker:
    def __init__(self, config, model_config=None, num_gpus: int | None = None, seq_len: int = 2048, rank: int = 0,
                 peak_tflops: float | None = None, *, gpu_peak_tflops: float | None = None) -> None:
        """``config`` is the metrics section; a whole job config works too (``MetricsTracker(job, num_gpus)``), in which
        case the model section, the sequence length and the calling process's rank are taken from it / the environment."""
        if hasattr(config, "metrics") and hasattr(config, "model"):
            job = config
            if isinstance(model_config, int):          # MetricsTracker(job, num_gpus[, gpu_peak_tflops])
                if num_gpus is not None and peak_tflops is None:
                    peak_tflops = float(num_gpus)
                num_gpus = model_config
            config, model_config, seq_len = job.metrics, job.model, job.train.seq_len
            rank = int(os.environ.get("RANK", rank))
        peak_tflops = peak_tflops if peak_tflops is not None else gpu_peak_tflops
        self.config = config
        self.model_config = model_config
        self.num_gpus = 1 if num_gpus is None else num_gpus
        self.seq_len = seq_len
        self.rank = rank
        self.backends: list = []
        self.peak_tflops = peak_tflops if peak_tflops is not None else get_gpu_peak_tflops()
        self._ema = 0.1
        self._smoothed_loss: float | None = None
        self._smoothed_tps: float | None = None
        self._t0 = 0.0
        self._use_events = torch.cuda.is_available()
        self._ev_start = self._ev_end = None
        self._pending: tuple | None = None
        self.last_step_time = 0.0
        self.wandb_run_id = ""

    def init_backends(self, job_config: dict | None = None) -> None:
        if self.rank != 0:
            return
        c = self.config
        if c.enable_wandb:
            try:
                be = WandBBackend(c.wandb_project, c.wandb_run_name, c.wandb_run_id, job_config)
                self.wandb_run_id = be.run_id
                self.backends.append(be)
            except Exception as exc:  # optional dependency / offline
                log.warning("W&B disabled: %s", exc)
        if c.enable_tensorboard:
            try:
                self.backends.append(TensorBoardBackend(c.tensorboard_dir))
            except Exception as exc:
                log.warning("TensorBoard disabled: %s", exc)

    # ------------------------------------------------------------------ timing
    def start_step(self) -> None:
        self._t0 = time.perf_counter()
        if self._use_events:
            self._ev_start = torch.cuda.Event(enable_timing=True)
            self._ev_end = torch.cuda.Event(enable_timing=True)
            self._ev_start.record()

    def _elapsed(self) -> float:
        host = time.perf_counter() - self._t0
        if not self._use_events:
            return host
        self._ev_end.record()
        prev = self._pending
        self._pending = (self._ev_start, self._ev_end)
        if prev is not None and prev[1].query():
            return prev[0].elapsed_time(prev[1]) / 1e3
        return host

    def end_step(self, step: int, loss: float, grad_norm: float, lr: float, tokens_in_step: int,
                 extra: dict | None = None) -> StepMetrics | None:
        dt = max(self._elapsed(), 1e-9)
        self.last_step_time = dt
        tps = tokens_in_step / dt
        a = self._ema
        self._smoothed_loss = loss if self._smoothed_loss is None else (1 - a) * self._smoothed_loss + a * loss
        self._smoothed_tps = tps if self._smoothed_tps is None else (1 - a) * self._smoothed_tps + a * tps
        if not (step % self.config.log_interval == 0 or step == 1):
            return None
        mfu = 0.0
        if self.model_config is not None:
            mfu = compute_mfu(self.model_config, tps, self.num_gpus, self.peak_tflops, self.seq_len)
        mem = get_memory_stats()
        m = StepMetrics(step, loss, grad_norm, lr, tps, mfu, dt, mem["peak_gb"], mem["total_gb"],
                        self._smoothed_loss, self._smoothed_tps)
        line = {"loss": loss, "lr": lr, "grad_norm": grad_norm, "tok/s": tps, "mfu": 100.0 * mfu,
                "mem": format_memory(mem), "step_time": dt}
        if extra:
            line.update(extra)
        log.info(format_metrics(step, line))
        payload = {
            "train/loss": loss, "train/grad_norm": grad_norm, "train/lr": lr, "train/tokens_per_sec": tps,
            "train/mfu": mfu, "train/step_time": dt, "train/peak_memory_gb": mem["peak_gb"],
            "train/smoothed_loss": self._smoothed_loss, "train/smoothed_tokens_per_sec": self._smoothed_tps,
        }
        if extra:
            payload.update({k: v for k, v in extra.items() if isinstance(v, (int, float))})
        for be in self.backends:
            be.log(payload, step)
        return m

    def log_eval(self, metrics: dict[str, float], step: int) -> None:
        log.info(format_metrics(step, metrics))
        for be in self.backends:
            be.log(metrics, step)

    def log_extra(self, metrics: dict[str, float], step: int) -> None:
        for be in self.backends:
            be.log(metrics, step)

    def close(self) -> None:
        for be in self.backends:
            be.close()
        self.backends = []
