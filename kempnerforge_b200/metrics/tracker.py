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
from kempnerforge_b200.metrics.memory import format_memory, get_memory_stats, get_memory_utilization
from kempnerforge_b200.metrics.mfu import compute_mfu, get_gpu_peak_tflops

log = get_logger("metrics")


@dataclass
class StepMetrics:
    """What one logged step reports.  Field names are those of the reference's record; ``step`` and the two smoothed
    values are additions, and ``step_time / peak_memory_gb / total_memory_gb`` read the same numbers under older names."""

    loss: float = 0.0
    grad_norm: float = 0.0
    lr: float = 0.0
    tokens_per_sec: float = 0.0
    mfu: float = 0.0
    step_time_sec: float = 0.0
    allocated_gb: float = 0.0
    peak_gb: float = 0.0
    reserved_gb: float = 0.0
    total_gb: float = 0.0
    mem_utilization: float = 0.0
    step: int = 0
    smoothed_loss: float = 0.0
    smoothed_tokens_per_sec: float = 0.0

    step_time = property(lambda self: self.step_time_sec)
    peak_memory_gb = property(lambda self: self.peak_gb)
    total_memory_gb = property(lambda self: self.total_gb)


class _LoggingBackend:
    """A sink for numeric metrics.  Back-ends are cheap to construct: the run / writer is created by the first
    ``log`` (or by ``_ensure_init``), and a missing package or a failed start only disables the back-end with a warning."""

    def _ensure_init(self) -> None:  # pragma: no cover - interface
        pass

    @property
    def active(self) -> bool:
        return True

    def log(self, metrics: dict, step: int) -> None:
        raise NotImplementedError

    def close(self) -> None:
        pass


class WandBBackend(_LoggingBackend):
    def __init__(self, project, run_name: str | None = None, run_id: str = "", config: dict | None = None) -> None:
        """``project`` is a project name, or a metrics config carrying ``wandb_project / wandb_run_name / wandb_run_id``
        (the id of the started run is written back to it, so that a checkpoint can record it).  ``config`` is the run's
        configuration as a dict, stored with the run."""
        if hasattr(project, "wandb_project"):
            self._config = project
        else:
            from types import SimpleNamespace

            self._config = SimpleNamespace(wandb_project=project, wandb_run_name=run_name, wandb_run_id=run_id)
        self._run_config = config
        self._run = None          # None: not started yet, False: could not start

    @property
    def run_id(self) -> str:
        return getattr(self._run, "id", "") or (self._config.wandb_run_id or "")

    @property
    def active(self) -> bool:
        return self._run is not False

    def _ensure_init(self) -> None:
        if self._run is not None:
            return
        try:
            import wandb

            kw = {"project": self._config.wandb_project, "name": self._config.wandb_run_name, "resume": "allow"}
            if self._config.wandb_run_id:
                kw["id"] = self._config.wandb_run_id
            if self._run_config is not None:
                kw["config"] = self._run_config
            self._run = wandb.init(**kw)
            self._config.wandb_run_id = self._run.id
            log.info("W&B run %s", getattr(self._run, "url", self._run.id))
        except ImportError:
            log.warning("wandb is not installed: W&B logging disabled")
            self._run = False
        except Exception as exc:  # noqa: BLE001  network, authentication, ...
            log.warning("W&B disabled: %s", exc)
            self._run = False

    def log(self, metrics: dict, step: int) -> None:
        self._ensure_init()
        if self._run is False:
            return
        import wandb

        wandb.log(metrics, step=step)

    def close(self) -> None:
        if self._run:
            import wandb

            wandb.finish()
            self._run = None


class TensorBoardBackend(_LoggingBackend):
    def __init__(self, log_dir) -> None:
        """``log_dir`` is a directory, or a metrics config carrying ``tensorboard_dir``."""
        self._log_dir = getattr(log_dir, "tensorboard_dir", log_dir)
        self._writer = None       # None: not opened yet, False: could not open

    @property
    def writer(self):
        self._ensure_init()
        return self._writer or None

    @property
    def active(self) -> bool:
        return self._writer is not False

    def _ensure_init(self) -> None:
        if self._writer is not None:
            return
        try:
            from torch.utils.tensorboard import SummaryWriter

            self._writer = SummaryWriter(log_dir=self._log_dir)
            log.info("TensorBoard writer -> %s", self._log_dir)
        except ImportError:
            log.warning("tensorboard is not installed: TensorBoard logging disabled")
            self._writer = False
        except Exception as exc:  # noqa: BLE001  unwritable directory, ...
            log.warning("TensorBoard disabled: %s", exc)
            self._writer = False

    def log(self, metrics: dict, step: int) -> None:
        self._ensure_init()
        if self._writer is False:
            return
        for k, v in metrics.items():
            if isinstance(v, (int, float)):
                self._writer.add_scalar(k, v, global_step=step)

    def close(self) -> None:
        if self._writer:
            self._writer.close()
            self._writer = None


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
        self._backends: list = []
        self._backends_initialized = False
        self.peak_tflops = peak_tflops if peak_tflops is not None else get_gpu_peak_tflops()
        self._ema = 0.1
        self._smoothed: dict[str, float] = {}      # loss, tokens_per_sec, mfu, step_time
        self._t0 = 0.0
        self._use_events = torch.cuda.is_available()
        self._ev_start = self._ev_end = None
        self._pending: tuple | None = None
        self.last_step_time = 0.0

    @property
    def backends(self) -> list:
        return self._backends

    @backends.setter
    def backends(self, value: list) -> None:
        self._backends = value

    @property
    def wandb_run_id(self) -> str:
        """Id of the started W&B run (back-ends write it into the metrics config), "" without one."""
        return getattr(self.config, "wandb_run_id", "") or ""

    @property
    def gpu_peak_tflops(self) -> float:
        return self.peak_tflops

    @property
    def metrics_config(self):
        return self.config

    def init_backends(self, job_config=None) -> None:
        """Create the W&B / TensorBoard back-ends once, on rank 0 only; later calls do nothing.  ``job_config`` is the
        run's configuration (a dict, or a job config object) that W&B stores with the run."""
        if self._backends_initialized:
            return
        self._backends_initialized = True
        import torch.distributed as dist

        if self.rank != 0 or (dist.is_available() and dist.is_initialized() and dist.get_rank() != 0):
            return
        c = getattr(job_config, "metrics", None) or self.config
        run_config = job_config if isinstance(job_config, dict) else None
        made = []
        if c.enable_wandb:
            made.append(WandBBackend(c) if run_config is None else WandBBackend(c, config=run_config))
        if c.enable_tensorboard:
            made.append(TensorBoardBackend(c))
        for be in made:            # start now: the run id is known before the first checkpoint, failures show at once
            be._ensure_init()
            if getattr(be, "active", True) is not False:
                self._backends.append(be)

    _init_backends = init_backends

    def _update_smoothed(self, key: str, value: float) -> None:
        prev = self._smoothed.get(key)
        self._smoothed[key] = value if prev is None else self._ema * value + (1 - self._ema) * prev

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
        mfu = 0.0
        if self.model_config is not None:
            mfu = compute_mfu(self.model_config, tps, self.num_gpus, self.peak_tflops, self.seq_len)
        for key, val in (("loss", loss), ("tokens_per_sec", tps), ("mfu", mfu), ("step_time", dt)):
            self._update_smoothed(key, val)
        if not (step % self.config.log_interval == 0 or step == 1):
            return None
        mem = get_memory_stats()
        m = StepMetrics(loss=loss, grad_norm=grad_norm, lr=lr, tokens_per_sec=tps, mfu=mfu, step_time_sec=dt,
                        allocated_gb=mem["allocated_gb"], peak_gb=mem["peak_gb"], reserved_gb=mem["reserved_gb"],
                        total_gb=mem["total_gb"], mem_utilization=get_memory_utilization(), step=step,
                        smoothed_loss=self._smoothed["loss"], smoothed_tokens_per_sec=self._smoothed["tokens_per_sec"])
        self._log_step(step, m, extra)
        return m

    def _log_step(self, step: int, m: StepMetrics, extra: dict | None = None) -> None:
        """One stdout line and one record per back-end.  Back-end keys are the reference's (``train/*``, ``gpu/*``,
        ``smoothed/*``), so dashboards built for it keep working."""
        line = {"loss": m.loss, "lr": m.lr, "grad_norm": m.grad_norm, "tok/s": m.tokens_per_sec, "mfu": 100.0 * m.mfu,
                "mem": format_memory({"peak_gb": m.peak_gb, "total_gb": m.total_gb}), "step_time": m.step_time_sec}
        if extra:
            line.update(extra)
        log.info(format_metrics(step, line))
        payload = {
            "train/loss": m.loss, "train/grad_norm": m.grad_norm, "train/lr": m.lr, "train/tokens_per_sec": m.tokens_per_sec,
            "train/mfu": m.mfu, "train/step_time_sec": m.step_time_sec, "gpu/allocated_gb": m.allocated_gb,
            "gpu/peak_gb": m.peak_gb, "gpu/reserved_gb": m.reserved_gb, "gpu/mem_utilization": m.mem_utilization,
        }
        payload.update({f"smoothed/{k}": v for k, v in self._smoothed.items()})
        if extra:
            payload.update({k: v for k, v in extra.items() if isinstance(v, (int, float))})
        for be in self._backends:
            be.log(payload, step=step)

    def log_eval(self, metrics: dict[str, float], step: int) -> None:
        log.info(format_metrics(step, metrics))
        for be in self._backends:
            be.log(metrics, step=step)

    def log_extra(self, metrics: dict[str, float], step: int) -> None:
        for be in self._backends:
            be.log(metrics, step=step)

    def close(self) -> None:
        for be in self._backends:
            be.close()
        self._backends = []
