"""Run-time health checks: non-finite loss tracking, GPU sanity, communication liveness.

``NaNDetector`` keeps all ranks in agreement (a flag all-reduce) so that either every rank skips a
step or none does.  ``check_nccl_health`` issues a tiny asynchronous all-reduce and waits for it
with a time limit, so a dead peer shows up as ``False`` instead of a hang.

Parity: kempnerforge/resilience/health.py:37-262.  Addition: ``check_values`` takes the finite flag
the training step already reduced on the device, which saves a second synchronisation per step.
"""

from __future__ import annotations

import logging
import math
from dataclasses import dataclass, field
from datetime import timedelta

import torch
import torch.distributed as dist

log = logging.getLogger(__name__)


@dataclass
class NaNState:
    consecutive_nans: int = 0
    total_nans: int = 0
    nan_steps: list[int] = field(default_factory=list)
    last_good_loss: float = float("inf")
    last_good_step: int = -1


class NaNDetector:
    def __init__(self, action: str = "warn", max_consecutive: int = 5, max_history: int = 100) -> None:
        if action not in ("warn", "skip", "raise"):
            raise ValueError(f"Invalid NaN action: {action!r} (expected warn/skip/raise)")
        self.action = action
        self.max_consecutive = max_consecutive
        self.max_history = max_history
        self.state = NaNState()

    def _record(self, ok: bool, local_bad: bool, loss: float, step: int) -> bool:
        st = self.state
        if ok:
            st.consecutive_nans = 0
            st.last_good_loss, st.last_good_step = loss, step
            return True
        st.consecutive_nans += 1
        st.total_nans += 1
        if len(st.nan_steps) < self.max_history:
            st.nan_steps.append(step)
        where = "loss" if local_bad else "loss on another rank"
        msg = (f"NaN/Inf {where} detected at step {step} (consecutive={st.consecutive_nans}, "
               f"total={st.total_nans}, last_good_step={st.last_good_step})")
        if self.action == "raise":
            raise RuntimeError(msg)
        log.warning(msg + (" — skipping optimizer step" if self.action == "skip" else ""))
        return False

    def check_loss(self, loss: float, step: int) -> bool:
        """True when the loss is finite on every rank (one flag all-reduce when distributed)."""
        local_bad = not math.isfinite(loss)
        any_bad = local_bad
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dev = "cuda" if torch.cuda.is_available() and dist.get_backend() != "gloo" else "cpu"
            flag = torch.tensor([1.0 if local_bad else 0.0], device=dev)
            dist.all_reduce(flag)
            any_bad = flag.item() > 0
        return self._record(not any_bad, local_bad, loss, step)

    def check_values(self, loss: float, grad_norm: float, all_ranks_finite: bool, step: int) -> bool:
        """Same bookkeeping as ``check_loss`` for a step whose finite flag was already reduced."""
        local_bad = not (math.isfinite(loss) and math.isfinite(grad_norm))
        return self._record(all_ranks_finite and not local_bad, local_bad, loss, step)

    def check_gradients(self, model: torch.nn.Module, step: int) -> bool:
        for name, p in model.named_parameters():
            if p.grad is not None and not torch.isfinite(p.grad).all():
                msg = f"NaN/Inf gradient in {name} at step {step}"
                if self.action == "raise":
                    raise RuntimeError(msg)
                log.warning(msg)
                return False
        return True

    @property
    def should_rollback(self) -> bool:
        return self.state.consecutive_nans >= self.max_consecutive

    @property
    def should_stop(self) -> bool:
        return self.should_rollback

    def reset(self) -> None:
        self.state = NaNState()


def check_gpu_health(device: int | None = None) -> dict:
    """Tiny compute + allocation probe of the current GPU; never raises."""
    out = {"healthy": False, "device": None, "error": None, "cuda_available": torch.cuda.is_available(),
           "device_accessible": False, "compute_ok": False, "memory_ok": False}
    if not out["cuda_available"]:
        out["error"] = "CUDA not available"
        return out
    try:
        dev = torch.cuda.current_device() if device is None else device
        out["device"] = torch.cuda.get_device_name(dev)
        out["device_accessible"] = True
        a = torch.ones(256, device=f"cuda:{dev}")
        ok = float((a + a).sum().item()) == 512.0
        out["compute_ok"] = ok
        buf = torch.empty(1 << 20, dtype=torch.uint8, device=f"cuda:{dev}")
        del buf
        out["memory_ok"] = True
        out["memory_allocated_gb"] = torch.cuda.memory_allocated(dev) / 1024**3
        out["healthy"] = ok
        if not ok:
            out["error"] = "arithmetic probe returned a wrong value"
    except RuntimeError as exc:
        out["error"] = str(exc)
    return out


def check_nccl_health(timeout_sec: float = 10.0, group=None) -> bool:
    """All-reduce of ones with a deadline; True when every rank answered and the sum is the world size."""
    if not (dist.is_available() and dist.is_initialized()):
        return True
    try:
        world = dist.get_world_size(group) if group is not None else dist.get_world_size()
        try:
            backend = dist.get_backend(group) if group is not None else dist.get_backend()
        except Exception:  # noqa: BLE001  no backend to ask (a stand-in process group): stay on the host
            backend = ""
        dev = "cuda" if torch.cuda.is_available() and "nccl" in str(backend) else "cpu"
        t = torch.ones(1, device=dev)
        work = dist.all_reduce(t, group=group, async_op=True)
        if not work.wait(timeout=timedelta(seconds=timeout_sec)):
            log.error("communication health check timed out after %.1fs", timeout_sec)
            return False
        if dev == "cuda":
            torch.cuda.synchronize()
        ok = abs(t.item() - world) < 1e-3
        if not ok:
            log.error("communication health check returned %s, expected %d", t.item(), world)
        return ok
    except Exception as exc:  # a broken process group raises rather than returning False
        log.error("communication health check failed: %s", exc)
        return False


def check_native_kernel_status() -> int:
    """Status word of the native kernel library: non-zero means a device-side wait gave up."""
    if not torch.cuda.is_available():
        return 0
    from kempnerforge_b200.ops import cuda as kcuda

    return kcuda.read_status() if kcuda.available() else 0
