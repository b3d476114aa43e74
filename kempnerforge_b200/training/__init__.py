"""Optimisation: optimizers, LR schedules, losses, hooks, gradient helpers, evaluation, the Trainer."""

from kempnerforge_b200.training.grad import maybe_no_sync
from kempnerforge_b200.training.hooks import HookRunner, StepContext, TrainingHook, load_hooks
from kempnerforge_b200.training.loss import build_loss_fn, chunked_cross_entropy, cross_entropy, z_loss
from kempnerforge_b200.training.optimizer import (
    FusedAdamW,
    Lion,
    Muon,
    ScheduleFreeAdamW,
    build_optimizer,
    is_muon_eligible,
    newton_schulz,
)
from kempnerforge_b200.training.scheduler import build_scheduler, lr_factor_fn

__all__ = [n for n in dir() if not n.startswith("_")]
