"""Four example training hooks and how to switch them on.

From a config file (no script edits needed):

    [train]
    hooks = ["examples.custom_hook:GradNormHistogramHook", "examples.custom_hook:EarlyStoppingHook"]

or from Python:

    from kempnerforge_b200.training.trainer import Trainer
    trainer = Trainer(cfg, hooks=[LearningDynamicsHook(every=50)])
    trainer.fit()

Each hook subclasses ``TrainingHook`` and overrides only the callbacks it needs; ``StepContext`` carries
step, loss, grad_norm, lr, tokens_seen, the model, the optimizer and a metrics dict whose entries are
logged with the step. Parity: examples/custom_hook.py:21-135 in the reference (same four hooks; there
the training script has to be edited to register them).
"""

from __future__ import annotations

import math

import torch

from kempnerforge_b200.training.hooks import StepContext, TrainingHook


class GradNormHistogramHook(TrainingHook):
    """Keeps a log-scale histogram of the global gradient norm and reports spikes."""

    def __init__(self, spike_factor: float = 5.0, window: int = 100) -> None:
        self.spike_factor, self.window = spike_factor, window
        self.history: list[float] = []
        self.bins: dict[int, int] = {}
        self.spikes: list[int] = []

    def on_step_end(self, ctx: StepContext) -> None:
        g = float(ctx.grad_norm)
        if not math.isfinite(g) or g <= 0:
            return
        self.bins[math.floor(math.log10(g) * 4)] = self.bins.get(math.floor(math.log10(g) * 4), 0) + 1
        recent = self.history[-self.window:]
        if len(recent) >= 10 and g > self.spike_factor * (sum(recent) / len(recent)):
            self.spikes.append(ctx.step)
            ctx.metrics["hooks/grad_norm_spike"] = 1.0
        self.history.append(g)

    def on_train_end(self, step: int, tokens_seen: int) -> None:
        for b in sorted(self.bins):
            print(f"grad_norm in [{10 ** (b / 4):.3g}, {10 ** ((b + 1) / 4):.3g}): {self.bins[b]}")
        print(f"{len(self.spikes)} spike(s) at steps {self.spikes[:20]}")


class LearningDynamicsHook(TrainingHook):
    """Every ``every`` steps: weight norm and update-to-weight ratio per top-level module."""

    def __init__(self, every: int = 100) -> None:
        self.every = every
        self._prev: dict[str, torch.Tensor] = {}

    @staticmethod
    def _bucket(name: str) -> str:
        parts = name.split(".")
        return ".".join(parts[:2]) if parts[0] == "layers" else parts[0]

    def on_step_end(self, ctx: StepContext) -> None:
        if ctx.model is None or ctx.step % self.every:
            return
        sq: dict[str, float] = {}
        dsq: dict[str, float] = {}
        with torch.no_grad():
            for name, p in ctx.model.named_parameters():
                key = self._bucket(name)
                cur = p.detach().float()
                sq[key] = sq.get(key, 0.0) + float(cur.pow(2).sum())
                old = self._prev.get(name)
                if old is not None:
                    dsq[key] = dsq.get(key, 0.0) + float((cur.cpu() - old).pow(2).sum())
                self._prev[name] = cur.cpu()
        for key, v in sq.items():
            ctx.metrics[f"dynamics/{key}/weight_norm"] = math.sqrt(v)
            if key in dsq and v > 0:
                ctx.metrics[f"dynamics/{key}/update_ratio"] = math.sqrt(dsq[key] / v)


class EarlyStoppingHook(TrainingHook):
    """Asks the trainer to stop when the eval loss has not improved ``patience`` evaluations in a row."""

    def __init__(self, patience: int = 3, min_delta: float = 0.0) -> None:
        self.patience, self.min_delta = patience, min_delta
        self.best = math.inf
        self.bad = 0
        self.should_stop = False

    def on_eval_end(self, eval_metrics: dict[str, float], step: int) -> None:
        loss = eval_metrics.get("eval/loss")
        if loss is None:
            return
        if loss < self.best - self.min_delta:
            self.best, self.bad = loss, 0
        else:
            self.bad += 1
            if self.bad >= self.patience:
                self.should_stop = True
                print(f"[early stopping] no improvement for {self.bad} evaluations (best {self.best:.4f}) at step {step}")

    def on_step_end(self, ctx: StepContext) -> None:
        if self.should_stop:
            ctx.metrics["hooks/stop_requested"] = 1.0


class ExpertLoadBalanceHook(TrainingHook):
    """For MoE models: coefficient of variation and max/mean of the per-expert token counts."""

    def __init__(self, every: int = 50) -> None:
        self.every = every

    def on_step_end(self, ctx: StepContext) -> None:
        model = ctx.model
        if model is None or ctx.step % self.every or not hasattr(model, "get_expert_counts"):
            return
        for layer, counts in model.get_expert_counts().items():
            c = counts.float()
            mean = c.mean().clamp_min(1e-9)
            ctx.metrics[f"moe/layer{layer}/load_cv"] = float(c.std(unbiased=False) / mean)
            ctx.metrics[f"moe/layer{layer}/load_max_over_mean"] = float(c.max() / mean)
