"""Activation capture for analysis: forward hooks that copy named sub-module outputs to the host.

``ActivationStore(model, ["layers.0.attention", "norm"])`` keeps, once enabled, the latest output of each
named module (the first element for tuple outputs) as a detached CPU tensor; ``extract_representations``
runs a model over batches and stacks what was captured; ``save_activations`` writes an ``.npz``.
Blocks with a capture hook run op by op (the fused block node is bypassed), so every named sub-module fires.

Parity: kempnerforge/model/hooks.py:26-180.
"""

from __future__ import annotations

from collections import defaultdict

import numpy as np
import torch
from torch import nn


class _MissingModule(KeyError, ValueError):
    """Raised for an unknown module name; both a KeyError (a lookup failed) and a ValueError (a bad argument)."""


class ActivationStore:
    """Forward hooks on named sub-modules that keep each module's LATEST output as a detached host tensor.

    Hooks are installed by ``enable()`` (or on entering a ``with`` block) and removed by ``disable()``; a module name
    that does not exist raises at ``enable()`` (a ``ValueError`` that is also a ``KeyError``).  ``get(name)`` returns the
    tensor captured by the last forward pass, or ``None``; every pass overwrites the previous capture.  With
    ``keep_history=True`` the store also keeps one tensor per pass (``history(name)``).  ``layer_names=`` is accepted
    as another spelling of ``layers``."""

    def __init__(self, model: nn.Module, layers: list[str] | None = None, detach_to_cpu: bool = True, *,
                 layer_names: list[str] | None = None, keep_history: bool = False) -> None:
        self.model = model
        self._layers = list(layers if layers is not None else (layer_names or []))
        self.to_cpu = detach_to_cpu
        self.keep_history = keep_history
        self._activations: dict[str, torch.Tensor] = {}
        self._history: dict[str, list[torch.Tensor]] = defaultdict(list)
        self._hooks = []
        self._on = False

    @property
    def enabled(self) -> bool:
        return self._on

    @property
    def layer_names(self) -> list[str]:
        return list(self._layers)

    @property
    def activations(self) -> dict[str, torch.Tensor]:
        """A copy of the captured activations (latest per module)."""
        return dict(self._activations)

    def enable(self) -> None:
        """Install the forward hooks (no-op while they are installed)."""
        if self._on:
            return
        modules = dict(self.model.named_modules())
        missing = [n for n in self._layers if n not in modules]
        if missing:
            raise _MissingModule(f"modules not found in model: {missing}; available e.g. {sorted(modules)[:8]}")
        for name in self._layers:
            self._hooks.append(modules[name].register_forward_hook(self._make_hook(name)))
            # make sure the parents of a hooked module run their ordinary (op-by-op) forward
            parts = name.split(".")
            for i in range(1, len(parts)):
                parent = modules.get(".".join(parts[:i]))
                if parent is not None and hasattr(parent, "ac_mode"):
                    self._hooks.append(parent.register_forward_hook(lambda *a: None))
        self._on = True

    def _make_hook(self, name: str):
        def hook(module, inputs, output):
            out = output[0] if isinstance(output, (tuple, list)) and len(output) else output
            if isinstance(out, dict):
                out = next(iter(out.values()))
            if torch.is_tensor(out):
                out = out.detach()
                out = out.cpu() if self.to_cpu else out
                self._activations[name] = out
                if self.keep_history:
                    self._history[name].append(out)

        return hook

    def clear(self) -> None:
        """Forget what was captured (the hooks stay installed)."""
        self._activations.clear()
        self._history.clear()

    def get(self, name: str) -> torch.Tensor | None:
        """The activation captured by the last forward pass for ``name``, or None."""
        return self._activations.get(name)

    def history(self, name: str) -> list[torch.Tensor]:
        """One tensor per forward pass since the last ``clear()`` (``keep_history=True`` only)."""
        return list(self._history.get(name, []))

    def disable(self) -> None:
        """Remove every hook."""
        for h in self._hooks:
            h.remove()
        self._hooks = []
        self._on = False

    remove = disable

    def __enter__(self):
        self.enable()
        return self

    def __exit__(self, *exc):
        self.disable()


@torch.no_grad()
def extract_representations(model: nn.Module, batches, layer_names: list[str], device=None,
                            batch_size: int | None = None, max_samples: int | None = None,
                            pool: str | None = None) -> dict[str, torch.Tensor]:
    """Run ``model`` over token batches; returns {layer: (N, ...) tensor} on the host.

    ``batches`` is an iterable of batches (tensors or dicts with ``input_ids``) or, with ``batch_size`` given or a
    ``torch.utils.data.Dataset`` passed, a map-style dataset of samples that is batched here in order.
    ``max_samples`` stops after that many samples and trims the result to it.  ``pool`` may be None, "mean" (over the
    sequence) or "last" (final position)."""
    from torch.utils.data import DataLoader, Dataset

    if batch_size is not None or isinstance(batches, Dataset):
        batches = DataLoader(batches, batch_size=batch_size or 32, shuffle=False)
    was_training = model.training
    model.eval()
    out: dict[str, list[torch.Tensor]] = defaultdict(list)
    seen = 0
    with ActivationStore(model, layer_names) as store:
        for batch in batches:
            if max_samples is not None and seen >= max_samples:
                break
            tokens = batch["input_ids"] if isinstance(batch, dict) else batch
            if device is not None:
                tokens = tokens.to(device)
            store.clear()
            model(tokens)
            for name in layer_names:
                act = store.get(name)
                if pool == "mean":
                    act = act.mean(dim=1)
                elif pool == "last":
                    act = act[:, -1]
                out[name].append(act)
            seen += tokens.shape[0]
    if was_training:
        model.train()
    return {k: torch.cat(v, dim=0)[:max_samples] for k, v in out.items()}


def save_activations(activations: dict[str, torch.Tensor], path) -> None:
    """One ``.npz`` (the suffix is added when missing, parent folders are created) keyed by the module names."""
    from pathlib import Path

    path = Path(path)
    if path.suffix != ".npz":
        path = path.with_suffix(".npz")
    path.parent.mkdir(parents=True, exist_ok=True)
    def as_array(v):
        if isinstance(v, (list, tuple)):          # per-pass lists (ActivationStore.history)
            v = torch.cat(list(v), dim=0)
        return v.float().numpy()                  # numpy has no bfloat16

    np.savez(str(path), **{k: as_array(v) for k, v in activations.items() if not isinstance(v, (list, tuple)) or len(v)})
