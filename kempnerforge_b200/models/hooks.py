"""Activation capture for analysis: forward hooks that copy named sub-module outputs to the host.

``ActivationStore(model, ["layers.0.attention", "norm"])`` records, per forward pass, the output of each
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


class ActivationStore:
    def __init__(self, model: nn.Module, layer_names: list[str], detach_to_cpu: bool = True) -> None:
        self.model = model
        self.layer_names = list(layer_names)
        self.to_cpu = detach_to_cpu
        self.activations: dict[str, list[torch.Tensor]] = defaultdict(list)
        self._handles = []
        modules = dict(model.named_modules())
        missing = [n for n in self.layer_names if n not in modules]
        if missing:
            raise KeyError(f"modules not found: {missing}; e.g. {sorted(modules)[:8]}")
        for name in self.layer_names:
            self._handles.append(modules[name].register_forward_hook(self._make_hook(name)))
            # make sure the parents of a hooked module run their ordinary (op-by-op) forward
            parts = name.split(".")
            for i in range(1, len(parts)):
                parent = modules.get(".".join(parts[:i]))
                if parent is not None and hasattr(parent, "ac_mode"):
                    self._handles.append(parent.register_forward_hook(lambda *a: None))

    def _make_hook(self, name: str):
        def hook(module, inputs, output):
            out = output[0] if isinstance(output, (tuple, list)) else output
            if isinstance(out, dict):
                out = next(iter(out.values()))
            if torch.is_tensor(out):
                out = out.detach()
                self.activations[name].append(out.float().cpu() if self.to_cpu else out)

        return hook

    def clear(self) -> None:
        self.activations.clear()

    def get(self, name: str, concat: bool = True):
        items = self.activations.get(name, [])
        if concat and items:
            return torch.cat(items, dim=0)
        return items

    def remove(self) -> None:
        for h in self._handles:
            h.remove()
        self._handles = []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.remove()


@torch.no_grad()
def extract_representations(model: nn.Module, batches, layer_names: list[str], device=None,
                            pool: str | None = None) -> dict[str, torch.Tensor]:
    """Run ``model`` over an iterable of token batches; returns {layer: (N, ...) tensor}.  ``pool`` may be
    None, "mean" (over the sequence) or "last" (final position)."""
    was_training = model.training
    model.eval()
    out: dict[str, list[torch.Tensor]] = defaultdict(list)
    with ActivationStore(model, layer_names) as store:
        for batch in batches:
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
    if was_training:
        model.train()
    return {k: torch.cat(v, dim=0) for k, v in out.items()}


def save_activations(activations: dict[str, torch.Tensor], path: str) -> None:
    np.savez(path, **{k.replace(".", "__"): v.float().numpy() for k, v in activations.items()})
