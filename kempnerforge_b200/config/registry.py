"""Name -> object registry used to plug components in without editing the core.

Categories are created lazily.  For the well-known categories the registry
exposes ``register_<cat>(name)`` decorators, ``get_<cat>(name)`` and
``list_<cat>s()`` accessors that are synthesised from one table instead of
being written out one by one.

Parity: kempnerforge/config/registry.py:25-257 (same categories and call
surface: ``registry.register_model("x")``, ``registry.get_optimizer("adamw")``,
``registry.register("router", name, obj)`` ...).
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

# category -> plural used by the ``list_*`` accessor
_KNOWN_CATEGORIES: dict[str, str] = {
    "model": "models",
    "optimizer": "optimizers",
    "scheduler": "schedulers",
    "loss": "losses",
    "router": "routers",
    "mlp": "mlps",
    "norm": "norms",
    "vision_encoder": "vision_encoders",
    "vlm_config": "vlm_configs",
    "modality_strategy": "modality_strategies",
    "adapter": "adapters",
    "video_dataset": "video_datasets",
    "sampling_policy": "sampling_policies",
    "dyn_ckpt_strategy": "dyn_ckpt_strategies",
    "hook": "hooks",
}


_UNSET: Any = object()


class Registry:
    """Two-level dictionary ``category -> name -> object`` with duplicate protection."""

    def __init__(self) -> None:
        self._tables: dict[str, dict[str, Any]] = {}

    # -- generic surface -------------------------------------------------
    def register(self, category: str, name: str, obj: Any = _UNSET) -> Any:
        """Register ``obj``; with ``obj`` omitted acts as a decorator factory."""
        if obj is _UNSET:
            return lambda o: self.register(category, name, o)
        table = self._tables.setdefault(category, {})
        if name in table:
            raise ValueError(f"{category}/{name} is already registered")
        table[name] = obj
        return obj

    def get(self, category: str, name: str) -> Any:
        table = self._tables.get(category, {})
        try:
            return table[name]
        except KeyError:
            raise KeyError(
                f"Unknown {category}: '{name}'. Available: {sorted(table)}"
            ) from None

    def list(self, category: str) -> list[str]:
        return list(self._tables.get(category, {}))

    def has(self, category: str, name: str) -> bool:
        return name in self._tables.get(category, {})

    def unregister(self, category: str, name: str) -> None:
        """Remove an entry (used by tests that register temporary components)."""
        self._tables.get(category, {}).pop(name, None)

    # -- synthesised per-category surface ----------------------------------
    def __getattr__(self, attr: str) -> Callable[..., Any]:
        for prefix in ("register_", "get_", "list_"):
            if not attr.startswith(prefix):
                continue
            tail = attr[len(prefix):]
            if prefix == "list_":
                for cat, plural in _KNOWN_CATEGORIES.items():
                    if tail == plural:
                        return lambda cat=cat: self.list(cat)
            elif tail in _KNOWN_CATEGORIES:
                if prefix == "register_":
                    return lambda name, cat=tail: self.register(cat, name)
                return lambda name, cat=tail: self.get(cat, name)
        raise AttributeError(attr)


registry = Registry()
