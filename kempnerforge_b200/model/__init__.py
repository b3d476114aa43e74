"""``kempnerforge_b200.model`` mirrors the reference's package name (kempnerforge/model): every sub-module of
``kempnerforge_b200.models`` is importable from here (``from kempnerforge_b200.model.transformer import Transformer``)."""

import importlib
import pkgutil
import sys

import kempnerforge_b200.models as _models

for _m in pkgutil.iter_modules(_models.__path__):
    sys.modules[f"{__name__}.{_m.name}"] = importlib.import_module(f"kempnerforge_b200.models.{_m.name}")
    globals()[_m.name] = sys.modules[f"{__name__}.{_m.name}"]
