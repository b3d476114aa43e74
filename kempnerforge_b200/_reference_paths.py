"""The reference's module paths, resolved to the modules of this package.

The reference spreads its configuration over one module per section (kempnerforge/config/model.py, optimizer.py, ...,
re-exported by kempnerforge/config/schema.py) and names two packages differently (kempnerforge/model,
kempnerforge/distributed).  Code written against that layout keeps working after changing only the top-level name:
``from kempnerforge_b200.config.model import ModelConfig``, ``from kempnerforge_b200.model.transformer import
Transformer``, ``from kempnerforge_b200.distributed.utils import clip_grad_norm_``.

One meta-path finder does this instead of a file per path.  An aliased name resolves to the very module object that
holds the definitions (no second copy is executed, so classes and module-level state are shared), and it is consulted
before the file finder: the aliased packages share ``__path__`` with their targets, so the file finder would otherwise
load ``models/transformer.py`` a second time under the name ``model.transformer``.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

ROOT = __name__.partition(".")[0]

# package prefixes: <ROOT>.<key>[.x] -> <ROOT>.<value>[.x]
PACKAGES = {"model": "models", "distributed": "parallel"}

# single modules: <ROOT>.<key> -> <ROOT>.<value>
MODULES = {
    "config.schema": "config",                    # every configuration class under one path
    "config.model": "config.sections",
    "config.training": "config.sections",
    "config.optimizer": "config.sections",
    "config.scheduler": "config.sections",
    "config.data": "config.sections",
    "config.distributed": "config.sections",
    "config.checkpoint": "config.sections",
    "config.eval": "config.sections",
    "config.metrics": "config.sections",
    "config.profiling": "config.sections",
    "config.adapter": "config.vlm",
    "config.vision": "config.vlm",
    "config.video": "config.vlm",
    "distributed.utils": "parallel",              # clip_grad_norm_, get_dp_info
}


def resolve(name: str) -> str | None:
    """The real module name behind an aliased one, or None when ``name`` is not an alias."""
    if not name.startswith(ROOT + "."):
        return None
    rel = name[len(ROOT) + 1:]
    if rel in MODULES:
        return f"{ROOT}.{MODULES[rel]}"
    head, _, tail = rel.partition(".")
    if head in PACKAGES:
        return f"{ROOT}.{PACKAGES[head]}" + (f".{tail}" if tail else "")
    return None


class ReferencePathFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, fullname, path=None, target=None):
        real = resolve(fullname)
        if real is None:
            return None
        return importlib.util.spec_from_loader(fullname, self, origin=real)

    def create_module(self, spec):
        return importlib.import_module(spec.origin)      # the target itself: attributes it already has are kept

    def exec_module(self, module) -> None:               # the target has been executed under its own name
        pass


def install() -> None:
    if not any(isinstance(f, ReferencePathFinder) for f in sys.meta_path):
        sys.meta_path.insert(0, ReferencePathFinder())
