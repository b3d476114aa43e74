"""Parameter freezing by module alias.

A ``FreezeSpec(module, frozen)`` names an alias (``vision_encoder``, ``adapter``, ``transformer`` ...);
``module_patterns`` maps the alias to fnmatch patterns over fully-qualified parameter names (a name that is not an
alias is a pattern itself).  Later specs override earlier ones.  ``canonical_freeze_meta`` is what gets stored in checkpoint metadata so a resume
can detect a changed freeze set-up.

Parity: kempnerforge/training/freeze.py:35-136.
"""

from __future__ import annotations

import fnmatch
from collections.abc import Iterable

from torch import nn


def freeze_params(model: nn.Module, patterns: Iterable[str], frozen: bool = True) -> int:
    """Set ``requires_grad = not frozen`` on every parameter whose fully-qualified name matches a pattern.  Only
    parameters whose state differs are touched, and the return value is the number of ELEMENTS flipped (so a second
    identical call returns 0)."""
    patterns = list(patterns)
    flipped = 0
    for name, p in model.named_parameters():
        if p.requires_grad == frozen and any(fnmatch.fnmatch(name, pat) for pat in patterns):
            p.requires_grad_(not frozen)
            flipped += p.numel()
    return flipped


def apply_freeze_specs(model: nn.Module, specs, module_patterns: dict[str, list[str]] | None = None, *,
                       pattern_map: dict[str, list[str]] | None = None) -> dict[str, int]:
    """``spec.module`` is an alias looked up in ``module_patterns`` (also ``pattern_map=``); a name that is not an
    alias is used as an fnmatch pattern itself.  Returns {spec.module: parameters matched}."""
    module_patterns = module_patterns if module_patterns is not None else (pattern_map or {})
    counts = {}
    for spec in specs:
        counts[spec.module] = freeze_params(model, module_patterns.get(spec.module, [spec.module]), spec.frozen)
    return counts


def canonical_freeze_meta(specs) -> list[dict]:
    """Order-independent, de-duplicated description of a freeze list: the sorted set of (module, frozen) pairs, so two
    lists with the same pairs give byte-equal JSON (the form the reference stores in checkpoint metadata)."""
    pairs = sorted({(spec.module, bool(spec.frozen)) for spec in specs})
    return [{"module": m, "frozen": f} for m, f in pairs]


def effective_freeze(step=None, base=None, schedule=None, valid_modules=None):
    """Static freeze list overlaid by every schedule stage whose start_step <= step (later stages win per module).

    Two call forms: ``effective_freeze(step, base, schedule, valid_modules=None)`` with explicit lists (also by
    keyword), which raises ValueError for a module key outside ``valid_modules``, and ``effective_freeze(vlm_config,
    step)`` which takes both lists from a VLM config (``None`` config: no freezing).
    Parity: kempnerforge/training/freeze.py:91-140.
    """
    if isinstance(step, int) and not isinstance(step, bool):
        base, stages = list(base or []), list(schedule or [])
    elif step is None:          # effective_freeze(None, step): a model without a VLM section freezes nothing
        return []
    else:
        vlm_config, step = step, base
        base, stages = list(vlm_config.freeze), list(vlm_config.freeze_schedule)
    applied = [("base", spec) for spec in base]
    for stage in sorted(stages, key=lambda s: s.start_step):
        if stage.start_step <= step:
            applied.extend((f"stage at step {stage.start_step}", spec) for spec in stage.specs)
    latest = {}
    for where, spec in applied:
        if valid_modules is not None and spec.module not in valid_modules:
            raise ValueError(f"freeze module {spec.module!r} (from {where}) is not one of {sorted(valid_modules)}")
        latest[spec.module] = spec
    return list(latest.values())   # one spec per module, in order of first appearance
