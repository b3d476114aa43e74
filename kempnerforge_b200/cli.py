"""Console entry points of the installed package (``kf-train``, ``kf-check-env``).

``kf-train configs/train/debug.toml --train.max_steps=20`` is ``python scripts/train.py ...`` without needing the
source tree on the path: first argument an optional TOML preset, then ``--section.key=value`` overrides
(the reference's scripts/train.py:4-18 contract).
"""

from __future__ import annotations

import sys


def train(argv: list[str] | None = None) -> int:
    from kempnerforge_b200.config import load_config
    from kempnerforge_b200.metrics.logger import get_logger
    from kempnerforge_b200.parallel.setup import destroy_distributed
    from kempnerforge_b200.resilience import log_job_info
    from kempnerforge_b200.training.trainer import Trainer

    argv = list(sys.argv[1:] if argv is None else argv)
    path = argv.pop(0) if argv and not argv[0].startswith("--") else None
    config = load_config(path, argv)
    get_logger("train")
    log_job_info()
    trainer = Trainer(config)
    try:
        result = trainer.fit()
    finally:
        destroy_distributed()
    return 0 if result.get("stop_reason") in (None, "signal") else 1


def check_env(argv: list[str] | None = None) -> int:
    """Environment report: interpreter, torch build, CUDA toolchain, GPUs, native library (scripts/check_env.py)."""
    import importlib.util
    from pathlib import Path

    script = Path(__file__).resolve().parent.parent / "scripts" / "check_env.py"
    if not script.exists():
        print("scripts/check_env.py is not part of this installation; run it from a source checkout", file=sys.stderr)
        return 2
    spec = importlib.util.spec_from_file_location("kf_check_env_cli", script)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return int(mod.main(argv))
