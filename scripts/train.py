#!/usr/bin/env python
"""Training entry point.

    python scripts/train.py configs/train/debug.toml --train.max_steps=20
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 scripts/train.py configs/train/7b.toml

The first argument is a TOML preset (optional); every further ``--section.key=value`` overrides it.
Same contract as the reference's scripts/train.py:4-18,69-77.
"""

from __future__ import annotations

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from kempnerforge_b200.config import load_config  # noqa: E402
from kempnerforge_b200.metrics.logger import get_logger  # noqa: E402
from kempnerforge_b200.parallel.setup import destroy_distributed  # noqa: E402
from kempnerforge_b200.resilience import log_job_info  # noqa: E402
from kempnerforge_b200.training.trainer import Trainer  # noqa: E402


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    path = None
    if argv and not argv[0].startswith("--"):
        path = argv.pop(0)
    config = load_config(path, argv)
    log = get_logger("train")
    log_job_info()
    trainer = Trainer(config)
    try:
        result = trainer.fit()
    finally:
        destroy_distributed()
    return 0 if result.get("stop_reason") in (None, "signal") else 1


if __name__ == "__main__":
    sys.exit(main())
