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

from kempnerforge_b200.cli import train as main  # noqa: E402

if __name__ == "__main__":
    sys.exit(main())
