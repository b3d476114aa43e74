#!/usr/bin/env python
"""Evaluate a checkpoint on held-out data and print JSON metrics.

    python scripts/eval.py cfg.toml --checkpoint.load_path=checkpoints/latest --eval.dataset_path=/data/val
    torchrun --nproc-per-node 4 scripts/eval.py cfg.toml ...

The model is built without activation checkpointing or fp8, the optimizer state is not loaded.
Same contract as the reference's scripts/eval.py:85-176.
"""

from __future__ import annotations

import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402

from kempnerforge_b200.checkpoint import CheckpointManager  # noqa: E402
from kempnerforge_b200.config import load_config  # noqa: E402
from kempnerforge_b200.parallel.parallel import build_parallel_model  # noqa: E402
from kempnerforge_b200.parallel.setup import destroy_distributed, get_dp_info, get_world_info, init_distributed  # noqa: E402
from kempnerforge_b200.training.eval import build_eval_dataloader, run_eval  # noqa: E402


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    path = argv.pop(0) if argv and not argv[0].startswith("--") else None
    cfg = load_config(path, argv)
    cfg.eval.enabled = True
    rank, _, world = get_world_info()
    mesh = init_distributed(cfg.distributed, cfg.train.seed)
    cfg.validate(world)
    device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    model = build_parallel_model(cfg.model, device, mesh, ac_mode="none", param_dtype=cfg.train.param_dtype, fp8=False)
    dummy = torch.optim.SGD([p for p in model.parameters() if p.requires_grad], lr=0.0)
    mgr = CheckpointManager(cfg.checkpoint, model, dummy)
    if mgr._resolve_load_path(None) is None:     # evaluating freshly initialised weights is never what was asked for
        where = cfg.checkpoint.load_path or cfg.checkpoint.dir
        print(f"error: no checkpoint found at {where!r}; set --checkpoint.load_path or --checkpoint.dir", file=sys.stderr)
        destroy_distributed()
        return 1
    step, tokens, _ = mgr.load(exclude_keys=["optimizer"])
    dp_rank, dp_size = get_dp_info(mesh)
    loader = build_eval_dataloader(cfg, dp_rank, dp_size)
    metrics = run_eval(model, loader, cfg, device)
    if rank == 0:
        print(json.dumps({"step": step, "tokens_seen": tokens, **metrics}))
    destroy_distributed()
    return 0


if __name__ == "__main__":
    sys.exit(main())
