"""One full training step per optimizer on the 125 M model.
Parity: benchmarks/bench_optimizer.py:24-56 in the reference (AdamW fused/unfused, Lion,
schedule-free AdamW, Muon)."""

from __future__ import annotations

import torch

from benchmarks._common import batch_shape, bench_model_config, dtype_for
from benchmarks.runner import Case, print_results, run_suite

SUITE = "optimizer"


def cases(device: torch.device):
    from kempnerforge_b200.config import OptimizerConfig
    from kempnerforge_b200.models.transformer import Transformer
    from kempnerforge_b200.training.optimizer import build_optimizer

    cfg = bench_model_config(device)
    dt = dtype_for(device)
    b, s = batch_shape(device)
    ids = torch.randint(0, cfg.vocab_size, (b, s), device=device)
    labels = torch.randint(0, cfg.vocab_size, (b, s), device=device)
    menu = [("AdamW (fused flat kernel)", OptimizerConfig(name="adamw", lr=3e-4, fused=True)),
            ("AdamW (unfused)", OptimizerConfig(name="adamw", lr=3e-4, fused=False)),
            ("Lion", OptimizerConfig(name="lion", lr=1e-4)),
            ("Schedule-free AdamW", OptimizerConfig(name="schedule_free_adamw", lr=3e-4)),
            ("Muon", OptimizerConfig(name="muon", lr=0.02))]
    for label, ocfg in menu:
        holder: dict = {}

        def setup(holder=holder, ocfg=ocfg):
            if "model" not in holder:
                holder["model"] = Transformer(cfg).to(device=device, dtype=dt)
                holder["opt"] = build_optimizer(holder["model"], ocfg)

        def step(holder=holder):
            m, o = holder["model"], holder["opt"]
            loss = m.compute_loss(ids, labels)
            (loss[0] if isinstance(loss, tuple) else loss).backward()
            o.step()
            o.zero_grad(set_to_none=True)

        yield Case(f"train step: {label}", step, tokens_per_iter=b * s, setup=setup, teardown=holder.clear)


if __name__ == "__main__":
    dev = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    print_results(run_suite(SUITE, dev), "optimizer")
