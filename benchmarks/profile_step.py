"""Per-kernel device time of one training step of the Llama-3-8B-shape benchmark (torch profiler, CUDA activities).

    python benchmarks/profile_step.py [--out step_profile.txt] [--model llama3_8b|tiny]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/profile_step.py
        (sharded data parallel over the ranks; rank 0 reports its own kernels and the gaps between them)

Three warm-up steps, one profiled step; kernels are listed by total device time.  The absolute times include profiler
overhead: use the shares, and `bench.py` for the step time itself.
"""

from __future__ import annotations

import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SHAPES = {
    "llama3_8b": dict(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, vocab_size=128256, ffn_hidden_dim=14336,
                      max_seq_len=4096, rope_theta=500000.0),
    "tiny": dict(dim=512, n_layers=4, n_heads=8, n_kv_heads=2, vocab_size=4096, ffn_hidden_dim=1536, max_seq_len=512),
}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3_8b", choices=sorted(SHAPES))
    ap.add_argument("--out", default=None)
    ap.add_argument("--top", type=int, default=40)
    args = ap.parse_args()
    from kempnerforge_b200.config import config_from_dict
    from kempnerforge_b200.training.trainer import Trainer

    shape = SHAPES[args.model]
    seq = shape["max_seq_len"]
    cfg = config_from_dict({"model": shape,
                            "train": {"batch_size": 2, "seq_len": seq, "max_steps": 100, "mixed_precision": "bf16",
                                      "activation_checkpointing": "full", "seed": 0},
                            "scheduler": {"warmup_steps": 10}, "metrics": {"log_interval": 1000},
                            "distributed": {"dp_shard": int(os.environ.get("WORLD_SIZE", "1"))}})
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    trainer = Trainer(cfg, init_dist=world > 1)

    def batch():
        tok = torch.randint(0, shape["vocab_size"], (2, seq + 1), device="cuda")
        return {"input_ids": tok[:, :-1].contiguous(), "labels": tok[:, 1:].contiguous()}

    for _ in range(3):
        trainer.train_step([batch()])
    torch.cuda.synchronize()
    acts = [torch.profiler.ProfilerActivity.CUDA, torch.profiler.ProfilerActivity.CPU]
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.profiler.profile(activities=acts) as prof:
        start.record()
        trainer.train_step([batch()])
        end.record()
        torch.cuda.synchronize()
    step_ms = start.elapsed_time(end)
    rows = []
    for e in prof.key_averages():
        us = getattr(e, "device_time_total", 0) or 0
        if us > 0 and e.device_type == torch.autograd.DeviceType.CUDA:
            rows.append((us, e.count, e.key))
    rows.sort(reverse=True)
    total = sum(r[0] for r in rows)
    lines = [f"ranks {world}; profiled step {step_ms:.1f} ms on the stream clock (with profiler overhead); "
             f"total device kernel time {total / 1e3:.1f} ms (kernels on different streams overlap)"]
    lines += [f"{us / 1e3:9.2f} ms {100 * us / total:5.1f}% x{n:5d} {key[:110]}" for us, n, key in rows[: args.top]]
    text = "\n".join(lines)
    if rank == 0:
        print(text)
    if args.out and rank == 0:
        with open(args.out, "w") as f:
            f.write(text + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
