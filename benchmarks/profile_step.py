"""Per-kernel device time of one training step of the Llama-3-8B-shape benchmark (torch profiler, CUDA activities).

    python benchmarks/profile_step.py [--out step_profile.txt] [--model llama3_8b|moe_8x|moe_fine|tiny] [--batch-size 2]
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
    # the mixture-of-experts benchmark models of bench.py, all experts on this rank unless launched with several ranks
    "moe_8x": dict(dim=2048, n_layers=24, n_heads=16, n_kv_heads=16, vocab_size=102400, ffn_hidden_dim=5632,
                   max_seq_len=4096, rope_theta=500000.0, num_experts=8, moe_top_k=2, moe_router="softmax_topk",
                   moe_packed_experts=True),
    "moe_fine": dict(dim=2048, n_layers=24, n_heads=16, n_kv_heads=16, vocab_size=102400, ffn_hidden_dim=10944,
                     max_seq_len=4096, rope_theta=500000.0, num_experts=64, moe_top_k=6, moe_router="sigmoid_topk",
                     moe_shared_experts=2, moe_router_z_loss_weight=1e-3, moe_first_k_dense=1,
                     moe_expert_ffn_multiplier=1408.0 / 10944.0, moe_packed_experts=True),
}


def stream_report(prof, n_gaps: int) -> list[str]:
    """Busy time per CUDA stream and the longest idle gaps of the busiest one (what the compute stream waited for)."""
    try:
        events = prof.profiler.kineto_results.events()
    except AttributeError:
        return []
    per_stream: dict[int, list] = {}
    for e in events:
        if str(e.device_type()).endswith("CUDA") and e.duration_ns() > 0 and "Memcpy" not in e.name() and "Memset" not in e.name():
            per_stream.setdefault(e.device_resource_id(), []).append((e.start_ns(), e.start_ns() + e.duration_ns(), e.name()))
    if not per_stream:
        return []
    out = ["", "streams (busy ms, kernels):"]
    busiest, best = None, -1
    for sid, evs in per_stream.items():
        busy = sum(b - a for a, b, _ in evs) / 1e6
        out.append(f"  stream {sid}: {busy:8.2f} ms in {len(evs)} kernels")
        if busy > best:
            busiest, best = sid, busy
    evs = sorted(per_stream[busiest])
    span = (evs[-1][1] - evs[0][0]) / 1e6
    gaps = sorted(((evs[i + 1][0] - evs[i][1], evs[i][2], evs[i + 1][2]) for i in range(len(evs) - 1)), reverse=True)
    idle = sum(g[0] for g in gaps if g[0] > 0) / 1e6
    out.append(f"busiest stream {busiest}: span {span:.2f} ms, idle inside the span {idle:.2f} ms; longest gaps:")
    for g, before, after in gaps[:n_gaps]:
        out.append(f"  {g / 1e6:7.3f} ms between {before[:60]} -> {after[:60]}")
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3_8b", choices=sorted(SHAPES))
    ap.add_argument("--out", default=None)
    ap.add_argument("--top", type=int, default=40)
    ap.add_argument("--batch-size", type=int, default=2)
    ap.add_argument("--param-sharding", default="resident", choices=("auto", "resident", "sharded"))
    ap.add_argument("--gaps", type=int, default=12, help="list this many of the longest idle gaps of the busiest stream")
    args = ap.parse_args()
    from kempnerforge_b200.config import config_from_dict
    from kempnerforge_b200.training.trainer import Trainer

    shape = SHAPES[args.model]
    seq = shape["max_seq_len"]
    cfg = config_from_dict({"model": shape,
                            "train": {"batch_size": args.batch_size, "seq_len": seq, "max_steps": 100, "mixed_precision": "bf16",
                                      "activation_checkpointing": "full", "seed": 0},
                            "scheduler": {"warmup_steps": 10}, "metrics": {"log_interval": 1000},
                            "distributed": {"dp_shard": int(os.environ.get("WORLD_SIZE", "1")),
                                            "param_sharding": args.param_sharding}})
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    trainer = Trainer(cfg, init_dist=world > 1)

    def batch():
        tok = torch.randint(0, shape["vocab_size"], (args.batch_size, seq + 1), device="cuda")
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
    lines += stream_report(prof, args.gaps)
    text = "\n".join(lines)
    if rank == 0:
        print(text)
    if args.out and rank == 0:
        with open(args.out, "w") as f:
            f.write(text + "\n")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
