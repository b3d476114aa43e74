"""``torch.profiler`` wrapper with a kernel-time breakdown.

The profile covers steps [start_step, end_step): wait = start_step - 1, warm-up = 1, active =
end_step - start_step, one repetition; traces go to ``trace_dir`` for TensorBoard / Perfetto.
The summary buckets device time by kernel name into matmul, fused compute+communication (our
``kf_*`` kernels that move data between GPUs), communication (NCCL), memory and other, and is also
written as ``summary.md``.

Parity: kempnerforge/profiling/profiler.py:21-255.
"""

from __future__ import annotations

import os

import torch

from kempnerforge_b200.metrics.logger import get_logger

log = get_logger("profiler")

_BUCKETS = (
    ("fused_comm", ("kf_ag_gemm", "kf_gemm_rs", "kf_rs_adamw", "kf_ep_put", "kf_ep_move", "kf_symm")),
    ("attention", ("kf_attn", "flash", "fmha", "sdpa")),
    ("matmul", ("gemm", "cublas", "nvjet", "cutlass", "tcgen05", "matmul", "_mm")),
    ("comm", ("nccl", "allreduce", "all_reduce", "allgather", "all_gather", "reduce_scatter", "alltoall")),
    ("memory", ("memcpy", "memset")),
)


def categorize_kernel(name: str) -> str:
    low = name.lower()
    for bucket, keys in _BUCKETS:
        if any(k in low for k in keys):
            return bucket
    return "other"


def build_profiler(config, rank: int = 0):
    """A configured ``torch.profiler.profile`` or None when profiling is off."""
    if not config.enable:
        return None
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    wait = max(0, config.start_step - 1)
    active = max(1, config.end_step - config.start_step)
    trace_dir = os.path.join(config.trace_dir, f"rank{rank}")
    os.makedirs(trace_dir, exist_ok=True)
    return torch.profiler.profile(
        activities=acts,
        schedule=torch.profiler.schedule(wait=wait, warmup=1, active=active, repeat=1),
        on_trace_ready=torch.profiler.tensorboard_trace_handler(trace_dir),
        record_shapes=True,
        profile_memory=True,
        with_flops=True,
    )


def analyze_profiler(prof) -> dict:
    totals = {"matmul": 0.0, "fused_comm": 0.0, "comm": 0.0, "memory": 0.0, "other": 0.0}
    kernels = []
    for evt in prof.key_averages():
        dev_us = getattr(evt, "device_time_total", None)
        if dev_us is None:
            dev_us = getattr(evt, "cuda_time_total", 0.0)
        if not dev_us:
            continue
        bucket = categorize_kernel(evt.key)
        totals[bucket] += dev_us
        kernels.append((evt.key, bucket, dev_us, evt.count))
    kernels.sort(key=lambda k: -k[2])
    total = sum(totals.values()) or 1.0
    return {"totals_us": totals, "fractions": {k: v / total for k, v in totals.items()},
            "top_kernels": kernels[:25], "total_us": total}


def print_profiler_summary(prof, trace_dir: str | None = None) -> dict:
    res = analyze_profiler(prof)
    lines = ["# Profiler summary", "", "| category | device time (ms) | share |", "|---|---:|---:|"]
    for k, v in res["totals_us"].items():
        lines.append(f"| {k} | {v / 1e3:.2f} | {100 * res['fractions'][k]:.1f}% |")
    lines += ["", "## Top kernels", "", "| kernel | category | device time (ms) | calls |", "|---|---|---:|---:|"]
    for name, bucket, us, n in res["top_kernels"]:
        lines.append(f"| `{name[:90]}` | {bucket} | {us / 1e3:.2f} | {n} |")
    text = "\n".join(lines)
    log.info("\n%s", text)
    if trace_dir:
        os.makedirs(trace_dir, exist_ok=True)
        with open(os.path.join(trace_dir, "summary.md"), "w") as fh:
            fh.write(text + "\n")
    return res
