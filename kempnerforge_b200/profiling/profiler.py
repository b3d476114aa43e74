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
    ("matmul", ("gemm", "cublas", "nvjet", "cutlass", "tcgen05", "matmul", "_mm", "::mm", "bmm", "addmm")),
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


def _self_device_us(evt) -> float:
    """An event's own device time (children excluded, so a sum over events counts each kernel once)."""
    for attr in ("self_device_time_total", "self_cuda_time_total"):
        v = getattr(evt, attr, None)
        if isinstance(v, (int, float)):
            return float(v)
    return 0.0


def analyze_profiler(prof) -> dict:
    """Aggregate device time and FLOPs of a finished profile.

    Keys: ``totals_us`` / ``fractions`` per bucket (matmul, attention, fused_comm, comm, memory, other),
    ``top_kernels`` (name, bucket, device us, calls), ``total_us``; and, under the reference's names
    (kempnerforge/profiling/profiler.py:71-127), ``total_cuda_time_us``, ``matmul_time_us`` (GEMM + attention),
    ``comm_time_us`` (NCCL + fused compute-communication kernels), ``memory_time_us``, ``other_time_us``, the four
    ``*_pct`` shares, ``total_flops``, ``achieved_tflops``, ``peak_tflops`` and ``kernel_efficiency_pct``."""
    from kempnerforge_b200.metrics.mfu import get_gpu_peak_tflops

    totals = {bucket: 0.0 for bucket, _ in _BUCKETS}
    totals["other"] = 0.0
    kernels = []
    flops = 0
    for evt in prof.key_averages():
        if "profilerstep" in str(evt.key).lower():
            continue
        flops += int(getattr(evt, "flops", 0) or 0)
        dev_us = _self_device_us(evt)
        if not dev_us:
            continue
        bucket = categorize_kernel(evt.key)
        totals[bucket] += dev_us
        kernels.append((evt.key, bucket, dev_us, getattr(evt, "count", 0)))
    kernels.sort(key=lambda k: -k[2])
    total = sum(totals.values())
    denom = total or 1.0
    peak = get_gpu_peak_tflops()
    achieved = flops / (total / 1e6) / 1e12 if total > 0 else 0.0
    flat = {"matmul": totals["matmul"] + totals["attention"], "comm": totals["comm"] + totals["fused_comm"],
            "memory": totals["memory"], "other": totals["other"]}
    out = {"totals_us": totals, "fractions": {k: v / denom for k, v in totals.items()}, "top_kernels": kernels[:25],
           "total_us": denom, "total_cuda_time_us": total, "total_flops": flops, "achieved_tflops": achieved,
           "peak_tflops": peak, "kernel_efficiency_pct": 100 * achieved / peak if peak > 0 else 0.0}
    for k, v in flat.items():
        out[f"{k}_time_us"] = v
        out[f"{k}_pct"] = 100 * v / denom
    return out


def save_profiler_summary(stats: dict, prof, trace_dir: str) -> str:
    """Write ``<trace_dir>/summary.md`` (bucket shares, FLOP rate against the peak, top kernels); returns its path."""
    from datetime import datetime

    lines = ["# Profiling Summary", "", f"Generated {datetime.now():%Y-%m-%d %H:%M:%S}", "",
             "| category | device time (ms) | share |", "|---|---:|---:|"]
    if "totals_us" in stats:
        for k, v in stats["totals_us"].items():
            lines.append(f"| {k} | {v / 1e3:.2f} | {100 * stats['fractions'][k]:.1f}% |")
    else:
        for k in ("matmul", "comm", "memory", "other"):
            lines.append(f"| {k} | {stats.get(f'{k}_time_us', 0) / 1e3:.2f} | {stats.get(f'{k}_pct', 0.0):.1f}% |")
    lines += ["", f"Total device time: {stats.get('total_cuda_time_us', 0) / 1e3:.2f} ms; "
                  f"{stats.get('achieved_tflops', 0.0):.1f} TFLOP/s counted by the profiler against a peak of "
                  f"{stats.get('peak_tflops', 0.0):.0f} ({stats.get('kernel_efficiency_pct', 0.0):.1f}%)."]
    top = stats.get("top_kernels")
    if top is None:
        top = sorted(((e.key, categorize_kernel(e.key), _self_device_us(e), getattr(e, "count", 0))
                      for e in prof.key_averages()), key=lambda k: -k[2])[:25]
    lines += ["", "## Top kernels", "", "| kernel | category | device time (ms) | calls |", "|---|---|---:|---:|"]
    for name, bucket, us, n in top:
        lines.append(f"| `{str(name)[:90]}` | {bucket} | {us / 1e3:.2f} | {n} |")
    os.makedirs(trace_dir, exist_ok=True)
    path = os.path.join(trace_dir, "summary.md")
    with open(path, "w") as fh:
        fh.write("\n".join(lines) + "\n")
    return path


def print_profiler_summary(prof, trace_dir: str | None = None) -> dict:
    res = analyze_profiler(prof)
    lines = ["GPU time by category:"]
    for k, v in res["totals_us"].items():
        lines.append(f"  {k:<11}{v / 1e3:>10.2f} ms {100 * res['fractions'][k]:>6.1f}%")
    lines.append(f"  {res['achieved_tflops']:.1f} TFLOP/s counted by the profiler, peak {res['peak_tflops']:.0f} "
                 f"({res['kernel_efficiency_pct']:.1f}%)")
    lines.append("Top kernels:")
    for name, bucket, us, n in res["top_kernels"][:15]:
        lines.append(f"  {us / 1e3:>9.2f} ms  x{n:<6} [{bucket}] {str(name)[:90]}")
    log.info("\n%s", "\n".join(lines))
    if trace_dir:
        save_profiler_summary(res, prof, trace_dir)
    return res


_analyze_profiler, _save_profiler_summary = analyze_profiler, save_profiler_summary   # the reference's private spellings
