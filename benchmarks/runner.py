"""Micro-benchmark harness: device-timed loops, a results table and JSON output.

    python benchmarks/runner.py                      # every suite
    python benchmarks/runner.py --suite forward moe  # a selection
    python benchmarks/runner.py --output results.json

Each suite module exposes ``SUITE`` (a name) and ``cases(device)`` which yields ``Case`` objects; the
harness owns warm-up, timing (CUDA events on the launching stream, one L2 flush between timed
iterations, a synchronize on both sides) and memory accounting, so every case is measured the same way.
On a machine without a GPU the same cases run on the CPU with wall-clock timing, which keeps the
harness testable.

Parity: benchmarks/runner.py:30-131 in the reference (``BenchmarkResult``, ``run_benchmark`` with
warmup=3 / iterations=10, table + JSON); the case/suite split and the L2 flush are ours.
"""

from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import sys
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Iterable, Iterator

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SUITES = ("forward", "moe", "optimizer", "data", "kernels")
_L2_BYTES = 192 << 20  # larger than the 126 MB L2 of a B200


@dataclass
class Case:
    """One thing to time. ``fn`` runs one iteration; ``setup`` (optional) runs before each, untimed."""

    name: str
    fn: Callable[[], None]
    tokens_per_iter: int = 0
    flops_per_iter: float = 0.0
    bytes_per_iter: float = 0.0
    host_timed: bool = False          # data-loading cases: wall clock, no device work
    setup: Callable[[], None] | None = None
    teardown: Callable[[], None] | None = None


@dataclass
class BenchmarkResult:
    name: str
    step_time_ms: float = 0.0
    step_time_ms_min: float = 0.0
    tokens_per_sec: float = 0.0
    peak_memory_gb: float = 0.0
    extra: dict[str, float] = field(default_factory=dict)

    def row(self) -> str:
        cells = [f"{self.name:<44}", f"{self.step_time_ms:>10.3f} ms"]
        cells.append(f"{self.tokens_per_sec:>14,.0f} tok/s" if self.tokens_per_sec else " " * 20)
        cells.append(f"{self.peak_memory_gb:>7.2f} GB" if self.peak_memory_gb else " " * 10)
        cells.extend(f"{k}={v:.4g}" for k, v in self.extra.items())
        return " | ".join(cells)

    __str__ = row


class _Flusher:
    """Writes a buffer larger than L2 so that the next timed iteration starts cold."""

    def __init__(self, device: torch.device) -> None:
        self.buf = torch.empty(_L2_BYTES // 4, dtype=torch.int32, device=device) if device.type == "cuda" else None

    def __call__(self) -> None:
        if self.buf is not None:
            self.buf.zero_()


def run_benchmark(case: Case | Callable[[], None], warmup: int = 3, iterations: int = 10, *,
                  name: str | None = None, tokens_per_iter: int = 0, device: torch.device | None = None,
                  flush_l2: bool = True) -> BenchmarkResult:
    """Times one case. Accepts a bare callable plus ``name``/``tokens_per_iter`` for quick use."""
    if not isinstance(case, Case):
        case = Case(name or "benchmark", case, tokens_per_iter=tokens_per_iter)
    device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
    on_gpu = device.type == "cuda" and not case.host_timed
    flush = _Flusher(device) if (on_gpu and flush_l2) else (lambda: None)
    for _ in range(max(warmup, 0)):
        if case.setup:
            case.setup()
        case.fn()
    times: list[float] = []
    if on_gpu:
        torch.cuda.synchronize(device)
        torch.cuda.reset_peak_memory_stats(device)
        for _ in range(iterations):
            if case.setup:
                case.setup()
            flush()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            case.fn()
            stop.record()
            torch.cuda.synchronize(device)
            times.append(start.elapsed_time(stop))
        peak = torch.cuda.max_memory_allocated(device) / 2**30
    else:
        for _ in range(iterations):
            if case.setup:
                case.setup()
            t0 = time.perf_counter()
            case.fn()
            times.append((time.perf_counter() - t0) * 1e3)
        peak = 0.0
    if case.teardown:
        case.teardown()
    mean = statistics.fmean(times)
    res = BenchmarkResult(case.name, step_time_ms=mean, step_time_ms_min=min(times), peak_memory_gb=peak)
    if case.tokens_per_iter:
        res.tokens_per_sec = case.tokens_per_iter / (mean * 1e-3)
    if case.flops_per_iter:
        res.extra["tflops"] = case.flops_per_iter / (mean * 1e-3) / 1e12
    if case.bytes_per_iter:
        res.extra["gb_per_s"] = case.bytes_per_iter / (mean * 1e-3) / 1e9
    return res


def run_suite(suite: str, device: torch.device, warmup: int = 3, iterations: int = 10) -> list[BenchmarkResult]:
    mod = importlib.import_module(f"benchmarks.bench_{suite}")
    out: list[BenchmarkResult] = []
    cases: Iterable[Case] = mod.cases(device)
    for case in cases:
        out.append(run_benchmark(case, warmup, iterations, device=device))
        if device.type == "cuda":
            torch.cuda.empty_cache()
    return out


def print_results(results: list[BenchmarkResult], title: str = "Benchmark results") -> None:
    bar = "=" * 110
    print(f"\n{bar}\n{title}\n{bar}")
    for r in results:
        print(r.row())
    print(bar)


def save_results(results: list[BenchmarkResult], path: str) -> None:
    meta = {"torch": torch.__version__, "device": torch.cuda.get_device_name(0) if torch.cuda.is_available() else "cpu",
            "time": time.strftime("%Y-%m-%dT%H:%M:%S")}
    with open(path, "w") as f:
        json.dump({"meta": meta, "results": [asdict(r) for r in results]}, f, indent=2)


def iter_suites(selected: list[str] | None) -> Iterator[str]:
    for s in selected or SUITES:
        if s not in SUITES:
            raise SystemExit(f"unknown suite '{s}' (choose from {', '.join(SUITES)})")
        yield s


def main(argv: list[str] | None = None) -> list[BenchmarkResult]:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--suite", nargs="*", default=None, help=f"subset of: {' '.join(SUITES)}")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iterations", type=int, default=10)
    ap.add_argument("--output", default=None, help="write results as JSON to this path")
    args = ap.parse_args(argv)
    device = torch.device("cuda" if torch.cuda.is_available() else "cpu")
    everything: list[BenchmarkResult] = []
    for suite in iter_suites(args.suite):
        res = run_suite(suite, device, args.warmup, args.iterations)
        print_results(res, f"{suite} ({device})")
        everything.extend(res)
    if args.output:
        save_results(everything, args.output)
        print(f"saved {len(everything)} results to {args.output}")
    return everything


if __name__ == "__main__":
    # run through the importable module so that suites and harness share one ``Case`` class
    from benchmarks.runner import main as _main

    _main()
