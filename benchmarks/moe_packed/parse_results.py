"""Tabulates logs of the packed-vs-unpacked MoE matrix: one row per expert count with both variants
and the speed-up. Parity: benchmarks/moe_packed/parse_results.py in the reference.

    python benchmarks/moe_packed/parse_results.py benchmarks/results/moe_packed
"""

from __future__ import annotations

import glob
import os
import re
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from benchmarks.cluster_bench import parse_log  # noqa: E402


def collect(directory: str) -> dict[int, dict[str, dict]]:
    table: dict[int, dict[str, dict]] = {}
    for path in sorted(glob.glob(os.path.join(directory, "*.log"))):
        m = re.search(r"_E(\d+)_(packed|unpacked)\.log$", path)
        if not m:
            continue
        parsed = parse_log(open(path).read())
        if parsed:
            table.setdefault(int(m[1]), {})[m[2]] = parsed
    return table


def main(argv: list[str]) -> int:
    directory = argv[1] if len(argv) > 1 else "benchmarks/results/moe_packed"
    table = collect(directory)
    if not table:
        print(f"no parsable logs in {directory}")
        return 1
    print(f"{'experts':>8}{'unpacked tok/s':>16}{'packed tok/s':>14}{'speed-up':>10}{'mem unpacked':>14}{'mem packed':>12}")
    for e in sorted(table):
        u, p = table[e].get("unpacked"), table[e].get("packed")
        cell = lambda r, k, fmt: format(r[k], fmt) if r else "-"  # noqa: E731
        ratio = f"{p['tokens_per_sec'] / u['tokens_per_sec']:.2f}x" if u and p else "-"
        print(f"{e:>8}{cell(u, 'tokens_per_sec', ',.0f'):>16}{cell(p, 'tokens_per_sec', ',.0f'):>14}{ratio:>10}"
              f"{cell(u, 'peak_mem_gb', '.1f'):>14}{cell(p, 'peak_mem_gb', '.1f'):>12}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main(sys.argv))
