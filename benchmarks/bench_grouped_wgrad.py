"""Native grouped weight-gradient kernel against torch._grouped_mm on the MoE 8-expert shapes, CUDA events with an L2
flush between launches:

    python benchmarks/bench_grouped_wgrad.py
"""
import sys
import torch
import os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kempnerforge_b200.ops import cuda as kc

torch.manual_seed(0)
def t(fn, it=10):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3): fn()
    ts = []
    for _ in range(it):
        flush.zero_()
        s, e = torch.cuda.Event(True), torch.cuda.Event(True)
        s.record(); fn(); e.record(); torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    return sorted(ts)[len(ts) // 2]

for E, rows, m, n in [(8, 16384, 2048, 5632), (8, 16384, 5632, 2048), (4, 16384, 2048, 5632)]:
    counts = torch.full((E,), rows // E, device="cuda")
    counts[0] -= 37; counts[-1] += 37
    offsets = torch.zeros(E + 1, dtype=torch.int32, device="cuda"); offsets[1:] = counts.cumsum(0)
    a = torch.randn(rows, m, device="cuda", dtype=torch.bfloat16)
    b = torch.randn(rows, n, device="cuda", dtype=torch.bfloat16)
    got = kc.grouped_wgrad(a, b, offsets)
    want = torch._grouped_mm(a.t(), b, offs=offsets[1:])
    err = ((got.float() - want.float()).norm() / want.float().norm()).item()
    t1 = t(lambda: kc.grouped_wgrad(a, b, offsets))
    t2 = t(lambda: torch._grouped_mm(a.t(), b, offs=offsets[1:]))
    fl = 2.0 * rows * m * n
    print(f"E={E} rows={rows} m={m} n={n}: native {t1:.3f} ms ({fl/t1/1e9:.0f} TF) library {t2:.3f} ms ({fl/t2/1e9:.0f} TF) rel err {err:.2e} status {kc.read_status()}")
