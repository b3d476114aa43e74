"""Attention backward on the Llama-3-8B shape in both dQ accumulation modes (per-element red.global, bulk tensor
reduction), CUDA events with an L2 flush between launches:

    python benchmarks/bench_attn_bwd_modes.py
"""
import math, sys, torch
import os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kempnerforge_b200.ops import cuda as K
b, s, h, hkv, hd = 2, 4096, 32, 8, 128
qkv = torch.randn(b, s, h + 2 * hkv, hd, device="cuda", dtype=torch.bfloat16)
q, k, v = qkv[:, :, :h], qkv[:, :, h:h + hkv], qkv[:, :, h + hkv:]
scale = 1 / math.sqrt(hd)
flush = torch.empty(64 << 20, dtype=torch.int32, device="cuda")
def timeit(fn, n=10):
    for _ in range(3): fn()
    ts = []
    for _ in range(n):
        flush.zero_()
        a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); e.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(e))
    return sorted(ts)[len(ts) // 2]
flops = 4 * b * h * s * s * hd / 2
dout = torch.randn(b, s, h, hd, device="cuda", dtype=torch.bfloat16)
out, lse = K.attn_fwd(q, k, v, True, None, scale)
res = {}
for mode in (0, 1, 0, 1):
    K.attn_bwd_dq_mode(mode)
    tb = timeit(lambda: K.attn_bwd(dout, q, k, v, out, lse, True, None, scale))
    res[mode] = K.attn_bwd(dout, q, k, v, out, lse, True, None, scale)
    print(f"native bwd dq_mode={mode}  {tb:.3f} ms  {2.5 * flops / tb / 1e9:.0f} TFLOP/s  status={K.read_status()}")
for a, c, n in zip(res[0], res[1], ("dq", "dk", "dv")):
    print(n, "rel diff between modes", ((a.float() - c.float()).norm() / a.float().norm()).item())
