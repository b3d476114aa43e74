"""tcgen05 GEMM against torch.matmul (cuBLAS) on the Llama-3-8B shapes: forward, input gradient and weight gradient of
every Linear, CUDA events, 256 MiB L2 flush between launches, median of 20:

    python benchmarks/bench_gemm_shapes.py [mode]      # mode 1: single-CTA tiles, 2: CTA pairs, 0: automatic
"""
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kempnerforge_b200.ops import cuda as kc
from kempnerforge_b200.ops.build import build
build()
dev = "cuda"
MODE = int(sys.argv[1]) if len(sys.argv) > 1 else 0
def timeit(fn, iters=20, warm=5):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(warm): fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record(); torch.cuda.synchronize()
        ts.append(s.elapsed_time(e))
    ts.sort()
    return ts[len(ts)//2]
T = 8192
shapes = [("qkv", T, 6144, 4096), ("o", T, 4096, 4096), ("gateup", T, 28672, 4096), ("down", T, 4096, 14336), ("head4k", 4096, 128256, 4096)]
res = []
for name, M, N, K in shapes:
    for mode in ("fwd", "dgrad", "wgrad"):
        if mode == "fwd":
            a = torch.randn(M, K, device=dev, dtype=torch.bfloat16); b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
            mine = lambda: kc.gemm(a, b, True, True, mode=MODE); ref = lambda: a @ b.t(); flops = 2*M*N*K
        elif mode == "dgrad":   # dX[M,K] = dY[M,N] W[N,K]
            a = torch.randn(M, N, device=dev, dtype=torch.bfloat16); b = torch.randn(N, K, device=dev, dtype=torch.bfloat16)
            mine = lambda: kc.gemm(a, b, True, False, mode=MODE); ref = lambda: a @ b; flops = 2*M*N*K
        else:                   # dW[N,K] = dY^T X
            a = torch.randn(M, N, device=dev, dtype=torch.bfloat16); b = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            mine = lambda: kc.gemm(a, b, False, False, mode=MODE); ref = lambda: a.t() @ b; flops = 2*M*N*K
        got, want = mine().float(), ref().float()
        err = ((got - want).abs().max() / want.abs().max()).item()
        tm, tr = timeit(mine), timeit(ref)
        r = dict(gemm_mode=MODE, name=name, mode=mode, M=M, N=N, K=K, ms_mine=tm, ms_cublas=tr, tf_mine=flops/tm/1e9, tf_cublas=flops/tr/1e9, relerr=err)
        print(json.dumps(r), flush=True); res.append(r)
print("status", kc.read_status())
if len(sys.argv) > 2:
    json.dump(res, open(sys.argv[2], "w"), indent=1)
