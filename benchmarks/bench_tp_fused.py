"""Fused tensor-parallel kernels (all-gather -> GEMM, GEMM -> reduce-scatter) against GEMM + NCCL, one rank per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 benchmarks/bench_tp_fused.py
"""
import os
import sys

import torch
import torch.distributed as dist
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl")
from kempnerforge_b200.comm.fused_tp import AgGemmContext, GemmRSContext
from kempnerforge_b200.ops import cuda as K
dev = torch.device("cuda")
B, S, D, F = 2, 4096, 4096, 14336
T = B * S
flush = torch.empty(64 << 20, dtype=torch.int32, device=dev)
def timeit(fn, n=8):
    for _ in range(3): fn()
    ts = []
    for _ in range(n):
        flush.zero_(); dist.barrier(); torch.cuda.synchronize()
        a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); e.record(); torch.cuda.synchronize(); ts.append(a.elapsed_time(e))
    t = torch.tensor(sum(ts) / len(ts), device=dev); dist.all_reduce(t, op=dist.ReduceOp.MAX); return t.item()
# row-parallel down projection: x [T, F/tp] @ w [D, F/tp]^T -> reduce-scatter
x = torch.randn(T, F // world, device=dev, dtype=torch.bfloat16); w = torch.randn(D, F // world, device=dev, dtype=torch.bfloat16) * 0.02
rs = GemmRSContext(dist.group.WORLD, dev, T, D)
out_rs = torch.empty(T // world, D, device=dev, dtype=torch.bfloat16)
t_f = timeit(lambda: K.gemm_reduce_scatter(x, w, rs, S, out=out_rs))
full = torch.empty(T, D, device=dev, dtype=torch.bfloat16)
def base_rs():
    K.gemm(x, w, out=full); dist.reduce_scatter_tensor(out_rs, full)
t_b = timeit(base_rs)
t_g = timeit(lambda: K.gemm(x, w, out=full)); t_g1 = timeit(lambda: K.gemm(x, w, out=full, mode=1))
if rank == 0: print(f"GEMM->RS  T={T} D={D} Kl={F//world}: fused {t_f:.3f} ms | gemm+nccl {t_b:.3f} ms | gemm alone {t_g:.3f} ms (1-CTA tiles {t_g1:.3f})")
# column-parallel gate|up: x_shard [T/tp, D] gathered, w [2F/tp, D]
xs = torch.randn(T // world, D, device=dev, dtype=torch.bfloat16); w2 = torch.randn(2 * F // world, D, device=dev, dtype=torch.bfloat16) * 0.02
ag = AgGemmContext(dist.group.WORLD, dev, T, D)
y = torch.empty(T, 2 * F // world, device=dev, dtype=torch.bfloat16)
t_f = timeit(lambda: K.all_gather_gemm(xs, w2, ag, S, out=y))
xg = torch.empty(T, D, device=dev, dtype=torch.bfloat16)
def base_ag():
    dist.all_gather_into_tensor(xg, xs); K.gemm(xg, w2, out=y)
t_b = timeit(base_ag)
t_g = timeit(lambda: K.gemm(xg, w2, out=y)); t_g1 = timeit(lambda: K.gemm(xg, w2, out=y, mode=1))
if rank == 0: print(f"AG->GEMM  T={T} K={D} Nl={2*F//world}: fused {t_f:.3f} ms | nccl+gemm {t_b:.3f} ms | gemm alone {t_g:.3f} ms (1-CTA tiles {t_g1:.3f})  status={K.read_status()}")
dist.destroy_process_group()
