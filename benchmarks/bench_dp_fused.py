"""Fused data-parallel kernels over NVLink peer memory, one rank per GPU, Llama-3-8B block shapes:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/bench_dp_fused.py

For every kernel: CUDA-event time (max over ranks, L2 flushed, barrier before each launch), the bytes that cross
NVLink into this GPU, and the fraction of the roofline  max(FLOPs / measured GEMM peak, NVLink bytes / link bandwidth).

  gemm_gather        weight-gathering GEMM (sharded parameters): QKV (+ rotary epilogue), O, gate|up (+ SwiGLU), down
                     against the plain GEMM on a resident weight and against pull-then-GEMM
  symm_rs_shard      reduce-scatter of one block's staged gradients into the gradient shard
  symm_rs_norm       resident plan: reduce-scatter fused with scaling, cast and the norm partial
  symm_adamw_bcast   resident plan: sharded AdamW fused with the publication of the new parameters

Peaks: MEASURED_PEAKS.json at the repository root when present (cuBLAS bf16 burst), else 1590 TFLOP/s; NVLink 770 GB/s
per direction (measured peer copy on this pool).  Prints one JSON line per kernel on rank 0.
"""

from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

LINK_GBS = 770.0


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    from kempnerforge_b200.comm import symmetric
    from kempnerforge_b200.ops import cuda as K

    dev = torch.device("cuda")
    peak = 1590.0
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as fh:
            peak = float(json.load(fh).get("bf16_tflops", peak))
    except OSError:
        pass
    flush = torch.empty(64 << 20, dtype=torch.int32, device=dev)

    def timeit(fn, n=8):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(n):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(e))
        t = torch.tensor(sorted(ts)[len(ts) // 2], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    def report(name, ms, flops, link_bytes, **extra):
        t_compute = flops / (peak * 1e12) * 1e3
        t_link = link_bytes / (LINK_GBS * 1e9) * 1e3
        bound = max(t_compute, t_link)
        if rank == 0:
            print(json.dumps({"kernel": name, "ranks": world, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1) if flops else None,
                              "nvlink_gb_in": round(link_bytes / 1e9, 4), "nvlink_gbs": round(link_bytes / ms / 1e6, 1),
                              "roofline_ms": round(bound, 4), "fraction_of_roofline": round(bound / ms, 3), **extra}), flush=True)

    alloc = symmetric.make_allocator(dist.group.WORLD)
    m, d, f, hq, hkv, hd, s = 8192, 4096, 14336, 32, 8, 128, 4096
    x = torch.randn(m, d, device=dev, dtype=torch.bfloat16)
    xf = torch.randn(m, f, device=dev, dtype=torch.bfloat16) * 0.1
    ang = torch.outer(torch.arange(s, device=dev).float(), 500000.0 ** (-torch.arange(0, hd, 2, device=dev).float() / hd))
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    flags = torch.zeros(8192, dtype=torch.int32, device=dev)

    def sharded(rows_list, k):
        """Symmetric shard buffer holding piece `rank` of every weight + a resident copy of the stacked operand."""
        total = sum(rows_list) * k
        full = torch.randn(sum(rows_list), k, device=dev, dtype=torch.bfloat16) * 0.02
        dist.broadcast(full, 0)
        shard = alloc(total // world, torch.bfloat16, dev)
        offs, acc, r0 = [], 0, 0
        for rows in rows_list:
            piece = rows * k // world
            offs.append(acc)
            shard[acc:acc + piece].copy_(full[r0:r0 + rows].reshape(-1)[rank * piece:(rank + 1) * piece])
            acc += piece
            r0 += rows
        symm = symmetric.lookup(shard)
        symm.barrier()
        stage = torch.empty(total, device=dev, dtype=torch.bfloat16)
        return full, {"symm": symm, "seg_rows": rows_list, "seg_src": offs, "stage": stage, "flags": flags}

    cases = [("qkv+rope", [hq * hd, hkv * hd, hkv * hd], d, 2), ("o", [d], d, 0), ("gate|up+swiglu", [f, f], d, 1), ("down", [d], f, 0)]
    for name, rows_list, k, epi in cases:
        full, plan = sharded(rows_list, k)
        a = xf if k == f else x
        n = rows_list[0] if epi == 1 else sum(rows_list)
        rope = (cos, sin, s, (hq + hkv) * hd, hd) if epi == 2 else None
        res = torch.randn(m, n, device=dev, dtype=torch.bfloat16) if epi == 0 else None

        def fused():
            return K.gemm_gather(a, plan, n, epi=epi, residual=res, rope=rope, want_gu=False)

        def plain():
            if epi == 1:
                return K.gemm_swiglu(a, full, want_gu=False)
            return K.gemm(a, full, residual=res, rope=rope, mode=2)

        offsets_full = [sum(rows_list[:i]) * k for i in range(len(rows_list))]

        def pull_then_gemm():
            K.symm_pull(plan["symm"], offsets_full, [r * k for r in rows_list], plan["seg_src"], plan["stage"])
            w = plan["stage"].view(sum(rows_list), k)
            if epi == 1:
                return K.gemm_swiglu(a, w, want_gu=False)
            return K.gemm(a, w, residual=res, rope=rope, mode=2)

        got, want = fused(), plain()
        got = got[0] if isinstance(got, tuple) else got
        want = want[0] if isinstance(want, tuple) else want
        same = bool(torch.equal(got, want))
        flops = 2.0 * m * sum(rows_list) * k
        link = sum(rows_list) * k * 2 * (world - 1) / world
        report(f"gemm_gather {name}", timeit(fused), flops, link, plain_gemm_ms=round(timeit(plain), 4),
               pull_then_gemm_ms=round(timeit(pull_then_gemm), 4), bit_identical_to_plain=same)
        del full, plan

    # gradient / parameter traffic of one block unit (218 M parameters)
    unit = 218_112_000 // (8 * world) * (8 * world)
    shard_n = unit // world
    gbuf = alloc(unit, torch.bfloat16, dev)
    gbuf.normal_()
    gs = symmetric.lookup(gbuf)
    gshard = torch.zeros(shard_n, device=dev, dtype=torch.bfloat16)
    gs.barrier()
    report("symm_rs_shard (one block)", timeit(lambda: K.symm_rs_shard(gs, [0], [unit], [0], gshard, False)), 0,
           shard_n * 2 * (world - 1))
    sq = torch.zeros(1, device=dev)
    report("symm_rs_norm (one block)", timeit(lambda: K.symm_rs_norm(gs, rank * shard_n, shard_n, sq, accumulate=False)), 0,
           shard_n * 2 * (world - 1))
    pbuf = alloc(unit, torch.bfloat16, dev)
    pbuf.normal_()
    ps = symmetric.lookup(pbuf)
    mom, var = torch.zeros(shard_n, device=dev, dtype=torch.bfloat16), torch.zeros(shard_n, device=dev, dtype=torch.bfloat16)
    ps.barrier()
    report("symm_adamw_bcast (one block)", timeit(lambda: K.symm_adamw_bcast(
        ps, gbuf[rank * shard_n:(rank + 1) * shard_n], mom, var, rank * shard_n, shard_n, unit, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1)),
        0, shard_n * 2 * (world - 1), note="bytes = what every GPU receives; multimem sends each value once")
    if rank == 0:
        print(json.dumps({"status_word": K.read_status(), "peak_tflops_used": peak, "link_gbs_used": LINK_GBS}))
    dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
