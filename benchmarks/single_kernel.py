"""One native kernel on one workload, timed with CUDA events (median of ``--iters`` launches after ``--warmup``,
L2 flushed between launches).  Each workload is small enough (a few hundred MB, a handful of launches) to be the
subject of a profiler capture as well:

    python benchmarks/single_kernel.py gemm
    python benchmarks/single_kernel.py attn_bwd --dq-mode red --iters 5

Workloads (Llama-3-8B shapes unless noted): gemm (CTA-pair tiles, 8192 x 6144 x 4096), gemm_1cta, gemm_swiglu,
gemm_rope (QKV projection with the rotary embedding in the epilogue), gemm_fp8 (tensorwise-scaled e4m3, same shape),
fp8_cast (abs-max + cast of the 8192 x 4096 activation, row-major + transposed), grouped / grouped_swiglu / grouped_wgrad (8 experts,
dim 2048 x 5632; ``grouped_single`` / ``grouped_swiglu_single``: the single-CTA tiling instead of CTA pairs), attn_fwd, attn_bwd (B=2, S=4096, 32 / 8 heads, head dim 128, causal; ``--dq-mode red|bulk``),
rmsnorm_bwd (16384 x 4096), adamw (one block's flat unit); gemm_symm / gemm_symm_plain (Gram matrix of a 4096 x 14336
weight from its upper-triangle tiles, and the plain GEMM it replaces; both report the full product's flops), muon_ns
(five Newton-Schulz iterations of that weight); gemm_wgrad_expert (one expert's weight gradient as a dense GEMM with both
operands MN-major: the dense counterpart of grouped_wgrad); gemm_gather (QKV projection whose weight is gathered
inside the kernel from 8 parameter shards; on one GPU the shards are 8 local buffers, so the kernel and its copy
warps run exactly as in a job but the "peer" loads stay on this GPU), symm_pull, symm_rs_shard (one block unit, 8
emulated ranks).  Prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def build(target: str, K, args):
    """(callable, flops, bytes) of the workload."""
    dev, bf = "cuda", torch.bfloat16
    if target in ("gemm", "gemm_1cta"):
        a = torch.randn(8192, 4096, device=dev, dtype=bf)
        w = torch.randn(6144, 4096, device=dev, dtype=bf) * 0.02
        out = torch.empty(8192, 6144, device=dev, dtype=bf)
        return (lambda: K.gemm(a, w, out=out, mode=1 if target == "gemm_1cta" else 2)), 2 * 8192 * 6144 * 4096, 0
    if target in ("gemm_fp8", "fp8_cast"):
        a = torch.randn(8192, 4096, device=dev, dtype=bf)
        w = torch.randn(6144, 4096, device=dev, dtype=bf) * 0.02
        if target == "fp8_cast":   # abs-max + cast of the activation, row-major and transposed copies
            def cast():
                sc = K.fp8_scale(a)
                return K.fp8_cast(a, sc, False, True, True)
            return cast, 0, a.numel() * (2 + 2 + 1 + 1)
        sa, sw = K.fp8_scale(a), K.fp8_scale(w)
        a8, _ = K.fp8_cast(a, sa, False, True, False)
        w8, _ = K.fp8_cast(w, sw, False, True, False)
        return (lambda: K.gemm_fp8(a8, w8, sa, sw)), 2 * 8192 * 6144 * 4096, 0
    if target == "gemm_swiglu":
        a = torch.randn(8192, 4096, device=dev, dtype=bf)
        w = torch.randn(2 * 14336, 4096, device=dev, dtype=bf) * 0.02
        return (lambda: K.gemm_swiglu(a, w, want_gu=True)), 2 * 8192 * 28672 * 4096, 0
    if target == "gemm_rope":
        s, h, hkv, hd = 4096, 32, 8, 128
        a = torch.randn(2 * s, 4096, device=dev, dtype=bf)
        w = torch.randn((h + 2 * hkv) * hd, 4096, device=dev, dtype=bf) * 0.02
        ang = torch.outer(torch.arange(s, device=dev).float(), 500000.0 ** (-torch.arange(0, hd, 2, device=dev).float() / hd))
        cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
        out = torch.empty(2 * s, w.shape[0], device=dev, dtype=bf)
        return (lambda: K.gemm(a, w, out=out, rope=(cos, sin, s, (h + hkv) * hd, hd))), 2 * 8192 * 6144 * 4096, 0
    if target in ("grouped", "grouped_wgrad", "grouped_single", "grouped_swiglu", "grouped_swiglu_single"):
        if target.endswith("_single"):
            K.grouped_pair_mode(0)
            target = target[:-7]
        counts = torch.tensor([4000, 5000, 3000, 4384, 4100, 3900, 4200, 4184], device=dev)
        offsets = torch.zeros(9, dtype=torch.int32, device=dev)
        offsets[1:] = counts.cumsum(0)
        rows = int(counts.sum())
        x = torch.randn(rows, 2048, device=dev, dtype=bf)
        if target == "grouped":
            w = torch.randn(8, 2048, 5632, device=dev, dtype=bf) * 0.02
            return (lambda: K.grouped_gemm(x, w, offsets, b_mn=True)), 2 * rows * 2048 * 5632, 0
        if target == "grouped_swiglu":
            wg = torch.randn(8, 2048, 5632, device=dev, dtype=bf) * 0.02
            wu = torch.randn(8, 2048, 5632, device=dev, dtype=bf) * 0.02
            return (lambda: K.grouped_swiglu(x, wg, wu, offsets, b_mn=True, want_gu=True)), 2 * 2 * rows * 2048 * 5632, 0
        dy = torch.randn(rows, 5632, device=dev, dtype=bf)
        return (lambda: K.grouped_wgrad(x, dy, offsets)), 2 * rows * 2048 * 5632, 0
    if target in ("attn_fwd", "attn_bwd"):
        b, s, h, hkv, hd = 2, 4096, 32, 8, 128
        qkv = torch.randn(b, s, h + 2 * hkv, hd, device=dev, dtype=bf)
        q, k, v = qkv[:, :, :h], qkv[:, :, h:h + hkv], qkv[:, :, h + hkv:]
        sc = 1 / math.sqrt(hd)
        fwd_flops = 4 * b * h * s * s * hd // 2
        if target == "attn_fwd":
            return (lambda: K.attn_fwd(q, k, v, True, None, sc)), fwd_flops, 0
        K.attn_bwd_dq_mode(0 if args.dq_mode == "red" else 1)
        out, lse = K.attn_fwd(q, k, v, True, None, sc)
        dout = torch.randn_like(out)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = dqkv[:, :, :h], dqkv[:, :, h:h + hkv], dqkv[:, :, h + hkv:]
        return (lambda: K.attn_bwd(dout, q, k, v, out, lse, True, None, sc, dq=dq, dk=dk, dv=dv)), fwd_flops * 5 // 2, 0
    if target in ("gemm_gather", "symm_pull", "symm_rs_shard"):
        import ctypes

        class Peers:   # stands in for a symmetric-memory buffer: eight local tensors play the eight ranks
            def __init__(self, tensors, rank):
                self.world, self.rank, self.multicast_ptr = len(tensors), rank, None
                self.peer_ptrs = (ctypes.c_longlong * 8)(*[t.data_ptr() for t in tensors])
                self.keep = tensors

        world = 8
        if target == "gemm_gather":
            s_len, h, hkv, hd, k = 4096, 32, 8, 128, 4096
            rows = [h * hd, hkv * hd, hkv * hd]
            a = torch.randn(2 * s_len, k, device=dev, dtype=bf)
            offs, acc = [], 0
            for r in rows:
                offs.append(acc)
                acc += r * k // world
            shards = [torch.randn(acc, device=dev, dtype=bf) * 0.02 for _ in range(world)]
            ang = torch.outer(torch.arange(s_len, device=dev).float(), 500000.0 ** (-torch.arange(0, hd, 2, device=dev).float() / hd))
            cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
            plan = {"symm": Peers(shards, 3), "seg_rows": rows, "seg_src": offs,
                    "stage": torch.empty(sum(rows) * k, device=dev, dtype=bf), "flags": torch.zeros(256, dtype=torch.int32, device=dev)}
            rope = (cos, sin, s_len, (h + hkv) * hd, hd)
            return (lambda: K.gemm_gather(a, plan, sum(rows), epi=2, rope=rope)), 2 * 8192 * 6144 * 4096, 0
        unit = 218_103_808
        if target == "symm_pull":
            shards = [torch.randn(unit // world, device=dev, dtype=bf) for _ in range(world)]
            dst = torch.empty(unit, device=dev, dtype=bf)
            return (lambda: K.symm_pull(Peers(shards, 3), [0], [unit], [0], dst)), 0, 2 * unit * 2
        grads = [torch.randn(unit, device=dev, dtype=bf) for _ in range(world)]
        out = torch.empty(unit // world, device=dev, dtype=bf)
        return (lambda: K.symm_rs_shard(Peers(grads, 3), [0], [unit], [0], out, False)), 0, (world + 1) * (unit // world) * 2
    if target == "gemm_wgrad_expert":   # one expert's weight gradient as a dense MN-major GEMM (2048 x 5632 over 4096 rows)
        x = torch.randn(4096, 2048, device=dev, dtype=bf)
        dy = torch.randn(4096, 5632, device=dev, dtype=bf)
        return (lambda: K.gemm(x, dy, a_kmajor=False, b_kmajor=False, mode=2)), 2 * 4096 * 2048 * 5632, 0
    if target in ("gemm_symm", "gemm_symm_plain", "muon_ns"):
        x = torch.randn(4096, 14336, device=dev, dtype=bf) * 0.01     # an MLP weight: Gram matrix on the short side
        if target == "muon_ns":   # five Newton-Schulz iterations of one MLP weight
            from kempnerforge_b200.training.optimizer import _newton_schulz_native
            return (lambda: _newton_schulz_native(x, 5)), 5 * (2 * 2 * 4096 * 4096 * 14336 + 2 * 4096 ** 3), 0
        if target == "gemm_symm_plain":
            return (lambda: K.gemm(x, x, mode=2)), 2 * 4096 * 4096 * 14336, 0
        return (lambda: K.gemm_symm(x)), 2 * 4096 * 4096 * 14336, 0   # flops of the full product: what it replaces
    if target == "rmsnorm_bwd":
        x = torch.randn(16384, 4096, device=dev, dtype=bf)
        w = torch.ones(4096, device=dev, dtype=bf)
        _, rstd = K.rmsnorm_fwd(x, w, 1e-5)
        dy = torch.randn_like(x)
        return (lambda: K.rmsnorm_bwd(dy, x, w, rstd, residual_grad=dy)), 0, 4 * x.numel() * 2
    if target == "adamw":
        n = 218_112_000
        p, g = torch.randn(n, device=dev, dtype=bf), torch.randn(n, device=dev, dtype=bf)
        m, v2 = torch.zeros(n, device=dev, dtype=bf), torch.zeros(n, device=dev, dtype=bf)
        return (lambda: K.adamw_flat(p, g, m, v2, n, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1)), 0, 7 * n * 2
    raise SystemExit(f"unknown workload {target!r}")


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("target")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--dq-mode", choices=("red", "bulk"), default="bulk")
    ap.add_argument("--no-flush", action="store_true", help="do not write a 256 MB buffer between launches")
    args = ap.parse_args()
    from kempnerforge_b200.ops import cuda as K

    fn, flops, nbytes = build(args.target, K, args)
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(args.warmup):
        fn()
    times = []
    for _ in range(args.iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    ms = sorted(times)[len(times) // 2]
    status = K.read_status()
    print(json.dumps({"workload": args.target, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1) if flops else None,
                      "gbs": round(nbytes / ms / 1e6, 1) if nbytes else None, "iters": args.iters, "status_word": status}))
    return 0 if status == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
