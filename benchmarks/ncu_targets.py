"""Small single-kernel workloads for Nsight Compute captures (one GPU, a few hundred MB, a handful of launches):

    python benchmarks/ncu_targets.py gemm                      # plain run first (must exit 0), then:
    ncu --set full --clock-control none -k regex:kf_gemm -s 2 -c 1 -o prof python benchmarks/ncu_targets.py gemm

Targets: gemm (CTA-pair tiling, 8192 x 6144 x 4096), gemm_1cta, gemm_swiglu, grouped, grouped_wgrad, attn_fwd, attn_bwd
(attn_bwd_bulk: dQ by bulk tensor reductions), rmsnorm_bwd, adamw.  Inputs are larger than the 126 MB L2 where the kernel is memory bound.
"""

from __future__ import annotations

import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main() -> int:
    from kempnerforge_b200.ops import cuda as K

    target = sys.argv[1] if len(sys.argv) > 1 else "gemm"
    dev, bf = "cuda", torch.bfloat16
    reps = 3
    if target in ("gemm", "gemm_1cta"):
        a = torch.randn(8192, 4096, device=dev, dtype=bf)
        w = torch.randn(6144, 4096, device=dev, dtype=bf) * 0.02
        out = torch.empty(8192, 6144, device=dev, dtype=bf)
        fn = lambda: K.gemm(a, w, out=out, mode=1 if target == "gemm_1cta" else 2)  # noqa: E731
    elif target == "gemm_swiglu":
        a = torch.randn(8192, 4096, device=dev, dtype=bf)
        w = torch.randn(2 * 14336, 4096, device=dev, dtype=bf) * 0.02
        fn = lambda: K.gemm_swiglu(a, w, want_gu=True)  # noqa: E731
    elif target == "grouped":
        counts = torch.tensor([4000, 5000, 3000, 4384, 4100, 3900, 4200, 4184], device=dev)
        offsets = torch.zeros(9, dtype=torch.int32, device=dev)
        offsets[1:] = counts.cumsum(0)
        x = torch.randn(int(counts.sum()), 2048, device=dev, dtype=bf)
        w = torch.randn(8, 2048, 5632, device=dev, dtype=bf) * 0.02
        fn = lambda: K.grouped_gemm(x, w, offsets, b_mn=True)  # noqa: E731
    elif target == "grouped_wgrad":
        counts = torch.tensor([4000, 5000, 3000, 4384, 4100, 3900, 4200, 4184], device=dev)
        offsets = torch.zeros(9, dtype=torch.int32, device=dev)
        offsets[1:] = counts.cumsum(0)
        x = torch.randn(int(counts.sum()), 2048, device=dev, dtype=bf)
        dy = torch.randn(int(counts.sum()), 5632, device=dev, dtype=bf)
        fn = lambda: K.grouped_wgrad(x, dy, offsets)  # noqa: E731
    elif target in ("attn_fwd", "attn_bwd", "attn_bwd_bulk"):
        b, s, h, hkv, hd = 2, 4096, 32, 8, 128
        qkv = torch.randn(b, s, h + 2 * hkv, hd, device=dev, dtype=bf)
        q, k, v = qkv[:, :, :h], qkv[:, :, h:h + hkv], qkv[:, :, h + hkv:]
        sc = 1 / math.sqrt(hd)
        if target == "attn_fwd":
            fn = lambda: K.attn_fwd(q, k, v, True, None, sc)  # noqa: E731
        else:
            K.attn_bwd_dq_mode(1 if target == "attn_bwd_bulk" else 0)
            out, lse = K.attn_fwd(q, k, v, True, None, sc)
            dout = torch.randn_like(out)
            fn = lambda: K.attn_bwd(dout, q, k, v, out, lse, True, None, sc)  # noqa: E731
    elif target == "rmsnorm_bwd":
        x = torch.randn(16384, 4096, device=dev, dtype=bf)
        w = torch.ones(4096, device=dev, dtype=bf)
        _, rstd = K.rmsnorm_fwd(x, w, 1e-5)
        dy = torch.randn_like(x)
        fn = lambda: K.rmsnorm_bwd(dy, x, w, rstd, residual_grad=dy)  # noqa: E731
    elif target == "adamw":
        n = 218_112_000
        p, g = torch.randn(n, device=dev, dtype=bf), torch.randn(n, device=dev, dtype=bf)
        m, v2 = torch.zeros(n, device=dev, dtype=bf), torch.zeros(n, device=dev, dtype=bf)
        fn = lambda: K.adamw_flat(p, g, m, v2, n, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1)  # noqa: E731
    else:
        print(f"unknown target {target!r}")
        return 2
    for _ in range(reps):
        fn()
    torch.cuda.synchronize()
    status = K.read_status()
    print(f"{target}: {reps} launches done, status word {status}")
    return 0 if status == 0 else 1


if __name__ == "__main__":
    raise SystemExit(main())
