"""The hand-written sm_100a kernels against their roofs: tcgen05 GEMMs at the Llama-3-8B shapes
(TFLOP/s, with the cuBLAS figure beside it) and the memory-bound kernels (GB/s). GPU only.
No counterpart in the reference, which ships no kernels of its own."""

from __future__ import annotations

import torch

from benchmarks.runner import Case, print_results, run_suite

SUITE = "kernels"

# (M, N, K): tokens x out x in for micro-batch 2 x 4096 of the 8B shape
GEMM_SHAPES = [(8192, 6144, 4096), (8192, 4096, 4096), (8192, 28672, 4096), (8192, 4096, 14336)]


def cases(device: torch.device):
    if device.type != "cuda":
        return
    from kempnerforge_b200.ops import cuda as K

    bf = torch.bfloat16
    for m, n, k in GEMM_SHAPES:
        a = torch.randn(m, k, device=device, dtype=bf)
        w = torch.randn(n, k, device=device, dtype=bf) * 0.02
        out = torch.empty(m, n, device=device, dtype=bf)
        flops = 2.0 * m * n * k
        yield Case(f"tcgen05 GEMM {m}x{n}x{k}", lambda a=a, w=w, out=out: K.gemm(a, w, out=out), flops_per_iter=flops)
        yield Case(f"cuBLAS  GEMM {m}x{n}x{k}", lambda a=a, w=w, out=out: torch.matmul(a, w.t(), out=out),
                   flops_per_iter=flops)

    # attention at the 8B shape: (B, S, H + 2 Hkv, hd) fused projection output, causal
    import math

    b, sq, h, hkv, hd = 2, 4096, 32, 8, 128
    qkv = torch.randn(b, sq, h + 2 * hkv, hd, device=device, dtype=bf)
    q, k, v = qkv[:, :, :h], qkv[:, :, h:h + hkv], qkv[:, :, h + hkv:]
    sc = 1.0 / math.sqrt(hd)
    aflops = 4.0 * b * h * sq * sq * hd / 2
    out, lse = K.attn_fwd(q, k, v, True, None, sc)
    dout = torch.randn_like(out)
    yield Case("tcgen05 attention fwd (2x32x4096x128, causal)", lambda: K.attn_fwd(q, k, v, True, None, sc),
               flops_per_iter=aflops)
    yield Case("tcgen05 attention bwd", lambda: K.attn_bwd(dout, q, k, v, out, lse, True, None, sc),
               flops_per_iter=2.5 * aflops)
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    yield Case("library attention fwd (SDPA)",
               lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt, is_causal=True, scale=sc,
                                                                        enable_gqa=True), flops_per_iter=aflops)

    t, d = 8192, 4096
    x = torch.randn(t, d, device=device, dtype=bf)
    wn = torch.ones(d, device=device, dtype=bf)
    yield Case("rmsnorm fwd (8192x4096)", lambda: K.rmsnorm_fwd(x, wn, 1e-5), bytes_per_iter=2 * x.numel() * 2)
    y0, rstd0 = K.rmsnorm_fwd(x, wn, 1e-5)
    dy0 = torch.randn_like(x)
    yield Case("rmsnorm bwd (8192x4096, with residual gradient)",
               lambda: K.rmsnorm_bwd(dy0, x, wn, rstd0, residual_grad=dy0), bytes_per_iter=4 * x.numel() * 2)
    h = torch.randn(t, 2 * 14336, device=device, dtype=bf)
    yield Case("swiglu fwd (8192x14336)", lambda: K.swiglu_fwd(h), bytes_per_iter=h.numel() * 2 * 1.5)
    nparam = 218_112_000
    p = torch.randn(nparam, device=device, dtype=bf)
    g = torch.randn(nparam, device=device, dtype=bf)
    m1 = torch.zeros(nparam, device=device, dtype=bf)
    m2 = torch.zeros(nparam, device=device, dtype=bf)
    yield Case("AdamW flat (one 8B block, 218M params)",
               lambda: K.adamw_flat(p, g, m1, m2, nparam, 1e-4, 0.9, 0.95, 1e-8, 0.1, 1),
               bytes_per_iter=nparam * 2 * 7)
    acc = torch.zeros(1, device=device, dtype=torch.float32)
    yield Case("sum of squares (218M bf16)", lambda: K.sumsq(g, acc), bytes_per_iter=nparam * 2)


if __name__ == "__main__":
    print_results(run_suite(SUITE, torch.device("cuda")), "kernels")
