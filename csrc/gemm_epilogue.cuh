// Epilogue helpers shared by the 1-CTA and 2-CTA tcgen05 GEMM kernels: conversion of one 32-column
// accumulator chunk (held by one thread for one output row) to bf16 / fp32 global stores, with
// optional accumulation into the destination and an optional residual operand; the SwiGLU forward / backward
// arithmetic of the fused epilogues.
#pragma once
#include "common.cuh"

namespace kf {

template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT* dst, const uint32_t (&acc)[32], int valid_cols,
                                            bool accumulate, const OutT* residual);

template <>
__device__ __forceinline__ void store_chunk<__nv_bfloat16>(__nv_bfloat16* dst, const uint32_t (&acc)[32],
                                                           int valid_cols, bool accumulate,
                                                           const __nv_bfloat16* residual) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    if (v * 8 >= valid_cols) break;
    uint4* p = reinterpret_cast<uint4*>(dst + v * 8);
    float f[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(acc[v * 8 + i]);
    if (accumulate) {
      uint4 old = *p;
      float2 a = unpack_bf16(old.x), b = unpack_bf16(old.y), c = unpack_bf16(old.z), d = unpack_bf16(old.w);
      f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y;
      f[4] += c.x; f[5] += c.y; f[6] += d.x; f[7] += d.y;
    }
    if (residual) {
      uint4 old = *reinterpret_cast<const uint4*>(residual + v * 8);
      float2 a = unpack_bf16(old.x), b = unpack_bf16(old.y), c = unpack_bf16(old.z), d = unpack_bf16(old.w);
      f[0] += a.x; f[1] += a.y; f[2] += b.x; f[3] += b.y;
      f[4] += c.x; f[5] += c.y; f[6] += d.x; f[7] += d.y;
    }
    uint4 out;
    out.x = pack_bf16(f[0], f[1]);
    out.y = pack_bf16(f[2], f[3]);
    out.z = pack_bf16(f[4], f[5]);
    out.w = pack_bf16(f[6], f[7]);
    *p = out;
  }
}

template <>
__device__ __forceinline__ void store_chunk<float>(float* dst, const uint32_t (&acc)[32], int valid_cols,
                                                   bool accumulate, const float* residual) {
#pragma unroll
  for (int v = 0; v < 8; ++v) {
    if (v * 4 >= valid_cols) break;
    float4* p = reinterpret_cast<float4*>(dst + v * 4);
    float4 o = make_float4(__uint_as_float(acc[v * 4]), __uint_as_float(acc[v * 4 + 1]),
                           __uint_as_float(acc[v * 4 + 2]), __uint_as_float(acc[v * 4 + 3]));
    if (accumulate) {
      float4 old = *p;
      o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
    }
    if (residual) {
      float4 r = *reinterpret_cast<const float4*>(residual + v * 4);
      o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
    }
    *p = o;
  }
}

// SwiGLU forward on one 32-column chunk: g <- silu(g) * u.  The activation sees the bf16-rounded pre-activations,
// like the two-kernel path (GEMM writes bf16 gate | up, the element-wise kernel reads them back).
__device__ __forceinline__ void swiglu_chunk(uint32_t (&g)[32], const uint32_t (&u)[32]) {
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const float gf = __bfloat162float(__float2bfloat16(__uint_as_float(g[i])));
    const float uf = __bfloat162float(__float2bfloat16(__uint_as_float(u[i])));
    g[i] = __float_as_uint(gf / (1.f + __expf(-gf)) * uf);
  }
}

// SwiGLU backward on one 32-column chunk: `dh` holds the gradient of the hidden activation (fp32 accumulator values),
// gate_row / up_row point at the saved bf16 pre-activations of these 32 hidden units, dgate_row / dup_row receive the
// gradients (they may be the same memory as gate_row / up_row: every element is read and written by one thread).
// The incoming gradient is rounded to bf16 first, like the two-kernel path.
__device__ __forceinline__ void swiglu_bwd_chunk(const uint32_t (&dh)[32], const __nv_bfloat16* gate_row,
                                                 const __nv_bfloat16* up_row, __nv_bfloat16* dgate_row,
                                                 __nv_bfloat16* dup_row, int valid_cols) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    if (q * 8 >= valid_cols) break;
    const uint4 gq = *reinterpret_cast<const uint4*>(gate_row + q * 8);
    const uint4 uq = *reinterpret_cast<const uint4*>(up_row + q * 8);
    const uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w}, uw[4] = {uq.x, uq.y, uq.z, uq.w};
    uint32_t dg[4], du[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 g2 = unpack_bf16(gw[e]), u2 = unpack_bf16(uw[e]);
      const float d0 = __bfloat162float(__float2bfloat16(__uint_as_float(dh[q * 8 + 2 * e])));
      const float d1 = __bfloat162float(__float2bfloat16(__uint_as_float(dh[q * 8 + 2 * e + 1])));
      const float s0 = 1.f / (1.f + __expf(-g2.x)), s1 = 1.f / (1.f + __expf(-g2.y));
      du[e] = pack_bf16(d0 * g2.x * s0, d1 * g2.y * s1);
      dg[e] = pack_bf16(d0 * u2.x * s0 * (1.f + g2.x * (1.f - s0)), d1 * u2.y * s1 * (1.f + g2.y * (1.f - s1)));
    }
    *reinterpret_cast<uint4*>(dgate_row + q * 8) = make_uint4(dg[0], dg[1], dg[2], dg[3]);
    *reinterpret_cast<uint4*>(dup_row + q * 8) = make_uint4(du[0], du[1], du[2], du[3]);
  }
}

}  // namespace kf
