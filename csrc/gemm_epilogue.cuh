// Epilogue helpers shared by the 1-CTA and 2-CTA tcgen05 GEMM kernels: conversion of one 32-column
// accumulator chunk (held by one thread for one output row) to bf16 / fp32 global stores, with
// optional accumulation into the destination and an optional residual operand.
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

}  // namespace kf
