// FP8 GEMM on the 5th-generation tensor cores (tcgen05.mma kind::f8f6f4) plus the casts that feed it.
//
//   C[M,N] (+)= alpha * A8[M,K] * B8[N,K]^T      alpha = 1 / (scale_a * scale_b), read from device memory
//
// A8 / B8 are e4m3 or e5m2 bytes with the reduction dim contiguous ("K-major"); tensorwise scales are
// computed on the device (abs-max -> scale) and never visit the host.  Same persistent warp-specialised
// structure as the bf16 kernel: TMA producer warp, one MMA-issuing thread, four epilogue warps, 4-stage
// 128B-swizzled ring (128 K-elements per stage), double-buffered fp32 accumulators in tensor memory.
// The transposed operands that dgrad / wgrad need are written by the cast kernel itself (one read of the
// bf16 source produces the row-major and the transposed fp8 copy), so every GEMM runs K-major.
//
// Covers the reference's float8 training path (torchao tensorwise scaling through
// kempnerforge/distributed/parallel.py:125-174): e4m3 for activations and weights, e5m2 for gradients.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tile_math.h"
#include <cuda_fp8.h>

namespace kf {
namespace f8 {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;       // fp8 elements = bytes per row of a stage
constexpr int UMMA_K = 32;    // K per tcgen05.mma for 8-bit inputs
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * BK;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK;  // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;
constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256;

// Instruction descriptor for kind::f8f6f4: fp32 accumulate, A/B format 0 = e4m3, 1 = e5m2, both K-major.
__host__ __device__ constexpr uint32_t idesc_f8(int m, int n, int a_fmt, int b_fmt) {
  return (1u << 4) | (uint32_t(a_fmt) << 7) | (uint32_t(b_fmt) << 10) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

__device__ __forceinline__ void tc_mma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void tile_coord(int t, int m_blocks, int n_blocks, int& tile_m, int& tile_n) {
  tilemath::raster(t, m_blocks, n_blocks, GROUP_M, tile_m, tile_n);
}

__global__ void __launch_bounds__(THREADS, 1)
kf_gemm_fp8_tcgen05(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    __nv_bfloat16* __restrict__ C, int M, int N, int K, int ldc, int accumulate, int a_fmt,
                    int b_fmt, const float* __restrict__ scale_a, const float* __restrict__ scale_b, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 4);
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 5);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_blocks = (M + BM - 1) / BM;
  const int n_blocks = (N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    mbar_init(drain_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coord(t, m_blocks, n_blocks, tm, tn);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * STAGE_BYTES;
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, full_bar(s), kb * BK, tm * BM);
          tma_load_2d(a_dst + A_STAGE_BYTES, &map_b, full_bar(s), kb * BK, tn * BN);
        }
      }
      for (int j = max(0, it - STAGES); j < it; ++j)
        mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1, status, KF_ERR_WAIT_DRAIN);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = idesc_f8(BM, BN, a_fmt, b_fmt);
      int it = 0, tile_iter = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
        const int acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1, status, KF_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(full_bar(s), ph, status, KF_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_src = smem_base + s * STAGE_BYTES;
          const uint32_t b_src = a_src + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // 32 one-byte elements per step = 32 B along the swizzled 128 B row
            tc_mma_f8(d_tmem, umma_desc_sw128(a_src + k * UMMA_K, 16, 1024),
                      umma_desc_sw128(b_src + k * UMMA_K, 16, 1024), idesc, (kb | k) != 0);
          }
          tc_commit(empty_bar(s));
        }
        if (ok) tc_commit(tfull_bar(acc));
      }
      tc_commit(drain_bar);
      mbar_wait(drain_bar, 0, status, KF_ERR_WAIT_DRAIN);
    }
  } else {
    const int quarter = warp & 3;
    const float alpha = 1.0f / (scale_a[0] * scale_b[0]);
    int tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
      int tm, tn;
      tile_coord(t, m_blocks, n_blocks, tm, tn);
      const int acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      if (!mbar_wait(tfull_bar(acc), acc_ph, status, KF_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + quarter * 32 + lane;
      const int col0 = tn * BN;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      __nv_bfloat16* c_row = C + size_t(row) * ldc + col0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_row + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
        const int valid = min(32, N - (col0 + c * 32));
        if (row < M && valid > 0) store_chunk<__nv_bfloat16>(c_row + c * 32, v, valid, accumulate != 0, nullptr);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// rows x cols one-byte matrix, row pitch ld bytes -> tensor map with (128 x box_rows) boxes, 128B swizzle
static int make_map_2d_u8(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                          uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// ------------------------------------------------------------------ abs-max -> scale, cast (+ transpose)
constexpr float E4M3_MAX = 448.f;
constexpr float E5M2_MAX = 57344.f;

__global__ void kf_absmax_bf16(const __nv_bfloat16* __restrict__ x, long long n, unsigned int* __restrict__ amax_bits) {
  float m = 0.f;
  const long long n8 = n / 8;
  const uint4* x8 = reinterpret_cast<const uint4*>(x);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = x8[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = unpack_bf16(w[j]);
      m = fmaxf(m, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  if (blockIdx.x == 0)
    for (long long i = n8 * 8 + threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, fabsf(__bfloat162float(x[i])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  // non-negative floats order like their bit patterns
  if ((threadIdx.x & 31) == 0) atomicMax(amax_bits, __float_as_uint(m));
}

// scale = fp8_max / max(amax, tiny); also resets nothing: the caller zeroes amax before the reduction.
__global__ void kf_scale_from_amax(const unsigned int* __restrict__ amax_bits, float* __restrict__ scale, float fp8_max) {
  const float a = __uint_as_float(amax_bits[0]);
  scale[0] = fp8_max / fmaxf(a, 1e-12f);
}

template <bool E5M2>
__device__ __forceinline__ uint8_t to_fp8(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, E5M2 ? __NV_E5M2 : __NV_E4M3);
}

// One 64 x 64 tile per block: reads bf16 x[rows][cols] (pitch ldx), writes the scaled fp8 copy row-major
// (out, pitch ld_out bytes, may be null) and transposed (out_t[cols][rows], pitch ld_t bytes, may be null).
template <bool E5M2>
__global__ void __launch_bounds__(256)
kf_cast_fp8(const __nv_bfloat16* __restrict__ x, int rows, int cols, long long ldx, const float* __restrict__ scale,
            uint8_t* __restrict__ out, long long ld_out, uint8_t* __restrict__ out_t, long long ld_t) {
  __shared__ uint8_t tile[64][64 + 4];
  const float s = scale[0];
  const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 15;   // 16 threads x 4 columns
  const int ty = threadIdx.x >> 4;   // 16 row groups
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
    const int r = r0 + ty + 16 * rr;
    const int c = c0 + tx * 4;
    uint8_t q[4] = {0, 0, 0, 0};
    if (r < rows) {
      if (c + 3 < cols && (ldx & 3) == 0) {
        const uint2 v = *reinterpret_cast<const uint2*>(x + size_t(r) * ldx + c);
        const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y);
        q[0] = to_fp8<E5M2>(a.x * s); q[1] = to_fp8<E5M2>(a.y * s);
        q[2] = to_fp8<E5M2>(b.x * s); q[3] = to_fp8<E5M2>(b.y * s);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (c + i < cols) q[i] = to_fp8<E5M2>(__bfloat162float(x[size_t(r) * ldx + c + i]) * s);
      }
      if (out) {
        if (c + 3 < cols && (ld_out & 3) == 0) {
          *reinterpret_cast<uint32_t*>(out + size_t(r) * ld_out + c) =
              uint32_t(q[0]) | (uint32_t(q[1]) << 8) | (uint32_t(q[2]) << 16) | (uint32_t(q[3]) << 24);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (c + i < cols) out[size_t(r) * ld_out + c + i] = q[i];
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) tile[ty + 16 * rr][tx * 4 + i] = q[i];
  }
  if (!out_t) return;
  __syncthreads();
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
    const int c = c0 + ty + 16 * rr;       // output row = source column
    const int r = r0 + tx * 4;             // 4 consecutive source rows = 4 output bytes
    if (c >= cols) continue;
    uint8_t q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = tile[tx * 4 + i][ty + 16 * rr];
    if (r + 3 < rows && (ld_t & 3) == 0) {
      *reinterpret_cast<uint32_t*>(out_t + size_t(c) * ld_t + r) =
          uint32_t(q[0]) | (uint32_t(q[1]) << 8) | (uint32_t(q[2]) << 16) | (uint32_t(q[3]) << 24);
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (r + i < rows) out_t[size_t(c) * ld_t + r + i] = q[i];
    }
  }
}

}  // namespace f8
}  // namespace kf

extern "C" void* kf_status_device_ptr();

extern "C" {

// C[M,N] (+)= A8[M,K] * B8[N,K]^T / (scale_a * scale_b).  Pitches lda / ldb in bytes (multiples of 16),
// ldc in elements (multiple of 8).  a_fmt / b_fmt: 0 = e4m3, 1 = e5m2.  scale_* are device pointers.
int kf_gemm_fp8(const void* A, const void* B, void* C, int M, int N, int K, long long lda, long long ldb, int ldc,
                int a_fmt, int b_fmt, const void* scale_a, const void* scale_b, int accumulate, int num_sms,
                void* stream) {
  using namespace kf;
  using namespace kf::f8;
  if ((lda & 15) || (ldb & 15) || (ldc & 7) || M <= 0 || N <= 0 || K <= 0) return 5;
  CUtensorMap ma, mb;
  int rc = make_map_2d_u8(&ma, A, M, K, lda, BM);
  if (rc) return 100 + rc;
  rc = make_map_2d_u8(&mb, B, N, K, ldb, BN);
  if (rc) return 200 + rc;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kf_gemm_fp8_tcgen05, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  kf_gemm_fp8_tcgen05<<<grid, THREADS, SMEM, (cudaStream_t)stream>>>(
      ma, mb, reinterpret_cast<__nv_bfloat16*>(C), M, N, K, ldc, accumulate, a_fmt, b_fmt,
      reinterpret_cast<const float*>(scale_a), reinterpret_cast<const float*>(scale_b),
      reinterpret_cast<int*>(kf_status_device_ptr()));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// scale[0] = fp8_max / absmax(x) for n bf16 values; amax_scratch is one 32-bit word of device memory.
int kf_fp8_scale_bf16(const void* x, long long n, int e5m2, void* amax_scratch, void* scale, void* stream) {
  using namespace kf::f8;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t e = cudaMemsetAsync(amax_scratch, 0, 4, st);
  if (e != cudaSuccess) return 400 + (int)e;
  long long blocks = (n / 8 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 1184) blocks = 1184;
  kf_absmax_bf16<<<(int)blocks, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), n,
                                              reinterpret_cast<unsigned int*>(amax_scratch));
  kf_scale_from_amax<<<1, 1, 0, st>>>(reinterpret_cast<const unsigned int*>(amax_scratch),
                                      reinterpret_cast<float*>(scale), e5m2 ? E5M2_MAX : E4M3_MAX);
  e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// fp8(x * scale) row-major into out (optional) and transposed into out_t (optional).
int kf_fp8_cast_bf16(const void* x, int rows, int cols, long long ldx, const void* scale, int e5m2, void* out,
                     long long ld_out, void* out_t, long long ld_t, void* stream) {
  using namespace kf::f8;
  dim3 grid((cols + 63) / 64, (rows + 63) / 64);
  auto xp = reinterpret_cast<const __nv_bfloat16*>(x);
  auto sp = reinterpret_cast<const float*>(scale);
  if (e5m2)
    kf_cast_fp8<true><<<grid, 256, 0, (cudaStream_t)stream>>>(xp, rows, cols, ldx, sp, (uint8_t*)out, ld_out,
                                                              (uint8_t*)out_t, ld_t);
  else
    kf_cast_fp8<false><<<grid, 256, 0, (cudaStream_t)stream>>>(xp, rows, cols, ldx, sp, (uint8_t*)out, ld_out,
                                                               (uint8_t*)out_t, ld_t);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // extern "C"
