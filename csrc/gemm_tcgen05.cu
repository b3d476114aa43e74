// bf16 GEMM on the 5th-generation tensor cores:  C[M,N] (+)= A[M,K] * B[N,K]^T.
//
// Persistent, warp-specialised kernel, one CTA per SM:
//   warp 0  : TMA producer   (cp.async.bulk.tensor -> 128B-swizzled smem ring, 4 stages)
//   warp 1  : MMA issuer     (one elected thread issues tcgen05.mma 128x256x16; owns TMEM)
//   warps 2-5: epilogue      (tcgen05.ld TMEM -> registers -> bf16/fp32 global stores)
// The fp32 accumulator lives in tensor memory and is double buffered (2 x 256 columns),
// so the epilogue of tile i overlaps the main loop of tile i+1.
//
// Each operand may be "K-major" (reduction dim contiguous: activations x[M,K], weights
// W[N,K]) or "MN-major" (reduction dim strided: the transposed uses in dgrad / wgrad),
// selected by template flags; the smem descriptors and the instruction descriptor carry
// the layout, so no operand is ever transposed in memory.
//
// Covers the Linear call sites of the reference model (attention q/k/v/o projections,
// SwiGLU gate/up/down, output head: kempnerforge/model/attention.py:150-152,236,
// kempnerforge/model/mlp.py:26, kempnerforge/model/embedding.py:51) and their backward.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tile_math.h"

namespace kf {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int STAGES = 4;
constexpr int UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int GEMM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;  // tile rasterisation: 8 row-blocks share each column-block sweep
constexpr size_t GEMM_SMEM = size_t(STAGES) * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/;

struct TileCoord {
  int m, n;
};

__device__ __forceinline__ TileCoord tile_coord(int t, int m_blocks, int n_blocks) {
  TileCoord tc;
  tilemath::raster(t, m_blocks, n_blocks, GROUP_M, tc.m, tc.n);
  return tc;
}

template <bool A_MN, bool B_MN, typename OutT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
kf_gemm_bf16_tcgen05(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                     OutT* __restrict__ C, const OutT* __restrict__ R, int M, int N, int K, int ldc, int ldr, int accumulate,
                     int* status) {
  extern __shared__ uint8_t smem_raw[];
  // 128B swizzle atoms are 1024 B; tile bases must be 1024-aligned
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  // barrier layout (8 B each): full[S], empty[S], tmem_full[2], tmem_empty[2], drain, then tmem ptr
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
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileCoord tc = tile_coord(t, m_blocks, n_blocks);
        const int m0 = tc.m * BM, n0 = tc.n * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_STAGE_BYTES;
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d(a_dst, &map_a, full_bar(s), k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c)
              tma_load_2d(a_dst + c * (64 * BK * 2), &map_a, full_bar(s), m0 + 64 * c, k0);
          }
          if (!B_MN) {
            tma_load_2d(b_dst, &map_b, full_bar(s), k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(b_dst + c * (64 * BK * 2), &map_b, full_bar(s), n0 + 64 * c, k0);
          }
        }
      }
      // never leave with copies still landing in this CTA's shared memory
      for (int j = max(0, it - STAGES); j < it; ++j)
        mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1, status, KF_ERR_WAIT_DRAIN);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
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
            const uint64_t ad = A_MN ? umma_desc_sw128(a_src + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                     : umma_desc_sw128(a_src + k * (UMMA_K * 2), 16, 1024);
            const uint64_t bd = B_MN ? umma_desc_sw128(b_src + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                     : umma_desc_sw128(b_src + k * (UMMA_K * 2), 16, 1024);
            tc_mma_f16(d_tmem, ad, bd, idesc, (kb | k) != 0);
          }
          tc_commit(empty_bar(s));  // stage is free once these MMAs have read it
        }
        if (ok) tc_commit(tfull_bar(acc));
      }
      // make sure every MMA retired before TMEM is released
      tc_commit(drain_bar);
      mbar_wait(drain_bar, 0, status, KF_ERR_WAIT_DRAIN);
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, 32*quarter+32) are visible to this warp
    int tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
      const TileCoord tc = tile_coord(t, m_blocks, n_blocks);
      const int acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      if (!mbar_wait(tfull_bar(acc), acc_ph, status, KF_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = tc.m * BM + quarter * 32 + lane;
      const int col0 = tc.n * BN;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      OutT* c_row = C + size_t(row) * ldc + col0;
      const OutT* r_row = R ? R + size_t(row) * ldr + col0 : nullptr;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_row + c * 32, v);
        tmem_ld_wait();
        const int valid = min(32, N - (col0 + c * 32));
        if (row < M && valid > 0)
          store_chunk<OutT>(c_row + c * 32, v, valid, accumulate != 0, r_row ? r_row + c * 32 : nullptr);
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

// ------------------------------------------------------------------ host side
static int* g_status[16] = {nullptr};

static int* status_ptr() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (!g_status[dev]) {
    cudaMalloc(&g_status[dev], 64);
    cudaMemset(g_status[dev], 0, 64);
  }
  return g_status[dev];
}

template <bool A_MN, bool B_MN, typename OutT>
static int launch_gemm(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb,
                       int ldc, int ldr, int accumulate, int num_sms, cudaStream_t stream) {
  CUtensorMap ma, mb;
  int rc;
  // K-major: rows = M (or N), cols = K, one (64 x rows) box.  MN-major: rows = K, cols = M (or N), 64x64 boxes.
  rc = A_MN ? make_map_2d_bf16(&ma, A, K, M, lda, 64, BK) : make_map_2d_bf16(&ma, A, M, K, lda, BK, BM);
  if (rc) return 100 + rc;
  rc = B_MN ? make_map_2d_bf16(&mb, B, K, N, ldb, 64, BK) : make_map_2d_bf16(&mb, B, N, K, ldb, BK, BN);
  if (rc) return 200 + rc;
  auto kern = kf_gemm_bf16_tcgen05<A_MN, B_MN, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GEMM_SMEM);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  kern<<<grid, GEMM_THREADS, GEMM_SMEM, stream>>>(ma, mb, reinterpret_cast<OutT*>(C),
                                                  reinterpret_cast<const OutT*>(R), M, N, K, ldc, ldr, accumulate,
                                                  status_ptr());
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // namespace kf

namespace kf2 {
int launch_gemm_2cta(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb,
                     int ldc, int ldr, int a_mn, int b_mn, int out_f32, int accumulate, int num_sms,
                     cudaStream_t stream, int* status);
}

namespace kf2 {
int launch_gemm_swiglu_2cta(const void* A, const void* W, void* H, void* GU, int M, int F, int K, int lda, int ldw, int ldh,
                            int ldgu, int num_sms, cudaStream_t stream, int* status);
}

namespace kf2 {
int launch_gemm_rope_2cta(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                          const float* cosT, const float* sinT, int S, int rope_cols, int hd, int num_sms,
                          cudaStream_t stream, int* status);
}

namespace kf2 {
int launch_gemm_symm_2cta(int x_mn, const void* X, void* C, const void* R, int n, int K, int ldx, int ldc, int ldr,
                          float alpha, float beta, float diag, int num_sms, cudaStream_t stream, int* status);
}

namespace kf2 {
int launch_gemm_swiglu_bwd_2cta(const void* DY, const void* W, const void* GU, void* DGU, int M, int F, int K, int lda,
                                int ldw, int ldgu, int num_sms, cudaStream_t stream, int* status);
}

namespace kf2 {
int launch_gemm_gather_2cta(int epi, const void* A, void* C, const void* R, int M, int N, int K, int lda, int ldc, int ldr,
                            const long long* peers, int world, int rank, int n_seg, const long long* seg_rows,
                            const long long* seg_src, void* stage, int* flags, const float* cosT, const float* sinT,
                            int S, int rope_cols, int hd, int num_sms, cudaStream_t stream, int* status);
}

extern "C" {

// Input gradient of a SwiGLU MLP's down projection fused with the SwiGLU gradient: dgu[M, 2F] (d gate | d up) from
// dy[M, K], the down weight w[K][F] (its stored layout) and the saved pre-activations gu[M, 2F]; dh is never written.
// dgu may alias gu.  Pitches in elements, multiples of 8; K % 64 == 0.
int kf_gemm_swiglu_bwd_bf16(const void* dy, const void* w, const void* gu, void* dgu, int M, int F, int K, int lda, int ldw,
                            int ldgu, int num_sms, void* stream) {
  if ((lda & 7) || (ldw & 7) || (ldgu & 7) || (F & 7) || (K % 64)) return 5;
  return kf2::launch_gemm_swiglu_bwd_2cta(dy, w, gu, dgu, M, F, K, lda, ldw, ldgu, num_sms, (cudaStream_t)stream,
                                          kf::status_ptr());
}

// Symmetric product with a polynomial epilogue (the Gram matrix and the quintic of Muon's Newton-Schulz iteration):
// c[n, n] = alpha * x x^T + beta * r + diag * I for x[n][K] (x_mn == 0) or alpha * x^T x + ... for x[K][n] (x_mn != 0).
// Only the tiles on and above the diagonal are computed, the rest is their transposed copy.  r (optional) must be
// symmetric; c must alias neither x nor r.  n % 8 == 0; pitches in elements, multiples of 8.
int kf_gemm_symm_bf16(int x_mn, const void* x, void* c, const void* r, int n, int K, int ldx, int ldc, int ldr, float alpha,
                      float beta, float diag, int num_sms, void* stream) {
  if ((ldx & 7) || (ldc & 7) || (r && (ldr & 7)) || c == x || c == r) return 5;
  return kf2::launch_gemm_symm_2cta(x_mn, x, c, r, n, K, ldx, ldc, ldr, alpha, beta, diag, num_sms, (cudaStream_t)stream,
                                    kf::status_ptr());
}

// GEMM whose weight operand is gathered from the data-parallel ranks' parameter shards by the same kernel
// (sharded parameters: rank r keeps piece r of every weight).  out = x W^T with W = the row stack of `n_seg`
// weights (seg_rows[i] rows of K elements); piece r of weight i is at shard_ptrs[r] + seg_src[i] (elements).
// epi 0: (+ residual R); epi 1: SwiGLU over [gate ; up] (N = hidden size F, out = h, R = optional pre-activations
// [M, 2F]); epi 2: rotary embedding on the first rope_cols columns.  `stage` (rows x K bf16) receives the assembled
// operand and stays valid afterwards; `flags`: rows / 128 + 1 ints of scratch.  K % 128 == 0, rows % 128 == 0,
// every piece a multiple of 16384 elements.
int kf_gemm_gather_bf16(int epi, const void* x, void* out, const void* R, int M, int N, int K, int lda, int ldc, int ldr,
                        const long long* shard_ptrs, int world, int rank, int n_seg, const long long* seg_rows,
                        const long long* seg_src, void* stage, void* flags, const void* cosT, const void* sinT, int S,
                        int rope_cols, int hd, int num_sms, void* stream) {
  if ((lda & 7) || (ldc & 7) || (R && (ldr & 7))) return 5;
  return kf2::launch_gemm_gather_2cta(epi, x, out, R, M, N, K, lda, ldc, ldr, shard_ptrs, world, rank, n_seg, seg_rows,
                                      seg_src, stage, (int*)flags, (const float*)cosT, (const float*)sinT, S, rope_cols,
                                      hd, num_sms, (cudaStream_t)stream, kf::status_ptr());
}

// Fused Q | K | V projection with the rotary embedding in the epilogue: out[M, N] = x W^T, then every head of `hd`
// columns inside the first `rope_cols` columns is rotated by the angle of position (row % S); cos / sin are fp32
// [S][hd / 2].  N and rope_cols multiples of hd (64, 128 or 256); pitches in elements, multiples of 8.
int kf_gemm_rope_bf16(const void* x, const void* w, void* out, int M, int N, int K, int lda, int ldw, int ldc,
                      const void* cosT, const void* sinT, int S, int rope_cols, int hd, int num_sms, void* stream) {
  if ((lda & 7) || (ldw & 7) || (ldc & 7)) return 5;
  return kf2::launch_gemm_rope_2cta(x, w, out, M, N, K, lda, ldw, ldc, (const float*)cosT, (const float*)sinT, S,
                                    rope_cols, hd, num_sms, (cudaStream_t)stream, kf::status_ptr());
}

// SwiGLU up-projection in one kernel: h[M, F] = silu(x Wg^T) * (x Wu^T), W = [Wg ; Wu] stacked as [2F][K] (K contiguous).
// gu (optional, [M, 2F]) receives the bf16 pre-activations (gate | up) for the backward pass.  F must be a multiple of
// 128; pitches in elements, multiples of 8.
int kf_gemm_swiglu_bf16(const void* x, const void* w, void* h, void* gu, int M, int F, int K, int lda, int ldw, int ldh,
                        int ldgu, int num_sms, void* stream) {
  if ((F % 128) || (lda & 7) || (ldw & 7) || (ldh & 7) || (gu && (ldgu & 7))) return 5;
  return kf2::launch_gemm_swiglu_2cta(x, w, h, gu, M, F, K, lda, ldw, ldh, ldgu, num_sms, (cudaStream_t)stream,
                                      kf::status_ptr());
}

// C[M,N] = op(A) * op(B)^T (+ C if accumulate) (+ R if given), bf16 inputs, fp32 accumulation.
//   a_mn == 0: A is stored [M][lda] (K contiguous);  a_mn == 1: A is stored [K][lda] (M contiguous)
//   b_mn == 0: B is stored [N][ldb] (K contiguous);  b_mn == 1: B is stored [K][ldb] (N contiguous)
//   out_f32: C (and R) are fp32 instead of bf16.  Leading dimensions in elements; A/B pitches must be
//   multiples of 8 elements and base pointers 16-byte aligned (TMA), ldc/ldr multiples of 8 (bf16) / 4 (fp32).
//   mode: 0 = pick automatically, 1 = one CTA per 128x256 tile, 2 = CTA pairs (cta_group::2) on 256x256 tiles.
// Returns 0 on success, otherwise a code identifying the failing step.
int kf_gemm_bf16(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb,
                 int ldc, int ldr, int a_mn, int b_mn, int out_f32, int accumulate, int mode, int num_sms,
                 void* stream) {
  using namespace kf;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (M <= 0 || N <= 0 || K <= 0) return 1;
  if (mode == 0) {
    // pairs pay off once there are enough 256x256 tiles to fill the machine a few times over
    const long long pair_tiles = (long long)((M + 255) / 256) * ((N + 255) / 256);
    mode = pair_tiles >= 2LL * (num_sms / 2) ? 2 : 1;
  }
  if (mode == 2)
    return kf2::launch_gemm_2cta(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, a_mn, b_mn, out_f32, accumulate, num_sms,
                                 st, status_ptr());
#define KF_DISPATCH(AM, BM_)                                                                                  \
  (out_f32 ? launch_gemm<AM, BM_, float>(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, accumulate, num_sms, st)    \
           : launch_gemm<AM, BM_, __nv_bfloat16>(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, accumulate, num_sms, st))
  if (!a_mn && !b_mn) return KF_DISPATCH(false, false);
  if (!a_mn && b_mn) return KF_DISPATCH(false, true);
  if (a_mn && !b_mn) return KF_DISPATCH(true, false);
  return KF_DISPATCH(true, true);
#undef KF_DISPATCH
}

// Status word shared by all kernels of this library on the current device (0 = healthy).
int kf_read_status() {
  int v = 0;
  cudaMemcpy(&v, kf::status_ptr(), sizeof(int), cudaMemcpyDeviceToHost);
  return v;
}
void kf_clear_status() { cudaMemset(kf::status_ptr(), 0, 64); }
void* kf_status_device_ptr() { return kf::status_ptr(); }

}  // extern "C"
