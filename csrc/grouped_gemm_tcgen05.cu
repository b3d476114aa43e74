// Ragged grouped GEMM for mixture-of-experts layers on the 5th-generation tensor cores:
//
//   C[rows of expert e, :] = A[rows of expert e, :] * op(B_e)        for every expert e
//
// A holds the token rows sorted by expert; `offsets[e] .. offsets[e+1]` (int32, on the DEVICE) are expert e's
// rows.  Nothing is padded and nothing is read back to the host: every CTA builds the table "first 128-row
// tile of each expert" in shared memory from the offsets and walks the tiles persistently.  A tile's TMA box
// may run past its expert's last row (into the next expert's rows); those accumulator rows are simply not
// stored.  B is either [E][N][K] (K contiguous, nn.Linear weights of stacked experts) or [E][K][N]
// (N contiguous, packed expert weights); the same kernel serves the forward and the input-gradient GEMM.
//
// Same pipeline as the dense kernel: TMA producer warp -> 4-stage 128B-swizzled ring -> one MMA-issuing
// thread -> double-buffered fp32 accumulators in TMEM -> four epilogue warps.
//
// Replaces the padded `torch._grouped_mm` call and its Python pack / unpack loops in the reference
// (kempnerforge/model/moe.py:20-145).
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tile_math.h"

namespace kf {
namespace grp {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2, B_STAGE_BYTES = BN * BK * 2, STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int THREADS = 192, TMEM_COLS = 512;
constexpr int MAX_EXPERTS = 256;
constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256 + (MAX_EXPERTS + 1) * 4;

using Tile = tilemath::GroupedTile;

__device__ __forceinline__ Tile decode(int t, int n_blocks, const int* tile_start, const int* offsets, int E) {
  return tilemath::grouped_decode(t, n_blocks, tile_start, offsets, E, BM);
}

// SWIGLU: the expert feed-forward's first half in one kernel.  Two weight operands (gate: map_b, up: map_b2) of N = F
// hidden units each; a tile covers 128 hidden units and its accumulator holds [gate 128 | up 128]; the epilogue writes
// h = silu(gate) * up to C[rows, F] and, when GU is given, the bf16 pre-activations to GU[rows, 2F] (gate | up) for the
// backward pass.  ACCUMULATE (plain variant): C += A * op(B_e) (the two input-gradient products of gate and up).
template <bool B_MN, bool SWIGLU>
__global__ void __launch_bounds__(THREADS, 1)
kf_grouped_gemm_tcgen05(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_b2, __nv_bfloat16* __restrict__ C,
                        __nv_bfloat16* __restrict__ GU, const int* __restrict__ offsets, int E, int N, int K,
                        long long ldc, long long ldgu, int accumulate, int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 4);
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 5);
  uint8_t* bar_gen = smem_raw + (bar_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(bar_gen + 8 * (2 * STAGES + 5));
  int* tile_start = reinterpret_cast<int*>(bar_gen + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int TN = SWIGLU ? BN / 2 : BN;  // output columns (hidden units) per tile
  const int n_blocks = (N + TN - 1) / TN;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
    mbar_init(drain_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (SWIGLU) tma_prefetch_desc(&map_b2);
    tilemath::grouped_tile_starts(offsets, E, BM, tile_start);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const int num_tiles = tile_start[E] * n_blocks;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tl = decode(t, n_blocks, tile_start, offsets, E);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * STAGE_BYTES, b_dst = a_dst + A_STAGE_BYTES;
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, full_bar(s), kb * BK, tl.row0);
          if constexpr (SWIGLU) {
            if (!B_MN) {  // rows 0..127 of the B tile: gate weights, rows 128..255: the matching up weights
              tma_load_2d(b_dst, &map_b, full_bar(s), kb * BK, tl.e * N + tl.nb * TN);
              tma_load_2d(b_dst + TN * BK * 2, &map_b2, full_bar(s), kb * BK, tl.e * N + tl.nb * TN);
            } else {
#pragma unroll
              for (int c = 0; c < TN / 64; ++c) {
                tma_load_2d(b_dst + c * (64 * BK * 2), &map_b, full_bar(s), tl.nb * TN + 64 * c, tl.e * K + kb * BK);
                tma_load_2d(b_dst + (TN / 64 + c) * (64 * BK * 2), &map_b2, full_bar(s), tl.nb * TN + 64 * c,
                            tl.e * K + kb * BK);
              }
            }
          } else if (!B_MN) {
            tma_load_2d(b_dst, &map_b, full_bar(s), kb * BK, tl.e * N + tl.nb * BN);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(b_dst + c * (64 * BK * 2), &map_b, full_bar(s), tl.nb * BN + 64 * c, tl.e * K + kb * BK);
          }
        }
      }
      for (int j = max(0, it - STAGES); j < it; ++j)
        mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1, status, KF_ERR_WAIT_DRAIN);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, false, B_MN);
      int it = 0, tile_iter = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
        const int acc = tile_iter & 1;
        if (!mbar_wait(tempty_bar(acc), ((tile_iter >> 1) & 1) ^ 1, status, KF_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(full_bar(s), (it / STAGES) & 1, status, KF_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_src = smem_base + s * STAGE_BYTES, b_src = a_src + A_STAGE_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t bd = B_MN ? umma_desc_sw128(b_src + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                     : umma_desc_sw128(b_src + k * (UMMA_K * 2), 16, 1024);
            tc_mma_f16(d_tmem, umma_desc_sw128(a_src + k * (UMMA_K * 2), 16, 1024), bd, idesc, (kb | k) != 0);
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
    int tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
      const Tile tl = decode(t, n_blocks, tile_start, offsets, E);
      const int acc = tile_iter & 1;
      if (!mbar_wait(tfull_bar(acc), (tile_iter >> 1) & 1, status, KF_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int r = quarter * 32 + lane;
      const int col0 = tl.nb * TN;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      __nv_bfloat16* c_row = C + size_t(tl.row0 + r) * ldc + col0;
      if constexpr (SWIGLU) {
        __nv_bfloat16* gu_row = GU ? GU + size_t(tl.row0 + r) * ldgu + col0 : nullptr;
#pragma unroll 1
        for (int c = 0; c < TN / 32; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(t_row + c * 32, g);
          tmem_ld_32x32(t_row + TN + c * 32, u);
          tmem_ld_wait();
          const int valid_cols = min(32, N - (col0 + c * 32));
          if (r < tl.valid && valid_cols > 0) {
            if (gu_row) {
              store_chunk<__nv_bfloat16>(gu_row + c * 32, g, valid_cols, false, nullptr);
              store_chunk<__nv_bfloat16>(gu_row + N + c * 32, u, valid_cols, false, nullptr);
            }
            swiglu_chunk(g, u);
            store_chunk<__nv_bfloat16>(c_row + c * 32, g, valid_cols, false, nullptr);
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_row + c * 32, v);
          tmem_ld_wait();
          const int valid_cols = min(32, N - (col0 + c * 32));
          if (r < tl.valid && valid_cols > 0)
            store_chunk<__nv_bfloat16>(c_row + c * 32, v, valid_cols, accumulate != 0, nullptr);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

}  // namespace grp
}  // namespace kf

extern "C" void* kf_status_device_ptr();

namespace kf {
namespace grp {
template <bool B_MN, bool SWIGLU>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, void* C, void* GU, const void* offsets,
                  int E, int N, int K, long long ldc, long long ldgu, int accumulate, int grid, cudaStream_t st) {
  auto kern = kf_grouped_gemm_tcgen05<B_MN, SWIGLU>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  int* status = reinterpret_cast<int*>(kf_status_device_ptr());
  kern<<<grid, THREADS, SMEM, st>>>(ma, mb, mb2, reinterpret_cast<__nv_bfloat16*>(C), reinterpret_cast<__nv_bfloat16*>(GU),
                                    reinterpret_cast<const int*>(offsets), E, N, K, ldc, ldgu, accumulate, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
}  // namespace grp
}  // namespace kf

namespace kf {
namespace grp2 {
int launch_grouped_gemm_2cta(const void* A, const void* B, void* C, const void* offsets, int rows, int E, int N, int K,
                             long long lda, long long ldc, int b_mn, int accumulate, int num_sms, cudaStream_t st, int* status);
int launch_grouped_swiglu_2cta(const void* A, const void* Wg, const void* Wu, void* H, void* GU, const void* offsets, int rows,
                               int E, int F, int K, long long lda, long long ldh, long long ldgu, int b_mn, int num_sms,
                               cudaStream_t st, int* status);
int launch_grouped_swiglu_bwd_2cta(const void* DY, const void* W, const void* GU, void* DGU, const void* offsets, int rows,
                                   int E, int F, int K, long long lda, long long ldgu, int b_mn, int num_sms, cudaStream_t st,
                                   int* status);
}  // namespace grp2
}  // namespace kf

// 1 (default): CTA-pair tiles (256 x 256; forward / input gradient when the call has at least 256 rows); 0: single-CTA
// 128 x 256 tiles.
int kf_grouped_pair_mode_value = 1;  // read by grouped_wgrad_tcgen05.cu as well

extern "C" {

void kf_grouped_pair_mode(int mode) { kf_grouped_pair_mode_value = mode; }

// C[rows, N] (+)= grouped A[rows, K] x B_e.  offsets: int32[E + 1] on the device (offsets[0] = 0, offsets[E] <= rows;
// rows past offsets[E] are neither read nor written, so C may be sized by an upper bound known on the host).
//   b_mn == 0: B is [E][N][K] (K contiguous);  b_mn == 1: B is [E][K][N] (N contiguous; K must be a multiple of 64).
//   lda / ldc in elements (multiples of 8); B is dense.  E <= 256.  accumulate != 0: add to C.
int kf_grouped_gemm_acc_bf16(const void* A, const void* B, void* C, const void* offsets, int rows, int E, int N, int K,
                             long long lda, long long ldc, int b_mn, int accumulate, int num_sms, void* stream) {
  using namespace kf;
  using namespace kf::grp;
  if (E < 1 || E > MAX_EXPERTS || (lda & 7) || (ldc & 7) || (K & 7) || (N & 7) || (b_mn && (K % BK))) return 5;
  if (rows <= 0) return 0;
  if (kf_grouped_pair_mode_value && rows >= 256 && num_sms >= 2)
    return grp2::launch_grouped_gemm_2cta(A, B, C, offsets, rows, E, N, K, lda, ldc, b_mn, accumulate, num_sms,
                                          (cudaStream_t)stream, reinterpret_cast<int*>(kf_status_device_ptr()));
  CUtensorMap ma, mb;
  int rc = make_map_2d_bf16(&ma, A, rows, K, lda, BK, BM);
  if (rc) return 100 + rc;
  rc = b_mn ? make_map_2d_bf16(&mb, B, uint64_t(E) * K, N, N, 64, BK) : make_map_2d_bf16(&mb, B, uint64_t(E) * N, K, K, BK, BN);
  if (rc) return 200 + rc;
  const int upper = ((rows + BM - 1) / BM + E) * ((N + BN - 1) / BN);  // at most one partial tile per expert
  const int grid = upper < num_sms ? upper : num_sms;
  cudaStream_t st = (cudaStream_t)stream;
  return b_mn ? launch<true, false>(ma, mb, mb, C, nullptr, offsets, E, N, K, ldc, 0, accumulate, grid, st)
              : launch<false, false>(ma, mb, mb, C, nullptr, offsets, E, N, K, ldc, 0, accumulate, grid, st);
}

int kf_grouped_gemm_bf16(const void* A, const void* B, void* C, const void* offsets, int rows, int E, int N, int K,
                         long long lda, long long ldc, int b_mn, int num_sms, void* stream) {
  return kf_grouped_gemm_acc_bf16(A, B, C, offsets, rows, E, N, K, lda, ldc, b_mn, 0, num_sms, stream);
}

// H[rows, F] = silu(A x Wg_e) * (A x Wu_e) per expert; GU (optional, [rows, 2F]) receives the pre-activations
// (gate | up).  Wg / Wu: [E][F][K] (b_mn == 0) or [E][K][F] (b_mn == 1).  F, K multiples of 8 (64 for K when b_mn).
int kf_grouped_swiglu_bf16(const void* A, const void* Wg, const void* Wu, void* H, void* GU, const void* offsets, int rows,
                           int E, int F, int K, long long lda, long long ldh, long long ldgu, int b_mn, int num_sms,
                           void* stream) {
  using namespace kf;
  using namespace kf::grp;
  if (E < 1 || E > MAX_EXPERTS || (lda & 7) || (ldh & 7) || (GU && (ldgu & 7)) || (K & 7) || (F & 7) || (b_mn && (K % BK)))
    return 5;
  if (rows <= 0) return 0;
  if (kf_grouped_pair_mode_value && rows >= 256 && num_sms >= 2)
    return grp2::launch_grouped_swiglu_2cta(A, Wg, Wu, H, GU, offsets, rows, E, F, K, lda, ldh, ldgu, b_mn, num_sms,
                                            (cudaStream_t)stream, reinterpret_cast<int*>(kf_status_device_ptr()));
  CUtensorMap ma, mg, mu;
  int rc = make_map_2d_bf16(&ma, A, rows, K, lda, BK, BM);
  if (rc) return 100 + rc;
  if (b_mn) {
    rc = make_map_2d_bf16(&mg, Wg, uint64_t(E) * K, F, F, 64, BK);
    if (!rc) rc = make_map_2d_bf16(&mu, Wu, uint64_t(E) * K, F, F, 64, BK);
  } else {
    rc = make_map_2d_bf16(&mg, Wg, uint64_t(E) * F, K, K, BK, BN / 2);
    if (!rc) rc = make_map_2d_bf16(&mu, Wu, uint64_t(E) * F, K, K, BK, BN / 2);
  }
  if (rc) return 200 + rc;
  const int upper = ((rows + BM - 1) / BM + E) * ((F + BN / 2 - 1) / (BN / 2));
  const int grid = upper < num_sms ? upper : num_sms;
  cudaStream_t st = (cudaStream_t)stream;
  return b_mn ? launch<true, true>(ma, mg, mu, H, GU, offsets, E, F, K, ldh, ldgu, 0, grid, st)
              : launch<false, true>(ma, mg, mu, H, GU, offsets, E, F, K, ldh, ldgu, 0, grid, st);
}

// d[gate | up] of an expert feed-forward from the output gradient: DGU[rows, 2F] (may alias GU) = SwiGLU'(GU) applied to
// dh = DY[rows, K] x W_e, with dh living only in tensor memory.  W: the down weights, [E][F][K] (b_mn == 0) or
// [E][K][F] (b_mn == 1).  F, K multiples of 8 (64 for K when b_mn); pitches multiples of 8.  CTA-pair tiles only.
int kf_grouped_swiglu_bwd_bf16(const void* DY, const void* W, const void* GU, void* DGU, const void* offsets, int rows, int E,
                               int F, int K, long long lda, long long ldgu, int b_mn, int num_sms, void* stream) {
  using namespace kf;
  if (E < 1 || E > grp::MAX_EXPERTS || (lda & 7) || (ldgu & 7) || (K & 7) || (F & 7) || (b_mn && (K % grp::BK)) || num_sms < 2)
    return 5;
  if (rows <= 0) return 0;
  return grp2::launch_grouped_swiglu_bwd_2cta(DY, W, GU, DGU, offsets, rows, E, F, K, lda, ldgu, b_mn, num_sms,
                                              (cudaStream_t)stream, reinterpret_cast<int*>(kf_status_device_ptr()));
}

}  // extern "C"
