// Weight gradient of the ragged grouped GEMM on the 5th-generation tensor cores:
//
//   Out[e] (M x N) = A[rows of expert e, :M]^T * B[rows of expert e, :N]        for every expert e
//
// A and B hold token rows sorted by expert (`offsets[e] .. offsets[e+1]`, int32 on the DEVICE), so the
// reduction dimension of each product is ragged.  Both operands are read "MN-major" (the reduction index is
// the slow one in memory), which is what TMA delivers for a {64 columns, 64 rows} box with the 128-byte swizzle.
// The last 64-row block of an expert usually runs into the next expert's rows (or past the end of the buffer's
// valid part): the MMA warp zeroes those rows of the landed stage in shared memory (a k-row is one 128-byte line
// of each 64-column block, whatever the swizzle), fences generic -> async proxy, and only then issues the MMAs.
// Experts without rows get a zero matrix.  Nothing is padded and nothing is read back to the host.
//
// Pipeline as in the other GEMMs: TMA producer warp -> 4-stage ring -> MMA warp (one issuing thread) ->
// double-buffered fp32 accumulators in TMEM -> four epilogue warps writing bf16.
//
// Replaces the per-expert weight-gradient products that autograd derives for the padded `torch._grouped_mm`
// call of the reference (kempnerforge/model/moe.py:20-145).
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tile_math.h"

namespace kf {
namespace gwg {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int BLOCK_BYTES = 64 * BK * 2;  // one {64 columns, BK rows} box
constexpr int A_STAGE_BYTES = (BM / 64) * BLOCK_BYTES, B_STAGE_BYTES = (BN / 64) * BLOCK_BYTES;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int THREADS = 192, TMEM_COLS = 512;
constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256;

using Tile = tilemath::WgradTile;

__device__ __forceinline__ Tile decode(int t, int m_blocks, int n_blocks, const int* offsets) {
  return tilemath::wgrad_decode(t, m_blocks, n_blocks, BM, BN, offsets);
}

__global__ void __launch_bounds__(THREADS, 1)
kf_grouped_wgrad_tcgen05(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         __nv_bfloat16* __restrict__ out, const int* __restrict__ offsets, int E, int M, int N,
                         int* status) {
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_blocks = (M + BM - 1) / BM, n_blocks = (N + BN - 1) / BN;
  const int num_tiles = E * m_blocks * n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
    mbar_init(drain_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const Tile tl = decode(t, m_blocks, n_blocks, offsets);
        const int k_blocks = (tl.rows + BK - 1) / BK;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * STAGE_BYTES, b_dst = a_dst + A_STAGE_BYTES;
          const int row = tl.row0 + kb * BK;
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
#pragma unroll
          for (int c = 0; c < BM / 64; ++c) tma_load_2d(a_dst + c * BLOCK_BYTES, &map_a, full_bar(s), tl.m0 + 64 * c, row);
#pragma unroll
          for (int c = 0; c < BN / 64; ++c) tma_load_2d(b_dst + c * BLOCK_BYTES, &map_b, full_bar(s), tl.n0 + 64 * c, row);
        }
      }
      for (int j = max(0, it - STAGES); j < it; ++j)
        mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1, status, KF_ERR_WAIT_DRAIN);
    }
  } else if (warp == 1) {
    // the whole warp walks the loop (the tail rows of a stage are zeroed by all lanes); lane 0 issues the MMAs
    constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, true, true);
    int it = 0, tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
      const Tile tl = decode(t, m_blocks, n_blocks, offsets);
      const int k_blocks = (tl.rows + BK - 1) / BK;
      const int acc = tile_iter & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(tempty_bar(acc), ((tile_iter >> 1) & 1) ^ 1, status, KF_ERR_WAIT_TMEM_EMPTY));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int s = it % STAGES;
        ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), (it / STAGES) & 1, status, KF_ERR_WAIT_FULL));
        if (!ok) break;
        const uint32_t a_src = smem_base + s * STAGE_BYTES, b_src = a_src + A_STAGE_BYTES;
        const int valid = tl.rows - kb * BK;
        if (valid < BK) {
          // rows valid..63 of every 64-column block belong to another expert (or to nobody): zero them
          constexpr int BLOCKS = STAGE_BYTES / BLOCK_BYTES;
          for (int i = lane; i < tilemath::tail_chunks(valid, BK, BLOCKS); i += 32) {
            const uint32_t addr = a_src + tilemath::tail_chunk_offset(i, valid, BK, BLOCK_BYTES);
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
          }
          fence_async_smem();
          __syncwarp();
        }
        if (lane == 0) {
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_f16(d_tmem, umma_desc_sw128(a_src + k * (UMMA_K * 128), BLOCK_BYTES, 1024),
                       umma_desc_sw128(b_src + k * (UMMA_K * 128), BLOCK_BYTES, 1024), idesc, (kb | k) != 0);
          tc_commit(empty_bar(s));
        }
        __syncwarp();
      }
      if (ok && lane == 0) tc_commit(tfull_bar(acc));
    }
    if (lane == 0) {
      tc_commit(drain_bar);
      mbar_wait(drain_bar, 0, status, KF_ERR_WAIT_DRAIN);
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    int tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
      const Tile tl = decode(t, m_blocks, n_blocks, offsets);
      const int acc = tile_iter & 1;
      if (!mbar_wait(tfull_bar(acc), (tile_iter >> 1) & 1, status, KF_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int r = quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      __nv_bfloat16* c_row = out + (size_t(tl.e) * M + tl.m0 + r) * N + tl.n0;
      const bool row_ok = tl.m0 + r < M;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        if (tl.rows > 0) {
          tmem_ld_32x32(t_row + c * 32, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        const int valid_cols = min(32, N - (tl.n0 + c * 32));
        if (row_ok && valid_cols > 0) store_chunk<__nv_bfloat16>(c_row + c * 32, v, valid_cols, false, nullptr);
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

}  // namespace gwg
}  // namespace kf

extern "C" void* kf_status_device_ptr();
extern int kf_grouped_pair_mode_value;

namespace kf {
namespace gwg2 {
int launch_grouped_wgrad_2cta(const void* A, const void* B, void* Out, const void* offsets, int rows, int E, int M, int N,
                              long long lda, long long ldb, int num_sms, cudaStream_t stream, int* status);
}
}  // namespace kf

extern "C" {

// Out[E][M][N] (bf16, dense) = per-expert A_e^T B_e.  A: [rows][lda] (M columns used), B: [rows][ldb] (N columns
// used), offsets: int32[E + 1] on the device (offsets[0] = 0, offsets[E] <= rows).  M, N, lda, ldb multiples of 8.
int kf_grouped_wgrad_bf16(const void* A, const void* B, void* Out, const void* offsets, int rows, int E, int M, int N,
                          long long lda, long long ldb, int num_sms, void* stream) {
  using namespace kf;
  using namespace kf::gwg;
  if (E < 1 || (lda & 7) || (ldb & 7) || (M & 7) || (N & 7) || rows < 1) return 5;
  if (kf_grouped_pair_mode_value && num_sms >= 2)
    return gwg2::launch_grouped_wgrad_2cta(A, B, Out, offsets, rows, E, M, N, lda, ldb, num_sms, (cudaStream_t)stream,
                                           reinterpret_cast<int*>(kf_status_device_ptr()));
  CUtensorMap ma, mb;
  int rc = make_map_2d_bf16(&ma, A, rows, M, lda, 64, BK);
  if (rc) return 100 + rc;
  rc = make_map_2d_bf16(&mb, B, rows, N, ldb, 64, BK);
  if (rc) return 200 + rc;
  int* status = reinterpret_cast<int*>(kf_status_device_ptr());
  const long long tiles = (long long)E * ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? (int)tiles : num_sms;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kf_grouped_wgrad_tcgen05, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  kf_grouped_wgrad_tcgen05<<<grid, THREADS, SMEM, (cudaStream_t)stream>>>(
      ma, mb, reinterpret_cast<__nv_bfloat16*>(Out), reinterpret_cast<const int*>(offsets), E, M, N, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // extern "C"
