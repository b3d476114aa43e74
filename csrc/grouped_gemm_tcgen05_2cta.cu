// Ragged grouped GEMM (mixture-of-experts feed-forward) with CTA pairs (tcgen05 cta_group::2):
//
//   C[rows of expert e, :N] (+)= A[rows of expert e, :K] * op(B_e)          for every expert e
//
// Same contract as the single-CTA kernel in grouped_gemm_tcgen05.cu (expert-sorted rows, int32 `offsets` on the
// device, nothing padded, no host read), with the tiling of the dense CTA-pair GEMM: two CTAs on neighbouring SMs own
// a 256 x 256 output tile, CTA r loads 128 of the tile's rows of A and 128 of its rows / columns of B, the leader
// issues 256 x 256 x 16 MMAs that read both CTAs' shared memory.  Per CTA and k-block 32 KB are loaded instead of the
// 48 KB of the 128 x 256 single-CTA tile, which leaves six pipeline stages and takes the shared-memory read port off
// the critical path.  A row tile never crosses an expert boundary: tiles are counted per expert (256 rows each, the
// last one partial) and the epilogue stores only the rows that belong to the expert.
//
// SWIGLU: two weight operands (gate: map_b, up: map_b2) of N = F hidden units each; a tile covers 128 hidden units,
// the leader CTA loads their gate weights and the peer the matching up weights, so every CTA's accumulator holds
// [gate 128 | up 128] for its 128 rows; the epilogue writes h = silu(gate) * up and optionally the pre-activations.
//
// EPI == 2: SwiGLU backward in the epilogue of the down projection's input-gradient product (see the launcher).
//
// Synchronisation as in gemm_tcgen05_2cta.cu (all waits bounded); TMA loads carry no cluster multicast.
// Replaces the padded torch._grouped_mm calls of the reference (kempnerforge/model/moe.py:20-145).
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tile_math.h"
#include "pair_common.cuh"

namespace kf {
namespace grp2 {

using namespace kf::pairops;

constexpr int CTA_M = 128, TILE_M = 256, TILE_N = 256, HALF_N = 128, BK = 64, STAGES = 6, UMMA_K = 16;
constexpr int A_BYTES = CTA_M * BK * 2, B_BYTES = HALF_N * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192, TMEM_COLS = 512;
constexpr int MAX_EXPERTS = 256;
constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256 + (MAX_EXPERTS + 1) * 4;

using Tile = tilemath::GroupedTile;

template <bool B_MN, int EPI>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
kf_grouped_gemm_tcgen05_2cta(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
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
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  constexpr bool SWIGLU = EPI == 1;
  constexpr int TN = SWIGLU ? HALF_N : TILE_N;  // output columns (hidden units) per tile
  const int n_blocks = (N + TN - 1) / TN;
  const int k_blocks = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
    }
    mbar_init(drain_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
    if (SWIGLU) tma_prefetch_desc(&map_b2);
    tilemath::grouped_tile_starts(offsets, E, TILE_M, tile_start);  // both CTAs of a pair compute the same table
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anyone signals across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const int num_tiles = tile_start[E] * n_blocks;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      // the leader fetches the gate weights (or the first 128 columns), the peer the up weights (or the last 128)
      const CUtensorMap* my_b = (SWIGLU && !leader) ? &map_b2 : &map_b;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        const Tile tl = tilemath::grouped_decode(t, n_blocks, tile_start, offsets, E, TILE_M);
        const int m0 = tl.row0 + int(rank) * CTA_M;
        const int n0 = SWIGLU ? tl.nb * TN : tl.nb * TN + int(rank) * HALF_N;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_BYTES;
          const uint32_t lead_full = full_bar(s) & PEER_BIT_MASK;
          if (leader) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
          const int k0 = kb * BK;
          tma_load_2d_pair(a_dst, &map_a, lead_full, k0, m0);
          if (!B_MN) {
            tma_load_2d_pair(b_dst, my_b, lead_full, k0, tl.e * N + n0);
          } else {
#pragma unroll
            for (int c = 0; c < HALF_N / 64; ++c)
              tma_load_2d_pair(b_dst + c * (64 * BK * 2), my_b, lead_full, n0 + 64 * c, tl.e * K + k0);
          }
        }
      }
      // Copies into this CTA's shared memory are complete once the stages they filled were consumed (empty
      // flipped) or, on the error path, once the leader's full barrier flipped.
      if (leader)
        for (int j = max(0, it - STAGES); j < it; ++j)
          mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1, status, KF_ERR_WAIT_DRAIN);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, TILE_N, false, B_MN);
      int it = 0, tile_iter = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tile_iter) {
        const int acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1;
        if (!mbar_wait(tempty_bar(acc), acc_ph ^ 1, status, KF_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * TILE_N;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(full_bar(s), ph, status, KF_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_src = smem_base + s * STAGE_BYTES;
          const uint32_t b_src = a_src + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t bd = B_MN ? umma_desc_sw128(b_src + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                     : umma_desc_sw128(b_src + k * (UMMA_K * 2), 16, 1024);
            mma_pair_f16(d_tmem, umma_desc_sw128(a_src + k * (UMMA_K * 2), 16, 1024), bd, idesc, (kb | k) != 0);
          }
          commit_pair(empty_bar(s));
        }
        if (ok) commit_pair(tfull_bar(acc));
      }
      // every MMA must have retired before either CTA gives up its shared or tensor memory
      asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(drain_bar)
                   : "memory");
      mbar_wait(drain_bar, 0, status, KF_ERR_WAIT_DRAIN);
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quarter = warp & 3;
    int tile_iter = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tile_iter) {
      const Tile tl = tilemath::grouped_decode(t, n_blocks, tile_start, offsets, E, TILE_M);
      const int acc = tile_iter & 1;
      if (!mbar_wait(tfull_bar(acc), (tile_iter >> 1) & 1, status, KF_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int r = int(rank) * CTA_M + quarter * 32 + lane;  // row inside the 256-row tile
      const int col0 = tl.nb * TN;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * TILE_N;
      __nv_bfloat16* c_row = C + size_t(tl.row0 + r) * ldc + col0;
      if constexpr (EPI == 2) {
        // SwiGLU backward: the accumulator is dh[rows, F] (never written); GU = the saved pre-activations [rows, 2F]
        // (gate | up), C = d[gate | up] [rows, 2F] (may be the same buffer: every element is read and written by one
        // thread)
        const __nv_bfloat16* gu_row = GU + size_t(tl.row0 + r) * ldgu + col0;
#pragma unroll 1
        for (int c = 0; c < TILE_N / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_row + c * 32, v);
          tmem_ld_wait();
          const int valid_cols = min(32, N - (col0 + c * 32));
          if (r < tl.valid && valid_cols > 0) {
            swiglu_bwd_chunk(v, gu_row + c * 32, gu_row + N + c * 32, c_row + c * 32, c_row + N + c * 32, valid_cols);
          }
        }
      } else if constexpr (SWIGLU) {
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
        for (int c = 0; c < TILE_N / 32; ++c) {
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
      if (lane == 0) arrive_on_cta(tempty_bar(acc), 0);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's shared and tensor memory stay alive until the leader's MMAs have retired
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <bool B_MN, int EPI>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& mb2, void* C, void* GU, const void* offsets,
                  int E, int N, int K, long long ldc, long long ldgu, int accumulate, int pairs, cudaStream_t st, int* status) {
  auto kern = kf_grouped_gemm_tcgen05_2cta<B_MN, EPI>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  kern<<<pairs * 2, THREADS, SMEM, st>>>(ma, mb, mb2, reinterpret_cast<__nv_bfloat16*>(C), reinterpret_cast<__nv_bfloat16*>(GU),
                                         reinterpret_cast<const int*>(offsets), E, N, K, ldc, ldgu, accumulate, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// Contracts of kf_grouped_gemm_acc_bf16 / kf_grouped_swiglu_bf16 (grouped_gemm_tcgen05.cu), which dispatch here.
int launch_grouped_gemm_2cta(const void* A, const void* B, void* C, const void* offsets, int rows, int E, int N, int K,
                             long long lda, long long ldc, int b_mn, int accumulate, int num_sms, cudaStream_t st, int* status) {
  CUtensorMap ma, mb;
  int rc = make_map_2d_bf16(&ma, A, rows, K, lda, BK, CTA_M);
  if (rc) return 100 + rc;
  rc = b_mn ? make_map_2d_bf16(&mb, B, uint64_t(E) * K, N, N, 64, BK) : make_map_2d_bf16(&mb, B, uint64_t(E) * N, K, K, BK, HALF_N);
  if (rc) return 200 + rc;
  const int upper = ((rows + TILE_M - 1) / TILE_M + E) * ((N + TILE_N - 1) / TILE_N);  // at most one partial tile per expert
  int pairs = num_sms / 2;
  if (upper < pairs) pairs = upper;
  return b_mn ? launch<true, 0>(ma, mb, mb, C, nullptr, offsets, E, N, K, ldc, 0, accumulate, pairs, st, status)
              : launch<false, 0>(ma, mb, mb, C, nullptr, offsets, E, N, K, ldc, 0, accumulate, pairs, st, status);
}

int launch_grouped_swiglu_2cta(const void* A, const void* Wg, const void* Wu, void* H, void* GU, const void* offsets, int rows,
                               int E, int F, int K, long long lda, long long ldh, long long ldgu, int b_mn, int num_sms,
                               cudaStream_t st, int* status) {
  CUtensorMap ma, mg, mu;
  int rc = make_map_2d_bf16(&ma, A, rows, K, lda, BK, CTA_M);
  if (rc) return 100 + rc;
  if (b_mn) {
    rc = make_map_2d_bf16(&mg, Wg, uint64_t(E) * K, F, F, 64, BK);
    if (!rc) rc = make_map_2d_bf16(&mu, Wu, uint64_t(E) * K, F, F, 64, BK);
  } else {
    rc = make_map_2d_bf16(&mg, Wg, uint64_t(E) * F, K, K, BK, HALF_N);
    if (!rc) rc = make_map_2d_bf16(&mu, Wu, uint64_t(E) * F, K, K, BK, HALF_N);
  }
  if (rc) return 200 + rc;
  const int upper = ((rows + TILE_M - 1) / TILE_M + E) * ((F + HALF_N - 1) / HALF_N);
  int pairs = num_sms / 2;
  if (upper < pairs) pairs = upper;
  return b_mn ? launch<true, 1>(ma, mg, mu, H, GU, offsets, E, F, K, ldh, ldgu, 0, pairs, st, status)
              : launch<false, 1>(ma, mg, mu, H, GU, offsets, E, F, K, ldh, ldgu, 0, pairs, st, status);
}

// d[gate | up] (rows x 2F, may alias GU) from dy (rows x K) and the down weights: W [E][F][K] (b_mn == 0: K
// contiguous) or [E][K][F] (b_mn == 1); the accumulator dh = dy W_e^T (resp. dy W_e) is consumed by the epilogue.
int launch_grouped_swiglu_bwd_2cta(const void* DY, const void* W, const void* GU, void* DGU, const void* offsets, int rows,
                                   int E, int F, int K, long long lda, long long ldgu, int b_mn, int num_sms, cudaStream_t st,
                                   int* status) {
  CUtensorMap ma, mb;
  int rc = make_map_2d_bf16(&ma, DY, rows, K, lda, BK, CTA_M);
  if (rc) return 100 + rc;
  rc = b_mn ? make_map_2d_bf16(&mb, W, uint64_t(E) * K, F, F, 64, BK) : make_map_2d_bf16(&mb, W, uint64_t(E) * F, K, K, BK, HALF_N);
  if (rc) return 200 + rc;
  const int upper = ((rows + TILE_M - 1) / TILE_M + E) * ((F + TILE_N - 1) / TILE_N);
  int pairs = num_sms / 2;
  if (upper < pairs) pairs = upper;
  void* gu = const_cast<void*>(GU);
  return b_mn ? launch<true, 2>(ma, mb, mb, DGU, gu, offsets, E, F, K, ldgu, ldgu, 0, pairs, st, status)
              : launch<false, 2>(ma, mb, mb, DGU, gu, offsets, E, F, K, ldgu, ldgu, 0, pairs, st, status);
}

}  // namespace grp2
}  // namespace kf
