// Weight gradient of the ragged grouped GEMM with CTA pairs (tcgen05 cta_group::2):
//
//   Out[e] (M x N) = A[rows of expert e, :M]^T * B[rows of expert e, :N]        for every expert e
//
// Same contract as the single-CTA kernel in grouped_wgrad_tcgen05.cu; a pair of CTAs owns a 256 x 256 tile of one
// expert's output.  CTA r loads, for every 64-row block of the expert's token range, columns [m0 + 128 r, + 128) of A
// and [n0 + 128 r, + 128) of B (both MN-major: the reduction index is the slow one in memory), 32 KB per CTA and
// k-block instead of the 48 KB of the 128 x 256 single-CTA tile.
//
// The ragged tail: the last 64-row block of an expert usually runs into the next expert's rows, and every CTA has to
// zero those rows of ITS OWN shared-memory stage before the MMAs read it.  Two hand-over protocols therefore:
//   full 64-row blocks   as in gemm_tcgen05_2cta.cu: both CTAs' TMA bytes are counted on the leader's full[s]
//   the tail block       (at most one per tile) each CTA's loads complete on its own full[s]; the peer's MMA warp waits
//                        for it, zeroes its tail rows, fences them towards the async proxy and arrives (remote,
//                        release) on the leader's ready[s]; the leader does the same with its own stage and its
//                        issuing thread then waits for ready[s] (cluster-scope acquire) before the MMAs
//   empty[s]             both CTAs: released by the leader's tcgen05.commit, multicast to the pair
//   tfull[a] / tempty[a] as in gemm_tcgen05_2cta.cu (8 epilogue-warp arrivals on the leader)
// The peer's full[s] and the leader's ready[s] complete one phase per TAIL use of stage s only; both sides keep one
// parity bit per stage for them.  (Relaying every block through the peer's warp was measured 2.4x slower than the
// single-CTA kernel.)
// All waits are bounded; TMA loads carry no cluster multicast.
//
// Replaces the per-expert weight-gradient products that autograd derives for the padded `torch._grouped_mm`
// call of the reference (kempnerforge/model/moe.py:20-145).
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tile_math.h"
#include "pair_common.cuh"

namespace kf {
namespace gwg2 {

using namespace kf::pairops;

constexpr int CTA_M = 128, TILE_M = 256, TILE_N = 256, HALF_N = 128, BK = 64, STAGES = 6, UMMA_K = 16;
constexpr int BLOCK_BYTES = 64 * BK * 2;  // one {64 columns, BK rows} box
constexpr int A_BYTES = (CTA_M / 64) * BLOCK_BYTES, B_BYTES = (HALF_N / 64) * BLOCK_BYTES;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192, TMEM_COLS = 512;
constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256;

using Tile = tilemath::WgradTile;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
kf_grouped_wgrad_tcgen05_2cta(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                              __nv_bfloat16* __restrict__ out, const int* __restrict__ offsets, int E, int M, int N,
                              int* status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto ready_bar = [&](int s) { return bar_base + 8u * (2 * STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (3 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (3 * STAGES + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (3 * STAGES + 4);
  const uint32_t tmem_slot = bar_base + 8u * (3 * STAGES + 5);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int m_blocks = (M + TILE_M - 1) / TILE_M, n_blocks = (N + TILE_N - 1) / TILE_N;
  const int num_tiles = E * m_blocks * n_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(ready_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);
    }
    mbar_init(drain_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&map_a);
    tma_prefetch_desc(&map_b);
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (lane == 0) {
      int it = 0, peer_tails = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        const Tile tl = tilemath::wgrad_decode(t, m_blocks, n_blocks, TILE_M, TILE_N, offsets);
        const int k_blocks = (tl.rows + BK - 1) / BK;
        const int m0 = tl.m0 + int(rank) * CTA_M, n0 = tl.n0 + int(rank) * HALF_N;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
          const int row = tl.row0 + kb * BK;
          if (tl.rows - kb * BK < BK) {
            // tail block: every CTA's bytes complete on its own barrier (its MMA warp zeroes the foreign rows)
            mbar_expect_tx(full_bar(s), STAGE_BYTES);
#pragma unroll
            for (int c = 0; c < CTA_M / 64; ++c) tma_load_2d(a_dst + c * BLOCK_BYTES, &map_a, full_bar(s), m0 + 64 * c, row);
#pragma unroll
            for (int c = 0; c < HALF_N / 64; ++c) tma_load_2d(b_dst + c * BLOCK_BYTES, &map_b, full_bar(s), n0 + 64 * c, row);
            if (!leader) ++peer_tails;
          } else {
            const uint32_t lead_full = full_bar(s) & PEER_BIT_MASK;
            if (leader) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
#pragma unroll
            for (int c = 0; c < CTA_M / 64; ++c) tma_load_2d_pair(a_dst + c * BLOCK_BYTES, &map_a, lead_full, m0 + 64 * c, row);
#pragma unroll
            for (int c = 0; c < HALF_N / 64; ++c) tma_load_2d_pair(b_dst + c * BLOCK_BYTES, &map_b, lead_full, n0 + 64 * c, row);
          }
        }
      }
      // Copies into this CTA's shared memory are complete once the stages they filled were consumed (empty flipped)
      // or, on the error path, once the barrier that counts them flipped.
      if (leader)
        for (int j = max(0, it - STAGES); j < it; ++j)
          mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1, status, KF_ERR_WAIT_DRAIN);
      (void)peer_tails;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ stage preparation (both CTAs) + MMA issue (leader)
    // the whole warp walks the loop (the tail rows of a stage are zeroed by all lanes); the peer's warp only acts on
    // tail blocks
    constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, TILE_N, true, true);
    int it = 0, tile_iter = 0;
    uint32_t tail_parity = 0;  // bit s: parity of the next tail use of stage s (peer: its full[s]; leader: ready[s])
    bool ok = true;
    auto zero_tail = [&](uint32_t a_src, int valid) {
      // rows valid..63 of every 64-column block belong to another expert (or to nobody)
      constexpr int BLOCKS = STAGE_BYTES / BLOCK_BYTES;
      for (int i = lane; i < tilemath::tail_chunks(valid, BK, BLOCKS); i += 32) {
        const uint32_t addr = a_src + tilemath::tail_chunk_offset(i, valid, BK, BLOCK_BYTES);
        asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
      }
      fence_async_smem();
      __syncwarp();
    };
    for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tile_iter) {
      const Tile tl = tilemath::wgrad_decode(t, m_blocks, n_blocks, TILE_M, TILE_N, offsets);
      const int k_blocks = (tl.rows + BK - 1) / BK;
      const int acc = tile_iter & 1;
      if (!leader) {
        // peer: only the tail block (the last one, when the expert's row count is not a multiple of 64)
        const int valid = tl.rows - (k_blocks - 1) * BK;
        if (k_blocks > 0 && valid < BK) {
          const int s = (it + k_blocks - 1) % STAGES;
          ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), (tail_parity >> s) & 1, status, KF_ERR_WAIT_FULL));
          if (!ok) break;
          tail_parity ^= 1u << s;
          zero_tail(smem_base + s * STAGE_BYTES, valid);
          if (lane == 0) arrive_on_cta(ready_bar(s), 0);  // this CTA's half of the stage is in place
        }
        it += k_blocks;
        continue;
      }
      ok = __all_sync(0xffffffffu, mbar_wait(tempty_bar(acc), ((tile_iter >> 1) & 1) ^ 1, status, KF_ERR_WAIT_TMEM_EMPTY));
      if (!ok) break;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * TILE_N;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(full_bar(s), ph, status, KF_ERR_WAIT_FULL));
        if (!ok) break;
        const uint32_t a_src = smem_base + s * STAGE_BYTES, b_src = a_src + A_BYTES;
        const int valid = tl.rows - kb * BK;
        const bool tail = valid < BK;
        if (tail) zero_tail(a_src, valid);
        if (lane == 0) {
          if (tail && !mbar_wait_cluster(ready_bar(s), (tail_parity >> s) & 1, status, KF_ERR_WAIT_FULL)) ok = false;
          if (ok) {
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              mma_pair_f16(d_tmem, umma_desc_sw128(a_src + k * (UMMA_K * 128), BLOCK_BYTES, 1024),
                           umma_desc_sw128(b_src + k * (UMMA_K * 128), BLOCK_BYTES, 1024), idesc, (kb | k) != 0);
            commit_pair(empty_bar(s));
          }
        }
        if (tail) {
          tail_parity ^= 1u << s;
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
      }
      if (ok && lane == 0) commit_pair(tfull_bar(acc));
    }
    if (leader && lane == 0) {
      // every MMA must have retired before either CTA gives up its shared or tensor memory
      asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(drain_bar)
                   : "memory");
      mbar_wait(drain_bar, 0, status, KF_ERR_WAIT_DRAIN);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quarter = warp & 3;
    int tile_iter = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tile_iter) {
      const Tile tl = tilemath::wgrad_decode(t, m_blocks, n_blocks, TILE_M, TILE_N, offsets);
      const int acc = tile_iter & 1;
      if (!mbar_wait(tfull_bar(acc), (tile_iter >> 1) & 1, status, KF_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int r = int(rank) * CTA_M + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * TILE_N;
      __nv_bfloat16* c_row = out + (size_t(tl.e) * M + tl.m0 + r) * N + tl.n0;
      const bool row_ok = tl.m0 + r < M;
#pragma unroll 1
      for (int c = 0; c < TILE_N / 32; ++c) {
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

// Contract of kf_grouped_wgrad_bf16 (grouped_wgrad_tcgen05.cu), which dispatches here.
int launch_grouped_wgrad_2cta(const void* A, const void* B, void* Out, const void* offsets, int rows, int E, int M, int N,
                              long long lda, long long ldb, int num_sms, cudaStream_t stream, int* status) {
  CUtensorMap ma, mb;
  int rc = make_map_2d_bf16(&ma, A, rows, M, lda, 64, BK);
  if (rc) return 100 + rc;
  rc = make_map_2d_bf16(&mb, B, rows, N, ldb, 64, BK);
  if (rc) return 200 + rc;
  const long long tiles = (long long)E * ((M + TILE_M - 1) / TILE_M) * ((N + TILE_N - 1) / TILE_N);
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = (int)tiles;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kf_grouped_wgrad_tcgen05_2cta, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  kf_grouped_wgrad_tcgen05_2cta<<<pairs * 2, THREADS, SMEM, stream>>>(
      ma, mb, reinterpret_cast<__nv_bfloat16*>(Out), reinterpret_cast<const int*>(offsets), E, M, N, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // namespace gwg2
}  // namespace kf
