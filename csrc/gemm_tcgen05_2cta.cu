// bf16 GEMM with CTA pairs (tcgen05 cta_group::2):  C[M,N] = A[M,K] * B[N,K]^T (+ C) (+ R).
//
// A cluster of two CTAs on neighbouring SMs owns one 256x256 output tile.  CTA r of the pair loads
// its 128 rows of A and its 128 rows of B (N-half r) with TMA; the leader CTA (rank 0) issues
// tcgen05.mma.cta_group::2 instructions of shape 256x256x16 that read both CTAs' shared memory and
// write each CTA's half of the accumulator (128 lanes x 256 columns) into that CTA's tensor memory.
// Per CTA and k-block only 32 KB are loaded (half of what the single-CTA 128x256 tile needs for the
// same math per SM), which leaves room for 6 pipeline stages.
//
// Synchronisation (all waits bounded, see common.cuh):
//   full[s]    leader only: armed by the leader's producer with the bytes of BOTH CTAs; the peer's TMA
//              loads complete on the leader's barrier (peer bit of the barrier address cleared)
//   empty[s]   both CTAs: released by the leader's tcgen05.commit, multicast to the pair
//   tfull[a]   both CTAs: accumulator a complete (multicast commit)
//   tempty[a]  leader only: 8 arrivals = 4 epilogue warps of each CTA (the peer arrives remotely)
// TMA loads carry no cluster multicast; every CTA fetches its own operands.
#include "common.cuh"
#include "gemm_epilogue.cuh"
#include "tile_math.h"
#include "pair_common.cuh"

namespace kf2 {

using namespace kf;
using namespace kf::pairops;

constexpr int CTA_M = 128;   // rows of A per CTA
constexpr int TILE_M = 256;  // rows per CTA pair
constexpr int TILE_N = 256;
constexpr int HALF_N = 128;  // rows of B per CTA
constexpr int BK = 64;
constexpr int STAGES = 6;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = CTA_M * BK * 2;   // 16 KB
constexpr int B_BYTES = HALF_N * BK * 2;  // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int THREADS_GATHER = 320;  // + four copy warps (6..9) in the weight-gathering variant
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;
constexpr size_t SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + 1024 + 256;

// ---- weight-gathering variant (sharded data parallelism: every rank keeps 1/world of each weight's rows) ------
// The B operand of the GEMM is a weight (or a row stack of weights: q | k | v, gate | up) that is NOT resident: each
// of its segments is cut into `world` equal contiguous pieces, piece r living in rank r's parameter shard.  The
// kernel's copy warps pull the pieces over NVLink (plain peer loads; the local piece by local loads) into a staging
// copy of the operand in this GPU's memory, chunk by chunk in the order in which the tiles will consume them (own
// rows first), and bump one counter per 128-row block; the TMA producer of a tile waits (bounded) for the counter
// of the row block it is about to load, so the transfer of later rows overlaps the math on earlier ones.  Nothing
// in here waits for another GPU: peers only have to keep their shards unchanged while the kernel runs.
constexpr int GATHER_CHUNK_ELEMS = 16384;  // 32 KB per copy step of one CTA's copy warps
constexpr int GATHER_MAX_SEG = 4;
constexpr int GATHER_GROUP_N = 4;          // column tiles that share one sweep over the row tiles
struct GatherArgs {
  const __nv_bfloat16* peer[8];            // every rank's parameter shard (this unit)
  __nv_bfloat16* stage;                    // local staging copy of the whole operand ([rows][K], rows contiguous)
  int* flags;                              // [row blocks] counters + [1] work counter, zeroed before the launch
  long long seg_dst[GATHER_MAX_SEG];       // first element of the segment inside the operand
  long long seg_len[GATHER_MAX_SEG];       // elements of the segment (all ranks together)
  long long seg_src[GATHER_MAX_SEG];       // first element of the segment's piece inside a rank's shard
  int n_seg, world;
  int chunks_per_rb;                       // chunks per 128-row block = K / 128
  int total_chunks, row_blocks;
  int n_tile_start;                        // rotation of the column-tile order: the tile that holds own rows
};

__device__ __forceinline__ void red_release_gpu_add(int* addr, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

struct TileCoord {
  int m, n;
};
__device__ __forceinline__ TileCoord tile_coord(int t, int m_blocks, int n_blocks) {
  TileCoord tc;
  tilemath::raster(t, m_blocks, n_blocks, GROUP_M, tc.m, tc.n);
  return tc;
}

// SWIGLU != 0 (bf16, K-major operands only): B is the stacked [gate ; up] weight of a SwiGLU MLP with F = N rows
// each.  The pair's B tile is made of 128 gate rows (loaded by the leader) and the matching 128 up rows (loaded by
// the peer), so every CTA's accumulator holds gate in columns 0..127 and up in columns 128..255 for the same 128
// hidden units; the epilogue writes h = silu(gate) * up to C[M, F] and, when R is given, the pre-activations to
// R[M, 2F] (gate | up) for the backward pass.
//
// SWIGLU == 2 (bf16, K-major operands only): rotary position embedding in the epilogue of a fused Q | K | V
// projection.  Output columns [0, rope.cols) are heads of `rope.hd` columns that get rotated (pairs (i, i + hd/2)
// with the angle of position `row % rope.S`), the remaining columns (V) are stored as they are.  The rotation is
// applied to the fp32 accumulators, so q and k are rounded to bf16 once.
//
// SWIGLU == 4 (bf16 output, A and B the same matrix X): symmetric product  C = alpha * X X^T + beta * R + diag * I
// (or X^T X with MN-major operands), N = M.  Only the tiles on and above the diagonal are computed; every tile
// above the diagonal is stored twice, as it is and transposed, so C comes out exactly symmetric at about half the
// tensor-core work.  R must be symmetric as well (it is read at the untransposed position only).
struct RopeArgs {
  const float* cosT;  // [S][hd / 2]
  const float* sinT;
  int S, cols, hd;
  float alpha, beta, diag;  // SWIGLU == 4 only
};

template <bool A_MN, bool B_MN, typename OutT, int SWIGLU = 0, bool GATHER = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GATHER ? THREADS_GATHER : THREADS, 1)
kf_gemm_bf16_tcgen05_2cta(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                          OutT* __restrict__ C, const OutT* __restrict__ R, int M, int N, int K, int ldc, int ldr,
                          int accumulate, int* status, RopeArgs rope, const __grid_constant__ GatherArgs ga) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };
  const uint32_t drain_bar = bar_base + 8u * (2 * STAGES + 4);
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 5);
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = leader
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int m_blocks = (M + TILE_M - 1) / TILE_M;
  const int n_blocks = SWIGLU == 1 ? (N + HALF_N - 1) / HALF_N : (N + TILE_N - 1) / TILE_N;
  const int num_tiles = SWIGLU == 4 ? m_blocks * (m_blocks + 1) / 2 : m_blocks * n_blocks;
  const int k_blocks = (K + BK - 1) / BK;
  // gathering variant: column tiles are the slow index (a weight row block is consumed completely soon after it
  // arrived), rotated so that the tile holding this rank's own rows comes first
  auto tile_at = [&](int t) {
    TileCoord tc;
    if constexpr (SWIGLU == 4) {  // upper triangle, row by row: consecutive tiles share their A rows
      int m = 0, rest = t;
      while (rest >= m_blocks - m) {
        rest -= m_blocks - m;
        ++m;
      }
      tc.m = m;
      tc.n = m + rest;
    } else if constexpr (GATHER) {
      int nr;
      tilemath::raster(t, n_blocks, m_blocks, GATHER_GROUP_N, nr, tc.m);
      tc.n = nr + ga.n_tile_start;
      if (tc.n >= n_blocks) tc.n -= n_blocks;
    } else {
      tc = tile_coord(t, m_blocks, n_blocks);
    }
    return tc;
  };

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
      int it = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        const TileCoord tc = tile_at(t);
        const int m0 = tc.m * TILE_M + int(rank) * CTA_M;
        const int n0 = SWIGLU == 1 ? tc.n * HALF_N + int(rank) * N  // leader: gate rows, peer: the matching up rows
                                   : tc.n * TILE_N + int(rank) * HALF_N;
        if constexpr (GATHER) {
          // the 128 weight rows this CTA loads must have landed in the staging copy
          if (n0 < N * (SWIGLU == 1 ? 2 : 1)) {
            if (!flag_wait_ge(ga.flags + n0 / HALF_N, ga.chunks_per_rb, status)) { ok = false; break; }
            asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy stores -> this thread's TMA reads
          }
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(empty_bar(s), ph ^ 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * STAGE_BYTES;
          const uint32_t b_dst = a_dst + A_BYTES;
          const uint32_t lead_full = full_bar(s) & PEER_BIT_MASK;
          if (leader) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
          const int k0 = kb * BK;
          if (!A_MN) {
            tma_load_2d_pair(a_dst, &map_a, lead_full, k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < CTA_M / 64; ++c)
              tma_load_2d_pair(a_dst + c * (64 * BK * 2), &map_a, lead_full, m0 + 64 * c, k0);
          }
          if (!B_MN) {
            tma_load_2d_pair(b_dst, &map_b, lead_full, k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < HALF_N / 64; ++c)
              tma_load_2d_pair(b_dst + c * (64 * BK * 2), &map_b, lead_full, n0 + 64 * c, k0);
          }
        }
      }
      // Copies into this CTA's shared memory are complete once the stages they filled were consumed
      // (empty flipped) or, on the error path, once the leader's full barrier flipped.
      if (leader)
        for (int j = max(0, it - STAGES); j < it; ++j)
          mbar_wait(full_bar(j % STAGES), (j / STAGES) & 1, status, KF_ERR_WAIT_DRAIN);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = umma_idesc_bf16(TILE_M, TILE_N, A_MN, B_MN);
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
            const uint64_t ad = A_MN ? umma_desc_sw128(a_src + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                     : umma_desc_sw128(a_src + k * (UMMA_K * 2), 16, 1024);
            const uint64_t bd = B_MN ? umma_desc_sw128(b_src + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                     : umma_desc_sw128(b_src + k * (UMMA_K * 2), 16, 1024);
            mma_pair_f16(d_tmem, ad, bd, idesc, (kb | k) != 0);
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
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quarter = warp & 3;
    int tile_iter = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += num_pairs, ++tile_iter) {
      const TileCoord tc = tile_at(t);
      const int acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      if (!mbar_wait(tfull_bar(acc), acc_ph, status, KF_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = tc.m * TILE_M + int(rank) * CTA_M + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * TILE_N;
      if constexpr (SWIGLU == 3) {
        // SwiGLU backward in the epilogue of the down projection's input-gradient GEMM: the accumulator is
        // dh[rows, F] (never written); R = the saved pre-activations [rows, 2F] (gate | up), C = d[gate | up]
        // [rows, 2F] (may be the same buffer: every element is read and written by one thread).
        const int col0 = tc.n * TILE_N;
        const __nv_bfloat16* gu_row = reinterpret_cast<const __nv_bfloat16*>(R) + size_t(row) * ldr + col0;
        __nv_bfloat16* d_row = reinterpret_cast<__nv_bfloat16*>(C) + size_t(row) * ldc + col0;
#pragma unroll 1
        for (int c = 0; c < TILE_N / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_row + c * 32, v);
          tmem_ld_wait();
          const int valid = min(32, N - (col0 + c * 32));
          if (row < M && valid > 0) {
            swiglu_bwd_chunk(v, gu_row + c * 32, gu_row + N + c * 32, d_row + c * 32, d_row + N + c * 32, valid);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_on_cta(tempty_bar(acc), 0);
        continue;
      }
      if constexpr (SWIGLU == 4) {
        const int col0 = tc.n * TILE_N;
        const bool mirror = tc.n != tc.m;
        __nv_bfloat16* c_out = reinterpret_cast<__nv_bfloat16*>(C);
        __nv_bfloat16* c_row = c_out + size_t(row) * ldc + col0;
        const __nv_bfloat16* r_row = R ? reinterpret_cast<const __nv_bfloat16*>(R) + size_t(row) * ldr + col0 : nullptr;
#pragma unroll 1
        for (int c = 0; c < TILE_N / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(t_row + c * 32, v);
          tmem_ld_wait();
          const int col = col0 + c * 32;
          const int valid = min(32, N - col);
          if (row < M && valid > 0) {
            uint32_t packed[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = rope.alpha * __uint_as_float(v[q * 8 + i]);
              if (r_row && q * 8 < valid) {
                const uint4 old = *reinterpret_cast<const uint4*>(r_row + c * 32 + q * 8);
                const float2 a = unpack_bf16(old.x), b = unpack_bf16(old.y), cc = unpack_bf16(old.z), d = unpack_bf16(old.w);
                f[0] += rope.beta * a.x; f[1] += rope.beta * a.y; f[2] += rope.beta * b.x; f[3] += rope.beta * b.y;
                f[4] += rope.beta * cc.x; f[5] += rope.beta * cc.y; f[6] += rope.beta * d.x; f[7] += rope.beta * d.y;
              }
#pragma unroll
              for (int i = 0; i < 8; ++i)
                if (col + q * 8 + i == row) f[i] += rope.diag;
#pragma unroll
              for (int i = 0; i < 4; ++i) packed[q * 4 + i] = pack_bf16(f[2 * i], f[2 * i + 1]);
              if (q * 8 < valid)
                *reinterpret_cast<uint4*>(c_row + c * 32 + q * 8) =
                    make_uint4(packed[q * 4], packed[q * 4 + 1], packed[q * 4 + 2], packed[q * 4 + 3]);
            }
            if (mirror) {
              // transposed copy: for a fixed column the 32 lanes of the warp write 32 consecutive elements
              unsigned short* t_col = reinterpret_cast<unsigned short*>(c_out) + size_t(col) * ldc + row;
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (i < valid)
                  t_col[size_t(i) * ldc] = (unsigned short)((i & 1) ? (packed[i >> 1] >> 16) : (packed[i >> 1] & 0xffffu));
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_on_cta(tempty_bar(acc), 0);
        continue;
      }
      if constexpr (SWIGLU == 2) {
        const int col0 = tc.n * TILE_N;
        __nv_bfloat16* c_row = reinterpret_cast<__nv_bfloat16*>(C) + size_t(row) * ldc + col0;
        const int half_chunks = rope.hd >> 6;       // 32-column chunks in half a head
        const int head_chunks = rope.hd >> 5;
        const int pos = row % rope.S;
        const float* cos_row = rope.cosT + size_t(pos) * (rope.hd >> 1);
        const float* sin_row = rope.sinT + size_t(pos) * (rope.hd >> 1);
#pragma unroll 1
        for (int c = 0; c < TILE_N / 32; ++c) {
          const int hc = c % head_chunks;           // chunk index inside its head
          if (hc >= half_chunks) continue;          // second halves are written together with their partners
          uint32_t lo[32], hi[32];
          tmem_ld_32x32(t_row + c * 32, lo);
          tmem_ld_32x32(t_row + (c + half_chunks) * 32, hi);
          tmem_ld_wait();
          const int col = col0 + c * 32;
          if (row < M && col < N) {
            if (col < rope.cols) {
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                const float4 cs = *reinterpret_cast<const float4*>(cos_row + hc * 32 + v * 4);
                const float4 sn = *reinterpret_cast<const float4*>(sin_row + hc * 32 + v * 4);
                const float cv[4] = {cs.x, cs.y, cs.z, cs.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float a = __uint_as_float(lo[v * 4 + i]), b = __uint_as_float(hi[v * 4 + i]);
                  lo[v * 4 + i] = __float_as_uint(a * cv[i] - b * sv[i]);
                  hi[v * 4 + i] = __float_as_uint(b * cv[i] + a * sv[i]);
                }
              }
            }
            store_chunk<__nv_bfloat16>(c_row + c * 32, lo, 32, false, nullptr);
            store_chunk<__nv_bfloat16>(c_row + (c + half_chunks) * 32, hi, 32, false, nullptr);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_on_cta(tempty_bar(acc), 0);
        continue;
      }
      if constexpr (SWIGLU == 1) {
        const int h0 = tc.n * HALF_N;  // first hidden unit of this tile
        __nv_bfloat16* h_row = reinterpret_cast<__nv_bfloat16*>(C) + size_t(row) * ldc + h0;
        __nv_bfloat16* gu_row = R ? const_cast<__nv_bfloat16*>(reinterpret_cast<const __nv_bfloat16*>(R)) + size_t(row) * ldr + h0
                                  : nullptr;
#pragma unroll 1
        for (int c = 0; c < HALF_N / 32; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(t_row + c * 32, g);
          tmem_ld_32x32(t_row + HALF_N + c * 32, u);
          tmem_ld_wait();
          const int valid = min(32, N - (h0 + c * 32));
          if (row < M && valid > 0) {
            if (gu_row) {
              store_chunk<__nv_bfloat16>(gu_row + c * 32, g, valid, false, nullptr);
              store_chunk<__nv_bfloat16>(gu_row + N + c * 32, u, valid, false, nullptr);
            }
            swiglu_chunk(g, u);
            store_chunk<__nv_bfloat16>(h_row + c * 32, g, valid, false, nullptr);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_on_cta(tempty_bar(acc), 0);
        continue;
      }
      const int col0 = tc.n * TILE_N;
      OutT* c_row = C + size_t(row) * ldc + col0;
      const OutT* r_row = R ? R + size_t(row) * ldr + col0 : nullptr;
#pragma unroll 1
      for (int c = 0; c < TILE_N / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_row + c * 32, v);
        tmem_ld_wait();
        const int valid = min(32, N - (col0 + c * 32));
        if (row < M && valid > 0)
          store_chunk<OutT>(c_row + c * 32, v, valid, accumulate != 0, r_row ? r_row + c * 32 : nullptr);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) arrive_on_cta(tempty_bar(acc), 0);
    }
  }

  else if constexpr (GATHER) {
    // ------------------------------------------------------------ copy warps 6..9: pull weight chunks into the staging copy
    const int c_tid = threadIdx.x - 192;  // 0..127
    volatile int* claim = reinterpret_cast<volatile int*>(smem_raw + (tmem_slot - smem_u32(smem_raw)) + 8);
    int* work = ga.flags + ga.row_blocks;
    const int f_blocks = SWIGLU == 1 ? N / HALF_N : 0;  // row blocks of the gate half (SwiGLU operand: [gate ; up])
    while (true) {
      if (c_tid == 0) *claim = atomicAdd(work, 1);
      asm volatile("bar.sync 2, 128;" ::: "memory");
      const int c = *claim;
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (c >= ga.total_chunks) break;
      // claimed position -> chunk, in the order in which the tiles consume the row blocks
      int rb, j;
      if constexpr (SWIGLU == 1) {
        const int per_tile = 2 * ga.chunks_per_rb;
        int n = c / per_tile + ga.n_tile_start;
        if (n >= f_blocks) n -= f_blocks;
        const int rem = c % per_tile;
        rb = n + (rem / ga.chunks_per_rb) * f_blocks;
        j = rem % ga.chunks_per_rb;
      } else {
        int q = c + 2 * ga.n_tile_start * ga.chunks_per_rb;
        if (q >= ga.total_chunks) q -= ga.total_chunks;
        rb = q / ga.chunks_per_rb;
        j = q - rb * ga.chunks_per_rb;
      }
      const long long d = (long long)(rb * ga.chunks_per_rb + j) * GATHER_CHUNK_ELEMS;  // element inside the operand
      int sg = 0;
#pragma unroll
      for (int i = 1; i < GATHER_MAX_SEG; ++i)
        if (i < ga.n_seg && d >= ga.seg_dst[i]) sg = i;
      const long long in_seg = d - ga.seg_dst[sg];
      const long long piece = ga.seg_len[sg] / ga.world;
      const int owner = int(in_seg / piece);
      const __nv_bfloat16* src = ga.peer[owner] + ga.seg_src[sg] + (in_seg - owner * piece);
      __nv_bfloat16* dst = ga.stage + d;
      // 2048 vectors of 16 bytes over 128 threads: eight loads in flight per thread before the first store
      constexpr int UNROLL = 8;
#pragma unroll 1
      for (int i0 = c_tid; i0 < GATHER_CHUNK_ELEMS / 8; i0 += 128 * UNROLL) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) v[u] = *reinterpret_cast<const uint4*>(src + size_t(i0 + u * 128) * 8);
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) *reinterpret_cast<uint4*>(dst + size_t(i0 + u * 128) * 8) = v[u];
      }
      __threadfence();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (c_tid == 0) red_release_gpu_add(ga.flags + rb, 1);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's shared memory / tensor memory stay valid until both CTAs are done
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

template <bool A_MN, bool B_MN, typename OutT>
static int launch(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb, int ldc,
                  int ldr, int accumulate, int num_sms, cudaStream_t stream, int* status) {
  CUtensorMap ma, mb;
  int rc = A_MN ? make_map_2d_bf16(&ma, A, K, M, lda, 64, BK) : make_map_2d_bf16(&ma, A, M, K, lda, BK, CTA_M);
  if (rc) return 100 + rc;
  rc = B_MN ? make_map_2d_bf16(&mb, B, K, N, ldb, 64, BK) : make_map_2d_bf16(&mb, B, N, K, ldb, BK, HALF_N);
  if (rc) return 200 + rc;
  auto kern = kf_gemm_bf16_tcgen05_2cta<A_MN, B_MN, OutT>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  const int tiles = ((M + TILE_M - 1) / TILE_M) * ((N + TILE_N - 1) / TILE_N);
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  kern<<<pairs * 2, THREADS, SMEM_BYTES, stream>>>(ma, mb, reinterpret_cast<OutT*>(C),
                                                   reinterpret_cast<const OutT*>(R), M, N, K, ldc, ldr, accumulate,
                                                   status, RopeArgs{nullptr, nullptr, 1, 0, 64}, GatherArgs{});
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// h[M, F] = silu(x Wg^T) * (x Wu^T) with W = [Wg ; Wu] stacked ([2F][K]); gu (optional) receives [M, 2F] pre-activations
int launch_gemm_swiglu_2cta(const void* A, const void* W, void* H, void* GU, int M, int F, int K, int lda, int ldw, int ldh,
                            int ldgu, int num_sms, cudaStream_t stream, int* status) {
  CUtensorMap ma, mb;
  int rc = make_map_2d_bf16(&ma, A, M, K, lda, BK, CTA_M);
  if (rc) return 100 + rc;
  rc = make_map_2d_bf16(&mb, W, 2 * (uint64_t)F, K, ldw, BK, HALF_N);
  if (rc) return 200 + rc;
  auto kern = kf_gemm_bf16_tcgen05_2cta<false, false, __nv_bfloat16, 1>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  const int tiles = ((M + TILE_M - 1) / TILE_M) * ((F + HALF_N - 1) / HALF_N);
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  kern<<<pairs * 2, THREADS, SMEM_BYTES, stream>>>(ma, mb, reinterpret_cast<__nv_bfloat16*>(H),
                                                   reinterpret_cast<const __nv_bfloat16*>(GU), M, F, K, ldh, ldgu, 0, status,
                                                   RopeArgs{nullptr, nullptr, 1, 0, 64}, GatherArgs{});
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// qkv[M, N] = x W^T with the rotary embedding applied to the first `rope_cols` output columns (heads of `hd` columns,
// position = row % S).  N and rope_cols must be multiples of hd; hd in {64, 128, 256}; tables fp32 [S][hd / 2].
int launch_gemm_rope_2cta(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                          const float* cosT, const float* sinT, int S, int rope_cols, int hd, int num_sms,
                          cudaStream_t stream, int* status) {
  if ((hd != 64 && hd != 128 && hd != 256) || N % hd || rope_cols % hd || rope_cols > N || S <= 0) return 6;
  CUtensorMap ma, mb;
  int rc = make_map_2d_bf16(&ma, A, M, K, lda, BK, CTA_M);
  if (rc) return 100 + rc;
  rc = make_map_2d_bf16(&mb, W, N, K, ldw, BK, HALF_N);
  if (rc) return 200 + rc;
  auto kern = kf_gemm_bf16_tcgen05_2cta<false, false, __nv_bfloat16, 2>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  const int tiles = ((M + TILE_M - 1) / TILE_M) * ((N + TILE_N - 1) / TILE_N);
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  kern<<<pairs * 2, THREADS, SMEM_BYTES, stream>>>(ma, mb, reinterpret_cast<__nv_bfloat16*>(C), nullptr, M, N, K, ldc, 0, 0,
                                                   status, RopeArgs{cosT, sinT, S, rope_cols, hd}, GatherArgs{});
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// Symmetric product with a polynomial epilogue: C[n, n] = alpha * X X^T + beta * R + diag * I for X[n][K] (K-major,
// x_mn == 0), or alpha * X^T X + ... for X[K][n] (x_mn != 0).  R (optional) must be symmetric; C must not alias X or R
// (the transposed stores of one tile land in the rows another tile may still be reading).  n % 8 == 0.
int launch_gemm_symm_2cta(int x_mn, const void* X, void* C, const void* R, int n, int K, int ldx, int ldc, int ldr,
                          float alpha, float beta, float diag, int num_sms, cudaStream_t stream, int* status) {
  if ((n & 7) || n <= 0 || K <= 0) return 6;
  CUtensorMap ma, mb;
  int rc = x_mn ? make_map_2d_bf16(&ma, X, K, n, ldx, 64, BK) : make_map_2d_bf16(&ma, X, n, K, ldx, BK, CTA_M);
  if (rc) return 100 + rc;
  rc = x_mn ? make_map_2d_bf16(&mb, X, K, n, ldx, 64, BK) : make_map_2d_bf16(&mb, X, n, K, ldx, BK, HALF_N);
  if (rc) return 200 + rc;
  const int nb = (n + TILE_M - 1) / TILE_M;
  const int tiles = nb * (nb + 1) / 2;
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  const RopeArgs ra{nullptr, nullptr, 1, 0, 64, alpha, beta, diag};
#define KF2_SYMM_LAUNCH(MN_)                                                                                         \
  {                                                                                                                  \
    auto kern = kf_gemm_bf16_tcgen05_2cta<MN_, MN_, __nv_bfloat16, 4>;                                               \
    static bool attr_set = false;                                                                                    \
    if (!attr_set) {                                                                                                 \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);      \
      if (e != cudaSuccess) return 300 + (int)e;                                                                     \
      attr_set = true;                                                                                               \
    }                                                                                                                \
    kern<<<pairs * 2, THREADS, SMEM_BYTES, stream>>>(ma, mb, reinterpret_cast<__nv_bfloat16*>(C),                    \
                                                     reinterpret_cast<const __nv_bfloat16*>(R), n, n, K, ldc, ldr, 0, \
                                                     status, ra, GatherArgs{});                                      \
  }
  if (x_mn) KF2_SYMM_LAUNCH(true) else KF2_SYMM_LAUNCH(false)
#undef KF2_SYMM_LAUNCH
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// Weight-gathering GEMM (see GatherArgs).  epi: 0 = C = A W^T (+ R), 1 = SwiGLU (W = [gate ; up], C = h, R = optional
// pre-activations), 2 = rotary epilogue.  W is described by `n_seg` segments (seg_rows[i] rows of K elements each,
// stacked in this order); segment i's piece of rank r is seg_rows[i] * K / world contiguous elements at
// peers[r] + seg_src[i].  `stage` receives the whole operand; `flags` needs rows / 128 + 1 ints.
int launch_gemm_gather_2cta(int epi, const void* A, void* C, const void* R, int M, int N, int K, int lda, int ldc, int ldr,
                            const long long* peers, int world, int rank, int n_seg, const long long* seg_rows,
                            const long long* seg_src, void* stage, int* flags, const float* cosT, const float* sinT,
                            int S, int rope_cols, int hd, int num_sms, cudaStream_t stream, int* status) {
  if (world < 1 || world > 8 || n_seg < 1 || n_seg > GATHER_MAX_SEG || (K % 128)) return 6;
  GatherArgs ga{};
  long long rows = 0;
  for (int i = 0; i < n_seg; ++i) {
    ga.seg_dst[i] = rows * K;
    ga.seg_len[i] = seg_rows[i] * K;
    ga.seg_src[i] = seg_src[i];
    if ((ga.seg_len[i] % world) || ((ga.seg_len[i] / world) % GATHER_CHUNK_ELEMS) || (seg_src[i] & 7)) return 7;
    rows += seg_rows[i];
  }
  const long long want_rows = epi == 1 ? 2LL * N : N;
  if (rows != want_rows || (rows % HALF_N)) return 8;
  if (epi == 1 && (n_seg != 2 || seg_rows[0] != N)) return 8;
  for (int r = 0; r < 8; ++r) ga.peer[r] = r < world ? reinterpret_cast<const __nv_bfloat16*>(peers[r]) : nullptr;
  ga.stage = reinterpret_cast<__nv_bfloat16*>(stage);
  ga.flags = flags;
  ga.n_seg = n_seg;
  ga.world = world;
  ga.chunks_per_rb = K / 128;
  ga.row_blocks = int(rows / HALF_N);
  ga.total_chunks = ga.row_blocks * ga.chunks_per_rb;
  const long long own_row = seg_rows[0] / world * rank;
  ga.n_tile_start = int(own_row / (epi == 1 ? HALF_N : TILE_N));
  cudaError_t me = cudaMemsetAsync(flags, 0, sizeof(int) * (ga.row_blocks + 1), stream);
  if (me != cudaSuccess) return 350 + (int)me;
  CUtensorMap ma, mb;
  int rc = make_map_2d_bf16(&ma, A, M, K, lda, BK, CTA_M);
  if (rc) return 100 + rc;
  rc = make_map_2d_bf16(&mb, stage, rows, K, K, BK, HALF_N);
  if (rc) return 200 + rc;
  const int n_tiles_n = epi == 1 ? (N + HALF_N - 1) / HALF_N : (N + TILE_N - 1) / TILE_N;
  const int tiles = ((M + TILE_M - 1) / TILE_M) * n_tiles_n;
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  RopeArgs ra{cosT, sinT, S > 0 ? S : 1, rope_cols, hd > 0 ? hd : 64};
  if (epi == 2 && ((hd != 64 && hd != 128 && hd != 256) || N % hd || rope_cols % hd || rope_cols > N || S <= 0)) return 6;
#define KF2_GATHER_LAUNCH(EPI_)                                                                                      \
  {                                                                                                                  \
    auto kern = kf_gemm_bf16_tcgen05_2cta<false, false, __nv_bfloat16, EPI_, true>;                                  \
    static bool attr_set = false;                                                                                    \
    if (!attr_set) {                                                                                                 \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);      \
      if (e != cudaSuccess) return 300 + (int)e;                                                                     \
      attr_set = true;                                                                                               \
    }                                                                                                                \
    kern<<<pairs * 2, THREADS_GATHER, SMEM_BYTES, stream>>>(ma, mb, reinterpret_cast<__nv_bfloat16*>(C),             \
                                                            reinterpret_cast<const __nv_bfloat16*>(R), M, N, K, ldc, ldr, \
                                                            0, status, ra, ga);                                      \
  }
  if (epi == 0) KF2_GATHER_LAUNCH(0) else if (epi == 1) KF2_GATHER_LAUNCH(1) else if (epi == 2) KF2_GATHER_LAUNCH(2) else return 6;
#undef KF2_GATHER_LAUNCH
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// d[gate | up][M, 2F] = SwiGLU'(gu) * (dy[M, K] x W[K, F]) with W stored [K][F] (F contiguous: the down projection's
// weight read for its input gradient); gu and dgu may be the same buffer.  F % 8 == 0, K % 64 == 0.
int launch_gemm_swiglu_bwd_2cta(const void* DY, const void* W, const void* GU, void* DGU, int M, int F, int K, int lda,
                                int ldw, int ldgu, int num_sms, cudaStream_t stream, int* status) {
  CUtensorMap ma, mb;
  int rc = make_map_2d_bf16(&ma, DY, M, K, lda, BK, CTA_M);
  if (rc) return 100 + rc;
  rc = make_map_2d_bf16(&mb, W, K, F, ldw, 64, BK);
  if (rc) return 200 + rc;
  auto kern = kf_gemm_bf16_tcgen05_2cta<false, true, __nv_bfloat16, 3>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  const int tiles = ((M + TILE_M - 1) / TILE_M) * ((F + TILE_N - 1) / TILE_N);
  int pairs = num_sms / 2;
  if (tiles < pairs) pairs = tiles;
  kern<<<pairs * 2, THREADS, SMEM_BYTES, stream>>>(ma, mb, reinterpret_cast<__nv_bfloat16*>(DGU),
                                                   reinterpret_cast<const __nv_bfloat16*>(GU), M, F, K, ldgu, ldgu, 0, status,
                                                   RopeArgs{nullptr, nullptr, 1, 0, 64}, GatherArgs{});
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

int launch_gemm_2cta(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int lda, int ldb,
                     int ldc, int ldr, int a_mn, int b_mn, int out_f32, int accumulate, int num_sms,
                     cudaStream_t stream, int* status) {
#define KF2_DISPATCH(AM, BM_)                                                                                         \
  (out_f32 ? launch<AM, BM_, float>(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, accumulate, num_sms, stream, status)     \
           : launch<AM, BM_, __nv_bfloat16>(A, B, C, R, M, N, K, lda, ldb, ldc, ldr, accumulate, num_sms, stream, status))
  if (!a_mn && !b_mn) return KF2_DISPATCH(false, false);
  if (!a_mn && b_mn) return KF2_DISPATCH(false, true);
  if (a_mn && !b_mn) return KF2_DISPATCH(true, false);
  return KF2_DISPATCH(true, true);
#undef KF2_DISPATCH
}

}  // namespace kf2
