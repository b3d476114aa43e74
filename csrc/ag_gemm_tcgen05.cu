// Column-parallel Linear fused with the all-gather of its sequence-sharded input over NVLink peer memory:
//
//   Y[T, N_local] = gather_seq(X_shard)[T, K] * W_local[N_local, K]^T
//
// ONE kernel does both.  Every CTA has two extra "copy" warps next to the usual TMA / MMA / epilogue warps.
// At kernel start they push this rank's shard into the gather buffers of all peers (plain peer stores through
// NVSwitch, 16 bytes per thread, one unit = 128 rows x one quarter of K) and bump a per-(source, row block)
// counter on the destination with a system-scope release.  The GEMM walks the row blocks in arrival order
// (own rows first, straight from the local shard through a second tensor map, then the rows of rank-1,
// rank-2, ...); its TMA producer waits (bounded) on the local counter of a row block before loading it from
// the local gather buffer, so the transfer of later blocks overlaps the math of earlier ones.  The remote
// data crosses NVLink once and is then read by TMA from this GPU's own memory.  Counters are monotonic and,
// like the gather buffer, double buffered by call parity.
//
// Row layout: rank r owns rows b * S + r * (S / tp) + s' of the (B, S) token grid; S / tp is a multiple of 128.
//
// Replaces DTensor's Shard(1) -> Replicate all-gather in front of the Colwise-parallel Linears of the
// reference (kempnerforge/distributed/tensor_parallel.py:60,69-71,79-80).
#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace kf {
namespace ag {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2, B_STAGE_BYTES = BN * BK * 2, STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int THREADS = 256;  // warps: 0 TMA, 1 MMA, 2-5 epilogue, 6-7 copy
constexpr int COPY_THREADS = 64;
constexpr int TMEM_COLS = 512;
constexpr int K_SLICES = 4;   // a row block is pushed in four column slices (finer load balance over CTAs)
constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256;
constexpr int MAX_PEERS = 8;

struct Peers {
  void* gather[MAX_PEERS];  // each rank's gather buffer: [2 parities][T][K] bf16
  int* flags[MAX_PEERS];    // each rank's counters: [2 parities][tp sources][T / tp / 128]
};

__device__ __forceinline__ void red_release_sys_add(int* addr, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

// Schedule position t -> row block.  Owners in the order rank, rank-1, ..., rank+1; all column blocks of a
// row block are adjacent so that a block that has arrived is consumed completely.
struct TileRef {
  int owner, local_mb, nb, row0;
};
__device__ __forceinline__ TileRef tile_ref(int t, int rank, int tp, int mb_per_owner, int n_blocks, int mb_per_seq_shard,
                                            int S) {
  const int per_owner = mb_per_owner * n_blocks;
  const int oi = t / per_owner;
  const int r = t - oi * per_owner;
  TileRef x;
  x.owner = (rank - oi + tp) % tp;
  // inside an owner's rows: eight row blocks share each sweep over the column blocks (weight tiles stay in L2)
  constexpr int GROUP_M = 8;
  const int per_group = GROUP_M * n_blocks;
  const int g = r / per_group;
  const int first = g * GROUP_M;
  const int rows = min(GROUP_M, mb_per_owner - first);
  const int rr = r - g * per_group;
  x.local_mb = first + rr % rows;
  x.nb = rr / rows;
  const int b = x.local_mb / mb_per_seq_shard;
  const int sb = x.local_mb - b * mb_per_seq_shard;
  x.row0 = b * S + x.owner * (mb_per_seq_shard * BM) + sb * BM;
  return x;
}

template <bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
kf_ag_gemm_tcgen05(const __grid_constant__ CUtensorMap map_local, const __grid_constant__ CUtensorMap map_gather,
                   const __grid_constant__ CUtensorMap map_b, Peers peers, const __nv_bfloat16* __restrict__ x_shard,
                   long long ldx, __nv_bfloat16* __restrict__ Y, long long ldy, int T, int N, int K, int S, int tp,
                   int rank, int call_no, int* status) {
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

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int Tl = T / tp;
  const int mb_per_owner = Tl / BM;
  const int mb_per_seq_shard = (S / tp) / BM;
  const int n_blocks = (N + BN - 1) / BN;
  const int num_tiles = tp * mb_per_owner * n_blocks;
  const int k_blocks = (K + BK - 1) / BK;
  const int parity = call_no & 1;
  const int flags_per_parity = tp * mb_per_owner;
  const int expected = (call_no / 2 + 1) * K_SLICES;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
    mbar_init(drain_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&map_local);
    tma_prefetch_desc(&map_gather);
    tma_prefetch_desc(&map_b);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (waits for remote row blocks)
    if (lane == 0) {
      int it = 0;
      bool ok = true;
      const int* my_flags = peers.flags[rank] + parity * flags_per_parity;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const TileRef tr = tile_ref(t, rank, tp, mb_per_owner, n_blocks, mb_per_seq_shard, S);
        const bool local = tr.owner == rank;
        if (!local) {
          if (!flag_wait_ge(my_flags + tr.owner * mb_per_owner + tr.local_mb, expected, status)) { ok = false; break; }
          // the rows were written by other GPUs' generic-proxy stores; order them before this thread's
          // asynchronous-proxy (TMA) reads
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        const CUtensorMap* ma = local ? &map_local : &map_gather;
        const int arow = local ? tr.local_mb * BM : parity * T + tr.row0;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * STAGE_BYTES;
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          tma_load_2d(a_dst, ma, full_bar(s), kb * BK, arow);
          if (!B_MN) {
            tma_load_2d(a_dst + A_STAGE_BYTES, &map_b, full_bar(s), kb * BK, tr.nb * BN);
          } else {  // B stored [K][N] (output dim contiguous): 64-column boxes
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(a_dst + A_STAGE_BYTES + c * (64 * BK * 2), &map_b, full_bar(s), tr.nb * BN + 64 * c, kb * BK);
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
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_f16(d_tmem, umma_desc_sw128(a_src + k * (UMMA_K * 2), 16, 1024),
                       B_MN ? umma_desc_sw128(b_src + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                            : umma_desc_sw128(b_src + k * (UMMA_K * 2), 16, 1024),
                       idesc, (kb | k) != 0);
          tc_commit(empty_bar(s));
        }
        if (ok) tc_commit(tfull_bar(acc));
      }
      tc_commit(drain_bar);
      mbar_wait(drain_bar, 0, status, KF_ERR_WAIT_DRAIN);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    int tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++tile_iter) {
      const TileRef tr = tile_ref(t, rank, tp, mb_per_owner, n_blocks, mb_per_seq_shard, S);
      const int acc = tile_iter & 1;
      if (!mbar_wait(tfull_bar(acc), (tile_iter >> 1) & 1, status, KF_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      const int row = tr.row0 + quarter * 32 + lane;
      const int col0 = tr.nb * BN;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      __nv_bfloat16* c_row = Y + size_t(row) * ldy + col0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_row + c * 32, v);
        tmem_ld_wait();
        const int valid = min(32, N - (col0 + c * 32));
        if (row < T && valid > 0) store_chunk<__nv_bfloat16>(c_row + c * 32, v, valid, false, nullptr);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
    }
  } else {
    // ------------------------------------------------------------ copy warps: push this rank's shard to the peers
    const int c_tid = threadIdx.x - 192;  // 0..63
    const int kslice = K / K_SLICES;      // elements (multiple of 8)
    const int units = (tp - 1) * mb_per_owner * K_SLICES;
    for (int u = blockIdx.x; u < units; u += gridDim.x) {
      // destinations in the order rank+1, rank+2, ...: the peer that consumes our rows first gets them first
      const int di = u / (mb_per_owner * K_SLICES);
      const int r = u - di * (mb_per_owner * K_SLICES);
      const int mb = r / K_SLICES, ks = r - mb * K_SLICES;
      const int dest = (rank + 1 + di) % tp;
      const int b = mb / mb_per_seq_shard, sb = mb - b * mb_per_seq_shard;
      const size_t drow0 = size_t(parity) * T + size_t(b) * S + size_t(rank) * (mb_per_seq_shard * BM) + size_t(sb) * BM;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(peers.gather[dest]) + drow0 * K + size_t(ks) * kslice;
      const __nv_bfloat16* src = x_shard + size_t(mb) * BM * ldx + size_t(ks) * kslice;
      const int vec_per_row = kslice / 8;
      const int total = BM * vec_per_row;
      // eight independent 16-byte loads in flight per thread before the first store (the loop is bound by
      // memory latency, not by issue)
      constexpr int UNROLL = 8;
      for (int i0 = c_tid; i0 < total; i0 += COPY_THREADS * UNROLL) {
        uint4 v[UNROLL];
#pragma unroll
        for (int u2 = 0; u2 < UNROLL; ++u2) {
          const int i = i0 + u2 * COPY_THREADS;
          if (i < total) {
            const int rr = i / vec_per_row, cc = (i - rr * vec_per_row) * 8;
            v[u2] = *reinterpret_cast<const uint4*>(src + size_t(rr) * ldx + cc);
          }
        }
#pragma unroll
        for (int u2 = 0; u2 < UNROLL; ++u2) {
          const int i = i0 + u2 * COPY_THREADS;
          if (i < total) {
            const int rr = i / vec_per_row, cc = (i - rr * vec_per_row) * 8;
            *reinterpret_cast<uint4*>(dst + size_t(rr) * K + cc) = v[u2];
          }
        }
      }
      __threadfence_system();
      asm volatile("bar.sync 2, 64;" ::: "memory");
      if (c_tid == 0) red_release_sys_add(peers.flags[dest] + parity * flags_per_parity + rank * mb_per_owner + mb, 1);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

}  // namespace ag
}  // namespace kf

extern "C" void* kf_status_device_ptr();

extern "C" {

// y[T, N] = all-gather over `tp` ranks (along the sequence) of x_shard[T/tp, K], times w[N, K]^T.
//   gather_ptrs / flag_ptrs: tp device addresses each, in rank order: every rank's gather buffer
//   (2 * T * K bf16) and counter array (2 * tp * (T / tp / 128) ints, zero before the first call).
//   K must be a multiple of 32, S / tp a multiple of 128, pitches multiples of 8 elements.
// Cross-rank waits are bounded and report through the status word.
int kf_ag_gemm_bf16(const void* x_shard, const void* w, const long long* gather_ptrs, const long long* flag_ptrs, void* y,
                    int T, int N, int K, int S, long long ldx, long long ldw, long long ldy, int tp, int rank,
                    int call_no, int b_mn, int num_sms, void* stream) {
  using namespace kf;
  using namespace kf::ag;
  if (tp < 1 || tp > MAX_PEERS || T % tp || S % tp || ((S / tp) % BM) || (T % S) || (K % (8 * K_SLICES)) || (ldx & 7) ||
      (ldw & 7) || (ldy & 7))
    return 5;
  CUtensorMap ml, mg, mb;
  int rc = make_map_2d_bf16(&ml, x_shard, T / tp, K, ldx, BK, BM);
  if (rc) return 100 + rc;
  rc = make_map_2d_bf16(&mg, reinterpret_cast<const void*>(gather_ptrs[rank]), uint64_t(2) * T, K, K, BK, BM);
  if (rc) return 150 + rc;
  // b_mn: w is stored [K][N] (N contiguous; K must be a multiple of 64), else [N][K]
  if (b_mn && (K % BK)) return 5;
  rc = b_mn ? make_map_2d_bf16(&mb, w, K, N, ldw, 64, BK) : make_map_2d_bf16(&mb, w, N, K, ldw, BK, BN);
  if (rc) return 200 + rc;
  Peers peers;
  for (int i = 0; i < MAX_PEERS; ++i) {
    peers.gather[i] = i < tp ? reinterpret_cast<void*>(gather_ptrs[i]) : nullptr;
    peers.flags[i] = i < tp ? reinterpret_cast<int*>(flag_ptrs[i]) : nullptr;
  }
  const int tiles = (T / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  int* status = reinterpret_cast<int*>(kf_status_device_ptr());
  auto xs = reinterpret_cast<const __nv_bfloat16*>(x_shard);
  auto yp = reinterpret_cast<__nv_bfloat16*>(y);
  if (b_mn) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(kf_ag_gemm_tcgen05<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
      if (e != cudaSuccess) return 300 + (int)e;
      attr_set = true;
    }
    kf_ag_gemm_tcgen05<true><<<grid, THREADS, SMEM, (cudaStream_t)stream>>>(ml, mg, mb, peers, xs, ldx, yp, ldy, T, N, K, S, tp,
                                                                          rank, call_no, status);
  } else {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(kf_ag_gemm_tcgen05<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
      if (e != cudaSuccess) return 300 + (int)e;
      attr_set = true;
    }
    kf_ag_gemm_tcgen05<false><<<grid, THREADS, SMEM, (cudaStream_t)stream>>>(ml, mg, mb, peers, xs, ldx, yp, ldy, T, N, K, S, tp,
                                                                           rank, call_no, status);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // extern "C"
