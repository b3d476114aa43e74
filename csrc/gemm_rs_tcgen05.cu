// Row-parallel Linear fused with its reduce-scatter over NVLink peer memory (tensor parallelism with
// sequence-sharded activations):
//
//   partial[T, D] = X_local[T, K/tp] * W_local[D, K/tp]^T          (tcgen05 GEMM, this rank's K slice)
//   out[T/tp, D]  = sum over ranks of partial[rows owned by me] (+ residual)
//
// ONE kernel does both.  The GEMM epilogue stores every finished 128 x 256 tile straight into the staging
// buffer of the rank that owns those rows (plain peer stores through NVSwitch; no library collective) and
// bumps a per-tile counter on that rank with a system-scope release.  Tiles are visited owner by owner,
// starting with the next rank, so pushes are spread over the whole GEMM and overlap the math; the CTA then
// turns to the output tiles of its own rows, waits (bounded) until all tp partials of a tile have landed
// and writes their sum.  Counters grow monotonically (expected value = call number x tp), so nothing has to
// be cleared between calls; staging and counters are double buffered by call parity, which is enough because no rank can
// complete call n before every rank has pushed its part of call n.
//
// Row ownership follows the (B, S, D) -> sequence-sharded layout: row t = b * S + s belongs to rank
// s / (S / tp) and lands at row b * (S / tp) + s % (S / tp) of that rank's output.  S / tp must be a multiple
// of 128 so that a tile has one owner.
//
// Replaces DTensor's Rowwise-parallel Linear + NCCL reduce-scatter of the reference
// (kempnerforge/distributed/tensor_parallel.py:61,72,81).
#include "common.cuh"
#include "gemm_epilogue.cuh"

namespace kf {
namespace rs {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2, B_STAGE_BYTES = BN * BK * 2, STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int THREADS = 192, TMEM_COLS = 512;
constexpr int XPOSE_BYTES = 4 * 32 * 144;  // per epilogue warp: 32 rows x 128 B (+16 B pad against bank conflicts)
constexpr size_t SMEM = size_t(STAGES) * STAGE_BYTES + 1024 + 256 + XPOSE_BYTES;
constexpr int MAX_PEERS = 8;

struct Peers {
  void* stage[MAX_PEERS];  // each rank's staging buffer: [2 parities][tp sources][T / tp][D] bf16
  int* flags[MAX_PEERS];   // each rank's per-output-tile counters
};

__device__ __forceinline__ void red_release_sys_add(int* addr, int v) {
  asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

// Tile t of this rank's schedule -> (global row block, column block).  Row blocks are grouped by owner,
// owners visited in the order rank+1, rank+2, ..., rank; within an owner: batch, then local row block.
struct TileRef {
  int owner, local_mb, nb, row0;  // row0: first row of the tile in the full [T, *] operand
};
__device__ __forceinline__ TileRef tile_ref(int t, int rank, int tp, int mb_per_owner, int n_blocks, int mb_per_seq_shard,
                                            int S) {
  const int per_owner = mb_per_owner * n_blocks;
  const int oi = t / per_owner;
  const int r = t - oi * per_owner;
  TileRef x;
  x.owner = (rank + 1 + oi) % tp;
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
kf_gemm_rs_tcgen05(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, Peers peers,
                   __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ residual, int T, int D, int K,
                   int S, int tp, int rank, int call_no, int* status) {
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
  const int Tl = T / tp;                       // rows per owner
  const int mb_per_owner = Tl / BM;
  const int mb_per_seq_shard = (S / tp) / BM;  // row blocks of one batch element's shard
  const int n_blocks = (D + BN - 1) / BN;
  const int num_tiles = tp * mb_per_owner * n_blocks;
  const int k_blocks = (K + BK - 1) / BK;
  const int parity = call_no & 1;
  const size_t slice_elems = size_t(Tl) * D;   // one source's partial of one owner

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
        const TileRef tr = tile_ref(t, rank, tp, mb_per_owner, n_blocks, mb_per_seq_shard, S);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(empty_bar(s), ((it / STAGES) & 1) ^ 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
          const uint32_t a_dst = smem_base + s * STAGE_BYTES;
          mbar_expect_tx(full_bar(s), STAGE_BYTES);
          tma_load_2d(a_dst, &map_a, full_bar(s), kb * BK, tr.row0);
          if (!B_MN) {
            tma_load_2d(a_dst + A_STAGE_BYTES, &map_b, full_bar(s), kb * BK, tr.nb * BN);
          } else {  // B stored [K][D] (output dim contiguous): 64-column boxes
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
  } else {
    // ------------------------------------------------------------ epilogue warps: push, then reduce
    const int quarter = warp & 3;
    const int e_tid = threadIdx.x - 64;  // 0..127
    int tile_iter = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tile_iter) {
      const TileRef tr = tile_ref(t, rank, tp, mb_per_owner, n_blocks, mb_per_seq_shard, S);
      const int acc = tile_iter & 1;
      if (ok && !mbar_wait(tfull_bar(acc), (tile_iter >> 1) & 1, status, KF_ERR_WAIT_TMEM_FULL)) ok = false;
      tc_fence_after();
      // destination: the owner's staging slice for source `rank`
      __nv_bfloat16* slice = reinterpret_cast<__nv_bfloat16*>(peers.stage[tr.owner]) +
                             (size_t(parity) * tp + rank) * slice_elems;
      const int col0 = tr.nb * BN;
      const uint32_t t_row = tmem_base + (uint32_t(quarter * 32) << 16) + acc * BN;
      // Peer stores want long contiguous runs (a 16-byte store per row would cross NVLink as a 16-byte
      // packet), so 64 columns at a time go through shared memory: thread = row on the way in, eight lanes per
      // row (128 contiguous bytes) on the way out.
      uint8_t* xp = smem_raw + (bar_base - smem_u32(smem_raw)) + 256 + quarter * (32 * 144);
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(t_row + c * 64, v0);
        tmem_ld_32x32(t_row + c * 64 + 32, v1);
        tmem_ld_wait();
        uint4* mine = reinterpret_cast<uint4*>(xp + lane * 144);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          mine[i] = make_uint4(pack_bf16(__uint_as_float(v0[8 * i]), __uint_as_float(v0[8 * i + 1])),
                               pack_bf16(__uint_as_float(v0[8 * i + 2]), __uint_as_float(v0[8 * i + 3])),
                               pack_bf16(__uint_as_float(v0[8 * i + 4]), __uint_as_float(v0[8 * i + 5])),
                               pack_bf16(__uint_as_float(v0[8 * i + 6]), __uint_as_float(v0[8 * i + 7])));
          mine[4 + i] = make_uint4(pack_bf16(__uint_as_float(v1[8 * i]), __uint_as_float(v1[8 * i + 1])),
                                   pack_bf16(__uint_as_float(v1[8 * i + 2]), __uint_as_float(v1[8 * i + 3])),
                                   pack_bf16(__uint_as_float(v1[8 * i + 4]), __uint_as_float(v1[8 * i + 5])),
                                   pack_bf16(__uint_as_float(v1[8 * i + 6]), __uint_as_float(v1[8 * i + 7])));
        }
        __syncwarp();
        const int cbase = col0 + c * 64;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = i * 4 + (lane >> 3), piece = lane & 7;  // row of this warp's 32, 16-byte piece of its 128 B
          const uint4 w = *reinterpret_cast<const uint4*>(xp + rr * 144 + piece * 16);
          const int col = cbase + piece * 8;
          if (ok && col < D)
            *reinterpret_cast<uint4*>(slice + size_t(tr.local_mb * BM + quarter * 32 + rr) * D + col) = w;
        }
        __syncwarp();
      }
      tc_fence_before();
      __threadfence_system();              // this thread's stores are visible system-wide ...
      asm volatile("bar.sync 1, 128;" ::: "memory");  // ... and so are those of the other 127 rows
      if (e_tid == 0) {
        mbar_arrive(tempty_bar(acc)); mbar_arrive(tempty_bar(acc)); mbar_arrive(tempty_bar(acc)); mbar_arrive(tempty_bar(acc));
        if (ok) red_release_sys_add(peers.flags[tr.owner] + parity * (mb_per_owner * n_blocks) + tr.local_mb * n_blocks + tr.nb, 1);
      }
    }
    // ---- reduce phase: output tiles of this rank's rows, summed over the tp staged partials
    const int my_tiles = mb_per_owner * n_blocks;
    const int expected = (call_no / 2 + 1) * tp;  // counters are kept per parity: a rank one call ahead never mixes in
    const __nv_bfloat16* mine = reinterpret_cast<const __nv_bfloat16*>(peers.stage[rank]) + size_t(parity) * tp * slice_elems;
    for (int t = blockIdx.x; t < my_tiles; t += gridDim.x) {
      const int mb = t / n_blocks, nb = t - mb * n_blocks;
      if (ok && !flag_wait_ge(peers.flags[rank] + parity * my_tiles + t, expected, status)) ok = false;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (!ok) continue;
      // 128 rows x 256 columns: thread handles 8 columns of 32 rows strided by 4
      const int cvec = (e_tid & 31) * 8;      // column offset inside the tile
      const int col = nb * BN + cvec;
      if (col >= D) continue;
      for (int r = e_tid >> 5; r < BM; r += 4) {
        const size_t off = size_t(mb * BM + r) * D + col;
        float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int src = 0; src < tp; ++src) {
          const uint4 w = *reinterpret_cast<const uint4*>(mine + size_t(src) * slice_elems + off);
          const float2 a = unpack_bf16(w.x), b2 = unpack_bf16(w.y), c2 = unpack_bf16(w.z), d2 = unpack_bf16(w.w);
          f[0] += a.x; f[1] += a.y; f[2] += b2.x; f[3] += b2.y; f[4] += c2.x; f[5] += c2.y; f[6] += d2.x; f[7] += d2.y;
        }
        if (residual) {
          const uint4 w = *reinterpret_cast<const uint4*>(residual + off);
          const float2 a = unpack_bf16(w.x), b2 = unpack_bf16(w.y), c2 = unpack_bf16(w.z), d2 = unpack_bf16(w.w);
          f[0] += a.x; f[1] += a.y; f[2] += b2.x; f[3] += b2.y; f[4] += c2.x; f[5] += c2.y; f[6] += d2.x; f[7] += d2.y;
        }
        uint4 o;
        o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]); o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
        *reinterpret_cast<uint4*>(out + off) = o;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

}  // namespace rs
}  // namespace kf

extern "C" void* kf_status_device_ptr();

extern "C" {

// out[T/tp, D] = reduce-scatter over `tp` ranks of X[T, K] * W[D, K]^T (+ residual[T/tp, D]).
//   x, w: this rank's operands (K = its slice of the reduction dim), bf16, pitches lda / ldb elements.
//   stage_ptrs / flag_ptrs: tp device addresses each (every rank's staging buffer and counter array, in
//   rank order); staging needs 2 * T * D bf16 per rank, counters 2 * (T / tp / 128) * ceil(D / 256) ints (zero before the first call).
//   S: sequence length of the (B, S) token grid behind the T rows; S / tp must be a multiple of 128 and D a
//   multiple of 8.  call_no: number of earlier calls that used these buffers (same on every rank).
// The kernel needs all CTAs of all ranks to make progress independently; its only cross-rank wait (for the
// tile counters) is bounded and reports through the status word.
int kf_gemm_rs_bf16(const void* x, const void* w, const long long* stage_ptrs, const long long* flag_ptrs, void* out,
                    const void* residual, int T, int D, int K, int S, long long lda, long long ldb, int tp, int rank,
                    int call_no, int b_mn, int num_sms, void* stream) {
  using namespace kf;
  using namespace kf::rs;
  if (tp < 1 || tp > MAX_PEERS || T % tp || S % tp || ((S / tp) % BM) || (T % S) || (D & 7) || (lda & 7) || (ldb & 7)) return 5;
  CUtensorMap ma, mb;
  int rc = make_map_2d_bf16(&ma, x, T, K, lda, BK, BM);
  if (rc) return 100 + rc;
  // b_mn: w is stored [K][D] (D contiguous; K must be a multiple of 64), else [D][K]
  if (b_mn && (K % BK)) return 5;
  rc = b_mn ? make_map_2d_bf16(&mb, w, K, D, ldb, 64, BK) : make_map_2d_bf16(&mb, w, D, K, ldb, BK, BN);
  if (rc) return 200 + rc;
  Peers peers;
  for (int i = 0; i < MAX_PEERS; ++i) {
    peers.stage[i] = i < tp ? reinterpret_cast<void*>(stage_ptrs[i]) : nullptr;
    peers.flags[i] = i < tp ? reinterpret_cast<int*>(flag_ptrs[i]) : nullptr;
  }
  const int tiles = (T / BM) * ((D + BN - 1) / BN);
  const int grid = tiles < num_sms ? tiles : num_sms;
  int* status = reinterpret_cast<int*>(kf_status_device_ptr());
  auto out_p = reinterpret_cast<__nv_bfloat16*>(out);
  auto res_p = reinterpret_cast<const __nv_bfloat16*>(residual);
  if (b_mn) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(kf_gemm_rs_tcgen05<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
      if (e != cudaSuccess) return 300 + (int)e;
      attr_set = true;
    }
    kf_gemm_rs_tcgen05<true><<<grid, THREADS, SMEM, (cudaStream_t)stream>>>(ma, mb, peers, out_p, res_p, T, D, K, S, tp, rank,
                                                                          call_no, status);
  } else {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(kf_gemm_rs_tcgen05<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM);
      if (e != cudaSuccess) return 300 + (int)e;
      attr_set = true;
    }
    kf_gemm_rs_tcgen05<false><<<grid, THREADS, SMEM, (cudaStream_t)stream>>>(ma, mb, peers, out_p, res_p, T, D, K, S, tp, rank,
                                                                           call_no, status);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // extern "C"
