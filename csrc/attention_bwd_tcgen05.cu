// Flash attention backward on the 5th-generation tensor cores (head dim 128).
//
// One CTA owns a tile of 128 keys of one (batch, KV head) and walks over every query head of the group and
// every 64-row query tile that can see those keys.  All five GEMMs of the backward pass run on tcgen05 with
// the *transposed* score tile, so that each softmax thread owns one key row and the products that feed the
// dK / dV accumulators can be taken straight from tensor memory / shared memory without a transpose:
//
//   S^T  = K  Q_i^T                      (128 keys x 64 queries, smem x smem -> TMEM)
//   dP^T = V  dO_i^T                     (128 x 64)
//   P^T  = exp2(S^T * c - lse_i),  dS^T = P^T * (dP^T - D_i) * scale        (softmax warps)
//   dV  += P^T  dO_i                     (A from TMEM, 128 x 128 accumulator, lives in TMEM for the whole CTA)
//   dK  += dS^T Q_i                      (A from smem, 128 x 128 accumulator)
//   dQ_i^T = K^T dS                      (128 head-dim rows x 64 queries; added to an fp32 dQ by a bulk reduction)
//
//   warp 0     : TMA producer (K, V once; Q_i / dO_i ring of three stages)
//   warp 1     : MMA issuer
//   warps 2-5  : softmax of queries 0..31 of the tile (one thread per key row) and the final dK / dV store
//   warps 10-13: softmax of queries 32..63 (the same key rows): two warps per scheduler hide each other's
//                exp2 / conversion latencies, and 32 scores + 32 dP per thread leave registers for instruction-level
//                parallelism (with 64 + 64 per thread the P / dS arithmetic was latency bound: 2400 of the 4100
//                cycles of an iteration)
//   warps 6-9  : dQ reduction (TMEM -> shared-memory tile -> one cp.reduce.async.bulk.tensor add per tile;
//                or, as a fallback mode, red.global.add.f32 per element)
//
// D_i = rowsum(dO_i * O_i) comes from a small pre-pass; a post-pass converts the fp32 dQ to bf16.
// Replaces the backward of F.scaled_dot_product_attention (kempnerforge/model/attention.py:227-231) for the
// causal / document-masked training path, without expanding grouped KV heads.
#include "common.cuh"

namespace kf {
namespace attnb {

constexpr int HD = 128;
constexpr int BLK_K = 128;  // keys per CTA
constexpr int BLK_Q = 64;   // queries per iteration
constexpr int THREADS = 448;
constexpr int TMEM_COLS = 512;
constexpr int ST_COL = 0;     // S^T buffers 0 / 1 (fp32, 64 cols each); P^T (bf16 pairs, 32 cols) aliases each start
constexpr int DPT_COL = 128;  // dP^T (fp32, 64 cols)
constexpr int DQT_COL = 192;  // dQ^T (fp32, 64 cols)
constexpr int DV_COL = 256;   // dV accumulator (fp32, 128 cols)
constexpr int DK_COL = 384;   // dK accumulator (fp32, 128 cols)
constexpr int KV_TILE_BYTES = BLK_K * HD * 2;   // 32 KB: two blocks of [128 rows x 128 B]
constexpr int KV_BLOCK_BYTES = BLK_K * 128;     // 16 KB
constexpr int Q_TILE_BYTES = BLK_Q * HD * 2;    // 16 KB: two blocks of [64 rows x 128 B]
constexpr int Q_BLOCK_BYTES = BLK_Q * 128;      // 8 KB
constexpr int DS_BYTES = BLK_K * BLK_Q * 2;     // 16 KB: [128 key rows x 128 B]
constexpr int STAGES = 3;  // Q_i / dO_i ring: a tile is loaded one whole iteration before its scores are issued
constexpr int AUX_BYTES = 2048;  // barriers, row statistics, doc ids
constexpr size_t SMEM = 2 * size_t(KV_TILE_BYTES) + STAGES * 2 * size_t(Q_TILE_BYTES) + 2 * DS_BYTES + 1024 /*align*/ +
                        AUX_BYTES;
constexpr int DQ_STAGE_BYTES = BLK_Q * HD * 4;  // 32 KB: one dQ tile [64 queries][128] fp32 for the bulk reduction
constexpr size_t SMEM_DQ_TMA = SMEM + DQ_STAGE_BYTES;

__device__ __forceinline__ void tmem_ld_32x32_at(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void group_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void red_add_f32(float* addr, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

// fp32 tile in shared memory (row-major, the tensor map's box) added to global memory by the TMA unit
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, uint32_t smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map),
               "r"(x), "r"(y), "r"(smem_src)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

template <bool CAUSAL, bool HAS_DOC>
__global__ void __launch_bounds__(THREADS, 1)
kf_attn_bwd_tcgen05(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                    const __grid_constant__ CUtensorMap map_dq, int dq_tma, const float* __restrict__ LSE, const float* __restrict__ Dsum, const int* __restrict__ doc_ids,
                    float* __restrict__ dQacc, __nv_bfloat16* __restrict__ dK, __nv_bfloat16* __restrict__ dV, int Sq,
                    int Sk, int H, int group, long long lddk, long long lddv, float scale, int* status,
                    const float* __restrict__ cosT, const float* __restrict__ sinT) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t k_smem = smem_base;
  const uint32_t v_smem = k_smem + KV_TILE_BYTES;
  const uint32_t q_smem = v_smem + KV_TILE_BYTES;                 // STAGES tiles
  const uint32_t do_smem = q_smem + STAGES * Q_TILE_BYTES;        // STAGES tiles
  const uint32_t ds_smem = do_smem + STAGES * Q_TILE_BYTES;
  const uint32_t bar_base = ds_smem + 2 * DS_BYTES;  // dS^T is double buffered
  uint8_t* ds_gen = smem_gen + 2 * KV_TILE_BYTES + STAGES * 2 * Q_TILE_BYTES;
  uint8_t* bar_gen = ds_gen + 2 * DS_BYTES;
  // barriers (8 B each)
  const uint32_t kv_full = bar_base;
  auto qdo_full = [&](int st) { return bar_base + 8u * (1 + st); };     // 3
  auto stage_free = [&](int st) { return bar_base + 8u * (4 + st); };   // 3
  auto ds_free = [&](int buf) { return bar_base + 8u * (7 + buf); };    // 2
  const uint32_t sdp_full = bar_base + 8u * 9, ds_ready = bar_base + 8u * 10, mma_done = bar_base + 8u * 11,
                 dq_free = bar_base + 8u * 12, drain_bar = bar_base + 8u * 13, sdp_taken = bar_base + 8u * 14,
                 final_bar = bar_base + 8u * 15, tmem_slot = bar_base + 8u * 16;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(bar_gen + 128);
  float* stat_smem = reinterpret_cast<float*>(bar_gen + 256);       // [2][lse2 | D][64]
  int* docq_smem = reinterpret_cast<int*>(bar_gen + 256 + 1024);    // [2][64]
  const uint32_t dq_stage = bar_base + AUX_BYTES;                   // only allocated when dq_tma

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // grid: x = (batch, KV head), y = key tile.  Blocks are handed out x-fastest, so with a causal mask all the
  // heaviest key tiles (the earliest: every query sees them) start first and the lightest ones fill the tail.
  const int n_kv_tiles = gridDim.y;
  const int kt = CAUSAL ? blockIdx.y : (n_kv_tiles - 1 - blockIdx.y);
  const int Hkv_ = H / group;
  const int hk = blockIdx.x % Hkv_, b = blockIdx.x / Hkv_;
  const int k0 = kt * BLK_K;
  const int n_q_tiles = (Sq + BLK_Q - 1) / BLK_Q;
  const int i_start = CAUSAL ? min(n_q_tiles, k0 / BLK_Q) : 0;
  const int n_i = n_q_tiles - i_start;
  const int n_iter = n_i * group;
  const float scale_log2 = scale * 1.4426950408889634f;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int st = 0; st < STAGES; ++st) {
      mbar_init(qdo_full(st), 1);
      mbar_init(stage_free(st), 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(ds_ready, 8);
    mbar_init(mma_done, 1);
    mbar_init(dq_free, 4);
    mbar_init(sdp_taken, 8);
    mbar_init(final_bar, 1);
    mbar_init(ds_free(0), 1);
    mbar_init(ds_free(1), 1);
    mbar_init(drain_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_do);
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
      bool ok = true;
      int issued = 0;
      mbar_expect_tx(kv_full, 2 * KV_TILE_BYTES);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        tma_load_2d(k_smem + c * KV_BLOCK_BYTES, &map_k, kv_full, hk * HD + 64 * c, b * Sk + k0);
        tma_load_2d(v_smem + c * KV_BLOCK_BYTES, &map_v, kv_full, hk * HD + 64 * c, b * Sk + k0);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int st = it % STAGES;
        const int use = it / STAGES;
        if (use > 0 && !mbar_wait(stage_free(st), (use - 1) & 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
        const int hq = hk * group + it / n_i;
        const int q0 = (i_start + it % n_i) * BLK_Q;
        mbar_expect_tx(qdo_full(st), 2 * Q_TILE_BYTES);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          tma_load_2d(q_smem + st * Q_TILE_BYTES + c * Q_BLOCK_BYTES, &map_q, qdo_full(st), hq * HD + 64 * c,
                      b * Sq + q0);
          tma_load_2d(do_smem + st * Q_TILE_BYTES + c * Q_BLOCK_BYTES, &map_do, qdo_full(st), hq * HD + 64 * c,
                      b * Sq + q0);
        }
        ++issued;
      }
      if (!ok) {
        mbar_wait(kv_full, 0, status, KF_ERR_WAIT_DRAIN);
        for (int it = max(0, issued - STAGES); it < issued; ++it)
          mbar_wait(qdo_full(it % STAGES), (it / STAGES) & 1, status, KF_ERR_WAIT_DRAIN);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_st = umma_idesc_bf16(128, BLK_Q, false, false);  // S^T, dP^T
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, HD, false, true);     // dV, dK (B = rows of Q_i / dO_i)
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, BLK_Q, true, true);    // dQ^T = K^T dS
      bool ok = mbar_wait(kv_full, 0, status, KF_ERR_WAIT_FULL);
      // S^T(t) = K Q^T into score buffer t & 1 and dP^T(t) = V dO^T: all operands with the head dim contiguous
      auto issue_scores = [&](int t) -> bool {
        const int st = t % STAGES, buf = t & 1;
        const uint32_t qs = q_smem + st * Q_TILE_BYTES, dos = do_smem + st * Q_TILE_BYTES;
        if (!mbar_wait(qdo_full(st), (t / STAGES) & 1, status, KF_ERR_WAIT_FULL)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t a_off = (kk / 4) * KV_BLOCK_BYTES + (kk % 4) * 32;
          const uint32_t b_off = (kk / 4) * Q_BLOCK_BYTES + (kk % 4) * 32;
          tc_mma_f16(tmem_base + ST_COL + buf * BLK_Q, umma_desc_sw128(k_smem + a_off, 16, 1024),
                     umma_desc_sw128(qs + b_off, 16, 1024), idesc_st, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t a_off = (kk / 4) * KV_BLOCK_BYTES + (kk % 4) * 32;
          const uint32_t b_off = (kk / 4) * Q_BLOCK_BYTES + (kk % 4) * 32;
          tc_mma_f16(tmem_base + DPT_COL, umma_desc_sw128(v_smem + a_off, 16, 1024),
                     umma_desc_sw128(dos + b_off, 16, 1024), idesc_st, kk != 0);
        }
        tc_commit(sdp_full);
        return true;
      };
      if (ok && n_iter > 0) ok = issue_scores(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int st = it % STAGES, buf = it & 1;
        const uint32_t qs = q_smem + st * Q_TILE_BYTES, dos = do_smem + st * Q_TILE_BYTES;
        const uint32_t dss = ds_smem + buf * DS_BYTES;
        // The next tile's scores run while the softmax warps work on this one.  S^T(it+1) goes to the other
        // score buffer (its old P^T was read by an MMA issued earlier by this thread); dP^T has one buffer,
        // free once the softmax warps have copied dP^T(it) into registers.
        if (it + 1 < n_iter) {
          if (!mbar_wait(sdp_taken, it & 1, status, KF_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          if (!issue_scores(it + 1)) { ok = false; break; }
        }
        if (!mbar_wait(ds_ready, it & 1, status, KF_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        if (it > 0 && !mbar_wait(dq_free, (it - 1) & 1, status, KF_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        // dV += P^T dO_i : A = P^T from TMEM (8 columns per 16 queries), B = dO_i rows (head dim contiguous)
#pragma unroll
        for (int kk = 0; kk < BLK_Q / 16; ++kk)
          tc_mma_f16_ts(tmem_base + DV_COL, tmem_base + ST_COL + buf * BLK_Q + kk * 8,
                        umma_desc_sw128(dos + kk * 2048, Q_BLOCK_BYTES, 1024), idesc_acc, (it | kk) != 0);
        // dK += dS^T Q_i : A = dS^T from smem (query dim contiguous), B = Q_i rows
#pragma unroll
        for (int kk = 0; kk < BLK_Q / 16; ++kk)
          tc_mma_f16(tmem_base + DK_COL, umma_desc_sw128(dss + kk * 32, 16, 1024),
                     umma_desc_sw128(qs + kk * 2048, Q_BLOCK_BYTES, 1024), idesc_acc, (it | kk) != 0);
        // dQ_i^T = K^T dS : A = K rows read with the head dim as M, B = dS^T rows read with the query dim as N
#pragma unroll
        for (int kk = 0; kk < BLK_K / 16; ++kk)
          tc_mma_f16(tmem_base + DQT_COL, umma_desc_sw128(k_smem + kk * 2048, KV_BLOCK_BYTES, 1024),
                     umma_desc_sw128(dss + kk * 2048, DS_BYTES, 1024), idesc_dq, kk != 0);
        tc_commit(stage_free(st));
        tc_commit(ds_free(buf));
        tc_commit(mma_done);
      }
      if (ok) tc_commit(final_bar);  // every MMA of this CTA has retired: dK / dV are final
      if (!ok) {
        tc_commit(drain_bar);
        mbar_wait(drain_bar, 0, status, KF_ERR_WAIT_DRAIN);
      }
    }
  } else if (warp < 6 || warp >= 10) {
    // ------------------------------------------------------------ softmax warps: one thread per (key row, half of the queries)
    constexpr int HQ = BLK_Q / 2;             // queries per thread
    const int half = warp >= 10 ? 1 : 0;
    const int quarter = warp & 3;
    const int r_local = quarter * 32 + lane;  // key row of this thread
    const int kpos = k0 + r_local;
    const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16);
    const int t128 = half == 0 ? threadIdx.x - 64 : 128;   // the first group's 128 threads fetch the row statistics
    int doc_k = 0;
    if (HAS_DOC) doc_k = kpos < Sk ? doc_ids[size_t(b) * Sk + kpos] : -2;
    bool ok = true;
    // statistics of the 64 queries of iteration `t` (lse in log2 units for threads 0..63, D for 64..127), fetched one
    // iteration ahead so that the global-memory latency hides under the arithmetic of the current tile
    auto fetch_stat = [&](int t) -> float {
      if (t128 >= 128 || t >= n_iter) return 0.f;
      const int hq_t = hk * group + t / n_i;
      const int qq = (i_start + t % n_i) * BLK_Q + (t128 & 63);
      const size_t idx = (size_t(b) * H + hq_t) * Sq + qq;
      if (t128 < 64) return qq < Sq ? LSE[idx] * 1.4426950408889634f : INFINITY;  // +inf -> P = 0 for padding rows
      return qq < Sq ? Dsum[idx] : 0.f;
    };
    float stat_next = fetch_stat(0);
    for (int it = 0; it < n_iter; ++it) {
      const int hq = hk * group + it / n_i;
      const int q0 = (i_start + it % n_i) * BLK_Q;
      float* stat = stat_smem + (it & 1) * 128;
      int* dq_doc = docq_smem + (it & 1) * 64;
      if (t128 < 128) {
        stat[t128] = stat_next;
        if (HAS_DOC && t128 < 64) {
          const int qq = q0 + t128;
          dq_doc[t128] = qq < Sq ? doc_ids[size_t(b) * Sq + qq] : -1;
        }
      }
      group_sync(1, 256);
      stat_next = fetch_stat(it + 1);
      if (ok && !mbar_wait(sdp_full, it & 1, status, KF_ERR_WAIT_TMEM_FULL)) ok = false;
      tc_fence_after();
      const uint32_t t_s = t_lane + ST_COL + (it & 1) * BLK_Q;
      uint32_t sv[HQ], dp[HQ];
      tmem_ld_32x32_at(t_s + half * HQ, sv);
      tmem_ld_32x32_at(t_lane + DPT_COL + half * HQ, dp);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sdp_taken);  // dP^T is in registers: the next tile's dP^T may be computed
      // P^T overwrites the first 32 columns of S^T: nobody may store before both warps of a key-row quarter have
      // loaded their scores
      group_sync(3, 256);
      const bool tile_masked = HAS_DOC || (CAUSAL && q0 < k0 + BLK_K - 1) || (k0 + BLK_K > Sk) || (q0 + BLK_Q > Sq);
      uint32_t pk[HQ / 2], dsk[HQ / 2];
#pragma unroll
      for (int i4 = 0; i4 < HQ / 4; ++i4) {
        // four queries per step: their lse / D come as two 16-byte broadcast reads instead of eight 4-byte ones
        const float4 l4 = *reinterpret_cast<const float4*>(stat + half * HQ + 4 * i4);
        const float4 d4 = *reinterpret_cast<const float4*>(stat + 64 + half * HQ + 4 * i4);
        const float lse4[4] = {l4.x, l4.y, l4.z, l4.w}, dd4[4] = {d4.x, d4.y, d4.z, d4.w};
        float p[4], ds[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int c = 4 * i4 + e;           // index inside this thread's half
          float pe = fast_exp2(fmaf(__uint_as_float(sv[c]), scale_log2, -lse4[e]));
          if (tile_masked) {
            const int qpos = q0 + half * HQ + c;
            bool vis = kpos < Sk && qpos < Sq;
            if (CAUSAL) vis = vis && kpos <= qpos;
            if (HAS_DOC) vis = vis && dq_doc[half * HQ + c] == doc_k;
            pe = vis ? pe : 0.f;
          }
          p[e] = pe;
          ds[e] = pe * (__uint_as_float(dp[c]) - dd4[e]) * scale;
        }
        pk[2 * i4] = pack_bf16(p[0], p[1]);
        pk[2 * i4 + 1] = pack_bf16(p[2], p[3]);
        dsk[2 * i4] = pack_bf16(ds[0], ds[1]);
        dsk[2 * i4 + 1] = pack_bf16(ds[2], ds[3]);
      }
      // P^T over the start of S^T (bf16 pairs: 16 columns per 32 queries)
      tmem_st_32x16(t_s + half * (HQ / 2), pk);
      // dS^T into shared memory, 128B-swizzled rows (16-byte chunk c of row r lives at chunk c ^ (r % 8));
      // the previous iteration's dK / dQ MMAs must have finished reading it
      // (two buffers: the MMAs of iteration it-2 were the last readers of this one)
      if (it > 1 && ok && !mbar_wait(ds_free(it & 1), ((it >> 1) - 1) & 1, status, KF_ERR_WAIT_TMEM_FULL)) ok = false;
      {
        uint8_t* row_ptr = ds_gen + (it & 1) * DS_BYTES + r_local * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {   // this thread's 32 queries = four 16-byte chunks of the row
          uint4 w = make_uint4(dsk[4 * c], dsk[4 * c + 1], dsk[4 * c + 2], dsk[4 * c + 3]);
          *reinterpret_cast<uint4*>(row_ptr + (((half * 4 + c) ^ (r_local & 7)) << 4)) = w;
        }
      }
      fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async-proxy reads
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
    }
    // ---- epilogue: dK / dV accumulators -> bf16 rows of the key tile (first softmax group: one thread per key row)
    if (half != 0) ok = false;
    if (ok && n_iter > 0 && !mbar_wait(final_bar, 0, status, KF_ERR_WAIT_TMEM_FULL)) ok = false;
    if (ok && cosT != nullptr && n_iter > 0) {
      // dK leaves through the inverse rotary embedding (the forward rotated K after the projection): columns
      // (i, i + 64) of a head are a pair, the angle is that of the key's position
      tc_fence_after();
      __nv_bfloat16* dst = dK + (size_t(b) * Sk + kpos) * lddk + size_t(hk) * HD;
      const float* cr = cosT + size_t(min(kpos, Sk - 1)) * (HD / 2);
      const float* sr = sinT + size_t(min(kpos, Sk - 1)) * (HD / 2);
#pragma unroll 1
      for (int c = 0; c < HD / 64; ++c) {
        uint32_t lo[32], hi[32];
        tmem_ld_32x32_at(t_lane + DK_COL + c * 32, lo);
        tmem_ld_32x32_at(t_lane + DK_COL + HD / 2 + c * 32, hi);
        tmem_ld_wait();
        if (kpos < Sk) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float a[8], bb[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float cv = cr[c * 32 + 8 * i + e], sv2 = sr[c * 32 + 8 * i + e];
              const float x = __uint_as_float(lo[8 * i + e]), y = __uint_as_float(hi[8 * i + e]);
              a[e] = x * cv + y * sv2;
              bb[e] = y * cv - x * sv2;
            }
            uint4 w0, w1;
            w0.x = pack_bf16(a[0], a[1]); w0.y = pack_bf16(a[2], a[3]); w0.z = pack_bf16(a[4], a[5]); w0.w = pack_bf16(a[6], a[7]);
            w1.x = pack_bf16(bb[0], bb[1]); w1.y = pack_bf16(bb[2], bb[3]); w1.z = pack_bf16(bb[4], bb[5]); w1.w = pack_bf16(bb[6], bb[7]);
            *reinterpret_cast<uint4*>(dst + c * 32 + 8 * i) = w0;
            *reinterpret_cast<uint4*>(dst + HD / 2 + c * 32 + 8 * i) = w1;
          }
        }
      }
    }
    if (ok) {
      tc_fence_after();
#pragma unroll 1
      for (int which = 0; which < ((cosT != nullptr && n_iter > 0) ? 1 : 2); ++which) {
        __nv_bfloat16* dst = which == 0 ? dV + (size_t(b) * Sk + kpos) * lddv + size_t(hk) * HD
                                        : dK + (size_t(b) * Sk + kpos) * lddk + size_t(hk) * HD;
        const uint32_t col0 = which == 0 ? DV_COL : DK_COL;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          if (n_iter > 0) {
            tmem_ld_32x32_at(t_lane + col0 + c * 32, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = 0u;
          }
          if (kpos < Sk) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(o[8 * i + 0]), __uint_as_float(o[8 * i + 1]));
              w.y = pack_bf16(__uint_as_float(o[8 * i + 2]), __uint_as_float(o[8 * i + 3]));
              w.z = pack_bf16(__uint_as_float(o[8 * i + 4]), __uint_as_float(o[8 * i + 5]));
              w.w = pack_bf16(__uint_as_float(o[8 * i + 6]), __uint_as_float(o[8 * i + 7]));
              *reinterpret_cast<uint4*>(dst + c * 32 + 8 * i) = w;
            }
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ dQ reduction warps (6..9)
    const int quarter = warp & 3;
    const int d = quarter * 32 + lane;  // head-dim index = TMEM lane of dQ^T
    const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16);
    const bool elected = threadIdx.x == 192;  // issues, commits and waits for the bulk reductions
    bool ok = true;
    for (int it = 0; it < n_iter; ++it) {
      const int hq = hk * group + it / n_i;
      const int q0 = (i_start + it % n_i) * BLK_Q;
      if (ok && !mbar_wait(mma_done, it & 1, status, KF_ERR_WAIT_TMEM_FULL)) ok = false;
      tc_fence_after();
      uint32_t v[BLK_Q];
      tmem_ld_32x32_at(t_lane + DQT_COL, v);
      tmem_ld_32x32_at(t_lane + DQT_COL + 32, v + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_free);  // the values are in registers: the next dQ^T may be computed
      if (dq_tma) {
        // transpose through shared memory into the [query][head dim] tile the tensor map describes, then one
        // bulk reduction adds the whole tile; rows past the end of the tensor are clipped by the TMA unit, rows
        // of padding queries hold exact zeros
        if (elected) bulk_wait_read_all();  // the previous reduction has read the staging tile
        group_sync(2, 128);
#pragma unroll
        for (int c = 0; c < BLK_Q; ++c)
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(dq_stage + uint32_t(c * HD + d) * 4u), "r"(v[c]) : "memory");
        fence_async_smem();
        group_sync(2, 128);
        if (elected && ok) {
          tma_reduce_add_2d(&map_dq, dq_stage, hq * HD, b * Sq + q0);
          bulk_commit();
        }
      } else if (ok) {
        float* base = dQacc + ((size_t(b) * Sq + q0) * H + hq) * HD + d;
#pragma unroll
        for (int c = 0; c < BLK_Q; ++c)
          if (q0 + c < Sq) red_add_f32(base + size_t(c) * H * HD, __uint_as_float(v[c]));
      }
    }
    if (dq_tma && elected) bulk_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// D[b, h, s] = sum_d O[b, s, h, d] * dO[b, s, h, d]  (one warp per (b, s, h) row)
__global__ void kf_attn_bwd_dot(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                float* __restrict__ D, int B, int S, int H, int hd, long long ldo, long long lddo) {
  const long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;  // over b, s, h
  const int lane = threadIdx.x & 31;
  if (row >= (long long)B * S * H) return;
  const int h = row % H;
  const long long bs = row / H;
  const __nv_bfloat16* o = O + bs * ldo + (long long)h * hd;
  const __nv_bfloat16* g = dO + bs * lddo + (long long)h * hd;
  float acc = 0.f;
  for (int c = lane * 4; c < hd; c += 128) {
    const uint2 a = *reinterpret_cast<const uint2*>(o + c);
    const uint2 bb = *reinterpret_cast<const uint2*>(g + c);
    const float2 a0 = unpack_bf16(a.x), a1 = unpack_bf16(a.y), b0 = unpack_bf16(bb.x), b1 = unpack_bf16(bb.y);
    acc += a0.x * b0.x + a0.y * b0.y + a1.x * b1.x + a1.y * b1.y;
  }
#pragma unroll
  for (int o2 = 16; o2 > 0; o2 >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
  if (lane == 0) {
    const long long b = bs / S, s = bs % S;
    D[(b * H + h) * S + s] = acc;
  }
}

// fp32 (rows x cols contiguous) -> bf16 rows with pitch ld
__global__ void kf_f32_to_bf16_rows(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long rows,
                                    int cols, long long ld) {
  const long long n4 = rows * (cols / 4);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / (cols / 4);
    const int c = (i % (cols / 4)) * 4;
    const float4 v = *reinterpret_cast<const float4*>(src + r * cols + c);
    uint2 w;
    w.x = pack_bf16(v.x, v.y);
    w.y = pack_bf16(v.z, v.w);
    *reinterpret_cast<uint2*>(dst + r * ld + c) = w;
  }
}

// fp32 dQ [rows][H * 128] -> bf16 rows with pitch ld, through the inverse rotary embedding of position (row % S)
__global__ void kf_dq_finish_rope(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long rows, int H,
                                  long long ld, const float* __restrict__ cosT, const float* __restrict__ sinT, int S) {
  constexpr int HALF = HD / 2;
  const long long n4 = rows * H * (HALF / 4);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const int j = (i % (HALF / 4)) * 4;
    const long long rh = i / (HALF / 4);
    const int h = rh % H;
    const long long r = rh / H;
    const int pos = r % S;
    const float4 a = *reinterpret_cast<const float4*>(src + (r * H + h) * HD + j);
    const float4 b = *reinterpret_cast<const float4*>(src + (r * H + h) * HD + HALF + j);
    const float4 c = *reinterpret_cast<const float4*>(cosT + size_t(pos) * HALF + j);
    const float4 s = *reinterpret_cast<const float4*>(sinT + size_t(pos) * HALF + j);
    uint2 lo, hi;
    lo.x = pack_bf16(a.x * c.x + b.x * s.x, a.y * c.y + b.y * s.y);
    lo.y = pack_bf16(a.z * c.z + b.z * s.z, a.w * c.w + b.w * s.w);
    hi.x = pack_bf16(b.x * c.x - a.x * s.x, b.y * c.y - a.y * s.y);
    hi.y = pack_bf16(b.z * c.z - a.z * s.z, b.w * c.w - a.w * s.w);
    *reinterpret_cast<uint2*>(dst + r * ld + h * HD + j) = lo;
    *reinterpret_cast<uint2*>(dst + r * ld + h * HD + HALF + j) = hi;
  }
}

}  // namespace attnb
}  // namespace kf

extern "C" void* kf_status_device_ptr();

namespace kf {
namespace attnb {
static int g_dq_mode = 1;  // 0: red.global per element, 1: bulk tensor reduction from shared memory (1.75x faster)

// fp32 [rows][cols] row-major -> tensor map with an unswizzled (box_cols x box_rows) box
inline int make_map_2d_f32_plain(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_cols,
                                 uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 4};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
}  // namespace attnb
}  // namespace kf

extern "C" {

// How the backward kernel adds its dQ tiles to the fp32 accumulator: 0 = red.global per element,
// 1 = one bulk tensor reduction per tile (default).  Returns the previous mode.
int kf_attn_bwd_dq_mode(int mode) {
  const int prev = kf::attnb::g_dq_mode;
  if (mode == 0 || mode == 1) kf::attnb::g_dq_mode = mode;
  return prev;
}

// Backward attention (head dim 128).  q / k / v / o / do: rows (b * S + s) with pitches ld*, heads side by
// side; lse: fp32 [B][H][Sq] from the forward; dsum: fp32 scratch [B][H][Sq]; dq_acc: fp32 scratch
// [B][Sq][H][128] (zeroed here); dq / dk / dv: bf16 outputs with pitches lddq / lddk / lddv (they may be
// slices of one fused gradient buffer).  doc: optional int32 [B][S].  Requires Sq == Sk when causal or doc.
// kf_attn_bwd_rope_bf16: the same, and dq / dk additionally pass through the inverse rotary embedding (cosT / sinT:
// fp32 [Sq][64], position = index inside the sequence), i.e. they are gradients with respect to the un-rotated
// projections when q / k were rotated after the projection.  Null tables = no rotation.
int kf_attn_bwd_rope_bf16(const void* q, const void* k, const void* v, const void* o, const void* d_o, const void* lse,
                          void* dsum, void* dq_acc, void* dq, void* dk, void* dv, const void* doc, int B, int Sq, int Sk,
                          int H, int Hkv, int hd, long long ldq, long long ldk, long long ldv, long long ldo,
                          long long lddo, long long lddq, long long lddk, long long lddv, float scale, int causal,
                          const void* cosT, const void* sinT, void* stream) {
  using namespace kf;
  using namespace kf::attnb;
  if (hd != HD || Hkv <= 0 || H % Hkv != 0) return 3;
  if ((causal || doc) && Sq != Sk) return 4;
  if ((ldq | ldk | ldv | ldo | lddo | lddq | lddk | lddv) & 7) return 5;
  cudaStream_t st = (cudaStream_t)stream;
  CUtensorMap mq, mk, mv, mdo;
  int rc = make_map_2d_bf16(&mq, q, uint64_t(B) * Sq, uint64_t(H) * hd, ldq, 64, BLK_Q);
  if (rc) return 100 + rc;
  rc = make_map_2d_bf16(&mk, k, uint64_t(B) * Sk, uint64_t(Hkv) * hd, ldk, 64, BLK_K);
  if (rc) return 200 + rc;
  rc = make_map_2d_bf16(&mv, v, uint64_t(B) * Sk, uint64_t(Hkv) * hd, ldv, 64, BLK_K);
  if (rc) return 250 + rc;
  rc = make_map_2d_bf16(&mdo, d_o, uint64_t(B) * Sq, uint64_t(H) * hd, lddo, 64, BLK_Q);
  if (rc) return 270 + rc;
  const int dq_tma = g_dq_mode;
  CUtensorMap mdq;
  rc = make_map_2d_f32_plain(&mdq, dq_acc, uint64_t(B) * Sq, uint64_t(H) * hd, HD, BLK_Q);
  if (rc) return 280 + rc;
  const size_t smem_bytes = dq_tma ? SMEM_DQ_TMA : SMEM;
  // pre-pass: D = rowsum(dO * O); zero the fp32 dQ accumulator
  {
    const long long rows = (long long)B * Sq * H;
    const int threads = 256;
    const long long blocks = (rows * 32 + threads - 1) / threads;
    kf_attn_bwd_dot<<<(unsigned)blocks, threads, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(o),
                                                          reinterpret_cast<const __nv_bfloat16*>(d_o),
                                                          reinterpret_cast<float*>(dsum), B, Sq, H, hd, ldo, lddo);
    cudaError_t e = cudaMemsetAsync(dq_acc, 0, size_t(B) * Sq * H * hd * sizeof(float), st);
    if (e != cudaSuccess) return 400 + (int)e;
  }
  int* status = reinterpret_cast<int*>(kf_status_device_ptr());
  dim3 grid(Hkv * B, (Sk + BLK_K - 1) / BLK_K);
#define KF_BWD_LAUNCH(C_, D_)                                                                                      \
  {                                                                                                                \
    auto kern = kf_attn_bwd_tcgen05<C_, D_>;                                                                       \
    static bool attr_set = false;                                                                                  \
    if (!attr_set) {                                                                                               \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_DQ_TMA);   \
      if (e != cudaSuccess) return 300 + (int)e;                                                                   \
      attr_set = true;                                                                                             \
    }                                                                                                              \
    kern<<<grid, THREADS, smem_bytes, st>>>(mq, mk, mv, mdo, mdq, dq_tma, reinterpret_cast<const float*>(lse),     \
                                      reinterpret_cast<const float*>(dsum), reinterpret_cast<const int*>(doc),     \
                                      reinterpret_cast<float*>(dq_acc), reinterpret_cast<__nv_bfloat16*>(dk),      \
                                      reinterpret_cast<__nv_bfloat16*>(dv), Sq, Sk, H, H / Hkv, lddk, lddv, scale, \
                                      status, reinterpret_cast<const float*>(cosT),                                \
                                      reinterpret_cast<const float*>(sinT));                                       \
  }
  if (doc) {
    if (causal) KF_BWD_LAUNCH(true, true) else KF_BWD_LAUNCH(false, true)
  } else {
    if (causal) KF_BWD_LAUNCH(true, false) else KF_BWD_LAUNCH(false, false)
  }
#undef KF_BWD_LAUNCH
  {
    const long long rows = (long long)B * Sq;
    const int cols = H * hd;
    if (cosT)
      kf_dq_finish_rope<<<1184, 256, 0, st>>>(reinterpret_cast<const float*>(dq_acc), reinterpret_cast<__nv_bfloat16*>(dq),
                                              rows, H, lddq, reinterpret_cast<const float*>(cosT),
                                              reinterpret_cast<const float*>(sinT), Sq);
    else
      kf_f32_to_bf16_rows<<<1184, 256, 0, st>>>(reinterpret_cast<const float*>(dq_acc),
                                                reinterpret_cast<__nv_bfloat16*>(dq), rows, cols, lddq);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

int kf_attn_bwd_bf16(const void* q, const void* k, const void* v, const void* o, const void* d_o, const void* lse,
                     void* dsum, void* dq_acc, void* dq, void* dk, void* dv, const void* doc, int B, int Sq, int Sk,
                     int H, int Hkv, int hd, long long ldq, long long ldk, long long ldv, long long ldo,
                     long long lddo, long long lddq, long long lddk, long long lddv, float scale, int causal,
                     void* stream) {
  return kf_attn_bwd_rope_bf16(q, k, v, o, d_o, lse, dsum, dq_acc, dq, dk, dv, doc, B, Sq, Sk, H, Hkv, hd, ldq, ldk, ldv,
                               ldo, lddo, lddq, lddk, lddv, scale, causal, nullptr, nullptr, stream);
}

}  // extern "C"
