// Flash attention on the 5th-generation tensor cores (forward pass).
//
//   O[b, s, h, :] = softmax_k( scale * Q[b, s, h, :] . K[b, k, h / group, :] + mask ) V[b, k, h / group, :]
//
// One CTA owns a 128-row query tile of one (batch, head) and walks the key/value sequence in tiles of
// 128 keys.  Grouped KV heads are indexed (h / group), never expanded; the causal mask skips whole
// tiles above the diagonal; a per-token document id (packed sequences) masks inside the kernel, so no
// S x S mask is ever built.  One CTA per SM; the score tile is double buffered in tensor memory so the
// tensor cores compute S_{j+1} while the softmax warps (the critical path: one exp2 per score on the
// special-function units) still work on S_j.
//
//   warp 0   : TMA producer   Q once, then K_j / V_j into two-stage 128B-swizzled rings
//   warp 1   : MMA issuer     S_{j+1} = Q K_{j+1}^T (smem x smem -> TMEM), then O += P_j V_j (TMEM x smem)
//   warps 2-5: softmax        one thread per query row: tcgen05.ld S, online max / sum with lazy
//                             rescaling of O (only when the row max grew by more than 2^8), exp2,
//                             bf16 P written back over S in TMEM (the A operand of the second MMA)
//
// Replaces F.scaled_dot_product_attention and the repeat_interleave GQA expansion of the reference
// (kempnerforge/model/attention.py:173-175,190-231) for the causal / document-masked cases.
#include "attention_common.cuh"

namespace kf {
namespace attn {

constexpr int BLK_M = 128;  // query rows per CTA
constexpr int BLK_N = 128;  // keys per tile
constexpr int THREADS = 320;  // TMA warp, MMA warp, 8 softmax warps
constexpr int TMEM_COLS = 512;
constexpr int S_COL = 0;    // S buffers 0 / 1 (fp32, 128 columns each); P (bf16 pairs) aliases each one's start
constexpr int O_COL = 256;  // O accumulator (fp32, HD columns)
constexpr int K_STAGES = 3;  // K is needed one tile earlier than V (S_{j+1} runs ahead), so it gets the deeper ring
constexpr int V_STAGES = 2;
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

template <int HD>
struct Cfg {
  static constexpr int BLOCKS = HD / 64;               // 64-column (128 B) swizzle blocks per row
  static constexpr int TILE_BYTES = BLK_N * HD * 2;    // one Q / K / V tile
  static constexpr int BLOCK_BYTES = BLK_N * 128;      // one 128-row x 128-byte block
  static constexpr int N_TILES_SMEM = 1 + K_STAGES + V_STAGES;  // Q, K ring, V ring
  static constexpr size_t SMEM = N_TILES_SMEM * size_t(TILE_BYTES) + 1024 /*align*/ + 4352 /*barriers, doc ids, row exchange*/;
};

// Named barriers: ids 1-4 join the two softmax warps that share a TMEM lane quarter (64 threads),
// id 5 joins all 256 softmax threads.
__device__ __forceinline__ void pair_sync(int quarter) {
  asm volatile("bar.sync %0, 64;" ::"r"(quarter + 1) : "memory");
}
__device__ __forceinline__ void softmax_all_sync() { asm volatile("bar.sync 5, 256;" ::: "memory"); }

template <int HD, bool CAUSAL, bool HAS_DOC>
__global__ void __launch_bounds__(THREADS, 1)
kf_attn_fwd_tcgen05(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ O,
                    float* __restrict__ LSE, const int* __restrict__ doc_ids, int Sq, int Sk, int H, int group,
                    long long ldo, float scale_log2, int* status) {
  using C = Cfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  const uint32_t k_smem = q_smem + C::TILE_BYTES;                // K_STAGES tiles
  const uint32_t v_smem = k_smem + K_STAGES * C::TILE_BYTES;    // V_STAGES tiles
  const uint32_t bar_base = v_smem + V_STAGES * C::TILE_BYTES;
  // barriers (8 B each): q_full, k_full[3], k_empty[3], v_full[2], v_empty[2], s_full[2], p_full, pv_done, drain
  const uint32_t q_full = bar_base;
  auto k_full = [&](int st) { return bar_base + 8u * (1 + st); };
  auto k_empty = [&](int st) { return bar_base + 8u * (4 + st); };
  auto v_full = [&](int st) { return bar_base + 8u * (7 + st); };
  auto v_empty = [&](int st) { return bar_base + 8u * (9 + st); };
  auto s_full = [&](int buf) { return bar_base + 8u * (11 + buf); };
  const uint32_t p_full = bar_base + 8u * 13, pv_done = bar_base + 8u * 14, drain_bar = bar_base + 8u * 15;
  const uint32_t o_final = bar_base + 8u * 17;  // every MMA of this CTA has retired (a phase of its own)
  uint8_t* aligned_generic = smem_raw + (smem_base - smem_u32(smem_raw));
  uint8_t* bar_generic = aligned_generic + C::N_TILES_SMEM * C::TILE_BYTES;
  const uint32_t tmem_slot = bar_base + 8u * 15 + 8u;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(bar_generic + 8 * 16);
  int* doc_smem = reinterpret_cast<int*>(bar_generic + 256);            // [2][128] key doc ids
  float* xch_smem = reinterpret_cast<float*>(bar_generic + 256 + 1024);  // [2][2][128] maxima, [2][128] sums

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_q_tiles = gridDim.x;
  const int qt = n_q_tiles - 1 - blockIdx.x;  // the longest (last) causal rows are scheduled first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / group;
  const int m0 = qt * BLK_M;
  const int kv_tiles_all = (Sk + BLK_N - 1) / BLK_N;
  const int n_tiles = CAUSAL ? min(kv_tiles_all, (m0 + BLK_M + BLK_N - 1) / BLK_N) : kv_tiles_all;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int st = 0; st < K_STAGES; ++st) {
      mbar_init(k_full(st), 1);
      mbar_init(k_empty(st), 1);
    }
    for (int st = 0; st < 2; ++st) {
      mbar_init(v_full(st), 1);
      mbar_init(v_empty(st), 1);
      mbar_init(s_full(st), 1);
    }
    mbar_init(p_full, 8);
    mbar_init(pv_done, 1);
    mbar_init(o_final, 1);
    mbar_init(drain_bar, 1);
    mbar_fence_init();
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
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
    // ------------------------------------------------------------ TMA producers
    // lane 0 feeds Q and the K ring, lane 1 the V ring: independent, so waiting for a V stage never
    // delays a K load (K_{j+1} is needed a whole tile before V_{j+1})
    if (lane == 0) {
      bool ok = true;
      int issued = 0;
      mbar_expect_tx(q_full, C::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < C::BLOCKS; ++c)
        tma_load_2d(q_smem + c * C::BLOCK_BYTES, &map_q, q_full, h * HD + 64 * c, b * Sq + m0);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % K_STAGES;
        const int use = j / K_STAGES;  // how many times this stage has been filled before
        if (use > 0 && !mbar_wait(k_empty(st), (use - 1) & 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(k_full(st), C::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < C::BLOCKS; ++c)
          tma_load_2d(k_smem + st * C::TILE_BYTES + c * C::BLOCK_BYTES, &map_k, k_full(st), hk * HD + 64 * c,
                      b * Sk + j * BLK_N);
        ++issued;
      }
      if (!ok) {
        // never leave with copies still landing in this CTA's shared memory
        mbar_wait(q_full, 0, status, KF_ERR_WAIT_DRAIN);
        for (int j = max(0, issued - K_STAGES); j < issued; ++j)
          mbar_wait(k_full(j % K_STAGES), (j / K_STAGES) & 1, status, KF_ERR_WAIT_DRAIN);
      }
    } else if (lane == 1) {
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % V_STAGES;
        const int use = j / V_STAGES;
        if (use > 0 && !mbar_wait(v_empty(st), (use - 1) & 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(v_full(st), C::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < C::BLOCKS; ++c)
          tma_load_2d(v_smem + st * C::TILE_BYTES + c * C::BLOCK_BYTES, &map_v, v_full(st), hk * HD + 64 * c,
                      b * Sk + j * BLK_N);
        ++issued;
      }
      if (!ok) {
        for (int j = max(0, issued - V_STAGES); j < issued; ++j)
          mbar_wait(v_full(j % V_STAGES), (j / V_STAGES) & 1, status, KF_ERR_WAIT_DRAIN);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BLK_M, BLK_N, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(BLK_M, HD, false, true);
      bool ok = mbar_wait(q_full, 0, status, KF_ERR_WAIT_FULL);
      // S_t = Q K_t^T into score buffer t & 1 : both operands K-major (head dim contiguous)
      auto issue_s = [&](int t) -> bool {
        const int st = t % K_STAGES, buf = t & 1;
        if (!mbar_wait(k_full(st), (t / K_STAGES) & 1, status, KF_ERR_WAIT_FULL)) return false;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * C::BLOCK_BYTES + (kk % 4) * 32;
          tc_mma_f16(tmem_base + S_COL + buf * BLK_N, umma_desc_sw128(q_smem + off, 16, 1024),
                     umma_desc_sw128(k_smem + st * C::TILE_BYTES + off, 16, 1024), idesc_s, kk != 0);
        }
        tc_commit(k_empty(st));  // K_t has been read
        tc_commit(s_full(buf));  // S_t is complete
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int st = j & 1;
        // the next score tile goes first: it overlaps the softmax of tile j.  Its buffer held P_{j-1}, whose
        // reader (O += P_{j-1} V_{j-1}) was issued earlier by this thread and therefore executes before it.
        if (j + 1 < n_tiles && !issue_s(j + 1)) { ok = false; break; }
        if (!mbar_wait(p_full, j & 1, status, KF_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        if (!mbar_wait(v_full(st), (j >> 1) & 1, status, KF_ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        // O += P V : A = P from tensor memory (bf16 pairs, 8 columns per 16 keys), B = V with the
        // head dim contiguous (MN-major): 64-column blocks BLOCK_BYTES apart, 16 keys = 2048 B
#pragma unroll
        for (int kk = 0; kk < BLK_N / 16; ++kk) {
          tc_mma_f16_ts(tmem_base + O_COL, tmem_base + S_COL + st * BLK_N + kk * 8,
                        umma_desc_sw128(v_smem + st * C::TILE_BYTES + kk * 2048, C::BLOCK_BYTES, 1024), idesc_o,
                        (j | kk) != 0);
        }
        tc_commit(v_empty(st));  // V_j has been read
        tc_commit(pv_done);      // O includes tile j
        if (j + 1 == n_tiles) tc_commit(o_final);
      }
      if (!ok) {
        tc_commit(drain_bar);
        mbar_wait(drain_bar, 0, status, KF_ERR_WAIT_DRAIN);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue (warps 2..9)
    // Two threads share a query row: warps 2-5 take score columns [0, 64), warps 6-9 columns [64, 128) of
    // the same TMEM lanes, so every scheduler has two softmax warps to interleave.  The pair exchanges
    // its row maximum through shared memory once per tile; everything else (sums, O columns) is split.
    // After a failed wait a warp keeps walking the loop (without waiting) so that its partner never
    // blocks on a named barrier.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r_local = quarter * 32 + lane;
    const int row = m0 + r_local;  // query position inside the sequence
    const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16);
    constexpr int HALF_N = BLK_N / 2;
    constexpr int O_HALF = HD / 2;
    const int col_base = half * HALF_N;
    const float NEG_INF = -INFINITY;
    float m_run = NEG_INF;  // running (possibly stale) row max, log2 units (identical in both threads of a row)
    float l_run = 0.f;      // running sum over this thread's columns, relative to m_run
    int doc_q = 0;
    if (HAS_DOC) doc_q = row < Sq ? doc_ids[size_t(b) * Sq + row] : -1;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int n0 = j * BLK_N;
      const int* dk = nullptr;
      if (HAS_DOC) {
        int* buf = doc_smem + (j & 1) * BLK_N;
        const int kpos = n0 + r_local;
        if (half == 0) buf[r_local] = kpos < Sk ? doc_ids[size_t(b) * Sk + kpos] : -2;
        softmax_all_sync();
        dk = buf + col_base;
      }
      const bool tile_masked = HAS_DOC || (CAUSAL && n0 + BLK_N - 1 > m0) || (n0 + BLK_N > Sk);
      const uint32_t t_s = t_lane + S_COL + (j & 1) * BLK_N;
      if (ok && !mbar_wait(s_full(j & 1), (j >> 1) & 1, status, KF_ERR_WAIT_TMEM_FULL)) ok = false;
      tc_fence_after();
      // ---- this thread's half of the score row (64 fp32) comes into registers with one wait
      uint32_t sv[HALF_N];
#pragma unroll
      for (int c = 0; c < HALF_N / 32; ++c) tmem_ld_32x32_at(t_s + col_base + c * 32, sv + c * 32);
      tmem_ld_wait();
      if (tile_masked) {
#pragma unroll
        for (int i = 0; i < HALF_N; ++i) {
          const int col = n0 + col_base + i;
          bool vis = col < Sk;
          if (CAUSAL) vis = vis && col <= row;
          if (HAS_DOC) vis = vis && dk[i] == doc_q;
          sv[i] = vis ? sv[i] : __float_as_uint(NEG_INF);  // exp2(-inf) = 0 later on
        }
      }
      float mx;
      {
        // four independent chains of three-input maxima (masked entries already hold -inf)
        float mx4[4] = {NEG_INF, NEG_INF, NEG_INF, NEG_INF};
#pragma unroll
        for (int i = 0; i < HALF_N; i += 8) {
#pragma unroll
          for (int q = 0; q < 4; ++q)
            mx4[q] = fmax3(mx4[q], __uint_as_float(sv[i + 2 * q]), __uint_as_float(sv[i + 2 * q + 1]));
        }
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      }
      // ---- exchange with the other half of the row.  Once both halves passed this barrier every score of
      // the row sits in registers, so P may overwrite the start of the S buffer.
      float* xch = xch_smem + (j & 1) * (2 * BLK_M);
      xch[half * BLK_M + r_local] = mx;
      pair_sync(quarter);
      mx = fmaxf(mx, xch[(half ^ 1) * BLK_M + r_local]);
      const float m_new = fmaxf(m_run, mx * scale_log2);
      // ---- lazy rescale: O and l follow the max only when it grew by more than the threshold
      const bool grow = m_new > m_run + RESCALE_THRESHOLD;  // true on the first visible tile (m_run = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? (m_run == NEG_INF ? 0.f : fast_exp2(m_run - m_new)) : 1.f;
        if (j > 0) {
          // O must be quiescent: wait until O += P_{j-1} V_{j-1} has retired (O += P_j V_j cannot start
          // before the softmax warps hand over P_j)
          if (ok && !mbar_wait(pv_done, (j - 1) & 1, status, KF_ERR_WAIT_TMEM_FULL)) ok = false;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < O_HALF / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(t_lane + O_COL + half * O_HALF + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(t_lane + O_COL + half * O_HALF + c * 32, o);
          }
        }
        if (grow) {
          l_run *= alpha;
          m_run = m_new;
        }
      }
      const float m_use = m_run == NEG_INF ? 0.f : m_run;
      // ---- P = exp2(S * scale - m), row sum, bf16 P over the start of the S buffer
      const uint64_t scale2 = pack2(scale_log2, scale_log2);
      const uint64_t neg_m2 = pack2(-m_use, -m_use);
      uint64_t lsum[4] = {0ull, 0ull, 0ull, 0ull};  // four independent chains of two-wide sums
#pragma unroll
      for (int c = 0; c < HALF_N / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint64_t x2 = ffma2(pack2(__uint_as_float(sv[c * 32 + 2 * i]), __uint_as_float(sv[c * 32 + 2 * i + 1])),
                                    scale2, neg_m2);
          float x0, x1;
          unpack2(x2, x0, x1);
          const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
          lsum[i & 3] = fadd2(lsum[i & 3], pack2(e0, e1));
          pk[i] = pack_bf16(e0, e1);
        }
        // keys [col_base + 32c, +32) -> packed columns [(col_base + 32c) / 2, +16)
        tmem_st_32x16(t_s + col_base / 2 + c * 16, pk);
      }
      {
        float a0, a1;
        unpack2(fadd2(fadd2(lsum[0], lsum[1]), fadd2(lsum[2], lsum[3])), a0, a1);
        l_run += a0 + a1;
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l -> bf16, log-sum-exp for the backward pass
    float* xl = xch_smem + 2 * (2 * BLK_M);  // [2][BLK_M] partial row sums
    xl[half * BLK_M + r_local] = l_run;
    pair_sync(quarter);
    const float l_tot = l_run + xl[(half ^ 1) * BLK_M + r_local];
    if (ok && n_tiles > 0 && !mbar_wait(o_final, 0, status, KF_ERR_WAIT_TMEM_FULL)) ok = false;
    if (ok) {
      tc_fence_after();
      const float inv_l = l_tot > 0.f ? 1.f / l_tot : 0.f;
      __nv_bfloat16* o_row = O + (size_t(b) * Sq + row) * ldo + size_t(h) * HD + half * O_HALF;
#pragma unroll 1
      for (int c = 0; c < O_HALF / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(t_lane + O_COL + half * O_HALF + c * 32, o);
        tmem_ld_wait();
        if (row < Sq) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(o[8 * i + 0]) * inv_l, __uint_as_float(o[8 * i + 1]) * inv_l);
            w.y = pack_bf16(__uint_as_float(o[8 * i + 2]) * inv_l, __uint_as_float(o[8 * i + 3]) * inv_l);
            w.z = pack_bf16(__uint_as_float(o[8 * i + 4]) * inv_l, __uint_as_float(o[8 * i + 5]) * inv_l);
            w.w = pack_bf16(__uint_as_float(o[8 * i + 6]) * inv_l, __uint_as_float(o[8 * i + 7]) * inv_l);
            *reinterpret_cast<uint4*>(o_row + c * 32 + 8 * i) = w;
          }
        }
      }
      if (row < Sq && half == 0) {
        // natural-log units of the scaled scores; -inf for a row that saw no key
        LSE[(size_t(b) * H + h) * Sq + row] =
            l_tot > 0.f ? (m_run + log2f(l_tot)) * 0.6931471805599453f : NEG_INF;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int HD, bool CAUSAL, bool HAS_DOC>
static int launch_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* O, float* LSE,
                      const int* doc, int B, int Sq, int Sk, int H, int Hkv, long long ldo, float scale,
                      int* status, cudaStream_t stream) {
  auto kern = kf_attn_fwd_tcgen05<HD, CAUSAL, HAS_DOC>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<HD>::SMEM);
    if (e != cudaSuccess) return 300 + (int)e;
    // two CTAs per SM need the largest shared-memory carve-out
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  dim3 grid((Sq + BLK_M - 1) / BLK_M, H, B);
  kern<<<grid, THREADS, Cfg<HD>::SMEM, stream>>>(mq, mk, mv, reinterpret_cast<__nv_bfloat16*>(O), LSE, doc, Sq, Sk,
                                                 H, H / Hkv, ldo, scale * 1.4426950408889634f, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // namespace attn
}  // namespace kf

extern "C" void* kf_status_device_ptr();

extern "C" {

// Resident CTAs per SM of the forward kernel for a head dim (a tuning aid: the design wants 2).
int kf_attn_fwd_occupancy(int hd) {
  using namespace kf::attn;
  int n = 0;
  cudaError_t e;
  if (hd == 128) {
    auto k = kf_attn_fwd_tcgen05<128, true, false>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<128>::SMEM);
    cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k, THREADS, Cfg<128>::SMEM);
  } else {
    auto k = kf_attn_fwd_tcgen05<64, true, false>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<64>::SMEM);
    cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, k, THREADS, Cfg<64>::SMEM);
  }
  return e == cudaSuccess ? n : -(int)e;
}

// Forward attention.  q: rows (b * Sq + s), row pitch ldq elements, head h at column h * hd; k / v likewise with
// Sk rows per batch and Hkv heads; o: pitch ldo; lse: fp32 [B][H][Sq].  doc (optional): int32 [B][S] document
// ids (requires Sq == Sk).  hd in {64, 128}; causal requires Sq == Sk.  Pitches must be multiples of 8
// elements and the base pointers 16-byte aligned.  Returns 0 or an error code; errors of bounded waits go
// to the library's status word.
int kf_attn_fwd_bf16(const void* q, const void* k, const void* v, void* o, void* lse, const void* doc, int B,
                     int Sq, int Sk, int H, int Hkv, int hd, long long ldq, long long ldk, long long ldv,
                     long long ldo, float scale, int causal, void* stream) {
  using namespace kf;
  using namespace kf::attn;
  if ((hd != 64 && hd != 128) || Hkv <= 0 || H % Hkv != 0) return 3;
  if ((causal || doc) && Sq != Sk) return 4;
  if ((ldq | ldk | ldv | ldo) & 7) return 5;
  CUtensorMap mq, mk, mv;
  int rc = make_map_2d_bf16(&mq, q, uint64_t(B) * Sq, uint64_t(H) * hd, ldq, 64, BLK_M);
  if (rc) return 100 + rc;
  rc = make_map_2d_bf16(&mk, k, uint64_t(B) * Sk, uint64_t(Hkv) * hd, ldk, 64, BLK_N);
  if (rc) return 200 + rc;
  rc = make_map_2d_bf16(&mv, v, uint64_t(B) * Sk, uint64_t(Hkv) * hd, ldv, 64, BLK_N);
  if (rc) return 250 + rc;
  int* status = reinterpret_cast<int*>(kf_status_device_ptr());
  cudaStream_t st = (cudaStream_t)stream;
  float* L = reinterpret_cast<float*>(lse);
  const int* D = reinterpret_cast<const int*>(doc);
#define KF_ATTN_LAUNCH(HD_, C_, D_) \
  return launch_fwd<HD_, C_, D_>(mq, mk, mv, o, L, D, B, Sq, Sk, H, Hkv, ldo, scale, status, st)
  if (hd == 128) {
    if (doc) { if (causal) KF_ATTN_LAUNCH(128, true, true); else KF_ATTN_LAUNCH(128, false, true); }
    if (causal) KF_ATTN_LAUNCH(128, true, false); else KF_ATTN_LAUNCH(128, false, false);
  } else {
    if (doc) { if (causal) KF_ATTN_LAUNCH(64, true, true); else KF_ATTN_LAUNCH(64, false, true); }
    if (causal) KF_ATTN_LAUNCH(64, true, false); else KF_ATTN_LAUNCH(64, false, false);
  }
#undef KF_ATTN_LAUNCH
}

}  // extern "C"
