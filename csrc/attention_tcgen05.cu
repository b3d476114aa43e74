// Flash attention on the 5th-generation tensor cores (forward pass).
//
//   O[b, s, h, :] = softmax_k( scale * Q[b, s, h, :] . K[b, k, h / group, :] + mask ) V[b, k, h / group, :]
//
// One CTA owns a 128-row query tile of one (batch, head) and walks the key/value sequence in tiles of
// 128 keys.  Grouped KV heads are indexed (h / group), never expanded; the causal mask skips whole
// tiles above the diagonal; a per-token document id (packed sequences) masks inside the kernel, so no
// S x S mask is ever built.  Two CTAs are resident per SM (96 KB of shared memory and 256 TMEM columns
// each), so one CTA's softmax overlaps the other's tensor-core work.
//
//   warp 0   : TMA producer   Q once, then K_j / V_j into single 128B-swizzled buffers
//   warp 1   : MMA issuer     S_j = Q K_j^T  (smem x smem -> TMEM),  O += P_j V_j  (TMEM x smem -> TMEM)
//   warps 2-5: softmax        one thread per query row: tcgen05.ld S, online max / sum with lazy
//                             rescaling of O (only when the row max grew by more than 2^8), exp2,
//                             bf16 P written back over S in TMEM (the A operand of the second MMA)
//
// Replaces F.scaled_dot_product_attention and the repeat_interleave GQA expansion of the reference
// (kempnerforge/model/attention.py:173-175,190-231) for the causal / document-masked cases.
#include "common.cuh"

namespace kf {
namespace attn {

constexpr int BLK_M = 128;  // query rows per CTA
constexpr int BLK_N = 128;  // keys per tile
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 256;
constexpr int S_COL = 0;    // S (fp32, 128 columns); P (bf16 pairs, 64 columns) aliases its start
constexpr int O_COL = 128;  // O accumulator (fp32, HD columns)
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

template <int HD>
struct Cfg {
  static constexpr int BLOCKS = HD / 64;               // 64-column (128 B) swizzle blocks per row
  static constexpr int TILE_BYTES = BLK_N * HD * 2;    // one Q / K / V tile
  static constexpr int BLOCK_BYTES = BLK_N * 128;      // one 128-row x 128-byte block
  static constexpr size_t SMEM = 3 * size_t(TILE_BYTES) + 1024 /*align*/ + 1280 /*barriers + doc ids*/;
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]),
        "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
        "r"(r[31])
      : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Named barrier among the 128 softmax threads only.
__device__ __forceinline__ void softmax_group_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int HD, bool CAUSAL, bool HAS_DOC>
__global__ void __launch_bounds__(THREADS, 2)
kf_attn_fwd_tcgen05(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                    const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ O,
                    float* __restrict__ LSE, const int* __restrict__ doc_ids, int Sq, int Sk, int H, int group,
                    long long ldo, float scale_log2, int* status) {
  using C = Cfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;
  const uint32_t k_smem = q_smem + C::TILE_BYTES;
  const uint32_t v_smem = k_smem + C::TILE_BYTES;
  const uint32_t bar_base = v_smem + C::TILE_BYTES;
  const uint32_t q_full = bar_base + 0, k_full = bar_base + 8, v_full = bar_base + 16, k_empty = bar_base + 24,
                 s_full = bar_base + 32, p_full = bar_base + 40, pv_done = bar_base + 48, drain_bar = bar_base + 56,
                 tmem_slot = bar_base + 64;
  uint8_t* aligned_generic = smem_raw + (smem_base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(aligned_generic + 3 * C::TILE_BYTES + 64);
  int* doc_smem = reinterpret_cast<int*>(aligned_generic + 3 * C::TILE_BYTES + 128);  // [2][128] key doc ids

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
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(s_full, 1);
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
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
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      int k_issued = 0, v_issued = 0;
      mbar_expect_tx(q_full, C::TILE_BYTES);
#pragma unroll
      for (int c = 0; c < C::BLOCKS; ++c)
        tma_load_2d(q_smem + c * C::BLOCK_BYTES, &map_q, q_full, h * HD + 64 * c, b * Sq + m0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j > 0 && !mbar_wait(k_empty, (j - 1) & 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(k_full, C::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < C::BLOCKS; ++c)
          tma_load_2d(k_smem + c * C::BLOCK_BYTES, &map_k, k_full, hk * HD + 64 * c, b * Sk + j * BLK_N);
        ++k_issued;
        if (j > 0 && !mbar_wait(pv_done, (j - 1) & 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(v_full, C::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < C::BLOCKS; ++c)
          tma_load_2d(v_smem + c * C::BLOCK_BYTES, &map_v, v_full, hk * HD + 64 * c, b * Sk + j * BLK_N);
        ++v_issued;
      }
      if (!ok) {
        // never leave with copies still landing in this CTA's shared memory
        mbar_wait(q_full, 0, status, KF_ERR_WAIT_DRAIN);
        if (k_issued) mbar_wait(k_full, (k_issued - 1) & 1, status, KF_ERR_WAIT_DRAIN);
        if (v_issued) mbar_wait(v_full, (v_issued - 1) & 1, status, KF_ERR_WAIT_DRAIN);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BLK_M, BLK_N, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(BLK_M, HD, false, true);
      bool ok = mbar_wait(q_full, 0, status, KF_ERR_WAIT_FULL);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(k_full, ph, status, KF_ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        // S = Q K^T : both operands K-major (head dim contiguous)
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * C::BLOCK_BYTES + (kk % 4) * 32;
          tc_mma_f16(tmem_base + S_COL, umma_desc_sw128(q_smem + off, 16, 1024),
                     umma_desc_sw128(k_smem + off, 16, 1024), idesc_s, kk != 0);
        }
        tc_commit(k_empty);  // K_j has been read
        tc_commit(s_full);   // S_j is complete (and so is every earlier MMA, O += P_{j-1} V_{j-1} included)
        if (!mbar_wait(p_full, ph, status, KF_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        if (!mbar_wait(v_full, ph, status, KF_ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        // O += P V : A = P from tensor memory (bf16 pairs, 8 columns per 16 keys), B = V with the
        // head dim contiguous (MN-major): 64-column blocks BLOCK_BYTES apart, 16 keys = 2048 B
#pragma unroll
        for (int kk = 0; kk < BLK_N / 16; ++kk) {
          tc_mma_f16_ts(tmem_base + O_COL, tmem_base + S_COL + kk * 8,
                        umma_desc_sw128(v_smem + kk * 2048, C::BLOCK_BYTES, 1024), idesc_o, (j | kk) != 0);
        }
        tc_commit(pv_done);  // V_j has been read; after the last tile: O is final
      }
      if (!ok) {
        tc_commit(drain_bar);
        mbar_wait(drain_bar, 0, status, KF_ERR_WAIT_DRAIN);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue (warps 2..5)
    const int quarter = warp & 3;
    const int r_local = quarter * 32 + lane;
    const int row = m0 + r_local;  // query position inside the sequence
    const uint32_t t_lane = tmem_base + (uint32_t(quarter * 32) << 16);
    const float NEG_INF = -INFINITY;
    float m_run = NEG_INF;  // running (possibly stale) row max, log2 units
    float l_run = 0.f;      // running row sum relative to m_run
    int doc_q = 0;
    if (HAS_DOC) doc_q = row < Sq ? doc_ids[size_t(b) * Sq + row] : -1;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int n0 = j * BLK_N;
      const int* dk = nullptr;
      if (HAS_DOC) {
        int* buf = doc_smem + (j & 1) * BLK_N;
        const int kpos = n0 + r_local;
        buf[r_local] = kpos < Sk ? doc_ids[size_t(b) * Sk + kpos] : -2;
        softmax_group_sync();
        dk = buf;
      }
      const bool tile_masked = HAS_DOC || (CAUSAL && n0 + BLK_N - 1 > m0) || (n0 + BLK_N > Sk);
      if (!mbar_wait(s_full, j & 1, status, KF_ERR_WAIT_TMEM_FULL)) { ok = false; break; }
      tc_fence_after();
      // ---- pass 1: row max of the visible scores
      float mx = NEG_INF;
#pragma unroll 1
      for (int c = 0; c < BLK_N / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_lane + S_COL + c * 32, v);
        tmem_ld_wait();
        if (tile_masked) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int col = n0 + c * 32 + i;
            bool vis = col < Sk;
            if (CAUSAL) vis = vis && col <= row;
            if (HAS_DOC) vis = vis && dk[c * 32 + i] == doc_q;
            mx = vis ? fmaxf(mx, __uint_as_float(v[i])) : mx;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(v[i]));
        }
      }
      const float m_new = fmaxf(m_run, mx * scale_log2);
      // ---- lazy rescale: O and l follow the max only when it grew by more than the threshold
      const bool grow = m_new > m_run + RESCALE_THRESHOLD;  // true on the first visible tile (m_run = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? (m_run == NEG_INF ? 0.f : fast_exp2(m_run - m_new)) : 1.f;
        if (j > 0) {
          // O += P_{j-1} V_{j-1} retired before s_full(j) flipped, so O is quiescent here
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32(t_lane + O_COL + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(t_lane + O_COL + c * 32, o);
          }
        }
        if (grow) {
          l_run *= alpha;
          m_run = m_new;
        }
      }
      const float m_use = m_run == NEG_INF ? 0.f : m_run;
      // ---- pass 2: P = exp2(S * scale - m), row sum, bf16 P over the start of S
      float l_add = 0.f;
#pragma unroll 1
      for (int c = 0; c < BLK_N / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_lane + S_COL + c * 32, v);
        tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = fast_exp2(fmaf(__uint_as_float(v[i]), scale_log2, -m_use));
          if (tile_masked) {
            const int col = n0 + c * 32 + i;
            bool vis = col < Sk;
            if (CAUSAL) vis = vis && col <= row;
            if (HAS_DOC) vis = vis && dk[c * 32 + i] == doc_q;
            e = vis ? e : 0.f;
          }
          p[i] = e;
          l_add += e;
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack_bf16(p[2 * i], p[2 * i + 1]);
        // chunk c of P lands on columns [16c, 16c+16): inside S columns already consumed
        tmem_st_32x16(t_lane + S_COL + c * 16, pk);
      }
      l_run += l_add;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l -> bf16, log-sum-exp for the backward pass
    if (ok && n_tiles > 0) ok = mbar_wait(pv_done, (n_tiles - 1) & 1, status, KF_ERR_WAIT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
      __nv_bfloat16* o_row = O + (size_t(b) * Sq + row) * ldo + size_t(h) * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t o[32];
        if (n_tiles > 0) {
          tmem_ld_32x32(t_lane + O_COL + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
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
      if (row < Sq) {
        // natural-log units of the scaled scores; -inf for a row that saw no key
        LSE[(size_t(b) * H + h) * Sq + row] =
            l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : NEG_INF;
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
