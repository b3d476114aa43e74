// Flash attention forward, two query tiles per CTA (256 query rows of one head).
//
// The softmax of a 128 x 128 score tile costs about as many cycles on the special-function units (one exp2 per
// score) as its two GEMMs cost on the tensor cores, and its other phases (TMEM load, row maximum, hand-over)
// cannot overlap its own exponentials.  This kernel therefore runs two query tiles A and B against the same K / V
// stream and interleaves them: while the softmax warps of A are in their exp2 phase, the warps of B load, reduce and
// hand over, and the tensor cores alternate  O_A += P_A V_j, S_A = Q_A K_{j+1}^T, O_B += P_B V_j, S_B = Q_B K_{j+1}^T.
// K and V tiles are fetched once for both query tiles.
//
//   warp 0    : TMA producers (lane 0: Q_A, Q_B and the K ring; lane 1: the V ring)
//   warp 1    : MMA issuer
//   warps 2-5 : softmax + epilogue of tile A (one thread per query row)
//   warps 6-9 : softmax + epilogue of tile B
//   TMEM      : S_A | S_B | O_A | O_B   (128 fp32 columns each; bf16 P aliases the start of its S)
//
// Masks, lazy rescaling and outputs are those of the single-tile kernel in attention_tcgen05.cu, which remains the
// path for short sequences.  Replaces F.scaled_dot_product_attention (kempnerforge/model/attention.py:227-231).
#include "attention_common.cuh"
#include <stdlib.h>

namespace kf {
namespace attn2 {

using namespace kf::attn;

constexpr int BLK_M = 128, BLK_N = 128;
constexpr int THREADS = 320;
constexpr int TMEM_COLS = 512;
constexpr int KV_STAGES = 2;
constexpr float RESCALE_THRESHOLD = 8.0f;

template <int HD>
struct Cfg {
  static constexpr int BLOCKS = HD / 64;
  static constexpr int TILE_BYTES = BLK_N * HD * 2;
  static constexpr int BLOCK_BYTES = BLK_N * 128;
  static constexpr int N_TILES_SMEM = 2 + 2 * KV_STAGES;  // Q_A, Q_B, K ring, V ring
  static constexpr size_t SMEM = N_TILES_SMEM * size_t(TILE_BYTES) + 1024 + 4352;
};

__device__ __forceinline__ void tile_group_sync(int tile) {
  asm volatile("bar.sync %0, 128;" ::"r"(tile + 1) : "memory");
}

// POLY: how many of every 16 pairs of exponentials are evaluated by exp2_poly2 on the FMA pipe (0 = all on the
// special-function unit).
template <int HD, bool CAUSAL, bool HAS_DOC, int POLY>
__global__ void __launch_bounds__(THREADS, 1)
kf_attn_fwd2_tcgen05(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ O,
                     float* __restrict__ LSE, const int* __restrict__ doc_ids, int Sq, int Sk, int H, int group,
                     long long ldo, float scale_log2, int* status, int n_super, int n_batch) {
  using C = Cfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;                                   // two tiles
  const uint32_t k_smem = q_smem + 2 * C::TILE_BYTES;
  const uint32_t v_smem = k_smem + KV_STAGES * C::TILE_BYTES;
  const uint32_t bar_base = v_smem + KV_STAGES * C::TILE_BYTES;
  // barriers: q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2 tiles], p_full[2], pv_done[2], drain
  const uint32_t q_full = bar_base;
  auto k_full = [&](int st) { return bar_base + 8u * (1 + st); };
  auto k_empty = [&](int st) { return bar_base + 8u * (3 + st); };
  auto v_full = [&](int st) { return bar_base + 8u * (5 + st); };
  auto v_empty = [&](int st) { return bar_base + 8u * (7 + st); };
  auto s_full = [&](int tile) { return bar_base + 8u * (9 + tile); };
  auto p_full = [&](int tile) { return bar_base + 8u * (11 + tile); };
  auto pv_done = [&](int tile) { return bar_base + 8u * (13 + tile); };
  const uint32_t drain_bar = bar_base + 8u * 15;
  auto o_final = [&](int tile) { return bar_base + 8u * (16 + tile); };  // every MMA of the tile has retired
  auto p_half = [&](int tile) { return bar_base + 8u * (19 + tile); };   // first 64 keys of P are in tensor memory
  const uint32_t tmem_slot = bar_base + 8u * 18;
  uint8_t* bar_generic = smem_raw + (smem_base - smem_u32(smem_raw)) + C::N_TILES_SMEM * C::TILE_BYTES;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(bar_generic + 8 * 18);
  int* doc_smem = reinterpret_cast<int*>(bar_generic + 256);  // [2 tiles][2][128] key doc ids

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // 1-D grid, query super-tile slowest: blocks are handed out in index order, so with a causal mask ALL the longest
  // rows (of every head and batch entry) start first and the short ones fill the tail of the last wave; the heads
  // of one KV group are neighbours and share their K / V tiles in L2
  const int n_hb = H * n_batch;
  const int qs = CAUSAL ? n_super - 1 - int(blockIdx.x) / n_hb : int(blockIdx.x) / n_hb;
  const int hb = int(blockIdx.x) % n_hb;
  const int h = hb % H, b = hb / H;
  const int hk = h / group;
  const int m0 = qs * 2 * BLK_M;
  const int kv_all = (Sk + BLK_N - 1) / BLK_N;
  // key tiles each query tile walks (tile B is absent when the sequence ends inside tile A)
  const int n_a = CAUSAL ? min(kv_all, (m0 + BLK_M + BLK_N - 1) / BLK_N) : kv_all;
  const int n_b = (m0 + BLK_M >= Sq) ? 0 : (CAUSAL ? min(kv_all, (m0 + 2 * BLK_M + BLK_N - 1) / BLK_N) : kv_all);
  const int n_max = max(n_a, n_b);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(k_full(i), 1);
      mbar_init(k_empty(i), 1);
      mbar_init(v_full(i), 1);
      mbar_init(v_empty(i), 1);
      mbar_init(s_full(i), 1);
      mbar_init(p_full(i), 4);
      mbar_init(p_half(i), 4);
      mbar_init(pv_done(i), 1);
      mbar_init(o_final(i), 1);
    }
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
  auto s_col = [&](int tile) { return tmem_base + uint32_t(tile * BLK_N); };
  auto o_col = [&](int tile) { return tmem_base + uint32_t(256 + tile * 128); };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producers
    if (lane == 0) {
      bool ok = true;
      int issued = 0;
      mbar_expect_tx(q_full, 2 * C::TILE_BYTES);
#pragma unroll
      for (int tile = 0; tile < 2; ++tile)
#pragma unroll
        for (int c = 0; c < C::BLOCKS; ++c)
          tma_load_2d(q_smem + tile * C::TILE_BYTES + c * C::BLOCK_BYTES, &map_q, q_full, h * HD + 64 * c,
                      b * Sq + m0 + tile * BLK_M);
      for (int j = 0; j < n_max; ++j) {
        const int st = j & 1, use = j >> 1;
        if (use > 0 && !mbar_wait(k_empty(st), (use - 1) & 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(k_full(st), C::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < C::BLOCKS; ++c)
          tma_load_2d(k_smem + st * C::TILE_BYTES + c * C::BLOCK_BYTES, &map_k, k_full(st), hk * HD + 64 * c,
                      b * Sk + j * BLK_N);
        ++issued;
      }
      if (!ok) {
        mbar_wait(q_full, 0, status, KF_ERR_WAIT_DRAIN);
        for (int j = max(0, issued - 2); j < issued; ++j) mbar_wait(k_full(j & 1), (j >> 1) & 1, status, KF_ERR_WAIT_DRAIN);
      }
    } else if (lane == 1) {
      bool ok = true;
      int issued = 0;
      for (int j = 0; j < n_max; ++j) {
        const int st = j & 1, use = j >> 1;
        if (use > 0 && !mbar_wait(v_empty(st), (use - 1) & 1, status, KF_ERR_WAIT_EMPTY)) { ok = false; break; }
        mbar_expect_tx(v_full(st), C::TILE_BYTES);
#pragma unroll
        for (int c = 0; c < C::BLOCKS; ++c)
          tma_load_2d(v_smem + st * C::TILE_BYTES + c * C::BLOCK_BYTES, &map_v, v_full(st), hk * HD + 64 * c,
                      b * Sk + j * BLK_N);
        ++issued;
      }
      if (!ok)
        for (int j = max(0, issued - 2); j < issued; ++j) mbar_wait(v_full(j & 1), (j >> 1) & 1, status, KF_ERR_WAIT_DRAIN);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(BLK_M, BLK_N, false, false);
      constexpr uint32_t idesc_o = umma_idesc_bf16(BLK_M, HD, false, true);
      bool ok = mbar_wait(q_full, 0, status, KF_ERR_WAIT_FULL);
      const int n_of[2] = {n_a, n_b};
      // S_tile = Q_tile K_t^T ; the caller has made sure K_t landed
      auto issue_s = [&](int tile, int t) {
        const int st = t & 1;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk / 4) * C::BLOCK_BYTES + (kk % 4) * 32;
          tc_mma_f16(s_col(tile), umma_desc_sw128(q_smem + tile * C::TILE_BYTES + off, 16, 1024),
                     umma_desc_sw128(k_smem + st * C::TILE_BYTES + off, 16, 1024), idesc_s, kk != 0);
        }
        tc_commit(s_full(tile));
      };
      if (ok && n_max > 0) {
        ok = mbar_wait(k_full(0), 0, status, KF_ERR_WAIT_FULL);
        if (ok) {
          tc_fence_after();
          if (n_a > 0) issue_s(0, 0);
          if (n_b > 0) issue_s(1, 0);
          tc_commit(k_empty(0));
        }
      }
      for (int j = 0; j < n_max && ok; ++j) {
        const int st = j & 1;
        bool k_next_ready = false;
        for (int tile = 0; tile < 2 && ok; ++tile) {
          if (j >= n_of[tile]) continue;
          // O_tile += P_tile V_j : A = P from tensor memory, B = V with the head dim contiguous (MN-major).  The
          // softmax warps hand P over in two halves: the products over the first 64 keys run while the
          // exponentials of the last 64 are still being computed.
          if (!mbar_wait(p_half(tile), j & 1, status, KF_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          if (!mbar_wait(v_full(st), (j >> 1) & 1, status, KF_ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < BLK_N / 32; ++kk)
            tc_mma_f16_ts(o_col(tile), s_col(tile) + kk * 8,
                          umma_desc_sw128(v_smem + st * C::TILE_BYTES + kk * 2048, C::BLOCK_BYTES, 1024), idesc_o,
                          (j | kk) != 0);
          if (!mbar_wait(p_full(tile), j & 1, status, KF_ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = BLK_N / 32; kk < BLK_N / 16; ++kk)
            tc_mma_f16_ts(o_col(tile), s_col(tile) + kk * 8,
                          umma_desc_sw128(v_smem + st * C::TILE_BYTES + kk * 2048, C::BLOCK_BYTES, 1024), idesc_o, 1u);
          tc_commit(pv_done(tile));
          if (j + 1 == n_of[tile]) tc_commit(o_final(tile));  // a phase of its own: cannot be mistaken for an earlier tile
          // the next score tile of this query tile follows at once (its buffer's P was read by the MMAs just issued)
          if (j + 1 < n_of[tile]) {
            if (!k_next_ready) {
              if (!mbar_wait(k_full((j + 1) & 1), ((j + 1) >> 1) & 1, status, KF_ERR_WAIT_FULL)) { ok = false; break; }
              tc_fence_after();
              k_next_ready = true;
            }
            issue_s(tile, j + 1);
          }
        }
        if (ok) {
          tc_commit(v_empty(st));                               // V_j read by both query tiles
          if (j + 1 < n_max) tc_commit(k_empty((j + 1) & 1));   // K_{j+1} read by every S that needs it
        }
      }
      if (!ok) {
        tc_commit(drain_bar);
        mbar_wait(drain_bar, 0, status, KF_ERR_WAIT_DRAIN);
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue: warps 2-5 tile A, 6-9 tile B
    const int tile = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int r_local = quarter * 32 + lane;
    const int t0 = m0 + tile * BLK_M;          // first query row of this tile
    const int row = t0 + r_local;
    const int n_tiles = tile == 0 ? n_a : n_b;
    const uint32_t lane_off = uint32_t(quarter * 32) << 16;
    const uint32_t t_s = s_col(tile) + lane_off;
    const uint32_t t_o = o_col(tile) + lane_off;
    const float NEG_INF = -INFINITY;
    float m_run = NEG_INF, l_run = 0.f;
    int doc_q = 0;
    if (HAS_DOC) doc_q = row < Sq ? doc_ids[size_t(b) * Sq + row] : -1;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int n0 = j * BLK_N;
      const int* dk = nullptr;
      if (HAS_DOC) {
        int* buf = doc_smem + tile * 256 + (j & 1) * BLK_N;
        const int kpos = n0 + r_local;
        buf[r_local] = kpos < Sk ? doc_ids[size_t(b) * Sk + kpos] : -2;
        tile_group_sync(tile);
        dk = buf;
      }
      const bool tile_masked = HAS_DOC || (CAUSAL && n0 + BLK_N - 1 > t0) || (n0 + BLK_N > Sk);
      if (ok && !mbar_wait(s_full(tile), j & 1, status, KF_ERR_WAIT_TMEM_FULL)) ok = false;
      tc_fence_after();
      uint32_t sv[BLK_N];
#pragma unroll
      for (int c = 0; c < BLK_N / 32; ++c) tmem_ld_32x32_at(t_s + c * 32, sv + c * 32);
      tmem_ld_wait();
      if (tile_masked) {
#pragma unroll
        for (int i = 0; i < BLK_N; ++i) {
          const int col = n0 + i;
          bool vis = col < Sk;
          if (CAUSAL) vis = vis && col <= row;
          if (HAS_DOC) vis = vis && dk[i] == doc_q;
          sv[i] = vis ? sv[i] : __float_as_uint(NEG_INF);
        }
      }
      float mx;
      {
        float mx4[4] = {NEG_INF, NEG_INF, NEG_INF, NEG_INF};
#pragma unroll
        for (int i = 0; i < BLK_N; i += 8)
#pragma unroll
          for (int q = 0; q < 4; ++q)
            mx4[q] = fmax3(mx4[q], __uint_as_float(sv[i + 2 * q]), __uint_as_float(sv[i + 2 * q + 1]));
        mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      }
      const float m_new = fmaxf(m_run, mx * scale_log2);
      const bool grow = m_new > m_run + RESCALE_THRESHOLD;
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? (m_run == NEG_INF ? 0.f : fast_exp2(m_run - m_new)) : 1.f;
        if (j > 0) {
          if (ok && !mbar_wait(pv_done(tile), (j - 1) & 1, status, KF_ERR_WAIT_TMEM_FULL)) ok = false;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32_at(t_o + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(t_o + c * 32, o);
          }
        }
        if (grow) {
          l_run *= alpha;
          m_run = m_new;
        }
      }
      const float m_use = m_run == NEG_INF ? 0.f : m_run;
      const uint64_t scale2 = pack2(scale_log2, scale_log2);
      const uint64_t neg_m2 = pack2(-m_use, -m_use);
      uint64_t lsum[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
      for (int c = 0; c < BLK_N / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const uint64_t x2 = ffma2(pack2(__uint_as_float(sv[c * 32 + 2 * i]), __uint_as_float(sv[c * 32 + 2 * i + 1])),
                                    scale2, neg_m2);
          float x0, x1, e0, e1;
          unpack2(x2, x0, x1);
          if (POLY > 0 && ((i * POLY) & 15) < POLY) {
            exp2_poly2(x0, x1, e0, e1);
          } else {
            e0 = fast_exp2(x0);
            e1 = fast_exp2(x1);
          }
          lsum[i & 3] = fadd2(lsum[i & 3], pack2(e0, e1));
          pk[i] = pack_bf16(e0, e1);
        }
        tmem_st_32x16(t_s + c * 16, pk);
        if (c == 1) {  // the first 64 keys are in place: the MMA warp may start O += P V on them
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(p_half(tile));
        }
      }
      {
        float a0, a1;
        unpack2(fadd2(fadd2(lsum[0], lsum[1]), fadd2(lsum[2], lsum[3])), a0, a1);
        l_run += a0 + a1;
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full(tile));
    }
    if (n_tiles > 0) {
      if (ok && !mbar_wait(o_final(tile), 0, status, KF_ERR_WAIT_TMEM_FULL)) ok = false;
      if (ok) {
        tc_fence_after();
        const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
        __nv_bfloat16* o_row = O + (size_t(b) * Sq + row) * ldo + size_t(h) * HD;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32_at(t_o + c * 32, o);
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
        if (row < Sq)
          LSE[(size_t(b) * H + h) * Sq + row] = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : NEG_INF;
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

template <int HD, bool CAUSAL, bool HAS_DOC, int POLY = 0>
static int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* O, float* LSE, const int* doc,
                  int B, int Sq, int Sk, int H, int Hkv, long long ldo, float scale, int* status, cudaStream_t stream) {
  auto kern = kf_attn_fwd2_tcgen05<HD, CAUSAL, HAS_DOC, POLY>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<HD>::SMEM);
    if (e != cudaSuccess) return 300 + (int)e;
    attr_set = true;
  }
  const int n_super = (Sq + 2 * BLK_M - 1) / (2 * BLK_M);
  dim3 grid((unsigned)(n_super * H * B));
  kern<<<grid, THREADS, Cfg<HD>::SMEM, stream>>>(mq, mk, mv, reinterpret_cast<__nv_bfloat16*>(O), LSE, doc, Sq, Sk, H,
                                                 H / Hkv, ldo, scale * 1.4426950408889634f, status, n_super, B);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // namespace attn2
}  // namespace kf

extern "C" void* kf_status_device_ptr();

extern "C" {

// Same contract as kf_attn_fwd_bf16 (attention_tcgen05.cu); two query tiles per CTA.
int kf_attn_fwd2_bf16(const void* q, const void* k, const void* v, void* o, void* lse, const void* doc, int B, int Sq,
                      int Sk, int H, int Hkv, int hd, long long ldq, long long ldk, long long ldv, long long ldo,
                      float scale, int causal, void* stream) {
  using namespace kf;
  using namespace kf::attn2;
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
#define KF_ATTN2_LAUNCH(HD_, C_, D_) return launch<HD_, C_, D_>(mq, mk, mv, o, L, D, B, Sq, Sk, H, Hkv, ldo, scale, status, st)
#define KF_ATTN2_POLY(C_, P_) return launch<128, C_, false, P_>(mq, mk, mv, o, L, D, B, Sq, Sk, H, Hkv, ldo, scale, status, st)
  if (hd == 128 && !doc) {
    // share of the exponentials on the FMA pipe (of 16): KF_ATTN_EXP_POLY = 0 (default), 4, 6 or 8.  On the 8B
    // shape the variants measured 0.307 / 0.313 / 0.313 / 0.320 ms: the two-tile kernel is paced by the per-tile
    // softmax -> MMA chain, not by the special-function unit, so the extra FMA-pipe instructions do not pay here.
    static int poly = -1;
    if (poly < 0) {
      const char* e = getenv("KF_ATTN_EXP_POLY");
      poly = e ? atoi(e) : 0;
    }
    if (causal) {
      if (poly == 4) KF_ATTN2_POLY(true, 4);
      if (poly == 6) KF_ATTN2_POLY(true, 6);
      if (poly == 8) KF_ATTN2_POLY(true, 8);
    } else {
      if (poly == 4) KF_ATTN2_POLY(false, 4);
      if (poly == 6) KF_ATTN2_POLY(false, 6);
      if (poly == 8) KF_ATTN2_POLY(false, 8);
    }
  }
  if (hd == 128) {
    if (doc) { if (causal) KF_ATTN2_LAUNCH(128, true, true); else KF_ATTN2_LAUNCH(128, false, true); }
    if (causal) KF_ATTN2_LAUNCH(128, true, false); else KF_ATTN2_LAUNCH(128, false, false);
  } else {
    if (doc) { if (causal) KF_ATTN2_LAUNCH(64, true, true); else KF_ATTN2_LAUNCH(64, false, true); }
    if (causal) KF_ATTN2_LAUNCH(64, true, false); else KF_ATTN2_LAUNCH(64, false, false);
  }
#undef KF_ATTN2_LAUNCH
#undef KF_ATTN2_POLY
}

}  // extern "C"
