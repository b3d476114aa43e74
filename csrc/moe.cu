// Mixture-of-experts routing and token movement, all on the device (no host reads):
//
//   kf_router_topk      one warp per token: softmax or sigmoid(+bias) over the expert logits, top-k by repeated
//                       warp arg-max, renormalised weights, per-expert token counts, per-expert probability sums
//                       (load-balancing loss) and the sum of logsumexp^2 (router z-loss) in one pass.
//   kf_moe_sort_*       stable counting sort of the (token, k) assignments by expert: per-block histograms,
//                       a scan, then ranks -> `row_of_slot` (destination row of every assignment),
//                       `slot_of_row` (its inverse) and the expert offsets the grouped GEMM consumes.
//   kf_moe_gather       expert-sorted activation rows from token rows.
//   kf_moe_combine      out[token] = sum_j weight[token, j] * y_sorted[row_of_slot[token, j]]  (+ gradients).
//
// Replaces softmax / topk / one_hot / argsort / bincount(.tolist()) / index_select / scatter_add_ call chains of
// the reference (kempnerforge/model/router.py:45-72,157-200, kempnerforge/model/moe.py:148-185,273-325).
#include "common.cuh"

namespace kf {
namespace moe {

constexpr int MAX_E_PER_LANE = 8;  // experts <= 256
constexpr int MAX_K = 8;

// ------------------------------------------------------------------ router
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T, bool SIGMOID>
__global__ void __launch_bounds__(256)
kf_router_topk(const T* __restrict__ logits, const float* __restrict__ bias, int tokens, int E, int k,
               long long* __restrict__ idx_out, float* __restrict__ w_out, float* __restrict__ counts,
               float* __restrict__ prob_sum, float* __restrict__ lse_sq_sum) {
  extern __shared__ float sh[];  // [E] probability sums of this block, [E] counts
  float* sh_prob = sh;
  float* sh_cnt = sh + E;
  for (int i = threadIdx.x; i < 2 * E; i += blockDim.x) sh[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  float zacc = 0.f;
  for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < tokens; t += gridDim.x * warps_per_block) {
    float raw[MAX_E_PER_LANE], score[MAX_E_PER_LANE], sel[MAX_E_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      raw[j] = e < E ? to_f<T>(logits[size_t(t) * E + e]) : -INFINITY;
      mx = fmaxf(mx, raw[j]);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float se = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) se += (lane + 32 * j) < E ? __expf(raw[j] - mx) : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
    const float lse = mx + __logf(se);
    if (lane == 0) zacc += lse * lse;
#pragma unroll
    for (int j = 0; j < MAX_E_PER_LANE; ++j) {
      const int e = lane + 32 * j;
      if (e < E) {
        if (SIGMOID) {
          score[j] = 1.f / (1.f + __expf(-(raw[j] + (bias ? bias[e] : 0.f))));
        } else {
          score[j] = __expf(raw[j] - mx) / se;
        }
        atomicAdd(&sh_prob[e], score[j]);
        sel[j] = score[j];
      } else {
        score[j] = 0.f;
        sel[j] = -INFINITY;
      }
    }
    // top-k: k rounds of warp arg-max (ties: the lower expert index wins, as torch.topk does for sorted input)
    float wsel[MAX_K];
    int isel[MAX_K];
    float wsum = 0.f;
#pragma unroll
    for (int r = 0; r < MAX_K; ++r) {
      if (r < k) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < MAX_E_PER_LANE; ++j) {
          const int e = lane + 32 * j;
          if (sel[j] > bv) { bv = sel[j]; bi = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
          if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        wsel[r] = bv;
        isel[r] = bi;
        wsum += bv;
#pragma unroll
        for (int j = 0; j < MAX_E_PER_LANE; ++j)
          if (lane + 32 * j == bi) sel[j] = -INFINITY;
      }
    }
    if (lane == 0) {
      const float inv = 1.f / wsum;
#pragma unroll
      for (int r = 0; r < MAX_K; ++r) {
        if (r < k) {
          idx_out[size_t(t) * k + r] = isel[r];
          w_out[size_t(t) * k + r] = wsel[r] * inv;
          atomicAdd(&sh_cnt[isel[r]], 1.f);
        }
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    if (sh_prob[e] != 0.f) atomicAdd(&prob_sum[e], sh_prob[e]);
    if (sh_cnt[e] != 0.f) atomicAdd(&counts[e], sh_cnt[e]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) zacc += __shfl_xor_sync(0xffffffffu, zacc, o);
  if (lane == 0 && zacc != 0.f) atomicAdd(lse_sq_sum, zacc);
}

// ------------------------------------------------------------------ stable counting sort by expert
constexpr int SORT_BLOCK = 256;

__global__ void __launch_bounds__(SORT_BLOCK)
kf_moe_sort_hist(const long long* __restrict__ expert_of_slot, int slots, int E, int* __restrict__ block_hist) {
  extern __shared__ int h[];
  for (int i = threadIdx.x; i < E; i += blockDim.x) h[i] = 0;
  __syncthreads();
  const int s = blockIdx.x * SORT_BLOCK + threadIdx.x;
  if (s < slots) atomicAdd(&h[(int)expert_of_slot[s]], 1);
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) block_hist[size_t(blockIdx.x) * E + i] = h[i];
}

// one block: offsets[e] (exclusive scan of the expert totals) and, in place, block_hist[b][e] -> first
// destination row of block b's assignments to expert e
__global__ void __launch_bounds__(256)
kf_moe_sort_scan(int* __restrict__ block_hist, int n_blocks, int E, int* __restrict__ offsets) {
  __shared__ int total[256];
  const int e = threadIdx.x;
  int sum = 0;
  if (e < E)
    for (int b = 0; b < n_blocks; ++b) {
      const int v = block_hist[size_t(b) * E + e];
      block_hist[size_t(b) * E + e] = sum;
      sum += v;
    }
  total[e] = e < E ? sum : 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < E; ++i) {
      const int v = total[i];
      total[i] = acc;
      offsets[i] = acc;
      acc += v;
    }
    offsets[E] = acc;
  }
  __syncthreads();
  if (e < E)
    for (int b = 0; b < n_blocks; ++b) block_hist[size_t(b) * E + e] += total[e];
}

__global__ void __launch_bounds__(SORT_BLOCK)
kf_moe_sort_place(const long long* __restrict__ expert_of_slot, int slots, int E, const int* __restrict__ block_base,
                  int* __restrict__ row_of_slot, int* __restrict__ slot_of_row) {
  __shared__ int ex[SORT_BLOCK];
  const int s = blockIdx.x * SORT_BLOCK + threadIdx.x;
  const int mine = s < slots ? (int)expert_of_slot[s] : -1;
  ex[threadIdx.x] = mine;
  __syncthreads();
  if (mine < 0) return;
  int rank = 0;  // assignments to the same expert earlier in this block (keeps the sort stable)
  for (int i = 0; i < threadIdx.x; ++i) rank += ex[i] == mine;
  const int row = block_base[size_t(blockIdx.x) * E + mine] + rank;
  row_of_slot[s] = row;
  slot_of_row[row] = s;
}

// ------------------------------------------------------------------ gather / combine
// dst[row] = src[slot_of_row[row] / k]   (rows of `cols` bf16, cols % 8 == 0)
__global__ void kf_moe_gather(const __nv_bfloat16* __restrict__ src, const int* __restrict__ slot_of_row, int rows, int k,
                              int cols, __nv_bfloat16* __restrict__ dst) {
  const int vec = cols / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)rows * vec;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = i / vec, c = (i - (long long)r * vec) * 8;
    const int tok = slot_of_row[r] / k;
    *reinterpret_cast<uint4*>(dst + size_t(r) * cols + c) = *reinterpret_cast<const uint4*>(src + size_t(tok) * cols + c);
  }
}

// out[t] = sum_j w[t, j] * y[row_of_slot[t * k + j]]   (w == nullptr: plain sum, the gradient of the gather)
__global__ void kf_moe_combine(const __nv_bfloat16* __restrict__ y, const int* __restrict__ row_of_slot,
                               const float* __restrict__ w, int tokens, int k, int cols, __nv_bfloat16* __restrict__ out) {
  const int vec = cols / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < (long long)tokens * vec;
       i += (long long)gridDim.x * blockDim.x) {
    const int t = i / vec, c = (i - (long long)t * vec) * 8;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int row = row_of_slot[size_t(t) * k + j];
      const float wj = w ? w[size_t(t) * k + j] : 1.f;
      const uint4 v = *reinterpret_cast<const uint4*>(y + size_t(row) * cols + c);
      const float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), cc = unpack_bf16(v.z), d = unpack_bf16(v.w);
      acc[0] += wj * a.x; acc[1] += wj * a.y; acc[2] += wj * b.x; acc[3] += wj * b.y;
      acc[4] += wj * cc.x; acc[5] += wj * cc.y; acc[6] += wj * d.x; acc[7] += wj * d.y;
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + size_t(t) * cols + c) = o;
  }
}

// backward of the combine, one warp per sorted row: dy[row] = w[slot] * dout[token],  dw[slot] = <dout[token], y[row]>
__global__ void kf_moe_combine_bwd(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                                   const int* __restrict__ slot_of_row, const float* __restrict__ w, int rows, int k, int cols,
                                   __nv_bfloat16* __restrict__ dy, float* __restrict__ dw) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
    const int slot = slot_of_row[r];
    const int tok = slot / k;
    const float ws = w[slot];
    float dot = 0.f;
    for (int c = lane * 8; c < cols; c += 256) {
      const uint4 g = *reinterpret_cast<const uint4*>(dout + size_t(tok) * cols + c);
      const uint4 v = *reinterpret_cast<const uint4*>(y + size_t(r) * cols + c);
      const float2 g0 = unpack_bf16(g.x), g1 = unpack_bf16(g.y), g2 = unpack_bf16(g.z), g3 = unpack_bf16(g.w);
      const float2 v0 = unpack_bf16(v.x), v1 = unpack_bf16(v.y), v2 = unpack_bf16(v.z), v3 = unpack_bf16(v.w);
      dot += g0.x * v0.x + g0.y * v0.y + g1.x * v1.x + g1.y * v1.y + g2.x * v2.x + g2.y * v2.y + g3.x * v3.x + g3.y * v3.y;
      uint4 o;
      o.x = pack_bf16(ws * g0.x, ws * g0.y); o.y = pack_bf16(ws * g1.x, ws * g1.y);
      o.z = pack_bf16(ws * g2.x, ws * g2.y); o.w = pack_bf16(ws * g3.x, ws * g3.y);
      *reinterpret_cast<uint4*>(dy + size_t(r) * cols + c) = o;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    if (lane == 0) dw[slot] = dot;
  }
}

}  // namespace moe
}  // namespace kf

extern "C" {

// logits [tokens][E] (dt 0 = bf16, 1 = fp32); bias fp32 [E] or null (sigmoid mode); outputs: idx int64 [tokens][k],
// w fp32 [tokens][k] (renormalised), and ACCUMULATED into: counts fp32 [E], prob_sum fp32 [E], lse_sq_sum fp32 [1]
// (zero them first).  E <= 256, k <= 8.
int kf_router_topk(const void* logits, int dt, const void* bias, int sigmoid, int tokens, int E, int k, void* idx, void* w,
                   void* counts, void* prob_sum, void* lse_sq_sum, void* stream) {
  using namespace kf::moe;
  if (E < 1 || E > 32 * MAX_E_PER_LANE || k < 1 || k > MAX_K || k > E) return 3;
  if (tokens <= 0) return 0;
  const int threads = 256, wpb = threads / 32;
  int blocks = (tokens + wpb - 1) / wpb;
  if (blocks > 1184) blocks = 1184;
  const size_t sh = 2 * size_t(E) * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
#define KF_ROUTER(T_, S_)                                                                                              \
  kf_router_topk<T_, S_><<<blocks, threads, sh, st>>>(reinterpret_cast<const T_*>(logits),                              \
                                                      reinterpret_cast<const float*>(bias), tokens, E, k,               \
                                                      reinterpret_cast<long long*>(idx), reinterpret_cast<float*>(w),   \
                                                      reinterpret_cast<float*>(counts), reinterpret_cast<float*>(prob_sum), \
                                                      reinterpret_cast<float*>(lse_sq_sum))
  if (dt == 0) {
    if (sigmoid) KF_ROUTER(__nv_bfloat16, true); else KF_ROUTER(__nv_bfloat16, false);
  } else {
    if (sigmoid) KF_ROUTER(float, true); else KF_ROUTER(float, false);
  }
#undef KF_ROUTER
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// Stable sort of `slots` assignments by expert.  scratch: int32 [ceil(slots / 256) * E].  Outputs: offsets int32
// [E + 1], row_of_slot int32 [slots], slot_of_row int32 [slots].
int kf_moe_sort(const void* expert_of_slot, int slots, int E, void* scratch, void* offsets, void* row_of_slot,
                void* slot_of_row, void* stream) {
  using namespace kf::moe;
  if (E < 1 || E > 256) return 3;
  cudaStream_t st = (cudaStream_t)stream;
  const int nb = (slots + SORT_BLOCK - 1) / SORT_BLOCK;
  if (nb == 0) {
    cudaMemsetAsync(offsets, 0, (E + 1) * sizeof(int), st);
    return 0;
  }
  auto ex = reinterpret_cast<const long long*>(expert_of_slot);
  kf_moe_sort_hist<<<nb, SORT_BLOCK, E * sizeof(int), st>>>(ex, slots, E, reinterpret_cast<int*>(scratch));
  kf_moe_sort_scan<<<1, 256, 0, st>>>(reinterpret_cast<int*>(scratch), nb, E, reinterpret_cast<int*>(offsets));
  kf_moe_sort_place<<<nb, SORT_BLOCK, 0, st>>>(ex, slots, E, reinterpret_cast<const int*>(scratch),
                                               reinterpret_cast<int*>(row_of_slot), reinterpret_cast<int*>(slot_of_row));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

int kf_moe_gather_bf16(const void* src, const void* slot_of_row, int rows, int k, int cols, void* dst, void* stream) {
  using namespace kf::moe;
  if (cols & 7) return 5;
  if (rows <= 0) return 0;
  long long work = (long long)rows * (cols / 8);
  int blocks = (int)((work + 255) / 256 < 2368 ? (work + 255) / 256 : 2368);
  kf_moe_gather<<<blocks, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const __nv_bfloat16*>(src),
                                                        reinterpret_cast<const int*>(slot_of_row), rows, k, cols,
                                                        reinterpret_cast<__nv_bfloat16*>(dst));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

int kf_moe_combine_bf16(const void* y, const void* row_of_slot, const void* w, int tokens, int k, int cols, void* out,
                        void* stream) {
  using namespace kf::moe;
  if (cols & 7) return 5;
  if (tokens <= 0) return 0;
  long long work = (long long)tokens * (cols / 8);
  int blocks = (int)((work + 255) / 256 < 2368 ? (work + 255) / 256 : 2368);
  kf_moe_combine<<<blocks, 256, 0, (cudaStream_t)stream>>>(reinterpret_cast<const __nv_bfloat16*>(y),
                                                         reinterpret_cast<const int*>(row_of_slot),
                                                         reinterpret_cast<const float*>(w), tokens, k, cols,
                                                         reinterpret_cast<__nv_bfloat16*>(out));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

int kf_moe_combine_bwd_bf16(const void* dout, const void* y, const void* slot_of_row, const void* w, int rows, int k,
                            int cols, void* dy, void* dw, void* stream) {
  using namespace kf::moe;
  if (cols & 7) return 5;
  if (rows <= 0) return 0;
  int blocks = (rows + 7) / 8 < 2368 ? (rows + 7) / 8 : 2368;
  kf_moe_combine_bwd<<<blocks, 256, 0, (cudaStream_t)stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(dout), reinterpret_cast<const __nv_bfloat16*>(y),
      reinterpret_cast<const int*>(slot_of_row), reinterpret_cast<const float*>(w), rows, k, cols,
      reinterpret_cast<__nv_bfloat16*>(dy), reinterpret_cast<float*>(dw));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // extern "C"

// ==================================================================== expert-parallel dispatch over peer memory
// Rows travel between the ranks of an expert-parallel group with plain peer stores (NVLink / NVSwitch); no
// library all-to-all, no host-side split sizes.
//
//   kf_ep_put      source side.  Rows sorted by GLOBAL expert (optionally gathered from token rows on the fly) are
//                  stored into the destination rank's receive window [source][cap][cols]; the per-expert counts
//                  and the source's base row of that destination are stored into the destination's table.
//   kf_ep_layout   destination side, one block: from the count table build the expert-major layout
//                  (offsets per local expert, first compact row of every (source, expert) chunk).
//   kf_ep_compact  destination side: windows -> expert-major rows (the A operand of the grouped GEMM).
//   kf_ep_return   destination side: expert-major rows -> the SOURCE's return buffer, at the row the source had
//                  them in its own sorted order.
// Between put and layout, and between return and the source's use of its return buffer, the ranks meet in a
// bounded symmetric-memory barrier on the stream (host side).  Replaces the count / token / expert-id / combine
// all-to-alls and their three host synchronisations (kempnerforge/distributed/expert_parallel.py:93-309).
namespace kf {
namespace ep {

constexpr int MAX_PEERS = 8;
struct Peers {
  void* p[MAX_PEERS];
};

// table layout on every rank, per source s: [n_local counts][1 base row] -> stride n_local + 1 ints
__global__ void kf_ep_put(const __nv_bfloat16* __restrict__ src, const int* __restrict__ slot_of_row, int k,
                          const int* __restrict__ offsets_g, int n_local, int ep, int me, int cols, long long cap,
                          Peers windows, Peers tables) {
  const int total = offsets_g[ep * n_local];
  // counts and base rows (a few ints per destination)
  if (blockIdx.x == 0) {
    for (int i = threadIdx.x; i < ep * (n_local + 1); i += blockDim.x) {
      const int d = i / (n_local + 1), j = i - d * (n_local + 1);
      int* tab = reinterpret_cast<int*>(tables.p[d]) + me * (n_local + 1);
      tab[j] = j < n_local ? offsets_g[d * n_local + j + 1] - offsets_g[d * n_local + j] : offsets_g[d * n_local];
    }
  }
  const int vec = cols / 8;
  const int lane_vecs = blockDim.x;
  for (int r = blockIdx.x; r < total; r += gridDim.x) {
    // destination rank: the one whose expert range contains sorted row r
    int d = 0;
    while (d + 1 < ep && offsets_g[(d + 1) * n_local] <= r) ++d;
    const int pos = r - offsets_g[d * n_local];
    const int srow = slot_of_row ? slot_of_row[r] / k : r;
    const __nv_bfloat16* s = src + size_t(srow) * cols;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(windows.p[d]) + (size_t(me) * cap + pos) * cols;
    for (int c = threadIdx.x; c < vec; c += lane_vecs)
      *reinterpret_cast<uint4*>(dst + c * 8) = *reinterpret_cast<const uint4*>(s + c * 8);
  }
}

// outputs: offsets_l int32 [n_local + 1]; chunk_dst int32 [ep][n_local] (first compact row of chunk (s, j));
// chunk_src int32 [ep][n_local] (first window row of chunk (s, j)); total_rows int32 [1]
__global__ void kf_ep_layout(const int* __restrict__ table, int ep, int n_local, int* __restrict__ offsets_l,
                             int* __restrict__ chunk_dst, int* __restrict__ chunk_src, int* __restrict__ total_rows) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int acc = 0;
  for (int j = 0; j < n_local; ++j) {
    offsets_l[j] = acc;
    for (int s = 0; s < ep; ++s) {
      chunk_dst[s * n_local + j] = acc;
      acc += table[s * (n_local + 1) + j];
    }
  }
  offsets_l[n_local] = acc;
  total_rows[0] = acc;
  for (int s = 0; s < ep; ++s) {
    int w = 0;
    for (int j = 0; j < n_local; ++j) {
      chunk_src[s * n_local + j] = w;
      w += table[s * (n_local + 1) + j];
    }
  }
}

// one block per (chunk, row slice): copies window rows of chunk (s, j) to their compact position (to_compact = 1)
// or compact rows back into a peer's return buffer at the source's own sorted row (to_compact = 0)
__global__ void kf_ep_move(const __nv_bfloat16* __restrict__ window, __nv_bfloat16* __restrict__ compact,
                           const int* __restrict__ table, const int* __restrict__ chunk_dst,
                           const int* __restrict__ chunk_src, int ep, int n_local, int cols, long long cap, int to_compact,
                           int my_local_start, Peers returns) {
  const int chunk = blockIdx.y;
  const int s = chunk / n_local, j = chunk - s * n_local;
  const int count = table[s * (n_local + 1) + j];
  const int base_in_source = table[s * (n_local + 1) + n_local];  // source's sorted row of its first row for this rank
  const int vec = cols / 8;
  for (int r = blockIdx.x; r < count; r += gridDim.x) {
    const size_t crow = size_t(chunk_dst[chunk]) + r;
    const int wrow = chunk_src[chunk] + r;
    if (to_compact) {
      const __nv_bfloat16* src = window + (size_t(s) * cap + wrow) * cols;
      __nv_bfloat16* dst = compact + crow * cols;
      for (int c = threadIdx.x; c < vec; c += blockDim.x)
        *reinterpret_cast<uint4*>(dst + c * 8) = *reinterpret_cast<const uint4*>(src + c * 8);
    } else {
      const __nv_bfloat16* src = compact + crow * cols;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(returns.p[s]) + (size_t(base_in_source) + wrow) * cols;
      for (int c = threadIdx.x; c < vec; c += blockDim.x)
        *reinterpret_cast<uint4*>(dst + c * 8) = *reinterpret_cast<const uint4*>(src + c * 8);
    }
  }
}

}  // namespace ep
}  // namespace kf

extern "C" {

// Source side of the dispatch.  src: token rows (slot_of_row given: row r comes from token slot_of_row[r] / k) or
// rows already in sorted order (slot_of_row null).  offsets_g: int32 [ep * n_local + 1] of the global-expert sort.
// window_ptrs / table_ptrs: ep device addresses each (every rank's receive windows [ep][cap][cols] bf16 and count
// table [ep][n_local + 1] int32).  max_rows: upper bound of the number of sorted rows (grid sizing only).
int kf_ep_put_bf16(const void* src, const void* slot_of_row, int k, const void* offsets_g, int n_local, int ep, int me,
                   int cols, long long cap, const long long* window_ptrs, const long long* table_ptrs, int max_rows,
                   void* stream) {
  using namespace kf::ep;
  if (ep < 1 || ep > MAX_PEERS || (cols & 7)) return 5;
  Peers w, t;
  for (int i = 0; i < MAX_PEERS; ++i) {
    w.p[i] = i < ep ? reinterpret_cast<void*>(window_ptrs[i]) : nullptr;
    t.p[i] = i < ep ? reinterpret_cast<void*>(table_ptrs[i]) : nullptr;
  }
  int blocks = max_rows < 1 ? 1 : (max_rows < 148 * 16 ? max_rows : 148 * 16);
  kf_ep_put<<<blocks, 128, 0, (cudaStream_t)stream>>>(reinterpret_cast<const __nv_bfloat16*>(src),
                                                     reinterpret_cast<const int*>(slot_of_row), k,
                                                     reinterpret_cast<const int*>(offsets_g), n_local, ep, me, cols, cap, w, t);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

int kf_ep_layout(const void* table, int ep, int n_local, void* offsets_l, void* chunk_dst, void* chunk_src,
                 void* total_rows, void* stream) {
  using namespace kf::ep;
  kf_ep_layout<<<1, 32, 0, (cudaStream_t)stream>>>(reinterpret_cast<const int*>(table), ep, n_local,
                                                  reinterpret_cast<int*>(offsets_l), reinterpret_cast<int*>(chunk_dst),
                                                  reinterpret_cast<int*>(chunk_src), reinterpret_cast<int*>(total_rows));
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// to_compact = 1: windows -> compact (local copy).  to_compact = 0: compact -> the sources' return buffers
// (return_ptrs: ep device addresses of every rank's [max sorted rows][cols] bf16 return buffer).
int kf_ep_move_bf16(const void* window, void* compact, const void* table, const void* chunk_dst, const void* chunk_src,
                    int ep, int n_local, int cols, long long cap, int to_compact, const long long* return_ptrs,
                    void* stream) {
  using namespace kf::ep;
  if (ep < 1 || ep > MAX_PEERS || (cols & 7)) return 5;
  Peers r;
  for (int i = 0; i < MAX_PEERS; ++i) r.p[i] = (i < ep && return_ptrs) ? reinterpret_cast<void*>(return_ptrs[i]) : nullptr;
  dim3 grid(64, ep * n_local);
  kf_ep_move<<<grid, 128, 0, (cudaStream_t)stream>>>(reinterpret_cast<const __nv_bfloat16*>(window),
                                                    reinterpret_cast<__nv_bfloat16*>(compact),
                                                    reinterpret_cast<const int*>(table), reinterpret_cast<const int*>(chunk_dst),
                                                    reinterpret_cast<const int*>(chunk_src), ep, n_local, cols, cap, to_compact,
                                                    0, r);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // extern "C"


// ------------------------------------------------------------------ expert capacity
// keep[t, j] = 1 when token t is among the first `cap` tokens (in sequence order) that slot j routes to its expert,
// else 0: the per-(slot, expert) capacity rule of the reference (kempnerforge/model/moe.py:148-185), evaluated on
// the device without data-dependent shapes.  One block per (slot, expert) scans the token column with a block-wide
// prefix count; the result does not depend on scheduling.
namespace kf {
namespace moe {
constexpr int CAP_THREADS = 256;
__global__ void __launch_bounds__(CAP_THREADS)
kf_moe_capacity_mask(const long long* __restrict__ indices, int T, int k, int cap, float* __restrict__ keep) {
  __shared__ int warp_tot[CAP_THREADS / 32];
  __shared__ int base;
  const int j = blockIdx.x % k, e = blockIdx.x / k;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) base = 0;
  __syncthreads();
  for (int t0 = 0; t0 < T; t0 += CAP_THREADS) {
    const int t = t0 + threadIdx.x;
    const bool hit = t < T && indices[size_t(t) * k + j] == e;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    const int before_in_warp = __popc(m & ((1u << lane) - 1u));
    if (lane == 0) warp_tot[warp] = __popc(m);
    __syncthreads();
    int before = base + before_in_warp;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    if (hit) keep[size_t(t) * k + j] = before < cap ? 1.f : 0.f;
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int w = 0; w < CAP_THREADS / 32; ++w) tot += warp_tot[w];
      base += tot;
    }
    __syncthreads();
  }
}
}  // namespace moe
}  // namespace kf

extern "C" int kf_moe_capacity_mask(const void* indices, int T, int k, int E, int cap, void* keep, void* stream) {
  using namespace kf::moe;
  if (T <= 0 || k <= 0 || E <= 0) return 0;
  kf_moe_capacity_mask<<<E * k, CAP_THREADS, 0, (cudaStream_t)stream>>>(reinterpret_cast<const long long*>(indices), T, k,
                                                                         cap, reinterpret_cast<float*>(keep));
  cudaError_t err = cudaGetLastError();
  return err == cudaSuccess ? 0 : 400 + (int)err;
}
