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
