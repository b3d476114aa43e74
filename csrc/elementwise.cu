// Memory-bound kernels of the transformer block and the optimizer: RMSNorm fwd/bwd,
// RoPE, SwiGLU fwd/bwd, embedding gather / scatter-add, fused softmax-cross-entropy
// (forward statistics and logits gradient in one sweep), fused AdamW on flat buffers,
// sum of squares.  All use 16-byte vector accesses, fp32 math and one read of every
// input; none needs shared-memory tiling beyond block reductions.
//
// Reference semantics: kempnerforge/model/norm.py:11-27, model/position.py:43-71,
// model/mlp.py:12-26, model/embedding.py:9-29, training/loss.py:19-102,
// training/optimizer.py:28-39 (torch.optim.AdamW update rule).
#include "common.cuh"

namespace kf {

// ------------------------------------------------------------------ reductions
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide sum; `red` holds >= 33 floats.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nw ? red[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

struct F8 {
  float v[8];
};
__device__ __forceinline__ F8 load8(const __nv_bfloat16* p) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  F8 r;
  float2 a = unpack_bf16(u.x), b = unpack_bf16(u.y), c = unpack_bf16(u.z), d = unpack_bf16(u.w);
  r.v[0] = a.x; r.v[1] = a.y; r.v[2] = b.x; r.v[3] = b.y;
  r.v[4] = c.x; r.v[5] = c.y; r.v[6] = d.x; r.v[7] = d.y;
  return r;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const F8& r) {
  uint4 u;
  u.x = pack_bf16(r.v[0], r.v[1]);
  u.y = pack_bf16(r.v[2], r.v[3]);
  u.z = pack_bf16(r.v[4], r.v[5]);
  u.w = pack_bf16(r.v[6], r.v[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// ------------------------------------------------------------------ RMSNorm
constexpr int NORM_THREADS = 256;
constexpr int NORM_CACHE = 4;  // vectors of 8 kept in registers per thread (covers D <= 8192)

__global__ void __launch_bounds__(NORM_THREADS)
kf_rmsnorm_fwd(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
               __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows, int D, float eps) {
  __shared__ float red[40];
  const int nvec = D >> 3;
  constexpr int CACHED = NORM_CACHE * NORM_THREADS;  // vectors kept in registers per row
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + size_t(row) * D;
    F8 cache[NORM_CACHE];
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < NORM_CACHE; ++c) {
      const int v = threadIdx.x + c * NORM_THREADS;
      if (v < nvec) {
        cache[c] = load8(xr + v * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += cache[c].v[i] * cache[c].v[i];
      }
    }
    for (int v = threadIdx.x + CACHED; v < nvec; v += NORM_THREADS) {
      const F8 t = load8(xr + v * 8);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += t.v[i] * t.v[i];
    }
    const float r = rsqrtf(block_sum(ss, red) / D + eps);
    if (threadIdx.x == 0 && rstd) rstd[row] = r;
    __nv_bfloat16* yr = y + size_t(row) * D;
#pragma unroll
    for (int c = 0; c < NORM_CACHE; ++c) {
      const int v = threadIdx.x + c * NORM_THREADS;
      if (v < nvec) {
        const F8 g = load8(w + v * 8);
        F8 t = cache[c];
#pragma unroll
        for (int i = 0; i < 8; ++i) t.v[i] = t.v[i] * r * g.v[i];
        store8(yr + v * 8, t);
      }
    }
    for (int v = threadIdx.x + CACHED; v < nvec; v += NORM_THREADS) {
      F8 t = load8(xr + v * 8);
      const F8 g = load8(w + v * 8);
#pragma unroll
      for (int i = 0; i < 8; ++i) t.v[i] = t.v[i] * r * g.v[i];
      store8(yr + v * 8, t);
    }
  }
}

// RMSNorm backward in two streaming passes (dw first, so that dx may overwrite dy in place):
//   kf_rmsnorm_bwd_dw   dw partial[chunk][d] = sum over the chunk's rows of dy * x * rstd   (column-parallel, fp32)
//   kf_rmsnorm_bwd_dx   dx = [dx_in +] r*g - x*r^3*mean(g*x) with g = dy*w                   (one block per row)
// Both keep many rows in flight per SM (few registers, no accumulators that live across rows), which is what lets
// them run at memory speed; the earlier single kernel carried the dw accumulators through the row loop and was
// latency bound.  dx_in (optional) is the gradient arriving over the residual connection; it may alias dx.
__global__ void __launch_bounds__(256)
kf_rmsnorm_bwd_dw(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                  const float* __restrict__ rstd, float* __restrict__ partial, int rows, int D, int rows_per_chunk) {
  const int nvec = D >> 3;
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  if (v >= nvec) return;
  const int r0 = blockIdx.y * rows_per_chunk;
  const int r1 = min(rows, r0 + rows_per_chunk);
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  int row = r0;
  for (; row + 4 <= r1; row += 4) {  // four rows in flight per thread
    F8 g[4], a[4];
    float r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      g[u] = load8(dy + size_t(row + u) * D + v * 8);
      a[u] = load8(x + size_t(row + u) * D + v * 8);
      r[u] = rstd[row + u];
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += g[u].v[i] * a[u].v[i] * r[u];
  }
  for (; row < r1; ++row) {
    const F8 g = load8(dy + size_t(row) * D + v * 8), a = load8(x + size_t(row) * D + v * 8);
    const float r = rstd[row];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += g.v[i] * a.v[i] * r;
  }
  float* out = partial + size_t(blockIdx.y) * D + v * 8;
  *reinterpret_cast<float4*>(out) = make_float4(acc[0], acc[1], acc[2], acc[3]);
  *reinterpret_cast<float4*>(out + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

constexpr int BWD_CACHE = 2;  // vectors of 8 per thread kept between the two passes over a row (D <= 4096)

__global__ void __launch_bounds__(NORM_THREADS)
kf_rmsnorm_bwd_dx(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                  const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                  __nv_bfloat16* __restrict__ dx, int rows, int D, const __nv_bfloat16* __restrict__ dx_in) {
  __shared__ float red[40];
  const int nvec = D >> 3;
  constexpr int CACHED = BWD_CACHE * NORM_THREADS;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + size_t(row) * D;
    const __nv_bfloat16* dyr = dy + size_t(row) * D;
    const float r = rstd[row];
    float dot = 0.f;
    F8 xc[BWD_CACHE], gc[BWD_CACHE];  // gc holds dy * w
#pragma unroll
    for (int c = 0; c < BWD_CACHE; ++c) {
      const int v = threadIdx.x + c * NORM_THREADS;
      if (v < nvec) {
        xc[c] = load8(xr + v * 8);
        gc[c] = load8(dyr + v * 8);
        const F8 ww = load8(w + v * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          gc[c].v[i] *= ww.v[i];
          dot += gc[c].v[i] * xc[c].v[i];
        }
      }
    }
    for (int v = threadIdx.x + CACHED; v < nvec; v += NORM_THREADS) {
      const F8 a = load8(xr + v * 8), g = load8(dyr + v * 8), ww = load8(w + v * 8);
#pragma unroll
      for (int i = 0; i < 8; ++i) dot += g.v[i] * ww.v[i] * a.v[i];
    }
    const float coef = block_sum(dot, red) / D * r * r * r;
    __nv_bfloat16* dxr = dx + size_t(row) * D;
    const __nv_bfloat16* dir = dx_in ? dx_in + size_t(row) * D : nullptr;
#pragma unroll
    for (int c = 0; c < BWD_CACHE; ++c) {
      const int v = threadIdx.x + c * NORM_THREADS;
      if (v < nvec) {
        F8 o;
        if (dir) o = load8(dir + v * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float d = r * gc[c].v[i] - xc[c].v[i] * coef;
          o.v[i] = dir ? o.v[i] + d : d;
        }
        store8(dxr + v * 8, o);
      }
    }
    // beyond the register cache: every element is re-read and then written by the same thread, so dx may alias dy
    for (int v = threadIdx.x + CACHED; v < nvec; v += NORM_THREADS) {
      const F8 a = load8(xr + v * 8), g = load8(dyr + v * 8), ww = load8(w + v * 8);
      F8 o;
      if (dir) o = load8(dir + v * 8);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float d = r * g.v[i] * ww.v[i] - a.v[i] * coef;
        o.v[i] = dir ? o.v[i] + d : d;
      }
      store8(dxr + v * 8, o);
    }
  }
}

// dw[d] = sum_b partial[b][d]  (fixed order -> deterministic)
__global__ void kf_colsum_partials(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out_bf16,
                                   float* __restrict__ out_f32, int nblocks, int D) {
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  float s = 0.f;
  for (int b = 0; b < nblocks; ++b) s += partial[size_t(b) * D + d];
  if (out_bf16) out_bf16[d] = __float2bfloat16(s);
  if (out_f32) out_f32[d] = s;
}

// ------------------------------------------------------------------ RoPE (half-split pairs)
// x, y: (B, S, Htot, hd) contiguous.  Heads [0, n_rot) are rotated, the rest copied.
// inverse != 0 applies the transpose rotation (the backward of the forward op).
__global__ void kf_rope(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                        const float* __restrict__ cosT, const float* __restrict__ sinT, long long tokens,
                        int S, int Htot, int n_rot, int hd, int inverse) {
  const int half = hd >> 1;
  const int vec_per_head = half >> 3;  // vectors of 8 in one half
  const long long total = tokens * Htot * vec_per_head;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = idx % vec_per_head;
    const long long th = idx / vec_per_head;
    const int h = th % Htot;
    const long long tok = th / Htot;
    const int pos = tok % S;
    const size_t base = (size_t(tok) * Htot + h) * hd + v * 8;
    F8 a = load8(x + base), b = load8(x + base + half);
    if (h < n_rot) {
      const float* cp = cosT + size_t(pos) * half + v * 8;
      const float* sp = sinT + size_t(pos) * half + v * 8;
      F8 oa, ob;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float c = cp[i], s = inverse ? -sp[i] : sp[i];
        oa.v[i] = a.v[i] * c - b.v[i] * s;
        ob.v[i] = b.v[i] * c + a.v[i] * s;
      }
      a = oa;
      b = ob;
    }
    store8(y + base, a);
    store8(y + base + half, b);
  }
}

// ------------------------------------------------------------------ SwiGLU on stacked [gate | up]
__global__ void kf_swiglu_fwd(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ h,
                              long long rows, int H) {
  const int vec = H >> 3;
  const long long total = rows * vec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / vec;
    const int v = idx % vec;
    const __nv_bfloat16* g = gu + size_t(r) * 2 * H + v * 8;
    F8 a = load8(g), b = load8(g + H), o;
#pragma unroll
    for (int i = 0; i < 8; ++i) o.v[i] = a.v[i] / (1.f + __expf(-a.v[i])) * b.v[i];
    store8(h + size_t(r) * H + v * 8, o);
  }
}

// rows_ptr (optional, device int): only the first min(rows, *rows_ptr) rows are touched (ragged expert activations
// whose buffers are sized by an upper bound known on the host).
__global__ void kf_swiglu_bwd(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ gu,
                              __nv_bfloat16* __restrict__ dgu, long long rows, int H, const int* __restrict__ rows_ptr) {
  const int vec = H >> 3;
  if (rows_ptr) rows = min(rows, (long long)*rows_ptr);
  const long long total = rows * vec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / vec;
    const int v = idx % vec;
    const size_t off = size_t(r) * 2 * H + v * 8;
    F8 a = load8(gu + off), b = load8(gu + off + H), d = load8(dh + size_t(r) * H + v * 8), da, db;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sg = 1.f / (1.f + __expf(-a.v[i]));
      const float silu = a.v[i] * sg;
      db.v[i] = d.v[i] * silu;
      da.v[i] = d.v[i] * b.v[i] * sg * (1.f + a.v[i] * (1.f - sg));
    }
    store8(dgu + off, da);
    store8(dgu + off + H, db);
  }
}

// ------------------------------------------------------------------ embedding
__global__ void kf_embedding_fwd(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, long long tokens, int D, int vocab) {
  const int vec = D >> 3;
  const long long total = tokens * vec;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / vec;
    const int v = idx % vec;
    long long id = ids[t];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    *reinterpret_cast<uint4*>(out + size_t(t) * D + v * 8) =
        *reinterpret_cast<const uint4*>(table + size_t(id) * D + v * 8);
  }
}

// dtable[ids[t]] += dy[t]   (bf16x2 atomics; dtable zeroed by the caller when not accumulating)
__global__ void kf_embedding_bwd(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dy,
                                 __nv_bfloat16* __restrict__ dtable, long long tokens, int D, int vocab) {
  const int pairs = D >> 1;
  const long long total = tokens * pairs;
  for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / pairs;
    const int p = idx % pairs;
    const long long id = ids[t];
    if (id < 0 || id >= vocab) continue;
    const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(dy + size_t(t) * D + p * 2);
    atomicAdd(reinterpret_cast<__nv_bfloat162*>(dtable + size_t(id) * D + p * 2), g);
  }
}

// ------------------------------------------------------------------ softmax cross entropy, fwd + dlogits
// One block per row.  logits are overwritten with d(loss)/d(logits) where
//   loss = inv_n * sum_valid (lse - logit[label]) + z_w * inv_n * sum_valid lse^2.
// row_nll / row_lse2 receive the per-row terms (0 for ignored rows) for a deterministic host-side sum.
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS)
kf_ce_fwd_bwd(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
              float* __restrict__ row_nll, float* __restrict__ row_lse2, const float* __restrict__ inv_n_ptr,
              float z_w, int V, int ld) {
  __shared__ float red[40];
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + size_t(row) * ld;
  const int nvec = V >> 3;
  // pass 1: online max / sum of exponentials
  float mx = -INFINITY, sum = 0.f;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    F8 t = load8(lr + v * 8);
    float m2 = mx;
#pragma unroll
    for (int i = 0; i < 8; ++i) m2 = fmaxf(m2, t.v[i]);
    float s2 = sum * __expf(mx - m2);
#pragma unroll
    for (int i = 0; i < 8; ++i) s2 += __expf(t.v[i] - m2);
    mx = m2;
    sum = s2;
  }
  for (int j = nvec * 8 + threadIdx.x; j < V; j += CE_THREADS) {  // ragged tail
    const float t = __bfloat162float(lr[j]);
    const float m2 = fmaxf(mx, t);
    sum = sum * __expf(mx - m2) + __expf(t - m2);
    mx = m2;
  }
  const float gmax = block_max(mx, red);
  const float gsum = block_sum(mx == -INFINITY ? 0.f : sum * __expf(mx - gmax), red);
  const float lse = gmax + __logf(gsum);
  const long long label = labels[row];
  const bool valid = label >= 0 && label < V;
  const float inv_n = *inv_n_ptr;
  if (threadIdx.x == 0) {
    const float picked = valid ? __bfloat162float(lr[label]) : 0.f;
    row_nll[row] = valid ? lse - picked : 0.f;
    row_lse2[row] = valid ? lse * lse : 0.f;
  }
  __syncthreads();  // the label logit was read before anyone overwrites it
  // pass 2: gradient
  const float gscale = valid ? inv_n * (1.f + 2.f * z_w * lse) : 0.f;
  const float onehot = valid ? inv_n : 0.f;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    F8 t = load8(lr + v * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float g = __expf(t.v[i] - lse) * gscale;
      if (v * 8 + i == label) g -= onehot;
      t.v[i] = g;
    }
    store8(lr + v * 8, t);
  }
  for (int j = nvec * 8 + threadIdx.x; j < V; j += CE_THREADS) {
    float g = __expf(__bfloat162float(lr[j]) - lse) * gscale;
    if (j == label) g -= onehot;
    lr[j] = __float2bfloat16(g);
  }
}

// ------------------------------------------------------------------ vocabulary-parallel cross entropy
// The vocabulary dimension of the logits is sharded over the tensor-parallel ranks (this rank holds columns
// [vocab_start, vocab_start + V)).  Phase 1 produces, per row, the local maximum, the local sum of exponentials
// relative to that maximum and the logit of the label when the label lives on this rank; the ranks then exchange
// those three numbers per row (one MAX and one SUM all-reduce of (T,) vectors) and phase 2 turns the logits into
// their gradient in place, given the global log-sum-exp.  No (T, V) temporary, no host read.
__global__ void __launch_bounds__(CE_THREADS)
kf_ce_vp_stats(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels, long long vocab_start,
               float* __restrict__ row_max, float* __restrict__ row_sum, float* __restrict__ row_picked, int V, int ld) {
  __shared__ float red[40];
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + size_t(row) * ld;
  const int nvec = V >> 3;
  float mx = -INFINITY, sum = 0.f;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    F8 t = load8(lr + v * 8);
    float m2 = mx;
#pragma unroll
    for (int i = 0; i < 8; ++i) m2 = fmaxf(m2, t.v[i]);
    float s2 = sum * __expf(mx - m2);
#pragma unroll
    for (int i = 0; i < 8; ++i) s2 += __expf(t.v[i] - m2);
    mx = m2;
    sum = s2;
  }
  for (int j = nvec * 8 + threadIdx.x; j < V; j += CE_THREADS) {
    const float t = __bfloat162float(lr[j]);
    const float m2 = fmaxf(mx, t);
    sum = sum * __expf(mx - m2) + __expf(t - m2);
    mx = m2;
  }
  const float gmax = block_max(mx, red);
  const float gsum = block_sum(mx == -INFINITY ? 0.f : sum * __expf(mx - gmax), red);
  if (threadIdx.x == 0) {
    const long long local = labels[row] - vocab_start;
    row_max[row] = gmax;
    row_sum[row] = gsum;
    row_picked[row] = (local >= 0 && local < V) ? __bfloat162float(lr[local]) : 0.f;
  }
}

// logits <- d loss / d logits = upstream * inv_n * (softmax * (1 + 2 z lse) - onehot) for rows with a valid label.
__global__ void __launch_bounds__(CE_THREADS)
kf_ce_vp_bwd(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels, long long vocab_start,
             const float* __restrict__ lse_rows, const float* __restrict__ inv_n_ptr, const float* __restrict__ upstream,
             float z_w, int V, int ld) {
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + size_t(row) * ld;
  const long long label = labels[row];
  const bool valid = label >= 0;
  const long long local = label - vocab_start;
  const float lse = lse_rows[row];
  const float scale = valid ? (*inv_n_ptr) * (upstream ? *upstream : 1.f) : 0.f;
  const float gscale = scale * (1.f + 2.f * z_w * lse);
  const int nvec = V >> 3;
  for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
    F8 t = load8(lr + v * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float g = __expf(t.v[i] - lse) * gscale;
      if (v * 8 + i == local) g -= scale;
      t.v[i] = g;
    }
    store8(lr + v * 8, t);
  }
  for (int j = nvec * 8 + threadIdx.x; j < V; j += CE_THREADS) {
    float g = __expf(__bfloat162float(lr[j]) - lse) * gscale;
    if (j == local) g -= scale;
    lr[j] = __float2bfloat16(g);
  }
}

// ------------------------------------------------------------------ fused AdamW on flat buffers
template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16(v); }

// Elements [0, n_decay) get weight decay `wd`, the rest none.  grad_scale (device scalar, may be
// null) multiplies every gradient (gradient clipping).  skip (device int, may be null) != 0 turns
// the whole update into a no-op (non-finite loss).
template <typename PT, typename GT, typename ST>
__global__ void kf_adamw(PT* __restrict__ p, const GT* __restrict__ g, ST* __restrict__ m, ST* __restrict__ v,
                         long long n, long long n_decay, float lr, float b1, float b2, float eps, float wd,
                         float bc1, float bc2_sqrt, const float* __restrict__ grad_scale,
                         const int* __restrict__ skip) {
  if (skip && *skip) return;
  const float gs = grad_scale ? *grad_scale : 1.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float gi = to_f<GT>(g[i]) * gs;
    float pi = to_f<PT>(p[i]);
    float mi = to_f<ST>(m[i]);
    float vi = to_f<ST>(v[i]);
    if (i < n_decay) pi *= 1.f - lr * wd;
    mi = b1 * mi + (1.f - b1) * gi;
    vi = b2 * vi + (1.f - b2) * gi * gi;
    const float denom = sqrtf(vi) / bc2_sqrt + eps;
    pi -= (lr / bc1) * mi / denom;
    p[i] = from_f<PT>(pi);
    m[i] = from_f<ST>(mi);
    v[i] = from_f<ST>(vi);
  }
}

// 8-wide bf16 variant (all of p, g, m, v bf16, 16-byte aligned, n % 8 == 0 handled by the tail kernel)
__global__ void kf_adamw_bf16x8(__nv_bfloat16* __restrict__ p, const __nv_bfloat16* __restrict__ g,
                                __nv_bfloat16* __restrict__ m, __nv_bfloat16* __restrict__ v, long long nvec,
                                long long n_decay, float lr, float b1, float b2, float eps, float wd,
                                float bc1, float bc2_sqrt, const float* __restrict__ grad_scale,
                                const int* __restrict__ skip) {
  if (skip && *skip) return;
  const float gs = grad_scale ? *grad_scale : 1.f;
  const float step = lr / bc1;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    F8 pp = load8(p + i * 8), gg = load8(g + i * 8), mm = load8(m + i * 8), vv = load8(v + i * 8);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gi = gg.v[k] * gs;
      float pi = pp.v[k];
      if (i * 8 + k < n_decay) pi *= 1.f - lr * wd;
      const float mi = b1 * mm.v[k] + (1.f - b1) * gi;
      const float vi = b2 * vv.v[k] + (1.f - b2) * gi * gi;
      pi -= step * mi / (sqrtf(vi) / bc2_sqrt + eps);
      pp.v[k] = pi;
      mm.v[k] = mi;
      vv.v[k] = vi;
    }
    store8(p + i * 8, pp);
    store8(m + i * 8, mm);
    store8(v + i * 8, vv);
  }
}

// ------------------------------------------------------------------ sum of squares (two deterministic stages)
template <typename T>
__global__ void kf_sumsq_stage1(const T* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[40];
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x) {
    const float t = to_f<T>(x[i]);
    s += t * t;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
// bf16, 16-byte aligned: 8 elements per load; the ragged tail (n % 8) is added by block 0
__global__ void kf_sumsq_stage1_bf16x8(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[40];
  const long long nvec = n >> 3;
  float s = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const F8 t = load8(x + i * 8);
#pragma unroll
    for (int k = 0; k < 8; ++k) s += t.v[k] * t.v[k];
  }
  if (blockIdx.x == 0)
    for (long long i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) {
      const float t = __bfloat162float(x[i]);
      s += t * t;
    }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void kf_sumsq_stage2(const float* __restrict__ partial, int nparts, float* __restrict__ out,
                                int accumulate) {
  __shared__ float red[40];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

static inline int grid_for(long long work, int threads, int cap = 148 * 16) {
  long long b = (work + threads - 1) / threads;
  if (b < 1) b = 1;
  return (int)(b > cap ? cap : b);
}

}  // namespace kf

// ------------------------------------------------------------------ C entry points
#define KF_LAUNCH_CHECK() \
  do { cudaError_t e_ = cudaGetLastError(); return e_ == cudaSuccess ? 0 : 400 + (int)e_; } while (0)

extern "C" {

int kf_rmsnorm_fwd_bf16(const void* x, const void* w, void* y, void* rstd, int rows, int D, float eps,
                        void* stream) {
  using namespace kf;
  if (D % 8) return 1;
  kf_rmsnorm_fwd<<<rows < 148 * 8 ? rows : 148 * 8, NORM_THREADS, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, (float*)rstd, rows, D, eps);
  KF_LAUNCH_CHECK();
}

// Number of fp32 partial rows rmsnorm_bwd writes (the workspace must hold nblocks * D floats).
int kf_rmsnorm_bwd_blocks(int rows) { return rows < 148 ? (rows < 1 ? 1 : rows) : 148; }

int kf_rmsnorm_bwd_bf16(const void* dy, const void* x, const void* w, const void* rstd, void* dx,
                        void* dw_partial, void* dw_bf16, void* dw_f32, int rows, int D, const void* dx_in,
                        void* stream) {
  using namespace kf;
  if (D % 8) return 1;
  cudaStream_t st = (cudaStream_t)stream;
  const int chunks = kf_rmsnorm_bwd_blocks(rows);
  const int rows_per_chunk = (rows + chunks - 1) / chunks;
  const int nvec = D / 8;
  // dw first: the dx pass may overwrite dy
  kf_rmsnorm_bwd_dw<<<dim3((nvec + 255) / 256, chunks), 256, 0, st>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const float*)rstd, (float*)dw_partial, rows, D, rows_per_chunk);
  kf_colsum_partials<<<(D + 255) / 256, 256, 0, st>>>((const float*)dw_partial, (__nv_bfloat16*)dw_bf16,
                                                      (float*)dw_f32, chunks, D);
  kf_rmsnorm_bwd_dx<<<rows < 148 * 8 ? rows : 148 * 8, NORM_THREADS, 0, st>>>(
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const float*)rstd,
      (__nv_bfloat16*)dx, rows, D, (const __nv_bfloat16*)dx_in);
  KF_LAUNCH_CHECK();
}

int kf_rope_bf16(const void* x, void* y, const void* cosT, const void* sinT, long long tokens, int S,
                 int Htot, int n_rot, int hd, int inverse, void* stream) {
  using namespace kf;
  if (hd % 16) return 1;
  const long long work = tokens * Htot * (hd / 16);
  kf_rope<<<grid_for(work, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)x, (__nv_bfloat16*)y, (const float*)cosT, (const float*)sinT, tokens, S, Htot,
      n_rot, hd, inverse);
  KF_LAUNCH_CHECK();
}

int kf_swiglu_fwd_bf16(const void* gu, void* h, long long rows, int H, void* stream) {
  using namespace kf;
  if (H % 8) return 1;
  kf_swiglu_fwd<<<grid_for(rows * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, (__nv_bfloat16*)h, rows, H);
  KF_LAUNCH_CHECK();
}

int kf_swiglu_bwd_bf16(const void* dh, const void* gu, void* dgu, long long rows, int H, void* stream) {
  using namespace kf;
  if (H % 8) return 1;
  kf_swiglu_bwd<<<grid_for(rows * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dh, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, rows, H, nullptr);
  KF_LAUNCH_CHECK();
}

int kf_swiglu_bwd_ragged_bf16(const void* dh, const void* gu, void* dgu, long long rows_bound, const void* rows_ptr, int H,
                              void* stream) {
  using namespace kf;
  if (H % 8) return 1;
  kf_swiglu_bwd<<<grid_for(rows_bound * (H / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)dh, (const __nv_bfloat16*)gu, (__nv_bfloat16*)dgu, rows_bound, H, (const int*)rows_ptr);
  KF_LAUNCH_CHECK();
}

int kf_embedding_fwd_bf16(const void* ids, const void* table, void* out, long long tokens, int D, int vocab,
                          void* stream) {
  using namespace kf;
  if (D % 8) return 1;
  kf_embedding_fwd<<<grid_for(tokens * (D / 8), 256), 256, 0, (cudaStream_t)stream>>>(
      (const long long*)ids, (const __nv_bfloat16*)table, (__nv_bfloat16*)out, tokens, D, vocab);
  KF_LAUNCH_CHECK();
}

int kf_embedding_bwd_bf16(const void* ids, const void* dy, void* dtable, long long tokens, int D, int vocab,
                          void* stream) {
  using namespace kf;
  if (D % 2) return 1;
  kf_embedding_bwd<<<grid_for(tokens * (D / 2), 256), 256, 0, (cudaStream_t)stream>>>(
      (const long long*)ids, (const __nv_bfloat16*)dy, (__nv_bfloat16*)dtable, tokens, D, vocab);
  KF_LAUNCH_CHECK();
}

int kf_ce_fwd_bwd_bf16(void* logits, const void* labels, void* row_nll, void* row_lse2, const void* inv_n,
                       float z_w, int rows, int V, int ld, void* stream) {
  using namespace kf;
  if (ld % 8) return 1;
  kf_ce_fwd_bwd<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)logits, (const long long*)labels, (float*)row_nll, (float*)row_lse2,
      (const float*)inv_n, z_w, V, ld);
  KF_LAUNCH_CHECK();
}

int kf_ce_vp_stats_bf16(const void* logits, const void* labels, long long vocab_start, void* row_max, void* row_sum,
                        void* row_picked, int rows, int V, int ld, void* stream) {
  using namespace kf;
  if (ld % 8) return 1;
  kf_ce_vp_stats<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)logits, (const long long*)labels,
                                                                vocab_start, (float*)row_max, (float*)row_sum,
                                                                (float*)row_picked, V, ld);
  KF_LAUNCH_CHECK();
}

int kf_ce_vp_bwd_bf16(void* logits, const void* labels, long long vocab_start, const void* lse, const void* inv_n,
                      const void* upstream, float z_w, int rows, int V, int ld, void* stream) {
  using namespace kf;
  if (ld % 8) return 1;
  kf_ce_vp_bwd<<<rows, CE_THREADS, 0, (cudaStream_t)stream>>>((__nv_bfloat16*)logits, (const long long*)labels,
                                                              vocab_start, (const float*)lse, (const float*)inv_n,
                                                              (const float*)upstream, z_w, V, ld);
  KF_LAUNCH_CHECK();
}

// dtype codes: 0 = bf16, 1 = fp32.  Supported (p, g, state): (0,0,0) (1,1,1) (0,0,1) (1,0,1).
int kf_adamw_flat(void* p, const void* g, void* m, void* v, long long n, long long n_decay, float lr,
                  float b1, float b2, float eps, float wd, float bc1, float bc2_sqrt, const void* grad_scale,
                  const void* skip, int p_dt, int g_dt, int s_dt, void* stream) {
  using namespace kf;
  cudaStream_t st = (cudaStream_t)stream;
  const float* gs = (const float*)grad_scale;
  const int* sk = (const int*)skip;
  if (n <= 0) return 0;
#define KF_ADAMW(PT, GT, ST)                                                                         \
  kf_adamw<PT, GT, ST><<<grid_for(n, 256), 256, 0, st>>>((PT*)p, (const GT*)g, (ST*)m, (ST*)v, n,    \
                                                         n_decay, lr, b1, b2, eps, wd, bc1, bc2_sqrt, \
                                                         gs, sk)
  if (p_dt == 0 && g_dt == 0 && s_dt == 0) {
    const bool aligned = (((uintptr_t)p | (uintptr_t)g | (uintptr_t)m | (uintptr_t)v) & 15) == 0;
    const long long nvec = aligned ? n / 8 : 0;
    if (nvec)
      kf_adamw_bf16x8<<<grid_for(nvec, 256), 256, 0, st>>>((__nv_bfloat16*)p, (const __nv_bfloat16*)g,
                                                           (__nv_bfloat16*)m, (__nv_bfloat16*)v, nvec,
                                                           n_decay, lr, b1, b2, eps, wd, bc1, bc2_sqrt, gs,
                                                           sk);
    const long long done = nvec * 8;
    if (done < n) {
      const long long rem = n - done;
      const long long nd = n_decay > done ? n_decay - done : 0;
      kf_adamw<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16><<<1, 256, 0, st>>>(
          (__nv_bfloat16*)p + done, (const __nv_bfloat16*)g + done, (__nv_bfloat16*)m + done,
          (__nv_bfloat16*)v + done, rem, nd, lr, b1, b2, eps, wd, bc1, bc2_sqrt, gs, sk);
    }
  } else if (p_dt == 1 && g_dt == 1 && s_dt == 1) {
    KF_ADAMW(float, float, float);
  } else if (p_dt == 0 && g_dt == 0 && s_dt == 1) {
    KF_ADAMW(__nv_bfloat16, __nv_bfloat16, float);
  } else if (p_dt == 1 && g_dt == 0 && s_dt == 1) {
    KF_ADAMW(float, __nv_bfloat16, float);
  } else {
    return 2;
  }
#undef KF_ADAMW
  KF_LAUNCH_CHECK();
}

// out[0] (+)= sum x^2.  `partial` must hold 1024 floats.
int kf_sumsq(const void* x, long long n, int dt, void* partial, void* out, int accumulate, void* stream) {
  using namespace kf;
  cudaStream_t st = (cudaStream_t)stream;
  const int nb = grid_for(dt == 0 ? n / 8 + 1 : n, 512, 1024);
  if (dt == 0 && ((uintptr_t)x & 15) == 0)
    kf_sumsq_stage1_bf16x8<<<nb, 512, 0, st>>>((const __nv_bfloat16*)x, n, (float*)partial);
  else if (dt == 0)
    kf_sumsq_stage1<__nv_bfloat16><<<nb, 512, 0, st>>>((const __nv_bfloat16*)x, n, (float*)partial);
  else
    kf_sumsq_stage1<float><<<nb, 512, 0, st>>>((const float*)x, n, (float*)partial);
  kf_sumsq_stage2<<<1, 256, 0, st>>>((const float*)partial, nb, (float*)out, accumulate);
  KF_LAUNCH_CHECK();
}

}  // extern "C"

// ------------------------------------------------------------------ bounded-wait self test
// Waits (at most `budget_cycles`) for *flag >= expected.  Used by the test-suite with a flag that
// nothing raises, to check that an expired wait ends in a status code and a healthy context.
namespace kf {
__global__ void kf_flag_wait_probe(const int* flag, int expected, long long budget, int* status) {
  flag_wait_ge(flag, expected, status, budget);
}
}  // namespace kf

extern "C" void* kf_status_device_ptr();

extern "C" int kf_test_flag_timeout(const void* flag, int expected, long long budget_cycles) {
  kf::kf_flag_wait_probe<<<1, 1>>>((const int*)flag, expected, budget_cycles,
                                   (int*)kf_status_device_ptr());
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// ------------------------------------------------------------------ sum of squares without caller scratch
// Same kernels as kf_sumsq; the partial sums live in a device array that is part of the library image.
#include "kf_noalloc.h"

namespace kf {
constexpr int SUMSQ_SCRATCH_FLOATS = 1024;
static __device__ __align__(256) float g_sumsq_scratch[SUMSQ_SCRATCH_FLOATS];
static float* g_sumsq_scratch_addr[64] = {nullptr};  // per device: the array's device address
}  // namespace kf

extern "C" int kf_sumsq_noalloc(const void* x, long long n, int dt, void* out, int accumulate, void* stream) {
  using namespace kf;
  if (n < 0 || n > KF_SUMSQ_NOALLOC_MAX_ELEMS) return 3;
  if (dt != 0 && dt != 1) return 4;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 500;
  if (!g_sumsq_scratch_addr[dev]) {
    // In host code `g_sumsq_scratch` names a host-side shadow, not device memory: ask the runtime for the
    // device address of this device's instance (once per device, with that device current).
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_sumsq_scratch);
    if (e != cudaSuccess || p == nullptr) return 500 + (int)e;
    g_sumsq_scratch_addr[dev] = p;
  }
  float* scratch = g_sumsq_scratch_addr[dev];
  cudaStream_t st = (cudaStream_t)stream;
  const int nb = grid_for(dt == 0 ? n / 8 + 1 : n, 512, SUMSQ_SCRATCH_FLOATS);
  // every slot that stage 2 reads (0 .. nb-1) is written by stage 1 of this call, so stale contents of the
  // shared array from an earlier call never enter the result
  if (dt == 0 && ((uintptr_t)x & 15) == 0)
    kf_sumsq_stage1_bf16x8<<<nb, 512, 0, st>>>((const __nv_bfloat16*)x, n, scratch);
  else if (dt == 0)
    kf_sumsq_stage1<__nv_bfloat16><<<nb, 512, 0, st>>>((const __nv_bfloat16*)x, n, scratch);
  else
    kf_sumsq_stage1<float><<<nb, 512, 0, st>>>((const float*)x, n, scratch);
  kf_sumsq_stage2<<<1, 256, 0, st>>>(scratch, nb, (float*)out, accumulate);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// ------------------------------------------------------------------ Lion and schedule-free AdamW updates
// One launch per parameter tensor, all tensors of one element type (bf16 or fp32), fp32 arithmetic.
// Same update rules as the reference's Python loops (kempnerforge/training/optimizer.py:76-114,177-246).
namespace kf {
template <typename T>
__device__ __forceinline__ float ld_f(const T* p, long long i);
template <>
__device__ __forceinline__ float ld_f<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T>
__device__ __forceinline__ void st_f(T* p, long long i, float v);
template <>
__device__ __forceinline__ void st_f<float>(float* p, long long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

template <typename T>
__global__ void kf_lion_kernel(T* __restrict__ p, const T* __restrict__ g, T* __restrict__ m, long long n, float lr,
                               float b1, float b2, float wd) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gi = ld_f(g, i), mi = ld_f(m, i);
    const float c = b1 * mi + (1.f - b1) * gi;
    const float dir = c > 0.f ? 1.f : (c < 0.f ? -1.f : 0.f);
    st_f(p, i, ld_f(p, i) * (1.f - lr * wd) - lr * dir);
    st_f(m, i, b2 * mi + (1.f - b2) * gi);
  }
}

// y (the parameter the model reads), z (base iterate), x (averaged iterate), v (second moment)
template <typename T>
__global__ void kf_sf_adamw_kernel(T* __restrict__ y, const T* __restrict__ g, T* __restrict__ z, T* __restrict__ v,
                                   T* __restrict__ x, long long n, float lr, float b1, float b2, float eps, float wd,
                                   float bc2, float ck, int first) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gi = ld_f(g, i);
    const float vi = b2 * ld_f(v, i) + (1.f - b2) * gi * gi;
    float zi = ld_f(z, i) - lr * gi / (sqrtf(vi / bc2) + eps);
    zi *= (1.f - lr * wd);
    const float xi = first ? zi : ld_f(x, i) + ck * (zi - ld_f(x, i));
    st_f(v, i, vi);
    st_f(z, i, zi);
    st_f(x, i, xi);
    st_f(y, i, zi + b1 * (xi - zi));
  }
}
}  // namespace kf

extern "C" int kf_lion(void* p, const void* g, void* m, long long n, int dt, float lr, float b1, float b2, float wd,
                       void* stream) {
  using namespace kf;
  if (n <= 0) return 0;
  const int blocks = grid_for(n, 256, 2368);
  cudaStream_t st = (cudaStream_t)stream;
  if (dt == 0)
    kf_lion_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((__nv_bfloat16*)p, (const __nv_bfloat16*)g, (__nv_bfloat16*)m, n, lr, b1, b2, wd);
  else if (dt == 1)
    kf_lion_kernel<float><<<blocks, 256, 0, st>>>((float*)p, (const float*)g, (float*)m, n, lr, b1, b2, wd);
  else
    return 4;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

extern "C" int kf_sf_adamw(void* y, const void* g, void* z, void* v, void* x, long long n, int dt, float lr, float b1,
                           float b2, float eps, float wd, float bc2, float ck, int first, void* stream) {
  using namespace kf;
  if (n <= 0) return 0;
  const int blocks = grid_for(n, 256, 2368);
  cudaStream_t st = (cudaStream_t)stream;
  if (dt == 0)
    kf_sf_adamw_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>((__nv_bfloat16*)y, (const __nv_bfloat16*)g, (__nv_bfloat16*)z,
                                                             (__nv_bfloat16*)v, (__nv_bfloat16*)x, n, lr, b1, b2, eps, wd, bc2, ck, first);
  else if (dt == 1)
    kf_sf_adamw_kernel<float><<<blocks, 256, 0, st>>>((float*)y, (const float*)g, (float*)z, (float*)v, (float*)x, n, lr, b1, b2, eps, wd, bc2, ck, first);
  else
    return 4;
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}
