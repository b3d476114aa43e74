// Fused communication + compute kernels over NVLink peer (symmetric) memory.
//
//   kf_symm_rs_norm      reduce-scatter fused with averaging, cast and the gradient-norm partial:
//                        every rank sums ITS shard of the flat gradient buffer over all ranks' buffers
//                        (plain peer loads, or one multimem.ld_reduce through NVSwitch), scales by 1/N,
//                        writes the result into its own buffer and accumulates sum(g^2).
//   kf_symm_adamw_bcast  sharded AdamW fused with the parameter all-gather: the rank updates its shard
//                        and stores the new bf16 parameters into every rank's parameter buffer
//                        (peer stores, or one multimem.st broadcast through NVSwitch).
//   kf_symm_gather       plain all-gather of a shard into every peer's buffer (initial broadcast, tests).
//
// The kernels contain no waits on other GPUs: ordering between ranks is established on the host side of
// the stream (a bounded signal-pad barrier before the reduce and after the publish).  Replaces FSDP2's
// NCCL reduce-scatter + copy-out + fused AdamW + next-step all-gather + copy-in
// (kempnerforge/distributed/parallel.py:72-87,250-302, kempnerforge/training/optimizer.py:28-39).
#include "common.cuh"

namespace kf {

constexpr int MAX_PEERS = 8;
constexpr int RS_UNROLL = 4;  // 16-byte vectors per thread and step in the peer-load kernels
struct PeerPtrs {
  void* p[MAX_PEERS];
};

__device__ __forceinline__ void ld_reduce_bf16x8(const void* mc_addr, float (&out)[8]) {
  uint32_t a, b, c, d;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
               : "l"(mc_addr)
               : "memory");
  float2 f;
  f = unpack_bf16(a); out[0] = f.x; out[1] = f.y;
  f = unpack_bf16(b); out[2] = f.x; out[3] = f.y;
  f = unpack_bf16(c); out[4] = f.x; out[5] = f.y;
  f = unpack_bf16(d); out[6] = f.x; out[7] = f.y;
}
__device__ __forceinline__ void multimem_st_16B(void* mc_addr, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float block_sum_f(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  if (warp == 0) {
    t = lane < nw ? red[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  return t;  // valid in thread 0
}

// grads: every rank's flat bf16 gradient buffer (same layout).  Elements [lo, lo + n) are this rank's shard.
// The averaged shard is written back into this rank's own buffer; partial[blockIdx.x] receives sum(avg^2).
__global__ void __launch_bounds__(512)
kf_symm_rs_norm(PeerPtrs grads, const void* mc_grad, int world, int rank, long long lo, long long n,
                float inv_world, float* __restrict__ partial) {
  __shared__ float red[32];
  const long long nvec = n >> 3;
  __nv_bfloat16* mine = reinterpret_cast<__nv_bfloat16*>(grads.p[rank]) + lo;
  float ss = 0.f;
  // RS_UNROLL vectors per thread and step, every rank's loads of a step issued before the first use: NVLink loads
  // take microseconds, so the bytes in flight per thread set the bandwidth
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * RS_UNROLL) {
    float acc[RS_UNROLL][8];
    if (mc_grad) {
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u) {
        const long long i = i0 + u * stride;
        if (i < nvec) ld_reduce_bf16x8(reinterpret_cast<const __nv_bfloat16*>(mc_grad) + lo + i * 8, acc[u]);
      }
    } else {
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[u][k] = 0.f;
      for (int r = 0; r < world; ++r) {  // fixed order: bit-identical results on every run
        const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(grads.p[r]) + lo;
        uint4 v[RS_UNROLL];
#pragma unroll
        for (int u = 0; u < RS_UNROLL; ++u) {
          const long long i = i0 + u * stride;
          v[u] = i < nvec ? *reinterpret_cast<const uint4*>(src + i * 8) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < RS_UNROLL; ++u) {
          float2 f;
          f = unpack_bf16(v[u].x); acc[u][0] += f.x; acc[u][1] += f.y;
          f = unpack_bf16(v[u].y); acc[u][2] += f.x; acc[u][3] += f.y;
          f = unpack_bf16(v[u].z); acc[u][4] += f.x; acc[u][5] += f.y;
          f = unpack_bf16(v[u].w); acc[u][6] += f.x; acc[u][7] += f.y;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < RS_UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
      uint4 o;
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[u][k] *= inv_world;
      o.x = pack_bf16(acc[u][0], acc[u][1]);
      o.y = pack_bf16(acc[u][2], acc[u][3]);
      o.z = pack_bf16(acc[u][4], acc[u][5]);
      o.w = pack_bf16(acc[u][6], acc[u][7]);
      *reinterpret_cast<uint4*>(mine + i * 8) = o;
      // the norm is taken of the values the optimizer will read (after rounding to bf16)
      float2 f;
      f = unpack_bf16(o.x); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16(o.y); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16(o.z); ss += f.x * f.x + f.y * f.y;
      f = unpack_bf16(o.w); ss += f.x * f.x + f.y * f.y;
    }
  }
  const float total = block_sum_f(ss, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = total;
}

__global__ void kf_sum_partials(const float* __restrict__ partial, int n, float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  const float t = block_sum_f(s, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + t : t;
}

// AdamW on the shard [lo, lo + n) (bf16 params / grads / moments) + broadcast of the new parameters.
__global__ void __launch_bounds__(256)
kf_symm_adamw_bcast(PeerPtrs params, void* mc_param, int world, int rank, const __nv_bfloat16* __restrict__ grad,
                    __nv_bfloat16* __restrict__ m, __nv_bfloat16* __restrict__ v, long long lo, long long n,
                    long long n_decay_global, float lr, float b1, float b2, float eps, float wd, float bc1,
                    float bc2_sqrt, const float* __restrict__ grad_scale, const int* __restrict__ skip) {
  if (skip && *skip) return;
  const float gs = grad_scale ? *grad_scale : 1.f;
  const float step = lr / bc1;
  const long long nvec = n >> 3;
  const __nv_bfloat16* mine = reinterpret_cast<const __nv_bfloat16*>(params.p[rank]) + lo;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 pu = *reinterpret_cast<const uint4*>(mine + i * 8);
    const uint4 gu = *reinterpret_cast<const uint4*>(grad + i * 8);
    const uint4 mu = *reinterpret_cast<const uint4*>(m + i * 8);
    const uint4 vu = *reinterpret_cast<const uint4*>(v + i * 8);
    const uint32_t pw[4] = {pu.x, pu.y, pu.z, pu.w}, gw[4] = {gu.x, gu.y, gu.z, gu.w};
    const uint32_t mw[4] = {mu.x, mu.y, mu.z, mu.w}, vw[4] = {vu.x, vu.y, vu.z, vu.w};
    uint32_t po[4], mo[4], vo[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 p2 = unpack_bf16(pw[k]), g2 = unpack_bf16(gw[k]), m2 = unpack_bf16(mw[k]), v2 = unpack_bf16(vw[k]);
      float pe[2] = {p2.x, p2.y}, ge[2] = {g2.x * gs, g2.y * gs}, me[2] = {m2.x, m2.y}, ve[2] = {v2.x, v2.y};
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        if (lo + i * 8 + k * 2 + e < n_decay_global) pe[e] *= 1.f - lr * wd;
        me[e] = b1 * me[e] + (1.f - b1) * ge[e];
        ve[e] = b2 * ve[e] + (1.f - b2) * ge[e] * ge[e];
        pe[e] -= step * me[e] / (sqrtf(ve[e]) / bc2_sqrt + eps);
      }
      po[k] = pack_bf16(pe[0], pe[1]);
      mo[k] = pack_bf16(me[0], me[1]);
      vo[k] = pack_bf16(ve[0], ve[1]);
    }
    *reinterpret_cast<uint4*>(m + i * 8) = make_uint4(mo[0], mo[1], mo[2], mo[3]);
    *reinterpret_cast<uint4*>(v + i * 8) = make_uint4(vo[0], vo[1], vo[2], vo[3]);
    const uint4 pn = make_uint4(po[0], po[1], po[2], po[3]);
    if (mc_param) {
      multimem_st_16B(reinterpret_cast<__nv_bfloat16*>(mc_param) + lo + i * 8, pn);
    } else {
      for (int r = 0; r < world; ++r)
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + lo + i * 8) = pn;
    }
  }
}

// Copy this rank's shard [lo, lo + n) of its own buffer into the same range of every peer's buffer.
__global__ void kf_symm_gather(PeerPtrs bufs, void* mc_buf, int world, int rank, long long lo, long long n) {
  const long long nvec = n >> 3;
  const __nv_bfloat16* mine = reinterpret_cast<const __nv_bfloat16*>(bufs.p[rank]) + lo;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 u = *reinterpret_cast<const uint4*>(mine + i * 8);
    if (mc_buf) {
      multimem_st_16B(reinterpret_cast<__nv_bfloat16*>(mc_buf) + lo + i * 8, u);
    } else {
      for (int r = 0; r < world; ++r)
        if (r != rank) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.p[r]) + lo + i * 8) = u;
    }
  }
}

// ---- sharded parameters (every rank keeps 1/world of each parameter) ---------------------------------------
// A unit's parameters are laid out one after another ("full layout"); parameter i occupies full[i] .. full[i] +
// len[i] and is cut into `world` equal contiguous pieces; rank r keeps piece r of every parameter, packed in the
// same order ("shard layout": the piece of parameter i starts at full[i] / world).  SegTable describes a subset
// of the parameters: where the segment starts in the destination / source full-layout buffer (`full`), its total
// length, and where its piece starts inside a rank's shard.  All values are multiples of 8 elements.
constexpr int MAX_SEGS = 16;
struct SegTable {
  long long full[MAX_SEGS];
  long long len[MAX_SEGS];
  long long shard[MAX_SEGS];
  long long vec_start[MAX_SEGS + 1];  // prefix sums of len / 8 (gather) or len / world / 8 (reduce)
  long long piece[MAX_SEGS];          // len / world
  int n;
};

__device__ __forceinline__ int seg_of(const SegTable& t, long long v) {
  int s = 0;
  for (int i = 1; i < t.n; ++i)
    if (v >= t.vec_start[i]) s = i;
  return s;
}

// All-gather of the listed parameters into a local full-layout buffer by plain peer loads (own piece: local loads).
// Nothing waits for another GPU; the peers' shards must not change while the kernel runs.
__global__ void __launch_bounds__(256)
kf_symm_pull(PeerPtrs shards, int world, SegTable t, __nv_bfloat16* __restrict__ dst) {
  const long long nvec = t.vec_start[t.n];
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * RS_UNROLL) {
    uint4 q[RS_UNROLL];
    long long dsti[RS_UNROLL];
#pragma unroll
    for (int u = 0; u < RS_UNROLL; ++u) {
      const long long v = v0 + u * stride;
      dsti[u] = -1;
      if (v < nvec) {
        const int s = seg_of(t, v);
        const long long e = (v - t.vec_start[s]) * 8;   // element inside the parameter
        const long long piece = t.piece[s];
        const int owner = int(e / piece);
        q[u] = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(shards.p[owner]) + t.shard[s] +
                                               (e - owner * piece));
        dsti[u] = t.full[s] + e;
      }
    }
#pragma unroll
    for (int u = 0; u < RS_UNROLL; ++u)
      if (dsti[u] >= 0) *reinterpret_cast<uint4*>(dst + dsti[u]) = q[u];
  }
}

// Reduce-scatter of full-layout gradient buffers into the shard layout: this rank sums ITS piece of every listed
// parameter over all ranks' buffers (peer loads, fixed order, fp32), scales by 1 / world and writes (or adds to)
// its gradient shard.  mc_grads != null: one multimem.ld_reduce through NVSwitch instead of `world` loads.
__global__ void __launch_bounds__(512)
kf_symm_rs_shard(PeerPtrs grads, const void* mc_grads, int world, int rank, SegTable t, float inv_world,
                 __nv_bfloat16* __restrict__ shard_grad, int accumulate) {
  const long long nvec = t.vec_start[t.n];
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * RS_UNROLL) {
    long long src[RS_UNROLL], dsti[RS_UNROLL];
    float acc[RS_UNROLL][8];
#pragma unroll
    for (int u = 0; u < RS_UNROLL; ++u) {
      const long long v = v0 + u * stride;
      src[u] = -1;
      if (v < nvec) {
        const int s = seg_of(t, v);
        const long long local = (v - t.vec_start[s]) * 8;        // element inside this rank's piece
        src[u] = t.full[s] + rank * t.piece[s] + local;           // element inside a full-layout buffer
        dsti[u] = t.shard[s] + local;
      }
    }
    if (mc_grads) {
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u)
        if (src[u] >= 0) ld_reduce_bf16x8(reinterpret_cast<const __nv_bfloat16*>(mc_grads) + src[u], acc[u]);
    } else {
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[u][k] = 0.f;
      for (int r = 0; r < world; ++r) {
        const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(grads.p[r]);
        uint4 q[RS_UNROLL];
#pragma unroll
        for (int u = 0; u < RS_UNROLL; ++u)
          q[u] = src[u] >= 0 ? *reinterpret_cast<const uint4*>(base + src[u]) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < RS_UNROLL; ++u) {
          float2 f;
          f = unpack_bf16(q[u].x); acc[u][0] += f.x; acc[u][1] += f.y;
          f = unpack_bf16(q[u].y); acc[u][2] += f.x; acc[u][3] += f.y;
          f = unpack_bf16(q[u].z); acc[u][4] += f.x; acc[u][5] += f.y;
          f = unpack_bf16(q[u].w); acc[u][6] += f.x; acc[u][7] += f.y;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < RS_UNROLL; ++u) {
      if (src[u] < 0) continue;
      __nv_bfloat16* out = shard_grad + dsti[u];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[u][k] *= inv_world;
      if (accumulate) {
        const uint4 old = *reinterpret_cast<const uint4*>(out);
        float2 f;
        f = unpack_bf16(old.x); acc[u][0] += f.x; acc[u][1] += f.y;
        f = unpack_bf16(old.y); acc[u][2] += f.x; acc[u][3] += f.y;
        f = unpack_bf16(old.z); acc[u][4] += f.x; acc[u][5] += f.y;
        f = unpack_bf16(old.w); acc[u][6] += f.x; acc[u][7] += f.y;
      }
      uint4 o;
      o.x = pack_bf16(acc[u][0], acc[u][1]);
      o.y = pack_bf16(acc[u][2], acc[u][3]);
      o.z = pack_bf16(acc[u][4], acc[u][5]);
      o.w = pack_bf16(acc[u][6], acc[u][7]);
      *reinterpret_cast<uint4*>(out) = o;
    }
  }
}

static inline int fill_seg_table(SegTable& t, int n, const long long* full, const long long* len, const long long* shard,
                                 int world, bool per_piece) {
  if (n < 1 || n > MAX_SEGS) return 1;
  t.n = n;
  long long acc = 0;
  for (int i = 0; i < n; ++i) {
    if ((full[i] & 7) || (shard[i] & 7) || (len[i] % (8LL * world))) return 2;
    t.full[i] = full[i];
    t.len[i] = len[i];
    t.shard[i] = shard[i];
    t.piece[i] = len[i] / world;
    t.vec_start[i] = acc;
    acc += (per_piece ? len[i] / world : len[i]) / 8;
  }
  for (int i = n; i <= MAX_SEGS; ++i) t.vec_start[i] = acc;
  return 0;
}

static inline PeerPtrs make_ptrs(const long long* ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < MAX_PEERS; ++i) pp.p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return pp;
}

}  // namespace kf

extern "C" {

// partial must hold 1024 floats; out[0] (+)= sum of squares of the averaged shard.  n % 8 == 0, lo % 8 == 0.
int kf_symm_rs_norm_bf16(const long long* peer_grad_ptrs, const void* mc_grad, int world, int rank, long long lo,
                         long long n, void* partial, void* out, int accumulate, int max_blocks, void* stream) {
  using namespace kf;
  if (world > MAX_PEERS || (n & 7) || (lo & 7)) return 1;
  cudaStream_t st = (cudaStream_t)stream;
  long long want = (n / 8 + 511) / 512;
  int nb = (int)(want < 1 ? 1 : (want > max_blocks ? max_blocks : want));
  if (nb > 1024) nb = 1024;
  kf_symm_rs_norm<<<nb, 512, 0, st>>>(make_ptrs(peer_grad_ptrs, world), mc_grad, world, rank, lo, n, 1.f / world,
                                      (float*)partial);
  kf_sum_partials<<<1, 256, 0, st>>>((const float*)partial, nb, (float*)out, accumulate);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

int kf_symm_adamw_bcast_bf16(const long long* peer_param_ptrs, void* mc_param, int world, int rank, const void* grad,
                             void* m, void* v, long long lo, long long n, long long n_decay_global, float lr, float b1,
                             float b2, float eps, float wd, float bc1, float bc2_sqrt, const void* grad_scale,
                             const void* skip, int max_blocks, void* stream) {
  using namespace kf;
  if (world > MAX_PEERS || (n & 7) || (lo & 7)) return 1;
  long long want = (n / 8 + 255) / 256;
  int nb = (int)(want < 1 ? 1 : (want > max_blocks ? max_blocks : want));
  kf_symm_adamw_bcast<<<nb, 256, 0, (cudaStream_t)stream>>>(
      make_ptrs(peer_param_ptrs, world), mc_param, world, rank, (const __nv_bfloat16*)grad, (__nv_bfloat16*)m,
      (__nv_bfloat16*)v, lo, n, n_decay_global, lr, b1, b2, eps, wd, bc1, bc2_sqrt, (const float*)grad_scale,
      (const int*)skip);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// dst[full[i] .. + len[i]) = parameter i assembled from every rank's piece at shard_ptrs[r] + shard[i].
int kf_symm_pull_bf16(const long long* shard_ptrs, int world, int n_seg, const long long* full, const long long* len,
                      const long long* shard, void* dst, int max_blocks, void* stream) {
  using namespace kf;
  if (world < 1 || world > MAX_PEERS) return 1;
  SegTable t;
  int rc = fill_seg_table(t, n_seg, full, len, shard, world, false);
  if (rc) return 10 + rc;
  const long long nvec = t.vec_start[t.n];
  long long want = (nvec + 255) / 256;
  int nb = (int)(want < 1 ? 1 : (want > max_blocks ? max_blocks : want));
  kf_symm_pull<<<nb, 256, 0, (cudaStream_t)stream>>>(make_ptrs(shard_ptrs, world), world, t, (__nv_bfloat16*)dst);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

// shard_grad[shard[i] .. + len[i] / world) (+)= mean over ranks of grad buffers [full[i] + rank * len[i] / world ..).
int kf_symm_rs_shard_bf16(const long long* grad_ptrs, const void* mc_grads, int world, int rank, int n_seg,
                          const long long* full, const long long* len, const long long* shard, void* shard_grad,
                          int accumulate, int max_blocks, void* stream) {
  using namespace kf;
  if (world < 1 || world > MAX_PEERS) return 1;
  SegTable t;
  int rc = fill_seg_table(t, n_seg, full, len, shard, world, true);
  if (rc) return 10 + rc;
  const long long nvec = t.vec_start[t.n];
  long long want = (nvec + 511) / 512;
  int nb = (int)(want < 1 ? 1 : (want > max_blocks ? max_blocks : want));
  kf_symm_rs_shard<<<nb, 512, 0, (cudaStream_t)stream>>>(make_ptrs(grad_ptrs, world), mc_grads, world, rank, t,
                                                         1.f / world, (__nv_bfloat16*)shard_grad, accumulate);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

int kf_symm_gather_bf16(const long long* peer_ptrs, void* mc_buf, int world, int rank, long long lo, long long n,
                        int max_blocks, void* stream) {
  using namespace kf;
  if (world > MAX_PEERS || (n & 7) || (lo & 7)) return 1;
  long long want = (n / 8 + 255) / 256;
  int nb = (int)(want < 1 ? 1 : (want > max_blocks ? max_blocks : want));
  kf_symm_gather<<<nb, 256, 0, (cudaStream_t)stream>>>(make_ptrs(peer_ptrs, world), mc_buf, world, rank, lo, n);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 400 + (int)e;
}

}  // extern "C"
