// Entry points of libkfb200 that never allocate.
//
// This header has no counterpart in the reference project: it exists for callers of this library that are
// not allowed to allocate device memory at the point where they need the result — a latency-critical loop
// that must not touch the allocator (an allocation can synchronise the device), a host process whose memory
// pool is owned and accounted by somebody else, or a C caller that simply has no PyTorch caching allocator
// to borrow a temporary from.  The regular entry points take their scratch buffers from
// the caller (`partial` arguments); the functions below keep the scratch inside the library instead.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest input (in elements) kf_sumsq_noalloc accepts.  The reduction uses at most 1024 partial sums, so
// the library holds a 4 KiB scratch array per GPU for the life of the process.
#define KF_SUMSQ_NOALLOC_MAX_ELEMS (1LL << 34)

// out[0] = sum(x[i]^2) (or out[0] += ... when accumulate != 0), fp32, fixed reduction order.
//   x      device pointer, n elements of bf16 (dt == 0) or fp32 (dt == 1)
//   out    device pointer to one float (caller-owned, like x)
//   stream cudaStream_t (0 = default stream)
// Returns 0 on success; 3 if n is negative or larger than KF_SUMSQ_NOALLOC_MAX_ELEMS; 4 if dt is unknown;
// 5xx if the address of the built-in scratch array could not be obtained; 4xx on a launch error.
//
// No cudaMalloc / cudaFree / allocating library call is made.  The scratch is one file-scope device array
// shared by every call on that GPU: the function overwrites the part it uses before reading it, and two
// calls that overlap on the GPU (different streams) race on it — serialise them.  The first call on each
// device does the set-up (it looks the array's device address up with cudaGetSymbolAddress): make that
// first call before any stream capture begins.  Nothing is claimed here about use inside a capture.
// Host threads: the per-device address is cached without a lock, so the first call on a device must not
// run concurrently with another host thread's call on that device; later calls may come from any thread.
int kf_sumsq_noalloc(const void* x, long long n, int dt, void* out, int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
