// coll_common.cuh -- pieces shared by the collective kernel files: the bounds-checking
// macro, copy-in / copy-out between user buffers and the staging window, the run-time
// pointer exchange for buffers outside symmetric windows, the shared-memory ring of the
// bulk-copy paths, and the flag helpers of the ring and point-to-point kernels.
// Everything is in an unnamed namespace: each kernel file gets its own copy.
#pragma once
#include <cuda_runtime.h>

#include "launch.h"
#include "prims.cuh"

namespace fcx {
namespace {

// ---------------------------------------------------------------------------
// bounds-checking build (make -C csrc bounds): takes the place of a memory checker
// ---------------------------------------------------------------------------
// Every kernel compares the extent of what it is about to read and write with the sizes
// the host recorded for the buffers.  A violation is reported through the status block
// (flagcxInvalidArgument from flagcxCommGetAsyncError) and the CTA returns WITHOUT making
// the access -- the index arithmetic is checked, the GPU never faults.
#ifdef FLAGCX_BOUNDS_CHECK
#define FCX_BOUNDS(c, end, limit, what)                                                              \
  do {                                                                                               \
    if ((limit) != 0 && (size_t)(end) > (size_t)(limit)) {                                           \
      if (threadIdx.x == 0)                                                                          \
        fcxdev::reportError((c).status, FLAGCX_DEV_BOUNDS, FLAGCX_DEV_AT_KERNEL, (unsigned)(what),   \
                            (unsigned long long)(end));                                              \
      return;                                                                                        \
    }                                                                                                \
  } while (0)
#else
#define FCX_BOUNDS(c, end, limit, what) do { } while (0)
#endif

// ---------------------------------------------------------------------------
// copy-in / copy-out between user buffers and the peer-visible staging
// ---------------------------------------------------------------------------
// nBlocks blocks of blockBytes; block j is read at src + j*srcStride and written
// at dst + j*dstStride.  This CTA moves its share of every block, so what CTA b
// stages is exactly what CTA b of a peer consumes.
__device__ void ctaCopyBlocks(char *dst, size_t dstStride, const char *src, size_t srcStride, int nBlocks,
                              size_t blockBytes, size_t totalBytes, int b, int g) {
  if (blockBytes == 0) return;
  for (int j = 0; j < nBlocks; ++j) {
    size_t len = blockBytes;
    if (totalBytes) { // back-to-back blocks, the last may be short or empty
      size_t start = (size_t)j * blockBytes;
      if (start >= totalBytes) break;
      if (totalBytes - start < len) len = totalBytes - start;
    }
    size_t ub, ue;
    ctaShare((len + 15) >> 4, b, g, &ub, &ue);
    size_t bb = ub << 4, be = (ue << 4) < len ? (ue << 4) : len;
    ctaCopy(dst + j * dstStride, src + j * srcStride, bb, be);
  }
}

__device__ __forceinline__ void copyIn(const CollArgs &a, int rank, int b, int g) {
  if (!a.userIn) return;
  size_t stageStride = a.inStride ? a.inStride : a.inBlockBytes;
  ctaCopyBlocks((char *)a.in[rank], stageStride, a.userIn, a.userInStride, a.nInBlocks, a.inBlockBytes,
                a.inTotalBytes, b, g);
}
__device__ __forceinline__ void copyOut(const CollArgs &a, int rank, int b, int g) {
  if (!a.userOut) return;
  size_t stageStride = a.outStride ? a.outStride : a.outBlockBytes;
  ctaCopyBlocks(a.userOut, a.userOutStride, a.out[rank], stageStride, a.nOutBlocks, a.outBlockBytes,
                a.outTotalBytes, b, g);
}

// ---------------------------------------------------------------------------
// run-time pointer exchange (buffers outside symmetric windows)
// ---------------------------------------------------------------------------
// The argument block lives in shared memory so that the peers' pointers can be
// filled in once they are known.
__device__ __forceinline__ CollArgs &stageArgs(const CollArgs &src) {
  static_assert(sizeof(CollArgs) % 8 == 0, "argument block is copied in 8-byte words");
  __shared__ __align__(16) unsigned long long words[sizeof(CollArgs) / 8];
  for (int i = threadIdx.x; i < (int)(sizeof(CollArgs) / 8); i += blockDim.x)
    words[i] = ((const unsigned long long *)&src)[i];
  __syncthreads();
  return *(CollArgs *)words;
}

// Before the first barrier: thread p tells rank p where this rank's input and output
// are in rank p's address space.  The same thread then raises the barrier flag at rank
// p with release semantics, so the pad is visible to whoever sees the flag.  CTA b only
// ever meets CTA b of a peer, hence one pad entry per (CTA, source rank); two parities
// because a fast rank may publish for its next launch while a slow one still has to
// read this launch's entry (it cannot be two launches ahead: that takes a barrier).
__device__ __forceinline__ void publishPointers(const flagcxDevComm &c, const CollArgs &a, int b) {
  const int t = threadIdx.x;
  if (a.xchg && t < c.nRanks && t != c.rank) {
    unsigned long long *pad =
        a.ptrPad[t] + (((size_t)a.xchgParity * FLAGCX_COLL_BARRIER_SLOTS + b) * FLAGCX_MAX_RANKS + c.rank) * 2;
    fcxdev::stRelaxedSys(pad, (unsigned long long)(uintptr_t)a.pubIn[t]);
    fcxdev::stRelaxedSys(pad + 1, (unsigned long long)(uintptr_t)a.pubOut[t]);
  }
}
// After the first barrier: take the peers' pointers out of the local pad.
__device__ __forceinline__ void learnPointers(const flagcxDevComm &c, CollArgs &a, int b) {
  if (!a.xchg) return;
  const int t = threadIdx.x;
  if (t < c.nRanks && t != c.rank) {
    const unsigned long long *pad =
        a.ptrPad[c.rank] + (((size_t)a.xchgParity * FLAGCX_COLL_BARRIER_SLOTS + b) * FLAGCX_MAX_RANKS + t) * 2;
    if (a.xchg & kXchgIn) a.in[t] = (const char *)(uintptr_t)fcxdev::ldRelaxedSys(pad);
    if (a.xchg & kXchgOut) a.out[t] = (char *)(uintptr_t)fcxdev::ldRelaxedSys(pad + 1);
  }
  __syncthreads();
}
// The bulk-copy engine needs 16-byte aligned addresses; pointers learnt at run time
// (or filled in by the emulated world's launcher) were not seen by the host's check.
__device__ __forceinline__ bool learntPointersAligned(const flagcxDevComm &c, const CollArgs &a) {
  uintptr_t bits = 0;
  for (int p = 0; p < c.nRanks; ++p) bits |= (uintptr_t)a.in[p] | (uintptr_t)a.out[p];
  return (bits & 15) == 0;
}

// ---------------------------------------------------------------------------
// shared-memory ring of the bulk-copy paths (dynamic shared memory of the launch)
// ---------------------------------------------------------------------------
constexpr int kBulkMaxStages = 12;
constexpr size_t kBulkRingBytes = 192u << 10;
extern __shared__ __align__(128) unsigned char bulkRing[];

__device__ __forceinline__ uint32_t smem32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Waits for the given phase parity of an mbarrier; gives up when `*abortS` is raised
// or the communicator's time limit passes (then raises it).
__device__ __forceinline__ bool mbarWaitBounded(const flagcxDevComm &c, uint64_t *bar, uint32_t parity,
                                                volatile int *abortS) {
  const uint32_t addr = smem32(bar);
  unsigned long long t0 = 0;
  for (unsigned spins = 0;; ++spins) {
    uint32_t done;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(done)
                 : "r"(addr), "r"(parity)
                 : "memory");
    if (done) return true;
    if ((spins & 255u) == 255u) {
      if (*abortS) return false;
      if (t0 == 0) t0 = fcxdev::globalTimerNs();
      else if (fcxdev::globalTimerNs() - t0 > c.timeoutNs) { *abortS = 1; return false; }
    }
  }
}

// ---------------------------------------------------------------------------
// flags between two ranks (ring steps, point-to-point chunks)
// ---------------------------------------------------------------------------
__device__ __forceinline__ bool ctaWaitFlag(const flagcxDevComm &c, const unsigned long long *flag,
                                            unsigned long long want, unsigned peer) {
  bool ok = true;
  if (threadIdx.x == 0) ok = fcxdev::waitGe(c, flag, want, FLAGCX_DEV_AT_SIGNAL, peer);
  return !__syncthreads_or(ok ? 0 : 1);
}
__device__ __forceinline__ void ctaRaiseFlag(unsigned long long *flag, unsigned long long v) {
  __syncthreads();
  if (threadIdx.x == 0) {
    fcxdev::fenceSys();
    fcxdev::stReleaseSys(flag, v);
  }
}

__device__ void ctaCopyShare(char *dst, const char *src, size_t bytes, int b, int g) {
  size_t ub, ue;
  ctaShare((bytes + 15) >> 4, b, g, &ub, &ue);
  size_t bb = ub << 4, be = (ue << 4) < bytes ? (ue << 4) : bytes;
  ctaCopy(dst, src, bb, be);
}

} // namespace
} // namespace fcx
