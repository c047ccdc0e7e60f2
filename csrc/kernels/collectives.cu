// collectives.cu -- the sm_100a collective kernels and their launch table.
//
// Every collective of the device path is ONE kernel launch per rank.  The kernel
// reads and writes the other ranks' buffers directly through their NVLink peer
// mappings; ranks meet only at per-CTA barriers made of release/acquire flags in
// peer memory (flagcx_device.cuh).  The adjacent element-wise work -- scaling
// (average, 1/world), bf16<->fp32 conversion of the result, a residual add -- is
// applied to the accumulator in registers before the single store.
//
// These kernels take the place of the FlagCX custom all-reduce kernels
// (flagcx/adaptor/kernel/nvidia/custom_allreduce.cu:337-467 in the FlagCX project:
// one-shot peer reduce, NVLS one-shot and NVLS two-shot) and of every NCCL call of
// its NCCL adaptor (flagcx/adaptor/ccl/nccl_adaptor.cc:228-382).  Differences:
// 16-byte accesses, fp32 accumulation in a fixed rank order (all ranks get
// bit-identical results), no staging copy when the buffers are registered, no
// size cap, all reductions and element types, and waits that give up with an
// error status instead of spinning forever.
#include <cuda_runtime.h>

#include "launch.h"
#include "prims.cuh"

namespace fcx {
namespace {

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

// ---------------------------------------------------------------------------
// reduce family
// ---------------------------------------------------------------------------
template <typename T, int OP, int NR>
struct Reducer {
  using Acc = typename Elem<T>::Acc;
  static constexpr int N = 16 / (int)sizeof(T);

  // Reduces the 16-byte pack at byte offset `off` of every rank's input, always in
  // rank order 0..n-1 so that every rank computes bit-identical sums.
  static __device__ __forceinline__ void loadReduce(const CollArgs &a, int nRanks, size_t off, Acc (&acc)[N]) {
    uint4 v[FLAGCX_MAX_RANKS];
    if (NR > 0) {
#pragma unroll
      for (int p = 0; p < NR; ++p) v[p] = ldSys16(a.in[p] + off);
    } else {
#pragma unroll
      for (int p = 0; p < FLAGCX_MAX_RANKS; ++p)
        if (p < nRanks) v[p] = ldSys16(a.in[p] + off);
    }
    const T *e0 = (const T *)&v[0];
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = toAcc<T>(e0[i]);
#pragma unroll
    for (int p = 1; p < (NR > 0 ? NR : FLAGCX_MAX_RANKS); ++p) {
      if (NR > 0 || p < nRanks) {
        const T *e = (const T *)&v[p];
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] = combine<OP, Acc>(acc[i], toAcc<T>(e[i]), a.redOp);
      }
    }
  }

  // Applies the epilogue and stores one pack at element index `e` (relative to
  // each destination base) to nDst destinations.
  static __device__ __forceinline__ void storePack(const CollArgs &a, char *const *dst, int nDst, size_t e,
                                                   Acc (&acc)[N]) {
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = finish<Acc>(acc[i], a.scale, a.divisor);
    if constexpr (sizeof(T) == 2) {
      if (a.outMode == kOutFloat) { // 8 x 16-bit in, 8 x fp32 out
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = (float)acc[i];
        if (a.residual) {
          const float *r = (const float *)a.residual + e;
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] += r[i];
        }
        for (int d = 0; d < nDst; ++d) {
          float *o = (float *)dst[d] + e;
          st16(o, *(uint4 *)&f[0]);
          st16(o + 4, *(uint4 *)&f[4]);
        }
        return;
      }
    }
    if constexpr (sizeof(T) == 4) {
      if (a.outMode == kOutBf16) { // 4 x fp32 in, 4 x bf16 out
        __align__(8) __nv_bfloat16 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float x = (float)acc[i];
          if (a.residual) x += __bfloat162float(((const __nv_bfloat16 *)a.residual)[e + i]);
          h[i] = __float2bfloat16_rn(x);
        }
        for (int d = 0; d < nDst; ++d) *(uint2 *)((__nv_bfloat16 *)dst[d] + e) = *(uint2 *)h;
        return;
      }
    }
    uint4 o;
    T *oe = (T *)&o;
    if (a.residual) {
      uint4 rv = ldLocal16((const T *)a.residual + e);
      const T *re = (const T *)&rv;
#pragma unroll
      for (int i = 0; i < N; ++i) oe[i] = fromAcc<T>(acc[i] + toAcc<T>(re[i]));
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) oe[i] = fromAcc<T>(acc[i]);
    }
    for (int d = 0; d < nDst; ++d) st16((T *)dst[d] + e, o);
  }

  static __device__ __forceinline__ void storeOne(const CollArgs &a, char *const *dst, int nDst, size_t e, Acc v) {
    v = finish<Acc>(v, a.scale, a.divisor);
    for (int d = 0; d < nDst; ++d) {
      if (a.outMode == kOutFloat && sizeof(T) == 2) {
        float x = (float)v;
        if (a.residual) x += ((const float *)a.residual)[e];
        ((float *)dst[d])[e] = x;
      } else if (a.outMode == kOutBf16 && sizeof(T) == 4) {
        float x = (float)v;
        if (a.residual) x += __bfloat162float(((const __nv_bfloat16 *)a.residual)[e]);
        ((__nv_bfloat16 *)dst[d])[e] = __float2bfloat16_rn(x);
      } else {
        Acc x = v;
        if (a.residual) x = x + toAcc<T>(((const T *)a.residual)[e]);
        ((T *)dst[d])[e] = fromAcc<T>(x);
      }
    }
  }

  // Reduces elements [sb, se) of the inputs (indices into in[p]) and stores them at
  // element index (i - sb + dstBase) of each destination.  The CTA takes its share
  // of the range in 16-byte units.
  static __device__ void slice(const CollArgs &a, int nRanks, size_t sb, size_t se, char *const *dst, int nDst,
                               size_t dstBase, int b, int g) {
    if (se <= sb) return;
    const size_t elems = se - sb;
    const size_t outSize = a.outMode == kOutFloat ? 4 : (a.outMode == kOutBf16 ? 2 : sizeof(T));
    bool vec = ((sb * sizeof(T)) & 15) == 0 && ((dstBase * outSize) & 15) == 0;
    for (int p = 0; p < nRanks; ++p) vec &= (((uintptr_t)a.in[p]) & 15) == 0;
    for (int d = 0; d < nDst; ++d) vec &= (((uintptr_t)dst[d]) & 15) == 0;
    if (a.residual) vec &= (((uintptr_t)a.residual) & 15) == 0;
    size_t ub, ue;
    ctaShare((elems * sizeof(T) + 15) >> 4, b, g, &ub, &ue);
    size_t eb = ub * N, ee = ue * N < elems ? ue * N : elems; // this CTA's elements, relative to sb
    if (vec) {
      const size_t fullEnd = ee / N * N; // whole packs only
      const size_t stride = (size_t)blockDim.x * N;
      size_t e = eb + (size_t)threadIdx.x * N;
      if constexpr (NR > 0) {
        // NVLink loads take microseconds: keep 16 of them in flight per thread
        constexpr int U = 16 / NR;
        for (; e + (U - 1) * stride < fullEnd; e += U * stride) {
          uint4 v[U][NR];
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int p = 0; p < NR; ++p) v[u][p] = ldSys16(a.in[p] + (sb + e + u * stride) * sizeof(T));
#pragma unroll
          for (int u = 0; u < U; ++u) {
            Acc acc[N];
            const T *e0 = (const T *)&v[u][0];
#pragma unroll
            for (int i = 0; i < N; ++i) acc[i] = toAcc<T>(e0[i]);
#pragma unroll
            for (int p = 1; p < NR; ++p) {
              const T *ep = (const T *)&v[u][p];
#pragma unroll
              for (int i = 0; i < N; ++i) acc[i] = combine<OP, Acc>(acc[i], toAcc<T>(ep[i]), a.redOp);
            }
            storePack(a, dst, nDst, dstBase + e + u * stride, acc);
          }
        }
      }
      for (; e < fullEnd; e += stride) {
        Acc acc[N];
        loadReduce(a, nRanks, (sb + e) * sizeof(T), acc);
        storePack(a, dst, nDst, dstBase + e, acc);
      }
      eb = fullEnd > eb ? fullEnd : eb;
    }
    for (size_t e = eb + threadIdx.x; e < ee; e += blockDim.x) {
      Acc acc = toAcc<T>(ldSysElem((const T *)a.in[0] + sb + e));
      for (int p = 1; p < nRanks; ++p)
        acc = combine<OP, Acc>(acc, toAcc<T>(ldSysElem((const T *)a.in[p] + sb + e)), a.redOp);
      storeOne(a, dst, nDst, dstBase + e, acc);
    }
  }

  // The same reduction with the inputs brought in by the bulk-copy engine: one thread
  // asks for a piece (16 bytes per thread) of every rank's input at once, peers
  // included, into one stage of the shared-memory ring; all threads then reduce
  // out of shared memory.  Needs NR > 0, 16-byte aligned inputs and whole packs.
  // Loads are plain bulk copies: none is multicast.  Returns false after a timeout.
  static __device__ bool sliceBulk(const flagcxDevComm &c, const CollArgs &a, size_t sb, size_t se, char *const *dst,
                                   int nDst, size_t dstBase, int b, int g) {
    constexpr int R = NR > 0 ? NR : 1;
    __shared__ __align__(8) uint64_t full[kBulkMaxStages], empty[kBulkMaxStages];
    __shared__ int abortS;
    const int nt = blockDim.x, tid = threadIdx.x;
    const uint32_t pieceBytes = (uint32_t)nt * 16u, stageBytes = pieceBytes * R;
    int stages = (int)(kBulkRingBytes / stageBytes);
    if (stages > kBulkMaxStages) stages = kBulkMaxStages;
    const int ahead = stages - 1;
    size_t ub, ue;
    ctaShare((se - sb) * sizeof(T) >> 4, b, g, &ub, &ue);
    const size_t nPieces = (ue - ub + nt - 1) / nt;
    const uint32_t ring = smem32(bulkRing);
    if (tid == 0) {
      abortS = 0;
      for (int s = 0; s < stages; ++s) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem32(&full[s])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem32(&empty[s])), "r"(nt >> 5) : "memory");
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async;" ::: "memory"); // a copy-in by this CTA's threads precedes the engine's reads
    __syncthreads();

    auto issue = [&](size_t j) {
      const int s = (int)(j % stages);
      const size_t first = ub + j * nt;
      const uint32_t sz = (uint32_t)((ue - first) < (size_t)nt ? (ue - first) : (size_t)nt) * 16u;
      const uint32_t bar = smem32(&full[s]);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(sz * R) : "memory");
      for (int k = 0; k < R; ++k) {
        int p = c.rank + 1 + k; // peers first, each rank starting with a different one
        if (p >= R) p -= R;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         ring + s * stageBytes + p * pieceBytes),
                     "l"(a.in[p] + sb * sizeof(T) + (first << 4)), "r"(sz), "r"(bar)
                     : "memory");
      }
    };

    if (tid == 0)
      for (size_t j = 0; j < nPieces && j < (size_t)ahead; ++j) issue(j);
    bool ok = true;
    for (size_t i = 0; i < nPieces; ++i) {
      if (tid == 0 && i + ahead < nPieces) {
        const size_t j = i + ahead;
        if (j >= (size_t)stages) ok = mbarWaitBounded(c, &empty[j % stages], (uint32_t)(j / stages - 1) & 1u, &abortS);
        if (ok) issue(j);
      }
      const int s = (int)(i % stages);
      if (ok) ok = mbarWaitBounded(c, &full[s], (uint32_t)(i / stages) & 1u, &abortS);
      if (!ok) break;
      const size_t pack = ub + i * nt + tid;
      if (pack < ue) {
        const uint4 *stage = (const uint4 *)(bulkRing + (size_t)s * stageBytes);
        uint4 v[R];
#pragma unroll
        for (int p = 0; p < R; ++p) v[p] = stage[p * nt + tid];
        Acc acc[N];
        const T *e0 = (const T *)&v[0];
#pragma unroll
        for (int i2 = 0; i2 < N; ++i2) acc[i2] = toAcc<T>(e0[i2]);
#pragma unroll
        for (int p = 1; p < R; ++p) {
          const T *ep = (const T *)&v[p];
#pragma unroll
          for (int i2 = 0; i2 < N; ++i2) acc[i2] = combine<OP, Acc>(acc[i2], toAcc<T>(ep[i2]), a.redOp);
        }
        storePack(a, dst, nDst, dstBase + pack * N, acc);
      }
      __syncwarp();
      if ((tid & 31) == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem32(&empty[s])) : "memory");
    }
    if (!ok && tid == 0) fcxdev::reportError(c.status, FLAGCX_DEV_TIMEOUT, FLAGCX_DEV_AT_KERNEL, (unsigned)b, 0);
    return !__syncthreads_or(ok ? 0 : 1);
  }
};

// Second phase of the casting two-shot all-reduce: `elems` 16-bit values of a reduced
// slice (local or a peer's scratch) become fp32 in the local output, plus an optional
// fp32 residual.  The CTA takes the share of the slice that the same CTA of the
// slice's owner produced (same partition as Reducer::slice).
template <typename T>
__device__ void widenSlice(const T *src, float *dst, size_t elems, const float *residual, int b, int g) {
  constexpr int N = 8;
  size_t ub, ue;
  ctaShare((elems * sizeof(T) + 15) >> 4, b, g, &ub, &ue);
  const size_t eb = ub * N, ee = ue * N < elems ? ue * N : elems;
  if (eb >= ee) return;
  const bool vec = ((((uintptr_t)src) | ((uintptr_t)dst) | ((uintptr_t)residual)) & 15) == 0;
  size_t done = eb;
  if (vec) {
    const size_t fullEnd = ee / N * N, stride = (size_t)blockDim.x * N;
    auto emit = [&](size_t e, uint4 v) {
      const T *h = (const T *)&v;
      float f[N];
#pragma unroll
      for (int i = 0; i < N; ++i) f[i] = toAcc<T>(h[i]);
      if (residual) {
        uint4 r0 = ldLocal16(residual + e), r1 = ldLocal16(residual + e + 4);
        const float *ra = (const float *)&r0, *rb = (const float *)&r1;
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[i] += ra[i]; f[4 + i] += rb[i]; }
      }
      st16(dst + e, *(uint4 *)&f[0]);
      st16(dst + e + 4, *(uint4 *)&f[4]);
    };
    size_t e = eb + (size_t)threadIdx.x * N;
    for (; e + 3 * stride < fullEnd; e += 4 * stride) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = ldSys16(src + e + u * stride);
#pragma unroll
      for (int u = 0; u < 4; ++u) emit(e + u * stride, v[u]);
    }
    for (; e < fullEnd; e += stride) emit(e, ldSys16(src + e));
    done = fullEnd > eb ? fullEnd : eb;
  }
  for (size_t e = done + threadIdx.x; e < ee; e += blockDim.x) {
    float x = toAcc<T>(ldSysElem(src + e));
    if (residual) x += residual[e];
    dst[e] = x;
  }
}

// One hop of a ring reduction: dst[i] = x[i] (op) y[i] over this CTA's share of `elems`
// elements (y may be null: a plain copy), accumulating in the wider type.  `last` applies
// the scale / integer division of the epilogue.  dst may be peer memory.
template <typename T, int OP>
__device__ void ringCombine(const CollArgs &a, T *dst, const T *x, const T *y, size_t elems, bool last, int b, int g) {
  using Acc = typename Elem<T>::Acc;
  constexpr int N = 16 / (int)sizeof(T);
  size_t ub, ue;
  ctaShare((elems * sizeof(T) + 15) >> 4, b, g, &ub, &ue);
  const size_t eb = ub * N, ee = ue * N < elems ? ue * N : elems;
  if (eb >= ee) return;
  const bool vec = ((((uintptr_t)dst) | ((uintptr_t)x) | ((uintptr_t)y)) & 15) == 0;
  size_t done = eb;
  if (vec) {
    const size_t fullEnd = ee / N * N, stride = (size_t)blockDim.x * N;
    auto emit = [&](size_t e, uint4 vx, uint4 vy) {
      const T *px = (const T *)&vx, *py = (const T *)&vy;
      uint4 o;
      T *po = (T *)&o;
#pragma unroll
      for (int i = 0; i < N; ++i) {
        Acc v = toAcc<T>(px[i]);
        if (y) v = combine<OP, Acc>(v, toAcc<T>(py[i]), a.redOp);
        if (last) v = finish<Acc>(v, a.scale, a.divisor);
        po[i] = fromAcc<T>(v);
      }
      st16(dst + e, o);
    };
    size_t e = eb + (size_t)threadIdx.x * N;
    for (; e + 3 * stride < fullEnd; e += 4 * stride) {
      uint4 vx[4], vy[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        vx[u] = ldSys16(x + e + u * stride);
        vy[u] = y ? ldSys16(y + e + u * stride) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) emit(e + u * stride, vx[u], vy[u]);
    }
    for (; e < fullEnd; e += stride) emit(e, ldSys16(x + e), y ? ldSys16(y + e) : make_uint4(0, 0, 0, 0));
    done = fullEnd > eb ? fullEnd : eb;
  }
  for (size_t e = done + threadIdx.x; e < ee; e += blockDim.x) {
    Acc v = toAcc<T>(ldSysElem(x + e));
    if (y) v = combine<OP, Acc>(v, toAcc<T>(ldSysElem(y + e)), a.redOp);
    if (last) v = finish<Acc>(v, a.scale, a.divisor);
    dst[e] = fromAcc<T>(v);
  }
}

// Ring reduce-scatter over blocks [blockBegin(i), blockBegin(i) + blockLen(i)) of the
// inputs; rank r ends up with the complete block r in `result` (n-1 hops, each adding the
// sender's own contribution to the partial sum it received).  Returns false after a
// timed-out wait.
template <typename T, int OP>
__device__ bool ringReduceScatter(const flagcxDevComm &c, const CollArgs &a, size_t blockElems, size_t totalElems,
                                  T *result, int b, int g) {
  const int rank = c.rank, n = c.nRanks, next = (rank + 1) % n, prev = (rank + n - 1) % n;
  const T *own = (const T *)a.in[rank];
  auto begin = [&](int i) { size_t s = blockElems * (size_t)i; return s < totalElems ? s : totalElems; };
  auto len = [&](int i) { size_t s = begin(i); return s + blockElems < totalElems ? blockElems : totalElems - s; };
  T *mine = (T *)a.aux[rank], *theirs = (T *)a.aux[next];
  for (int s = 0; s < n - 1; ++s) {
    int ci = rank - s - 1; while (ci < 0) ci += n;
    ringCombine<T, OP>(a, theirs + (size_t)s * a.ringSlotElems, own + begin(ci),
                       s > 0 ? mine + (size_t)(s - 1) * a.ringSlotElems : (const T *)nullptr, len(ci), false, b, g);
    ctaRaiseFlag(a.ringNext + b, a.ringBase + s + 1);
    if (!ctaWaitFlag(c, a.ringMine + b, a.ringBase + s + 1, (unsigned)prev)) return false;
  }
  ringCombine<T, OP>(a, result, own + begin(rank), n > 1 ? mine + (size_t)(n - 2) * a.ringSlotElems : (const T *)nullptr,
                     len(rank), true, b, g);
  return true;
}

template <typename T, int OP, int NR>
__device__ void reduceBody(const flagcxDevComm &c, CollArgs &a) {
  const int b = blockIdx.x, g = gridDim.x, rank = c.rank, n = c.nRanks;
  using R = Reducer<T, OP, NR>;

  copyIn(a, rank, b, g);
  publishPointers(c, a, b);
  if (a.flags & kFlagBeginBarrier)
    if (!ctaBarrier(c, b)) return;
  learnPointers(c, a, b);
  const bool bulk = NR > 0 && a.bulkStage && learntPointersAligned(c, a);

  char *local[1] = {a.out[rank]};
  switch (a.kind) {
    case kAllReduceOneShot:
      R::slice(a, n, 0, a.count, local, 1, 0, b, g);
      break;
    case kAllReduceTwoShot: {
      size_t s = sliceElems(a.count, n, sizeof(T));
      size_t sb = s * rank < a.count ? s * rank : a.count;
      size_t se = sb + s < a.count ? sb + s : a.count;
      if (bulk) {
        if (!R::sliceBulk(c, a, sb, se, a.out, n, sb, b, g)) return;
      } else {
        R::slice(a, n, sb, se, a.out, n, sb, b, g);
      }
      break;
    }
    case kReduceScatter: {
      size_t sb = a.inStride / sizeof(T) * rank;
      if (bulk) {
        if (!R::sliceBulk(c, a, sb, sb + a.count, local, 1, 0, b, g)) return;
      } else {
        R::slice(a, n, sb, sb + a.count, local, 1, 0, b, g);
      }
      break;
    }
    case kReduceToRoot:
      if (rank == a.root) R::slice(a, n, 0, a.count, local, 1, 0, b, g);
      break;
    case kReduceScatterRing:
      if (!ringReduceScatter<T, OP>(c, a, a.count, a.count * (size_t)n, (T *)a.out[rank], b, g)) return;
      break;
    case kAllReduceRing: {
      // reduce-scatter into this rank's block of its own output, then pass the finished
      // blocks round the ring: after step s a rank holds blocks rank, rank-1, .., rank-s-1
      const size_t s = sliceElems(a.count, n, sizeof(T));
      auto begin = [&](int i) { size_t x = s * (size_t)i; return x < a.count ? x : a.count; };
      auto len = [&](int i) { size_t x = begin(i); return x + s < a.count ? s : a.count - x; };
      T *myOut = (T *)a.out[rank];
      if (!ringReduceScatter<T, OP>(c, a, s, a.count, myOut + begin(rank), b, g)) return;
      const int next = (rank + 1) % n, prev = (rank + n - 1) % n;
      for (int st = 0; st < n - 1; ++st) {
        int bi = rank - st; while (bi < 0) bi += n;
        ringCombine<T, OP>(a, (T *)a.out[next] + begin(bi), myOut + begin(bi), (const T *)nullptr, len(bi), false, b, g);
        ctaRaiseFlag(a.ringNext + b, a.ringBase + (n - 1) + st + 1);
        if (!ctaWaitFlag(c, a.ringMine + b, a.ringBase + (n - 1) + st + 1, (unsigned)prev)) return;
      }
      break;
    }
    case kAllReduceTwoShotCast: {
      // 16-bit inputs, fp32 result.  Sending fp32 to every peer would double the NVLink
      // bytes, so each rank rounds its reduced (and scaled) slice once to the input type
      // into its own scratch, and every rank then pulls all slices and widens them while
      // writing its output: the same bytes cross NVLink as in the plain all-reduce, and
      // all ranks end up with identical values.
      if constexpr (sizeof(T) == 2) {
        const size_t s = sliceElems(a.count, n, sizeof(T));
        const size_t sb = s * rank < a.count ? s * rank : a.count;
        const size_t se = sb + s < a.count ? sb + s : a.count;
        const char *residual = a.residual;
        __syncthreads();
        if (threadIdx.x == 0) { a.outMode = kOutSame; a.residual = nullptr; }
        __syncthreads();
        char *scratch[1] = {a.aux[rank]};
        if (bulk) {
          if (!R::sliceBulk(c, a, sb, se, scratch, 1, 0, b, g)) return;
        } else {
          R::slice(a, n, sb, se, scratch, 1, 0, b, g);
        }
        if (!ctaBarrier(c, b)) return;
        for (int k = 0; k < n; ++k) {
          int p = rank + k; if (p >= n) p -= n;
          const size_t pb = s * p < a.count ? s * p : a.count;
          const size_t pe = pb + s < a.count ? pb + s : a.count;
          widenSlice<T>((const T *)a.aux[p], (float *)a.out[rank] + pb, pe - pb,
                        residual ? (const float *)residual + pb : nullptr, b, g);
        }
      }
      break;
    }
    default: break;
  }

  if (a.flags & kFlagEndBarrier)
    if (!ctaBarrier(c, b)) return;
  copyOut(a, rank, b, g);
}

// ---------------------------------------------------------------------------
// LL family: small messages without any barrier
// ---------------------------------------------------------------------------
// Every 8 bytes of data travel in one 16-byte store {data0, flag, data1, flag} into a
// slot that the receiver owns per sender; the receiver spins (bounded) until both
// flags carry this operation's value, so data and "it has arrived" are one message.
// Slots alternate between two parities: a rank can be at most one operation ahead of
// a peer (it needs the peer's data to finish the current one), so the slot of operation
// k is free again when operation k+2 writes it.  Only kinds in which every rank
// receives from every rank may use this (all-reduce, all-gather).
__device__ __forceinline__ void llLoadUnit(const char *src, size_t bytes, size_t u, uint32_t &d0, uint32_t &d1) {
  const size_t off = u << 3;
  if (off + 8 <= bytes && (((uintptr_t)src) & 7) == 0) {
    uint2 v = *(const uint2 *)(src + off);
    d0 = v.x;
    d1 = v.y;
    return;
  }
  unsigned char t[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (int i = 0; i < 8; ++i)
    if (off + i < bytes) t[i] = (unsigned char)src[off + i];
  d0 = (uint32_t)t[0] | ((uint32_t)t[1] << 8) | ((uint32_t)t[2] << 16) | ((uint32_t)t[3] << 24);
  d1 = (uint32_t)t[4] | ((uint32_t)t[5] << 8) | ((uint32_t)t[6] << 16) | ((uint32_t)t[7] << 24);
}
__device__ __forceinline__ void llStoreUnit(char *dst, size_t bytes, size_t u, uint32_t d0, uint32_t d1) {
  const size_t off = u << 3;
  if (off + 8 <= bytes && (((uintptr_t)dst) & 7) == 0) {
    *(uint2 *)(dst + off) = make_uint2(d0, d1);
    return;
  }
  for (int i = 0; i < 8; ++i)
    if (off + i < bytes) dst[off + i] = (char)(((i < 4 ? d0 : d1) >> (8 * (i & 3))) & 0xffu);
}
__device__ __forceinline__ void llSend(char *slot, uint32_t d0, uint32_t d1, uint32_t flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(slot), "r"(d0), "r"(flag), "r"(d1), "r"(flag)
               : "memory");
}
__device__ __forceinline__ bool llRecv(const flagcxDevComm &c, const char *slot, uint32_t flag, uint32_t &d0,
                                       uint32_t &d1, unsigned peer) {
  unsigned long long t0 = 0;
  for (unsigned spins = 0;; ++spins) {
    uint32_t f0, f1;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(d0), "=r"(f0), "=r"(d1), "=r"(f1)
                 : "l"(slot)
                 : "memory");
    if (f0 == flag && f1 == flag) return true;
    if ((spins & 1023u) == 1023u) {
      if (c.status && fcxdev::ldVolatileU32(&c.status->abortFlag)) {
        fcxdev::reportError(c.status, FLAGCX_DEV_ABORTED, FLAGCX_DEV_AT_KERNEL, peer, flag);
        return false;
      }
      if (t0 == 0) t0 = fcxdev::globalTimerNs();
      else if (fcxdev::globalTimerNs() - t0 > c.timeoutNs) {
        fcxdev::reportError(c.status, FLAGCX_DEV_TIMEOUT, FLAGCX_DEV_AT_KERNEL, peer, flag);
        return false;
      }
    }
  }
}

template <typename T>
__device__ void llBody(const flagcxDevComm &c, const CollArgs &a) {
  using Acc = typename Elem<T>::Acc;
  constexpr int N = 8 / (int)sizeof(T);
  const int rank = c.rank, n = c.nRanks;
  const size_t bytes = a.count * sizeof(T); // all-reduce: the message; all-gather: one rank's block
  const size_t units = (bytes + 7) >> 3;
  const size_t parityOff = (size_t)(a.llEpoch & 1u) * FLAGCX_MAX_RANKS * a.llSlotBytes;
  const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nt = (size_t)gridDim.x * blockDim.x;
  const char *in = a.in[rank];
  for (size_t u = t; u < units; u += nt) {
    uint32_t d0, d1;
    llLoadUnit(in, bytes, u, d0, d1);
    for (int k = 1; k < n; ++k) {
      int p = rank + k; if (p >= n) p -= n;
      llSend(a.aux[p] + parityOff + (size_t)rank * a.llSlotBytes + (u << 4), d0, d1, a.llEpoch);
    }
  }
  const char *mine = a.aux[rank] + parityOff;
  for (size_t u = t; u < units; u += nt) {
    if (a.kind == kLlAllReduce) {
      Acc acc[N];
      for (int p = 0; p < n; ++p) { // rank order: every rank computes bit-identical results
        uint32_t w[2];
        if (p == rank) llLoadUnit(in, bytes, u, w[0], w[1]);
        else if (!llRecv(c, mine + (size_t)p * a.llSlotBytes + (u << 4), a.llEpoch, w[0], w[1], (unsigned)p)) return;
        const T *e = (const T *)w;
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] = p == 0 ? toAcc<T>(e[i]) : combine<kOpRuntime, Acc>(acc[i], toAcc<T>(e[i]), a.redOp);
      }
      uint32_t o[2];
      T *oe = (T *)o;
#pragma unroll
      for (int i = 0; i < N; ++i) oe[i] = fromAcc<T>(finish<Acc>(acc[i], a.scale, a.divisor));
      llStoreUnit(a.out[rank], bytes, u, o[0], o[1]);
    } else {
      for (int k = 0; k < n; ++k) {
        int p = rank + k; if (p >= n) p -= n;
        uint32_t d0, d1;
        if (p == rank) llLoadUnit(in, bytes, u, d0, d1);
        else if (!llRecv(c, mine + (size_t)p * a.llSlotBytes + (u << 4), a.llEpoch, d0, d1, (unsigned)p)) return;
        llStoreUnit(a.out[rank] + a.outStride * p, bytes, u, d0, d1);
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    llKernel(const __grid_constant__ flagcxDevComm c, const __grid_constant__ CollArgs a) {
  llBody<T>(c, a);
}
template <typename T>
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    llKernelEmu(const flagcxDevComm *cs, const CollArgs *as) {
  llBody<T>(cs[blockIdx.y], as[blockIdx.y]);
}

template <typename T, int OP, int NR>
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    reduceKernel(const __grid_constant__ flagcxDevComm c, const __grid_constant__ CollArgs a) {
  reduceBody<T, OP, NR>(c, stageArgs(a));
}

// Emulated world: one cooperative launch, blockIdx.y plays the rank.
template <typename T, int OP, int NR>
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    reduceKernelEmu(const flagcxDevComm *cs, const CollArgs *as) {
  reduceBody<T, OP, NR>(cs[blockIdx.y], stageArgs(as[blockIdx.y]));
}

// ---------------------------------------------------------------------------
// copy family (no arithmetic: byte movers)
// ---------------------------------------------------------------------------
// One read of the source, one store per destination.
__device__ void ctaFanOut(char *const *dst, int nDst, const char *src, size_t bytes, int b, int g) {
  size_t ub, ue;
  ctaShare((bytes + 15) >> 4, b, g, &ub, &ue);
  size_t bb = ub << 4, be = (ue << 4) < bytes ? (ue << 4) : bytes;
  if (bb >= be) return;
  bool vec = (((uintptr_t)src) & 15) == 0;
  for (int d = 0; d < nDst; ++d) vec &= (((uintptr_t)dst[d]) & 15) == 0;
  const int t = threadIdx.x, nt = blockDim.x;
  size_t done = bb;
  if (vec) {
    size_t ve = be >> 4;
    size_t i = ub + t;
    // The stores to the peers are posted; what bounds a CTA's rate is how many local
    // loads it keeps in flight.  Eight 16-byte loads per thread (64 KiB per CTA) let a
    // dozen or so CTAs fill the links, which matters when GEMMs want the other SMs.
    for (; i + 7 * (size_t)nt < ve; i += 8 * (size_t)nt) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = ldSys16(src + ((i + u * (size_t)nt) << 4));
      for (int d = 0; d < nDst; ++d) {
#pragma unroll
        for (int u = 0; u < 8; ++u) st16(dst[d] + ((i + u * (size_t)nt) << 4), v[u]);
      }
    }
    for (; i < ve; i += nt) {
      uint4 v = ldSys16(src + (i << 4));
      for (int d = 0; d < nDst; ++d) st16(dst[d] + (i << 4), v);
    }
    done = ve > ub ? (ve << 4) : bb;
  }
  for (size_t i = done + t; i < be; i += nt) {
    char v = src[i];
    for (int d = 0; d < nDst; ++d) dst[d][i] = v;
  }
}

// ---- bulk-copy path of the push kinds ---------------------------------------------
// One thread per CTA drives the copy engine: untiled bulk copies bring 16 KiB pieces
// of LOCAL memory into a ring of shared-memory stages (completion on an mbarrier), and
// bulk stores send each stage on to its destination(s) in peer memory.  The loads run
// half a ring ahead of the stores; a stage is reloaded only after the stores
// that read it have left shared memory (wait_group.read).  No load here names a
// peer and none is multicast; sources, destinations and sizes are multiples of 16.

// K destinations; sameSrc: every piece of src[0] goes to all of them (all-gather,
// broadcast), else piece i of src[k] goes to dst[k] (all-to-all), peers interleaved.
// Runs in ONE thread.  Returns false after a timed-out wait.
__device__ bool bulkMoveThread(const flagcxDevComm &c, uint64_t *full, const char *const *src, char *const *dst, int K,
                               bool sameSrc, size_t bb, size_t be, uint32_t stageBytes, int stages) {
  if (bb >= be || K == 0) return true;
  const int ahead = stages / 2;
  for (int s = 0; s < stages; ++s)
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem32(&full[s])) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async;" ::: "memory");
  const size_t chunks = (be - bb + stageBytes - 1) / stageBytes;
  const size_t items = sameSrc ? chunks : chunks * (size_t)K;
  const uint32_t ring = smem32(bulkRing);

  auto issueLoad = [&](size_t it) {
    const size_t ch = sameSrc ? it : it / K;
    const int k = sameSrc ? 0 : (int)(it % K);
    const size_t off = bb + ch * stageBytes;
    const uint32_t sz = (uint32_t)((be - off) < stageBytes ? (be - off) : stageBytes);
    const int s = (int)(it % stages);
    const uint32_t bar = smem32(&full[s]);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(sz) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     ring + s * stageBytes),
                 "l"(src[k] + off), "r"(sz), "r"(bar)
                 : "memory");
  };

  for (size_t it = 0; it < items && it < (size_t)ahead; ++it) issueLoad(it);
  bool ok = true;
  for (size_t it = 0; it < items; ++it) {
    if (it + ahead < items) {
      // the stage about to be reloaded was last read by the stores of item it+ahead-stages
      // (at most stages - ahead - 1 younger store groups may still be reading)
      if (stages == 8) asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory");
      else asm volatile("cp.async.bulk.wait_group.read 5;" ::: "memory");
      issueLoad(it + ahead);
    }
    const int s = (int)(it % stages);
    const uint32_t bar = smem32(&full[s]), parity = (uint32_t)(it / stages) & 1u;
    uint32_t done = 0;
    unsigned long long t0 = 0;
    for (unsigned spins = 0; !done; ++spins) {
      asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                   : "=r"(done)
                   : "r"(bar), "r"(parity)
                   : "memory");
      if (!done && (spins & 255u) == 255u) {
        if (t0 == 0) t0 = fcxdev::globalTimerNs();
        else if (fcxdev::globalTimerNs() - t0 > c.timeoutNs) { ok = false; break; }
      }
    }
    if (!ok) {
      fcxdev::reportError(c.status, FLAGCX_DEV_TIMEOUT, FLAGCX_DEV_AT_KERNEL, (unsigned)blockIdx.x, it);
      break;
    }
    const size_t ch = sameSrc ? it : it / K;
    const size_t off = bb + ch * stageBytes;
    const uint32_t sz = (uint32_t)((be - off) < stageBytes ? (be - off) : stageBytes);
    const uint32_t from = ring + s * stageBytes;
    if (sameSrc) {
      for (int k = 0; k < K; ++k)
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst[k] + off), "r"(from), "r"(sz)
                     : "memory");
    } else {
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst[it % K] + off), "r"(from),
                   "r"(sz)
                   : "memory");
    }
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  }
  // every store has been written before the closing barrier releases the peers
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  asm volatile("fence.proxy.async;" ::: "memory");
  return ok;
}

// All threads call this; returns false (in all of them) after a timed-out wait.
__device__ bool ctaBulkMove(const flagcxDevComm &c, const char *const *src, char *const *dst, int K, bool sameSrc,
                            size_t bytes, int b, int g, uint32_t stageBytes, int stages) {
  __shared__ __align__(8) uint64_t full[kBulkMaxStages];
  __shared__ int okShared;
  size_t ub, ue;
  ctaShare(bytes >> 4, b, g, &ub, &ue);
  asm volatile("fence.proxy.async;" ::: "memory"); // a copy-in by this CTA's threads precedes the engine's reads
  __syncthreads();
  if (threadIdx.x == 0) okShared = bulkMoveThread(c, full, src, dst, K, sameSrc, ub << 4, ue << 4, stageBytes, stages) ? 1 : 0;
  __syncthreads();
  return okShared != 0;
}

__device__ void ctaCopyShare(char *dst, const char *src, size_t bytes, int b, int g) {
  size_t ub, ue;
  ctaShare((bytes + 15) >> 4, b, g, &ub, &ue);
  size_t bb = ub << 4, be = (ue << 4) < bytes ? (ue << 4) : bytes;
  ctaCopy(dst, src, bb, be);
}

__device__ void copyBody(const flagcxDevComm &c, CollArgs &a) {
  const int b = blockIdx.x, g = gridDim.x, rank = c.rank, n = c.nRanks;
  const size_t es = a.elemSize;
  const size_t blk = a.count * es;

  if (a.kind == kAllToAllvPull) {
    // publish where each peer finds its block in my input (every CTA writes the
    // same values: its peers' CTAs of the same index read them after the barrier)
    unsigned long long *m = a.meta[rank];
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
      m[i] = a.sendDispls[i];
      m[FLAGCX_MAX_RANKS + i] = a.sendCounts[i];
    }
  }
  copyIn(a, rank, b, g);
  publishPointers(c, a, b);
  if (a.flags & kFlagBeginBarrier)
    if (!ctaBarrier(c, b)) return;
  learnPointers(c, a, b);
  const bool bulk = a.bulkStage && learntPointersAligned(c, a);

  switch (a.kind) {
    case kAllGatherPush: {
      char *dst[FLAGCX_MAX_RANKS];
      int nd = 0;
      for (int k = 0; k < n; ++k) {
        int p = rank + k; if (p >= n) p -= n;
        char *d = a.out[p] + a.outStride * rank;
        if (p == rank && d == a.in[rank]) continue; // in place
        dst[nd++] = d;
      }
      if (bulk) {
        const char *src0 = a.in[rank];
        if (!ctaBulkMove(c, &src0, dst, nd, true, blk, b, g, a.bulkStage, a.bulkDepth)) return;
      } else {
        ctaFanOut(dst, nd, a.in[rank], blk, b, g);
      }
      break;
    }
    case kAllGatherRing: {
      // step s: pass block (rank - s) on to the next rank; own block first, then whatever
      // arrived in the step before
      const int next = (rank + 1) % n, prev = (rank + n - 1) % n;
      char *mine = a.out[rank];
      if (a.in[rank] != mine + a.outStride * rank) ctaCopyShare(mine + a.outStride * rank, a.in[rank], blk, b, g);
      for (int s = 0; s < n - 1; ++s) {
        int bi = rank - s; while (bi < 0) bi += n;
        ctaCopyShare(a.out[next] + a.outStride * bi, s == 0 ? a.in[rank] : mine + a.outStride * bi, blk, b, g);
        ctaRaiseFlag(a.ringNext + b, a.ringBase + s + 1);
        if (!ctaWaitFlag(c, a.ringMine + b, a.ringBase + s + 1, (unsigned)prev)) return;
      }
      break;
    }
    case kAllGatherPull:
      for (int k = 0; k < n; ++k) {
        int p = rank + k; if (p >= n) p -= n;
        char *d = a.out[rank] + a.outStride * p;
        if (p == rank && a.in[p] == d) continue;
        ctaCopyShare(d, a.in[p], blk, b, g);
      }
      break;
    case kBroadcastPush:
      if (rank == a.root) {
        char *dst[FLAGCX_MAX_RANKS];
        int nd = 0;
        for (int k = 0; k < n; ++k) {
          int p = rank + k; if (p >= n) p -= n;
          if (p == rank && a.in[rank] == a.out[rank]) continue;
          dst[nd++] = a.out[p];
        }
        if (bulk) {
          const char *src0 = a.in[rank];
          if (!ctaBulkMove(c, &src0, dst, nd, true, blk, b, g, a.bulkStage, a.bulkDepth)) return;
        } else {
          ctaFanOut(dst, nd, a.in[rank], blk, b, g);
        }
      }
      break;
    case kBroadcastPull:
      if (!(rank == a.root && a.in[rank] == a.out[rank])) ctaCopyShare(a.out[rank], a.in[a.root], blk, b, g);
      break;
    case kGatherPull:
      if (rank == a.root)
        for (int k = 0; k < n; ++k) {
          int p = rank + k; if (p >= n) p -= n;
          ctaCopyShare(a.out[rank] + a.outStride * p, a.in[p], blk, b, g);
        }
      break;
    case kScatterPull:
      ctaCopyShare(a.out[rank], a.in[a.root] + a.inStride * rank, blk, b, g);
      break;
    case kAllToAllPush:
    case kAllToAllPull: {
      // one block per peer; all peers' blocks advance together so that every link is
      // busy at once and each thread keeps one access per peer in flight
      const char *src[FLAGCX_MAX_RANKS];
      char *dst[FLAGCX_MAX_RANKS];
      bool vec = true;
      for (int k = 0; k < n; ++k) {
        int p = rank + k; if (p >= n) p -= n;
        if (a.kind == kAllToAllPush) {
          src[k] = a.in[rank] + a.inStride * p;
          dst[k] = a.out[p] + a.outStride * rank;
        } else {
          src[k] = a.in[p] + a.inStride * rank;
          dst[k] = a.out[rank] + a.outStride * p;
        }
        vec &= ((((uintptr_t)src[k]) | ((uintptr_t)dst[k])) & 15) == 0;
      }
      if (bulk && a.kind == kAllToAllPush) {
        if (!ctaBulkMove(c, src, dst, n, false, blk, b, g, a.bulkStage, a.bulkDepth)) return;
        break;
      }
      if (!vec) {
        for (int k = 0; k < n; ++k) ctaCopyShare(dst[k], src[k], blk, b, g);
        break;
      }
      size_t ub, ue;
      ctaShare((blk + 15) >> 4, b, g, &ub, &ue);
      const size_t ve = blk >> 4 < ue ? blk >> 4 : ue; // whole 16-byte packs of this CTA's share
      const int t = threadIdx.x, nt = blockDim.x;
      size_t i = ub + t;
      for (; i + nt < ve; i += 2 * (size_t)nt) {
        uint4 v0[FLAGCX_MAX_RANKS], v1[FLAGCX_MAX_RANKS];
#pragma unroll
        for (int k = 0; k < FLAGCX_MAX_RANKS; ++k)
          if (k < n) { v0[k] = ldSys16(src[k] + (i << 4)); v1[k] = ldSys16(src[k] + ((i + nt) << 4)); }
#pragma unroll
        for (int k = 0; k < FLAGCX_MAX_RANKS; ++k)
          if (k < n) { st16(dst[k] + (i << 4), v0[k]); st16(dst[k] + ((i + nt) << 4), v1[k]); }
      }
      for (; i < ve; i += nt) {
#pragma unroll
        for (int k = 0; k < FLAGCX_MAX_RANKS; ++k)
          if (k < n) st16(dst[k] + (i << 4), ldSys16(src[k] + (i << 4)));
      }
      // bytes past the last whole pack of the block (the last CTA share only)
      const size_t tailBegin = (blk >> 4) << 4;
      if (ub < ue && ue * 16 >= blk && tailBegin < blk)
        for (int k = 0; k < n; ++k)
          for (size_t j = tailBegin + t; j < blk; j += nt) dst[k][j] = src[k][j];
      break;
    }
    case kAllToAllvPull:
      for (int k = 0; k < n; ++k) {
        int p = rank + k; if (p >= n) p -= n;
        unsigned long long displ = fcxdev::ldRelaxedSys(a.meta[p] + rank);
        unsigned long long cnt = fcxdev::ldRelaxedSys(a.meta[p] + FLAGCX_MAX_RANKS + rank);
        if (cnt != a.recvCounts[p]) {
          if (threadIdx.x == 0 && b == 0)
            fcxdev::reportError(c.status, FLAGCX_DEV_BOUNDS, FLAGCX_DEV_AT_KERNEL, (unsigned)p, cnt);
          continue;
        }
        ctaCopyShare(a.out[rank] + a.recvDispls[p] * es, a.in[p] + displ * es, cnt * es, b, g);
      }
      break;
    default: break;
  }

  if (a.flags & kFlagEndBarrier)
    if (!ctaBarrier(c, b)) return;
  copyOut(a, rank, b, g);
}

__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    copyKernel(const __grid_constant__ flagcxDevComm c, const __grid_constant__ CollArgs a) {
  copyBody(c, stageArgs(a));
}
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    copyKernelEmu(const flagcxDevComm *cs, const CollArgs *as) {
  copyBody(cs[blockIdx.y], stageArgs(as[blockIdx.y]));
}

// ---------------------------------------------------------------------------
// grouped point-to-point (see P2pArgs)
// ---------------------------------------------------------------------------
__device__ void p2pBody(const flagcxDevComm &c, const P2pArgs &a) {
  const int b = blockIdx.x, g = gridDim.x, rank = c.rank, n = c.nRanks;
  const size_t slot = a.slotBytes;
  if (a.sendSrc[rank] && a.recvDst[rank] && a.sendBytes[rank])
    ctaCopyShare(a.recvDst[rank], a.sendSrc[rank], a.sendBytes[rank], b, g);
  size_t maxIter = 0;
  for (int p = 0; p < n; ++p) {
    if (p == rank) continue;
    size_t s = a.sendSrc[p] ? (a.sendBytes[p] + slot - 1) / slot : 0;
    size_t r = a.recvDst[p] ? (a.recvBytes[p] + slot - 1) / slot : 0;
    maxIter = s > maxIter ? s : maxIter;
    maxIter = r > maxIter ? r : maxIter;
  }
  for (size_t i = 0; i < maxIter; ++i) {
    for (int k = 1; k < n; ++k) { // sends of this step
      int p = rank + k; if (p >= n) p -= n;
      if (!a.sendSrc[p] || i * slot >= a.sendBytes[p]) continue;
      size_t len = a.sendBytes[p] - i * slot < slot ? a.sendBytes[p] - i * slot : slot;
      unsigned long long seq = a.sendSeq[p] + i + 1;
      // the receiver must have drained the previous chunk out of this slot
      if (!ctaWaitFlag(c, a.done[rank] + p * FLAGCX_P2P_CTAS + b, seq - 1, (unsigned)p)) return;
      ctaCopyShare(a.stage[rank] + slot * p, a.sendSrc[p] + i * slot, len, b, g);
      ctaRaiseFlag(a.ready[p] + rank * FLAGCX_P2P_CTAS + b, seq);
    }
    for (int k = 1; k < n; ++k) { // receives of this step
      int p = rank - k; if (p < 0) p += n;
      if (!a.recvDst[p] || i * slot >= a.recvBytes[p]) continue;
      size_t len = a.recvBytes[p] - i * slot < slot ? a.recvBytes[p] - i * slot : slot;
      unsigned long long seq = a.recvSeq[p] + i + 1;
      if (!ctaWaitFlag(c, a.ready[rank] + p * FLAGCX_P2P_CTAS + b, seq, (unsigned)p)) return;
      ctaCopyShare(a.recvDst[p] + i * slot, a.stage[p] + slot * rank, len, b, g);
      ctaRaiseFlag(a.done[p] + rank * FLAGCX_P2P_CTAS + b, seq);
    }
  }
}
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA) p2pKernel(const flagcxDevComm c, const P2pArgs a) {
  p2pBody(c, a);
}
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    p2pKernelEmu(const flagcxDevComm *cs, const P2pArgs *as) {
  p2pBody(cs[blockIdx.y], as[blockIdx.y]);
}

// ---------------------------------------------------------------------------
// NVLS family: the switch reduces (multimem.ld_reduce) and broadcasts (multimem.st)
// ---------------------------------------------------------------------------
template <typename T> struct Mm;
template <> struct Mm<float> {
  // the switch adds fp32 but has no fp32 min/max; the host never routes those here
  static __device__ __forceinline__ uint4 ldReduce(const void *p, int) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(void *p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct Mm<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ldReduce(const void *p, int op) {
    uint4 v;
    if (op == kOpMin)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    else if (op == kOpMax)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    else
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(void *p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w) : "memory");
  }
};
template <> struct Mm<__half> {
  static __device__ __forceinline__ uint4 ldReduce(const void *p, int op) {
    uint4 v;
    if (op == kOpMin)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    else if (op == kOpMax)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    else
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
  static __device__ __forceinline__ void st(void *p, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w) : "memory");
  }
};

template <typename T>
__device__ __forceinline__ uint4 scalePack(uint4 v, float scale) {
  if (scale == 1.0f) return v;
  constexpr int N = 16 / (int)sizeof(T);
  T *e = (T *)&v;
#pragma unroll
  for (int i = 0; i < N; ++i) e[i] = fromAcc<T>(toAcc<T>(e[i]) * scale);
  return v;
}

// Streams packs [ub, ue) from src (+srcBase packs) to dst (+dstBase packs), eight loads in
// flight per thread: through the switch (multimem.ld_reduce / multimem.st) or plainly.
template <typename T, bool MC_LOAD, bool MC_STORE>
__device__ __forceinline__ void nvlsStream(const char *src, char *dst, size_t ub, size_t ue, size_t srcBase,
                                           size_t dstBase, int redOp, float scale, int t, int nt) {
  constexpr int U = 8;
  size_t i = ub + t;
  for (; i + (U - 1) * (size_t)nt < ue; i += U * (size_t)nt) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const char *p = src + ((srcBase + i + u * (size_t)nt) << 4);
      v[u] = MC_LOAD ? Mm<T>::ldReduce(p, redOp) : ldSys16(p);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      char *q = dst + ((dstBase + i + u * (size_t)nt) << 4);
      uint4 o = scalePack<T>(v[u], scale);
      if (MC_STORE) Mm<T>::st(q, o); else st16(q, o);
    }
  }
  for (; i < ue; i += nt) {
    const char *p = src + ((srcBase + i) << 4);
    uint4 o = scalePack<T>(MC_LOAD ? Mm<T>::ldReduce(p, redOp) : ldSys16(p), scale);
    char *q = dst + ((dstBase + i) << 4);
    if (MC_STORE) Mm<T>::st(q, o); else st16(q, o);
  }
}

// All sizes here are whole 16-byte packs (the host falls back otherwise).
template <typename T>
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA) nvlsKernel(const flagcxDevComm c, const CollArgs a) {
  const int b = blockIdx.x, g = gridDim.x, rank = c.rank, n = c.nRanks;
  constexpr int N = 16 / (int)sizeof(T);
  const int t = threadIdx.x, nt = blockDim.x;
  copyIn(a, rank, b, g);
  if (a.flags & kFlagBeginBarrier)
    if (!ctaBarrier(c, b)) return;
  size_t ub, ue;
  switch (a.kind) {
    case kAllReduceNvlsOneShot: {
      ctaShare(a.count / N, b, g, &ub, &ue);
      nvlsStream<T, true, false>(a.mcIn, a.out[rank], ub, ue, 0, 0, a.redOp, a.scale, t, nt);
      break;
    }
    case kAllReduceNvlsTwoShot: {
      size_t s = sliceElems(a.count, n, sizeof(T));
      size_t sb = s * rank < a.count ? s * rank : a.count;
      size_t se = sb + s < a.count ? sb + s : a.count;
      ctaShare((se - sb) / N, b, g, &ub, &ue);
      size_t base = sb / N;
      nvlsStream<T, true, true>(a.mcIn, a.mcOut, ub, ue, base, base, a.redOp, a.scale, t, nt);
      break;
    }
    case kReduceScatterNvls: {
      ctaShare(a.count / N, b, g, &ub, &ue);
      nvlsStream<T, true, false>(a.mcIn, a.out[rank], ub, ue, a.inStride * rank >> 4, 0, a.redOp, a.scale, t, nt);
      break;
    }
    case kAllGatherNvls: {
      ctaShare(a.count / N, b, g, &ub, &ue);
      nvlsStream<T, false, true>(a.in[rank], a.mcOut, ub, ue, 0, a.outStride * rank >> 4, a.redOp, 1.0f, t, nt);
      break;
    }
    default: break;
  }
  if (a.flags & kFlagEndBarrier)
    if (!ctaBarrier(c, b)) return;
  copyOut(a, rank, b, g);
}

// ---------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------
template <typename T, int OP, int NR>
cudaError_t launchReduceT(const LaunchCtx &lc, const CollArgs &a) {
  dim3 grid(lc.nCtas, lc.emuRanks > 0 ? lc.emuRanks : 1), block(lc.nThreads);
  if (lc.emuRanks > 0) {
    void *params[] = {(void *)&lc.emuComms, (void *)&lc.emuArgs};
    size_t emuSmem = 0;
    if (NR > 0 && lc.emuBulk) {
      emuSmem = kBulkRingBytes;
      static bool emuConfigured = false; // one per instantiation
      if (!emuConfigured) {
        cudaError_t e = cudaFuncSetAttribute(reduceKernelEmu<T, OP, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)emuSmem);
        if (e != cudaSuccess) return e;
        emuConfigured = true;
      }
    }
    return cudaLaunchCooperativeKernel((const void *)reduceKernelEmu<T, OP, NR>, grid, block, params, emuSmem,
                                       lc.stream);
  }
  size_t smem = 0;
  if (NR > 0 && a.bulkStage) {
    smem = kBulkRingBytes;
    static bool configured = false; // one per instantiation
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(reduceKernel<T, OP, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      configured = true;
    }
  }
  reduceKernel<T, OP, NR><<<grid, block, smem, lc.stream>>>(*lc.comm, a);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launchReduceHot(const LaunchCtx &lc, const CollArgs &a, int nRanks) {
  // sum (and average, which is sum with a scale) at the common world sizes get the
  // fully unrolled instantiation; everything else takes the generic one
  if (a.redOp == kOpSum) {
    switch (nRanks) {
      case 2: return launchReduceT<T, kOpSum, 2>(lc, a);
      case 4: return launchReduceT<T, kOpSum, 4>(lc, a);
      case 8: return launchReduceT<T, kOpSum, 8>(lc, a);
      default: break;
    }
  }
  return launchReduceT<T, kOpRuntime, 0>(lc, a);
}

} // namespace

cudaError_t launchReduceKernel(const LaunchCtx &lc, const CollArgs &a, int nRanks) {
  switch ((flagcxDataType_t)a.dtype) {
    case flagcxFloat32: return launchReduceHot<float>(lc, a, nRanks);
    case flagcxBfloat16: return launchReduceHot<__nv_bfloat16>(lc, a, nRanks);
    case flagcxFloat16: return launchReduceHot<__half>(lc, a, nRanks);
    case flagcxFloat64: return launchReduceT<double, kOpRuntime, 0>(lc, a);
    case flagcxInt8: return launchReduceT<signed char, kOpRuntime, 0>(lc, a);
    case flagcxUint8: return launchReduceT<unsigned char, kOpRuntime, 0>(lc, a);
    case flagcxInt32: return launchReduceT<int, kOpRuntime, 0>(lc, a);
    case flagcxUint32: return launchReduceT<unsigned int, kOpRuntime, 0>(lc, a);
    case flagcxInt64: return launchReduceT<long long, kOpRuntime, 0>(lc, a);
    case flagcxUint64: return launchReduceT<unsigned long long, kOpRuntime, 0>(lc, a);
    default: return cudaErrorInvalidValue;
  }
}

namespace {
template <typename T>
cudaError_t launchLlT(const LaunchCtx &lc, const CollArgs &a) {
  dim3 grid(lc.nCtas, lc.emuRanks > 0 ? lc.emuRanks : 1), block(lc.nThreads);
  if (lc.emuRanks > 0) {
    void *params[] = {(void *)&lc.emuComms, (void *)&lc.emuArgs};
    return cudaLaunchCooperativeKernel((const void *)llKernelEmu<T>, grid, block, params, 0, lc.stream);
  }
  llKernel<T><<<grid, block, 0, lc.stream>>>(*lc.comm, a);
  return cudaGetLastError();
}
} // namespace

cudaError_t launchLlKernel(const LaunchCtx &lc, const CollArgs &a) {
  if (a.kind == kLlAllGather) return launchLlT<unsigned char>(lc, a); // bytes
  switch ((flagcxDataType_t)a.dtype) {
    case flagcxFloat32: return launchLlT<float>(lc, a);
    case flagcxBfloat16: return launchLlT<__nv_bfloat16>(lc, a);
    case flagcxFloat16: return launchLlT<__half>(lc, a);
    case flagcxFloat64: return launchLlT<double>(lc, a);
    case flagcxInt8: return launchLlT<signed char>(lc, a);
    case flagcxUint8: return launchLlT<unsigned char>(lc, a);
    case flagcxInt32: return launchLlT<int>(lc, a);
    case flagcxUint32: return launchLlT<unsigned int>(lc, a);
    case flagcxInt64: return launchLlT<long long>(lc, a);
    case flagcxUint64: return launchLlT<unsigned long long>(lc, a);
    default: return cudaErrorInvalidValue;
  }
}

cudaError_t launchCopyKernel(const LaunchCtx &lc, const CollArgs &a) {
  dim3 grid(lc.nCtas, lc.emuRanks > 0 ? lc.emuRanks : 1), block(lc.nThreads);
  if (lc.emuRanks > 0) {
    void *params[] = {(void *)&lc.emuComms, (void *)&lc.emuArgs};
    size_t emuSmem = 0;
    if (lc.emuBulk) {
      emuSmem = kBulkRingBytes;
      static bool emuConfigured = false;
      if (!emuConfigured) {
        cudaError_t e = cudaFuncSetAttribute(copyKernelEmu, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)emuSmem);
        if (e != cudaSuccess) return e;
        emuConfigured = true;
      }
    }
    return cudaLaunchCooperativeKernel((const void *)copyKernelEmu, grid, block, params, emuSmem, lc.stream);
  }
  size_t smem = 0;
  if (a.bulkStage) {
    smem = kBulkRingBytes;
    static bool configured = false;
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(copyKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      configured = true;
    }
  }
  copyKernel<<<grid, block, smem, lc.stream>>>(*lc.comm, a);
  return cudaGetLastError();
}

cudaError_t launchP2pKernel(const LaunchCtx &lc, const P2pArgs &a) {
  dim3 grid(FLAGCX_P2P_CTAS, lc.emuRanks > 0 ? lc.emuRanks : 1), block(lc.nThreads);
  if (lc.emuRanks > 0) {
    void *params[] = {(void *)&lc.emuComms, (void *)&lc.emuP2p};
    return cudaLaunchCooperativeKernel((const void *)p2pKernelEmu, grid, block, params, 0, lc.stream);
  }
  p2pKernel<<<grid, block, 0, lc.stream>>>(*lc.comm, a);
  return cudaGetLastError();
}

cudaError_t launchNvlsKernel(const LaunchCtx &lc, const CollArgs &a) {
  if (lc.emuRanks > 0) return cudaErrorNotSupported; // multimem needs a real multicast object
  dim3 grid(lc.nCtas), block(lc.nThreads);
  switch ((flagcxDataType_t)a.dtype) {
    case flagcxFloat32: nvlsKernel<float><<<grid, block, 0, lc.stream>>>(*lc.comm, a); break;
    case flagcxBfloat16: nvlsKernel<__nv_bfloat16><<<grid, block, 0, lc.stream>>>(*lc.comm, a); break;
    case flagcxFloat16: nvlsKernel<__half><<<grid, block, 0, lc.stream>>>(*lc.comm, a); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

int maxCoresidentCtas(int nThreads) {
  int dev = 0, sms = 0, perSm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, (const void *)copyKernelEmu, nThreads, 0);
  int reduceOcc = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&reduceOcc, (const void *)reduceKernelEmu<double, kOpRuntime, 0>,
                                                nThreads, 0);
  if (reduceOcc < perSm) perSm = reduceOcc;
  // other instantiations may fit fewer blocks per SM than these two: count one
  // per SM so that the cooperative launch is accepted for all of them
  return sms * (perSm > 0 ? 1 : 0);
}

} // namespace fcx
