// copy_kernels.cu -- the collectives that only move bytes: all-gather (push, pull, ring),
// broadcast, gather, scatter, all-to-all and all-to-all-v, and grouped point-to-point.
// Large pushes go through the bulk-copy engine (one thread per CTA drives a ring of
// shared-memory stages); everything else uses 16-byte loads and posted stores.  They take
// the place of the non-reducing NCCL calls of the FlagCX NCCL adaptor
// (flagcx/adaptor/ccl/nccl_adaptor.cc:228-382 in the FlagCX project).
#include "coll_common.cuh"

namespace fcx {
namespace {

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
  {
    size_t inEnd = blk, outEnd = blk;
    switch (a.kind) {
      case kAllGatherPush: case kAllGatherPull: case kAllGatherRing: case kGatherPull:
        outEnd = a.outStride * (size_t)(n - 1) + blk; break;
      case kScatterPull: inEnd = a.inStride * (size_t)(n - 1) + blk; break;
      case kAllToAllPush: case kAllToAllPull:
        inEnd = a.inStride * (size_t)(n - 1) + blk; outEnd = a.outStride * (size_t)(n - 1) + blk; break;
      case kAllToAllvPull:
        inEnd = outEnd = 0;
        for (int p = 0; p < n; ++p) {
          if ((a.sendDispls[p] + a.sendCounts[p]) * es > inEnd) inEnd = (a.sendDispls[p] + a.sendCounts[p]) * es;
          if ((a.recvDispls[p] + a.recvCounts[p]) * es > outEnd) outEnd = (a.recvDispls[p] + a.recvCounts[p]) * es;
        }
        break;
      case kBarrierOnly: inEnd = outEnd = 0; break;
      default: break;
    }
    (void)inEnd;
    (void)outEnd;
    FCX_BOUNDS(c, inEnd, a.inBytes, 1);
    FCX_BOUNDS(c, outEnd, a.outBytes, 2);
  }

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

} // namespace

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

int reduceEmuOccupancy(int nThreads);

int maxCoresidentCtas(int nThreads) {
  int dev = 0, sms = 0, perSm = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, (const void *)copyKernelEmu, nThreads, 0);
  const int reduceOcc = reduceEmuOccupancy(nThreads);
  if (reduceOcc < perSm) perSm = reduceOcc;
  // other instantiations may fit fewer blocks per SM than these two: count one
  // per SM so that the cooperative launch is accepted for all of them
  return sms * (perSm > 0 ? 1 : 0);
}

} // namespace fcx
