// moe.cu -- expert-parallel dispatch and combine as NVLink kernels.
//
// dispatch: every (token, chosen expert) pair ends up in the destination rank's receive
// buffer, already grouped by expert (rows of expert e from rank 0, then rank 1, ...),
// i.e. the all-to-all and the token permutation are one pass over the data.  A token that
// several experts of ONE rank want crosses NVLink once; the receiver makes the other
// copies locally.  Counting the routing table and exchanging the counts that place the
// rows happen inside the same kernel.
// combine: every token gathers its top-k expert outputs from the ranks that hold
// them, weights them in fp32 and stores one bf16 row: the all-to-all back and the
// weighted sum are one pass, and the un-permutation is implicit.
//
// FlagCX offers only flagcxAlltoAllv for this (plugin/torch/flagcx/src/
// backend_flagcx.cpp:926-993 in the FlagCX project); permutation and the weighted
// sum are separate framework kernels there.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "launch.h"
#include "moe_args.h"
#include "prims.cuh"

namespace fcx {
namespace {

// One warp copies one row (H bf16) with 16-byte accesses, four loads in flight per lane.
__device__ __forceinline__ void warpCopyRow(char *dst, const char *src, int vecs, int lane, bool srcIsPeerWritten) {
  const uint4 *s = (const uint4 *)src;
  uint4 *d = (uint4 *)dst;
  int v = lane;
  for (; v + 96 < vecs; v += 128) {
    uint4 r0, r1, r2, r3;
    if (srcIsPeerWritten) { r0 = ldSys16(s + v); r1 = ldSys16(s + v + 32); r2 = ldSys16(s + v + 64); r3 = ldSys16(s + v + 96); }
    else { r0 = s[v]; r1 = s[v + 32]; r2 = s[v + 64]; r3 = s[v + 96]; }
    st16(d + v, r0); st16(d + v + 32, r1); st16(d + v + 64, r2); st16(d + v + 96, r3);
  }
  for (; v < vecs; v += 32) st16(d + v, srcIsPeerWritten ? ldSys16(s + v) : s[v]);
}

// The whole dispatch is this one kernel: histogram of the routing, exchange of the
// counts, the copies, and the local fan-out of rows that several experts of one rank want.
__device__ void dispatchBody(const flagcxDevComm &c, const MoeArgs &a) {
  __shared__ int tot[FLAGCX_MOE_MAX_EXPERTS], base[FLAGCX_MOE_MAX_EXPERTS], before[FLAGCX_MOE_MAX_EXPERTS],
      mineCnt[FLAGCX_MOE_MAX_EXPERTS];
  __shared__ int dupN[FLAGCX_MAX_RANKS];
  const int b = blockIdx.x, g = gridDim.x, rank = c.rank, n = c.nRanks;
  const int t = threadIdx.x, nt = blockDim.x;
  // this CTA's tokens: a contiguous range, so that "how many earlier pairs chose expert e"
  // splits into the pairs of earlier CTAs' ranges and the pairs of this range
  const int tpc = (a.T + g - 1) / g;
  const int tlo = b * tpc < a.T ? b * tpc : a.T, thi = tlo + tpc < a.T ? tlo + tpc : a.T;
  const int lo = tlo * a.K, hi = thi * a.K, items = a.T * a.K;
  // 0. every CTA counts the whole routing table (a few dozen shared-memory atomics per
  // thread): no separate counting kernel, no global atomics, no memset
  for (int e = t; e < a.E; e += nt) tot[e] = before[e] = mineCnt[e] = 0;
  if (t < FLAGCX_MAX_RANKS) dupN[t] = 0;
  __syncthreads();
  for (int i = t; i < items; i += nt) {
    const int e = a.topkIdx[i];
    const bool valid = e >= 0 && e < a.E;
    if (i < lo) { if (valid) atomicAdd(&before[e], 1); }
    else if (i < hi) {
      if (valid) a.pos[i] = atomicAdd(&mineCnt[e], 1); // index within this CTA's range, completed below
      else {
        a.pos[i] = -1;
        fcxdev::reportError(c.status, FLAGCX_DEV_BOUNDS, FLAGCX_DEV_AT_KERNEL, 0xffffffffu, (unsigned long long)i);
      }
    } else if (valid) atomicAdd(&tot[e], 1);
  }
  __syncthreads();
  for (int e = t; e < a.E; e += nt) tot[e] += before[e] + mineCnt[e];
  __syncthreads();
  // 1. publish my per-expert counts in every rank's table (row `rank`), mine included;
  // every CTA writes the same values and reads them back from its own peers' CTA
  for (int p = 0; p < n; ++p) {
    int *dst = a.countsAll[p] + (size_t)rank * a.E;
    for (int e = t; e < a.E; e += nt) dst[e] = tot[e];
  }
  if (!ctaBarrier(c, b)) return;
  // 2. where my rows start inside each destination's expert-grouped buffer
  const int *tab = a.countsAll[rank];
  for (int e = t; e < a.E; e += nt) {
    int s = 0;
    // rows written by peers: system-scope loads, never a stale cached line
    for (int q = 0; q < n; ++q) s += ldSysElem(tab + (size_t)q * a.E + e);
    tot[e] = s;
  }
  __syncthreads();
  for (int e = t; e < a.E; e += nt) {
    int d = e / a.EPR, s = 0;
    for (int e2 = d * a.EPR; e2 < e; ++e2) s += tot[e2];
    for (int q = 0; q < rank; ++q) s += ldSysElem(tab + (size_t)q * a.E + e);
    base[e] = s + before[e]; // pairs of earlier CTAs' ranges come first
  }
  __syncthreads();
  if (b == 0) {
    // this rank's own expert boundaries, for whoever runs the experts
    for (int le = t; le <= a.EPR; le += nt) {
      int s = 0;
      for (int e2 = 0; e2 < le; ++e2) s += tot[rank * a.EPR + e2];
      a.expertOffsets[le] = s;
    }
    if (t == 0) {
      long total = 0;
      for (int le = 0; le < a.EPR; ++le) total += tot[rank * a.EPR + le];
      if ((size_t)total > a.capacity)
        fcxdev::reportError(c.status, FLAGCX_DEV_BOUNDS, FLAGCX_DEV_AT_KERNEL, (unsigned)rank, (unsigned long long)total);
    }
  }
  // 3. one warp per token.  The first expert of each destination rank gets the row over
  // NVLink, straight into its final place; for further experts on the same rank the
  // receiver is left a (source row, destination row) record and copies locally.
  const int warpsPerCta = nt >> 5, warp = t >> 5, lane = t & 31;
  const int vecs = a.H / 8; // 16-byte vectors per row
  const size_t rowBytes = (size_t)a.H * 2;
  const int capPer = ((a.maxT + g - 1) / g) * (a.K > 1 ? a.K - 1 : 1);
  for (int tok = tlo + warp; tok < thi; tok += warpsPerCta) {
    int d = -1, row = 0;
    bool valid = false;
    if (lane < a.K) {
      const int i = tok * a.K + lane, e = a.topkIdx[i], rel = a.pos[i];
      valid = rel >= 0;
      if (valid) {
        d = e / a.EPR;
        row = base[e] + rel;
        a.pos[i] = row; // any value >= 0 tells combine that the pair is real
        a.route[2 * i] = d;
        a.route[2 * i + 1] = row;
      }
    }
    int firstLane = lane;
    for (int j = a.K - 1; j >= 0; --j) { // the smallest earlier lane with the same destination wins
      const int dj = __shfl_sync(0xffffffffu, d, j);
      if (a.dedup && j < lane && dj == d && d >= 0) firstLane = j;
    }
    const bool isFirst = valid && firstLane == lane;
    const int firstRow = __shfl_sync(0xffffffffu, row, firstLane);
    if (valid && !isFirst && (size_t)row < a.capacity && (size_t)firstRow < a.capacity) {
      const int idx = atomicAdd(&dupN[d], 1);
      if (idx < capPer) {
        int2 *rec = a.dupList[d] + (size_t)rank * a.dupRecordsPerSender + (size_t)b * capPer + idx;
        *rec = make_int2(firstRow, row);
      }
    }
    const char *src = (const char *)(a.x + (size_t)tok * a.H);
    for (int k = 0; k < a.K; ++k) {
      const int dk = __shfl_sync(0xffffffffu, d, k), rowk = __shfl_sync(0xffffffffu, row, k);
      const bool fk = __shfl_sync(0xffffffffu, isFirst ? 1 : 0, k) != 0;
      if (fk && (size_t)rowk < a.capacity) // rows past the capacity are reported by the receiver
        warpCopyRow(a.recv[dk] + (size_t)rowk * rowBytes, src, vecs, lane, false);
    }
  }
  __syncthreads();
  if (t < n) a.dupCount[t][(size_t)rank * FLAGCX_COLL_BARRIER_SLOTS + b] = dupN[t] < capPer ? dupN[t] : capPer;
  if (!ctaBarrier(c, b)) return;
  // 4. the copies the senders' CTA b left to this rank: row to row inside my own buffer
  for (int q = 0; q < n; ++q) {
    const int cnt = ldSysElem(a.dupCount[rank] + (size_t)q * FLAGCX_COLL_BARRIER_SLOTS + b);
    const int2 *recs = a.dupList[rank] + (size_t)q * a.dupRecordsPerSender + (size_t)b * capPer;
    for (int r = warp; r < cnt; r += warpsPerCta) {
      const unsigned long long raw = fcxdev::ldRelaxedSys((const unsigned long long *)(recs + r));
      const int srcRow = (int)(raw & 0xffffffffu), dstRow = (int)(raw >> 32);
      if ((size_t)srcRow >= a.capacity || (size_t)dstRow >= a.capacity) continue;
      warpCopyRow(a.recv[rank] + (size_t)dstRow * rowBytes, a.recv[rank] + (size_t)srcRow * rowBytes, vecs, lane, true);
    }
  }
}

__device__ void combineBody(const flagcxDevComm &c, const MoeArgs &a) {
  const int b = blockIdx.x, g = gridDim.x;
  const int t = threadIdx.x, nt = blockDim.x;
  if (!ctaBarrier(c, b)) return; // every rank's expert outputs are complete
  const int warpsPerCta = nt >> 5, warp = t >> 5, lane = t & 31;
  const int vecs = a.H / 8;
  const size_t rowBytes = (size_t)a.H * 2;
  for (int tok = b * warpsPerCta + warp; tok < a.T; tok += g * warpsPerCta) {
    const char *rows[FLAGCX_MOE_MAX_TOPK];
    float w[FLAGCX_MOE_MAX_TOPK];
#pragma unroll
    for (int k = 0; k < FLAGCX_MOE_MAX_TOPK; ++k) {
      if (k < a.K) {
        int i = tok * a.K + k;
        int d = a.route[2 * i], row = a.route[2 * i + 1];
        bool ok = a.pos[i] >= 0 && (size_t)row < a.capacity;
        rows[k] = ok ? a.expertOut[d] + (size_t)row * rowBytes : nullptr;
        w[k] = ok ? a.topkW[i] : 0.f;
      } else {
        rows[k] = nullptr;
        w[k] = 0.f;
      }
    }
    uint4 *dst = (uint4 *)(a.out + (size_t)tok * a.H);
    for (int v = lane; v < vecs; v += 32) {
      uint4 r[FLAGCX_MOE_MAX_TOPK];
#pragma unroll
      for (int k = 0; k < FLAGCX_MOE_MAX_TOPK; ++k)
        if (rows[k]) r[k] = ldSys16(rows[k] + (size_t)v * 16);
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int k = 0; k < FLAGCX_MOE_MAX_TOPK; ++k)
        if (rows[k]) {
          const __nv_bfloat16 *e = (const __nv_bfloat16 *)&r[k];
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += w[k] * __bfloat162float(e[j]);
        }
      uint4 o;
      __nv_bfloat16 *oe = (__nv_bfloat16 *)&o;
#pragma unroll
      for (int j = 0; j < 8; ++j) oe[j] = __float2bfloat16_rn(acc[j]);
      dst[v] = o;
    }
  }
  ctaBarrier(c, b); // peers may overwrite their expert outputs only after everyone has read them
}

__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA) moeDispatchKernel(const flagcxDevComm c, const MoeArgs a) {
  dispatchBody(c, a);
}
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    moeDispatchKernelEmu(const flagcxDevComm *cs, const MoeArgs *as) {
  dispatchBody(cs[blockIdx.y], as[blockIdx.y]);
}
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA) moeCombineKernel(const flagcxDevComm c, const MoeArgs a) {
  combineBody(c, a);
}
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    moeCombineKernelEmu(const flagcxDevComm *cs, const MoeArgs *as) {
  combineBody(cs[blockIdx.y], as[blockIdx.y]);
}

} // namespace

cudaError_t launchMoeDispatch(const LaunchCtx &lc, const MoeArgs &a) {
  dim3 grid(lc.nCtas, lc.emuRanks > 0 ? lc.emuRanks : 1), block(lc.nThreads);
  const size_t smem = 0;
  (void)a;
  if (lc.emuRanks > 0) {
    const void *blob = lc.emuBlob;
    void *params[] = {(void *)&lc.emuComms, (void *)&blob};
    return cudaLaunchCooperativeKernel((const void *)moeDispatchKernelEmu, grid, block, params, smem, lc.stream);
  }
  moeDispatchKernel<<<grid, block, smem, lc.stream>>>(*lc.comm, a);
  return cudaGetLastError();
}

cudaError_t launchMoeCombine(const LaunchCtx &lc, const MoeArgs &a) {
  dim3 grid(lc.nCtas, lc.emuRanks > 0 ? lc.emuRanks : 1), block(lc.nThreads);
  if (lc.emuRanks > 0) {
    const void *blob = lc.emuBlob;
    void *params[] = {(void *)&lc.emuComms, (void *)&blob};
    return cudaLaunchCooperativeKernel((const void *)moeCombineKernelEmu, grid, block, params, 0, lc.stream);
  }
  moeCombineKernel<<<grid, block, 0, lc.stream>>>(*lc.comm, a);
  return cudaGetLastError();
}

} // namespace fcx
