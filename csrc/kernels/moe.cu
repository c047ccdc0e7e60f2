// moe.cu -- expert-parallel dispatch and combine as NVLink kernels.
//
// dispatch: every (token, chosen expert) pair ends up in the destination rank's receive
// buffer, already grouped by expert (rows of expert e from rank 0, then rank 1, ...),
// i.e. the all-to-all and the token permutation are one pass over the data.  A token that
// several experts of ONE rank want crosses NVLink once; the receiver makes the other
// copies locally.  Counting the routing table and exchanging the counts that place the
// rows happen inside the same kernel.
// combine: the mirror image.  The token's owner pushes the gate weights to the expert
// ranks; each expert rank adds up, in fp32, the weighted outputs a token has on it (one
// bf16 row per token and rank); the owner pulls those rows and sums them: one row per
// (token, rank) crosses NVLink instead of one per (token, expert), the all-to-all back and
// the weighted sum are one kernel, and the un-permutation is implicit.  With
// preReduce = 0 the owner pulls every (token, expert) row and weights it itself.
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

// CTAs of 8 warps: the combine keeps eight 16-byte loads per lane in flight and wants the
// registers for them; the host launches twice as many CTAs as it would of the 512-thread kind.
constexpr int kMoeThreads = 256;

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

// A group record (FLAGCX_MOE_MAX_TOPK ints written by a peer) as two 16-byte loads.
__device__ __forceinline__ void loadGroup(const int *rec, int rows[FLAGCX_MOE_MAX_TOPK]) {
  static_assert(FLAGCX_MOE_MAX_TOPK == 8, "a group record is two 16-byte vectors");
  const uint4 lo = ldSys16(rec), hi = ldSys16(rec + 4);
  rows[0] = (int)lo.x; rows[1] = (int)lo.y; rows[2] = (int)lo.z; rows[3] = (int)lo.w;
  rows[4] = (int)hi.x; rows[5] = (int)hi.y; rows[6] = (int)hi.z; rows[7] = (int)hi.w;
}

// dst row = sum over M rows of w[j] * rows[j], fp32 accumulation, one warp.  U vectors of
// every row are loaded before any is used, so a lane has M*U 16-byte loads in flight.
template <int M, int U>
__device__ __forceinline__ void rowSumFixed(const char *const *rows, const float *w, uint4 *dst, int vecs, int lane,
                                            bool peerWritten) {
  for (int v0 = lane; v0 < vecs; v0 += 32 * U) {
    uint4 r[U][M];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + 32 * u;
      if (v < vecs) {
#pragma unroll
        for (int j = 0; j < M; ++j)
          r[u][j] = peerWritten ? ldSys16(rows[j] + (size_t)v * 16) : *(const uint4 *)(rows[j] + (size_t)v * 16);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int v = v0 + 32 * u;
      if (v < vecs) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int j = 0; j < M; ++j) {
          const __nv_bfloat16 *e = (const __nv_bfloat16 *)&r[u][j];
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] += w[j] * __bfloat162float(e[i]);
        }
        uint4 o;
        __nv_bfloat16 *oe = (__nv_bfloat16 *)&o;
#pragma unroll
        for (int i = 0; i < 8; ++i) oe[i] = __float2bfloat16_rn(acc[i]);
        st16(dst + v, o);
      }
    }
  }
}

// dst row = sum of the first m rows, weighted (m = 0: zeros).  Few rows mean more vectors
// per row in flight: 8 loads per lane either way.  m is the same for all lanes of the warp.
__device__ __forceinline__ void weightedRowSum(const char *rows[FLAGCX_MOE_MAX_TOPK], float w[FLAGCX_MOE_MAX_TOPK], int m,
                                               uint4 *dst, int vecs, int lane, bool rowsArePeerWritten) {
  if (m == 0) {
    for (int v = lane; v < vecs; v += 32) st16(dst + v, make_uint4(0, 0, 0, 0));
  } else if (m == 1) {
    rowSumFixed<1, 8>(rows, w, dst, vecs, lane, rowsArePeerWritten);
  } else if (m == 2) {
    rowSumFixed<2, 4>(rows, w, dst, vecs, lane, rowsArePeerWritten);
  } else if (m <= 4) {
#pragma unroll
    for (int j = 2; j < 4; ++j)
      if (j >= m) { rows[j] = rows[0]; w[j] = 0.f; } // pad with a weightless repeat of a valid row
    rowSumFixed<4, 2>(rows, w, dst, vecs, lane, rowsArePeerWritten);
  } else {
#pragma unroll
    for (int j = 4; j < FLAGCX_MOE_MAX_TOPK; ++j)
      if (j >= m) { rows[j] = rows[0]; w[j] = 0.f; }
    rowSumFixed<8, 1>(rows, w, dst, vecs, lane, rowsArePeerWritten);
  }
}

// The whole dispatch is this one kernel: histogram of the routing, exchange of the
// counts, the copies, and the local fan-out of rows that several experts of one rank want.
__device__ void dispatchBody(const flagcxDevComm &c, const MoeArgs &a) {
  __shared__ int tot[FLAGCX_MOE_MAX_EXPERTS], base[FLAGCX_MOE_MAX_EXPERTS], before[FLAGCX_MOE_MAX_EXPERTS],
      mineCnt[FLAGCX_MOE_MAX_EXPERTS];
  __shared__ int grpN[FLAGCX_MAX_RANKS];
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
  if (t < FLAGCX_MAX_RANKS) grpN[t] = 0;
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
  // NVLink, straight into its final place; the destination is left a group record (all rows
  // of that token there, leader first) from which it makes the other copies locally.
  const int warpsPerCta = nt >> 5, warp = t >> 5, lane = t & 31;
  const int vecs = a.H / 8; // 16-byte vectors per row
  const size_t rowBytes = (size_t)a.H * 2;
  const int capPer = ((a.maxT + g - 1) / g) * a.K;
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
        valid = (size_t)row < a.capacity; // rows past the capacity are reported by the receiver and dropped
      }
    }
    int firstLane = lane;
    for (int j = a.K - 1; j >= 0; --j) { // the smallest earlier lane with the same destination wins
      const int dj = __shfl_sync(0xffffffffu, valid ? d : -1, j);
      if (a.dedup && valid && j < lane && dj == d) firstLane = j;
    }
    // lanes of one group find each other; the others (no pair, bad pair) are alone
    const unsigned members = __match_any_sync(0xffffffffu, valid ? firstLane : 32 + lane);
    const int member = __popc(members & ((1u << lane) - 1u)), groupSize = __popc(members);
    const bool isFirst = valid && member == 0;
    int idx = 0;
    if (isFirst) idx = atomicAdd(&grpN[d], 1);
    idx = __shfl_sync(0xffffffffu, idx, firstLane);
    // the token's groups, packed: entry j = pair index of the j-th leader, -1 after the last
    const unsigned leaders = __ballot_sync(0xffffffffu, isFirst);
    if (lane < a.K) a.lead[tok * a.K + lane] = -1;
    __syncwarp();
    if (isFirst) a.lead[tok * a.K + __popc(leaders & ((1u << lane) - 1u))] = lane;
    if (valid && idx < capPer) {
      int *rec = a.grpList[d] + ((size_t)rank * a.grpRecordsPerSender + (size_t)b * capPer + idx) * FLAGCX_MOE_MAX_TOPK;
      rec[member] = row;
      if (isFirst)
        for (int j = groupSize; j < FLAGCX_MOE_MAX_TOPK; ++j) rec[j] = -1;
    }
    const char *src = (const char *)(a.x + (size_t)tok * a.H);
    for (int k = 0; k < a.K; ++k) {
      const int dk = __shfl_sync(0xffffffffu, d, k), rowk = __shfl_sync(0xffffffffu, row, k);
      const bool fk = __shfl_sync(0xffffffffu, isFirst ? 1 : 0, k) != 0;
      if (fk) warpCopyRow(a.recv[dk] + (size_t)rowk * rowBytes, src, vecs, lane, false);
    }
  }
  __syncthreads();
  if (t < n) a.grpCount[t][(size_t)rank * FLAGCX_COLL_BARRIER_SLOTS + b] = grpN[t] < capPer ? grpN[t] : capPer;
  if (!ctaBarrier(c, b)) return;
  // 4. the copies the senders' CTA b left to this rank: row to row inside my own buffer
  for (int q = 0; q < n; ++q) {
    const int cnt = ldSysElem(a.grpCount[rank] + (size_t)q * FLAGCX_COLL_BARRIER_SLOTS + b);
    const int *recs = a.grpList[rank] + ((size_t)q * a.grpRecordsPerSender + (size_t)b * capPer) * FLAGCX_MOE_MAX_TOPK;
    for (int r = warp; r < cnt; r += warpsPerCta) {
      int rows[FLAGCX_MOE_MAX_TOPK];
      loadGroup(recs + (size_t)r * FLAGCX_MOE_MAX_TOPK, rows);
      if ((size_t)rows[0] >= a.capacity) continue;
#pragma unroll
      for (int j = 1; j < FLAGCX_MOE_MAX_TOPK; ++j)
        if (rows[j] >= 0 && (size_t)rows[j] < a.capacity)
          warpCopyRow(a.recv[rank] + (size_t)rows[j] * rowBytes, a.recv[rank] + (size_t)rows[0] * rowBytes, vecs, lane, true);
    }
  }
}

// Pull-everything combine: the token's owner reads each (token, expert) row and weights it.
// Independent of the dispatch's CTA layout (it needs only the route), so it runs as CTAs of
// 512 threads: measured faster that way (402 against 527 us on two B200s for the same
// number of warps in 256-thread CTAs).
__device__ void combinePullBody(const flagcxDevComm &c, const MoeArgs &a) {
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

// Pre-reducing combine.  Everything is organised per CTA index, like the dispatch: the
// groups that sender q's CTA b recorded here are reduced by this rank's CTA b and pulled
// by q's CTA b, so the per-CTA barriers across ranks are all the ordering it needs.
__device__ void combineReduceBody(const flagcxDevComm &c, const MoeArgs &a) {
  const int b = blockIdx.x, g = gridDim.x, rank = c.rank, n = c.nRanks;
  const int t = threadIdx.x, nt = blockDim.x;
  const int warpsPerCta = nt >> 5, warp = t >> 5, lane = t & 31;
  const int vecs = a.H / 8;
  const size_t rowBytes = (size_t)a.H * 2;
  const int tpc = (a.T + g - 1) / g; // the dispatch's token ranges
  const int tlo = b * tpc < a.T ? b * tpc : a.T, thi = tlo + tpc < a.T ? tlo + tpc : a.T;
  const int capPer = ((a.maxT + g - 1) / g) * a.K;
  // 0. the gate weight of each of my pairs goes next to the row it weights
  for (int i = tlo * a.K + t; i < thi * a.K; i += nt) {
    const int d = a.route[2 * i], row = a.route[2 * i + 1];
    if (a.pos[i] >= 0 && (size_t)row < a.capacity) a.wRow[d][row] = a.topkW[i];
  }
  if (!ctaBarrier(c, b)) return; // weights have landed; every rank's expert outputs are complete
  // A. one row per group: the weighted sum of the group's expert outputs, all local reads
  for (int q = 0; q < n; ++q) {
    const int cnt = ldSysElem(a.grpCount[rank] + (size_t)q * FLAGCX_COLL_BARRIER_SLOTS + b);
    const int *recs = a.grpList[rank] + ((size_t)q * a.grpRecordsPerSender + (size_t)b * capPer) * FLAGCX_MOE_MAX_TOPK;
    for (int r = warp; r < cnt; r += warpsPerCta) {
      int rowIdx[FLAGCX_MOE_MAX_TOPK];
      loadGroup(recs + (size_t)r * FLAGCX_MOE_MAX_TOPK, rowIdx);
      if ((size_t)rowIdx[0] >= a.capacity) continue;
      const char *rows[FLAGCX_MOE_MAX_TOPK];
      float w[FLAGCX_MOE_MAX_TOPK];
      int m = 0; // the record is packed: valid rows first
#pragma unroll
      for (int j = 0; j < FLAGCX_MOE_MAX_TOPK; ++j) {
        const bool ok = j == m && rowIdx[j] >= 0 && (size_t)rowIdx[j] < a.capacity;
        rows[j] = ok ? a.expertOut[rank] + (size_t)rowIdx[j] * rowBytes : nullptr;
        w[j] = ok ? ldSysElem(a.wRow[rank] + rowIdx[j]) : 0.f;
        m += ok ? 1 : 0;
      }
      weightedRowSum(rows, w, m, (uint4 *)(a.partial[rank] + (size_t)rowIdx[0] * rowBytes), vecs, lane, false);
    }
  }
  if (!ctaBarrier(c, b)) return; // the partial rows of my tokens are complete on every rank
  // B. each token adds up one row per rank it has experts on
  for (int tok = tlo + warp; tok < thi; tok += warpsPerCta) {
    const char *rows[FLAGCX_MOE_MAX_TOPK];
    float w[FLAGCX_MOE_MAX_TOPK];
    int m = 0;
#pragma unroll
    for (int j = 0; j < FLAGCX_MOE_MAX_TOPK; ++j) {
      rows[j] = nullptr;
      w[j] = 1.f;
      if (j < a.K) {
        const int k = a.lead[tok * a.K + j]; // pair index of this token's j-th group, -1 after the last
        if (j == m && k >= 0) {
          const int i = tok * a.K + k;
          rows[j] = a.partial[a.route[2 * i]] + (size_t)a.route[2 * i + 1] * rowBytes;
          ++m;
        }
      }
    }
    weightedRowSum(rows, w, m, (uint4 *)(a.out + (size_t)tok * a.H), vecs, lane, true);
  }
  ctaBarrier(c, b); // weights and partial rows may be overwritten only after everyone has read them
}


__global__ void __launch_bounds__(kMoeThreads) moeDispatchKernel(const flagcxDevComm c, const MoeArgs a) {
  dispatchBody(c, a);
}
__global__ void __launch_bounds__(kMoeThreads)
    moeDispatchKernelEmu(const flagcxDevComm *cs, const MoeArgs *as) {
  dispatchBody(cs[blockIdx.y], as[blockIdx.y]);
}
__global__ void __launch_bounds__(kMoeThreads) moeCombineKernel(const flagcxDevComm c, const MoeArgs a) {
  combineReduceBody(c, a);
}
__global__ void __launch_bounds__(kMoeThreads)
    moeCombineKernelEmu(const flagcxDevComm *cs, const MoeArgs *as) {
  combineReduceBody(cs[blockIdx.y], as[blockIdx.y]);
}
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA) moeCombinePullKernel(const flagcxDevComm c, const MoeArgs a) {
  combinePullBody(c, a);
}
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    moeCombinePullKernelEmu(const flagcxDevComm *cs, const MoeArgs *as) {
  combinePullBody(cs[blockIdx.y], as[blockIdx.y]);
}

} // namespace

cudaError_t launchMoeDispatch(const LaunchCtx &lc, const MoeArgs &a) {
  dim3 grid(lc.nCtas, lc.emuRanks > 0 ? lc.emuRanks : 1), block(kMoeThreads);
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

// a.preReduce picks the kernel; the pull kind takes half as many CTAs of twice the threads.
// In the emulated world every rank's arguments carry the same choice (lc.emuPull).
cudaError_t launchMoeCombine(const LaunchCtx &lc, const MoeArgs &a, bool pull) {
  const int ctas = pull ? (lc.nCtas + 1) / 2 : lc.nCtas;
  dim3 grid(ctas, lc.emuRanks > 0 ? lc.emuRanks : 1), block(pull ? FLAGCX_DEVICE_THREADS_PER_CTA : kMoeThreads);
  if (lc.emuRanks > 0) {
    const void *blob = lc.emuBlob;
    void *params[] = {(void *)&lc.emuComms, (void *)&blob};
    return cudaLaunchCooperativeKernel(pull ? (const void *)moeCombinePullKernelEmu : (const void *)moeCombineKernelEmu, grid, block,
                                       params, 0, lc.stream);
  }
  if (pull) moeCombinePullKernel<<<grid, block, 0, lc.stream>>>(*lc.comm, a);
  else moeCombineKernel<<<grid, block, 0, lc.stream>>>(*lc.comm, a);
  return cudaGetLastError();
}

} // namespace fcx
