// moe.cu -- expert-parallel dispatch and combine as NVLink kernels.
//
// dispatch: every (token, chosen expert) pair is copied straight from the local
// activation matrix into the destination rank's receive buffer, already grouped
// by expert (rows of expert e from rank 0, then rank 1, ...), i.e. the all-to-all
// and the token permutation are one pass over the data.  The counts each rank
// needs to place its rows are exchanged inside the same kernel before the first
// barrier.
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

__global__ void moeCountKernel(const int *__restrict__ topkIdx, int *__restrict__ counts, int *__restrict__ pos,
                               int items, int nExperts, flagcxDevStatus *status) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < items; i += gridDim.x * blockDim.x) {
    int e = topkIdx[i];
    if (e < 0 || e >= nExperts) {
      fcxdev::reportError(status, FLAGCX_DEV_BOUNDS, FLAGCX_DEV_AT_KERNEL, 0xffffffffu, (unsigned long long)i);
      pos[i] = -1;
      continue;
    }
    pos[i] = atomicAdd(&counts[e], 1);
  }
}

__device__ void dispatchBody(const flagcxDevComm &c, const MoeArgs &a) {
  __shared__ int tot[FLAGCX_MOE_MAX_EXPERTS], base[FLAGCX_MOE_MAX_EXPERTS];
  const int b = blockIdx.x, g = gridDim.x, rank = c.rank, n = c.nRanks;
  const int t = threadIdx.x, nt = blockDim.x;
  // 1. publish my per-expert counts in every rank's table (row `rank`)
  const int *mine = a.countsAll[rank] + (size_t)rank * a.E;
  for (int p = 0; p < n; ++p) {
    if (p == rank) continue;
    int *dst = a.countsAll[p] + (size_t)rank * a.E;
    for (int e = t; e < a.E; e += nt) dst[e] = mine[e];
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
    base[e] = s;
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
  // 3. one warp per (token, k): copy the row to its place on the destination rank
  const int warpsPerCta = nt >> 5, warp = t >> 5, lane = t & 31;
  const int items = a.T * a.K;
  const int vecs = a.H / 8; // 16-byte vectors per row
  const size_t rowBytes = (size_t)a.H * 2;
  for (int i = b * warpsPerCta + warp; i < items; i += g * warpsPerCta) {
    int e = a.topkIdx[i], p = a.pos[i];
    if (p < 0) continue;
    int d = e / a.EPR;
    size_t row = (size_t)base[e] + p;
    if (lane == 0) { a.route[2 * i] = d; a.route[2 * i + 1] = (int)row; }
    if (row >= a.capacity) continue; // reported above by the receiver
    const uint4 *src = (const uint4 *)(a.x + (size_t)(i / a.K) * a.H);
    uint4 *dst = (uint4 *)(a.recv[d] + row * rowBytes);
    int v = lane;
    for (; v + 96 < vecs; v += 128) {
      uint4 r0 = src[v], r1 = src[v + 32], r2 = src[v + 64], r3 = src[v + 96];
      st16(dst + v, r0); st16(dst + v + 32, r1); st16(dst + v + 64, r2); st16(dst + v + 96, r3);
    }
    for (; v < vecs; v += 32) st16(dst + v, src[v]);
  }
  ctaBarrier(c, b);
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

cudaError_t launchMoeCount(cudaStream_t s, const int *topkIdx, int *counts, int *pos, int items, int nExperts,
                           flagcxDevStatus *status) {
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * nExperts, s);
  if (e != cudaSuccess) return e;
  if (items == 0) return cudaSuccess;
  int blocks = (items + 255) / 256;
  moeCountKernel<<<blocks > 1024 ? 1024 : blocks, 256, 0, s>>>(topkIdx, counts, pos, items, nExperts, status);
  return cudaGetLastError();
}

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
