// prims.cuh -- building blocks of the collective kernels: 16-byte peer loads and
// stores, per-type pack arithmetic with fp32 accumulation for 16-bit floats, the
// CTA partition of a slice, and the per-CTA cross-rank barrier wrapper.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "coll_args.h"
#include "flagcx.h"
#include "flagcx_device.cuh"

namespace fcx {

// ---- 16-byte accesses ---------------------------------------------------------
// Peer (and staged) data is read with system-scope relaxed loads: they bypass L1,
// so a line fetched before the producer's release can never be served stale.
__device__ __forceinline__ uint4 ldSys16(const void *p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st16(void *p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// Local streaming read of data no other GPU writes during this kernel.
__device__ __forceinline__ uint4 ldLocal16(const void *p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// One element of any supported type with a system-scope relaxed load.
template <typename T>
__device__ __forceinline__ T ldSysElem(const T *p) {
  T out;
  if constexpr (sizeof(T) == 1) {
    unsigned int v;
    asm volatile("ld.relaxed.sys.global.u8 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    unsigned char b = (unsigned char)v;
    memcpy(&out, &b, 1);
  } else if constexpr (sizeof(T) == 2) {
    unsigned short v;
    asm volatile("ld.relaxed.sys.global.u16 %0, [%1];" : "=h"(v) : "l"(p) : "memory");
    memcpy(&out, &v, 2);
  } else if constexpr (sizeof(T) == 4) {
    unsigned int v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    memcpy(&out, &v, 4);
  } else {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    memcpy(&out, &v, 8);
  }
  return out;
}

// ---- element traits -----------------------------------------------------------------
template <typename T> struct Elem { using Acc = T; };
template <> struct Elem<__half> { using Acc = float; };
template <> struct Elem<__nv_bfloat16> { using Acc = float; };

template <typename T> __device__ __forceinline__ typename Elem<T>::Acc toAcc(T v) { return v; }
template <> __device__ __forceinline__ float toAcc<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float toAcc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T fromAcc(typename Elem<T>::Acc v) { return v; }
template <> __device__ __forceinline__ __half fromAcc<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 fromAcc<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <int OP, typename A>
__device__ __forceinline__ A combine(A a, A b, int runtimeOp) {
  const int op = OP == kOpRuntime ? runtimeOp : OP;
  switch (op) {
    case kOpProd: return a * b;
    case kOpMax: return a > b ? a : b;
    case kOpMin: return a < b ? a : b;
    default: return a + b;
  }
}

template <typename A> __device__ __forceinline__ A finish(A v, float scale, int divisor) {
  // integer types: average is an integer division; scale does not apply
  return divisor ? (A)(v / (A)divisor) : v;
}
template <> __device__ __forceinline__ float finish<float>(float v, float scale, int) { return v * scale; }
// double keeps its precision: the average divides exactly instead of using the fp32 scale
template <> __device__ __forceinline__ double finish<double>(double v, float scale, int divisor) {
  if (divisor) v /= (double)divisor;
  return scale == 1.0f ? v : v * (double)scale;
}

// ---- partitioning ---------------------------------------------------------------------
// Contiguous share of [0, n) that CTA `b` of `g` owns.  Every rank computes the same
// split, so CTA b of one rank consumes exactly what CTA b of a peer produced, and
// a barrier between same-index CTAs is all the ordering that is needed.
__device__ __forceinline__ void ctaShare(size_t n, int b, int g, size_t *begin, size_t *end) {
  size_t per = (n + g - 1) / g;
  size_t s = per * (size_t)b;
  *begin = s < n ? s : n;
  *end = (s + per) < n ? (s + per) : n;
}

// ---- barrier wrapper ---------------------------------------------------------------------
__device__ __forceinline__ bool ctaBarrier(const flagcxDevComm &c, int slot) {
  if (c.nRanks == 1) { __syncthreads(); return true; }
  if (c.nvlsBarrier) { // one multimem.red through the switch instead of a store per peer
    flagcxDevBarrierNvls bar(c, slot);
    return bar.sync(flagcxCoopBlock());
  }
  flagcxDevBarrierIntra bar(c, slot);
  return bar.sync(flagcxCoopBlock());
}

// ---- local copy -----------------------------------------------------------------------------
// Copies bytes [begin, end) of src to dst with the whole CTA.
__device__ __forceinline__ void ctaCopy(char *dst, const char *src, size_t begin, size_t end) {
  if (begin >= end) return;
  const int t = threadIdx.x, n = blockDim.x;
  if ((((uintptr_t)dst | (uintptr_t)src) & 15) == 0) {
    size_t vb = (begin + 15) >> 4, ve = end >> 4;
    if (vb > ve) vb = ve = (begin + 15) >> 4;
    // head and tail bytes outside the 16-byte aligned middle
    size_t headEnd = (vb << 4) < end ? (vb << 4) : end;
    for (size_t i = begin + t; i < headEnd; i += n) dst[i] = src[i];
    if (ve > vb) {
      const uint4 *s = (const uint4 *)src;
      uint4 *d = (uint4 *)dst;
      size_t i = vb + t;
      // peer loads take microseconds: keep eight in flight per thread
      for (; i + 7 * (size_t)n < ve; i += 8 * (size_t)n) {
        uint4 r[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) r[u] = ldSys16(s + i + u * (size_t)n);
#pragma unroll
        for (int u = 0; u < 8; ++u) st16(d + i + u * (size_t)n, r[u]);
      }
      for (; i < ve; i += n) st16(d + i, ldSys16(s + i));
    }
    const size_t tailBegin = ve > vb ? (ve << 4) : headEnd;
    for (size_t j = tailBegin + t; j < end; j += n) dst[j] = src[j];
  } else {
    for (size_t i = begin + t; i < end; i += n) dst[i] = src[i];
  }
}

} // namespace fcx
