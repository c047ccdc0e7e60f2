// nvls_kernels.cu -- collectives through the NVLink switch: multimem.ld_reduce lets the
// switch add the ranks' copies of an address, multimem.st writes all copies at once.
// Needs windows bound to a multicast object (FLAGCX_NVLS_ENABLE=1).  Counterpart of the NVLS
// kernels of the FlagCX project (flagcx/adaptor/kernel/nvidia/custom_allreduce.cu:337-467).
#include "coll_common.cuh"

namespace fcx {
namespace {

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

} // namespace

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

} // namespace fcx
