// ll_kernels.cu -- small messages without any barrier: data and "it has arrived" travel in
// the same 16-byte store (all-reduce, all-gather, reduce-scatter, all-to-all).
#include "coll_common.cuh"

namespace fcx {
namespace {

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
  // a.count elements make one message: the whole input (all-reduce), one rank's block
  // (all-gather), or the block destined to one rank (reduce-scatter, all-to-all)
  const size_t bytes = a.count * sizeof(T);
  const size_t units = (bytes + 7) >> 3;
  const bool perPeer = a.kind == kLlReduceScatter || a.kind == kLlAllToAll; // every peer gets its own block
  const bool reduces = a.kind == kLlAllReduce || a.kind == kLlReduceScatter;
  FCX_BOUNDS(c, units << 4, a.llSlotBytes, 3); // the encoded message must fit one slot
  FCX_BOUNDS(c, perPeer ? a.inStride * (size_t)(n - 1) + bytes : bytes, a.inBytes, 1);
  FCX_BOUNDS(c, reduces ? bytes : a.outStride * (size_t)(n - 1) + bytes, a.outBytes, 2);
  const size_t parityOff = (size_t)(a.llEpoch & 1u) * FLAGCX_MAX_RANKS * a.llSlotBytes;
  const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nt = (size_t)gridDim.x * blockDim.x;
  const char *in = a.in[rank];
  for (size_t u = t; u < units; u += nt) {
    uint32_t d0, d1;
    if (!perPeer) llLoadUnit(in, bytes, u, d0, d1);
    for (int k = 1; k < n; ++k) {
      int p = rank + k; if (p >= n) p -= n;
      if (perPeer) llLoadUnit(in + a.inStride * p, bytes, u, d0, d1);
      llSend(a.aux[p] + parityOff + (size_t)rank * a.llSlotBytes + (u << 4), d0, d1, a.llEpoch);
    }
  }
  const char *mine = a.aux[rank] + parityOff;
  const char *own = perPeer ? in + a.inStride * rank : in; // what this rank contributes to itself
  for (size_t u = t; u < units; u += nt) {
    if (reduces) {
      Acc acc[N];
      for (int p = 0; p < n; ++p) { // rank order: every rank computes bit-identical results
        uint32_t w[2];
        if (p == rank) llLoadUnit(own, bytes, u, w[0], w[1]);
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
        if (p == rank) llLoadUnit(own, bytes, u, d0, d1);
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

} // namespace

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
  if (a.kind == kLlAllGather || a.kind == kLlAllToAll) return launchLlT<unsigned char>(lc, a); // bytes
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

} // namespace fcx
