// tcgen05.cuh -- inline-PTX wrappers for the Blackwell tensor-core path used by the
// fused GEMM+collective kernels: mbarriers with bounded waits, TMA tile loads
// (never multicast), TMEM allocation, tcgen05.mma / commit / ld, and the shared-memory
// and instruction descriptors for bf16 operands in K-major, 128-byte-swizzled tiles.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fcx {
namespace tc {

__device__ __forceinline__ uint32_t smemAddr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ---------------------------------------------------------------------
__device__ __forceinline__ void mbarInit(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbarInitFence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbarExpectTx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool mbarTryWait(uint64_t *bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smemAddr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long timerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits for the phase with the given parity; gives up after limitNs or once *abortFlag
// is set by another warp of the CTA.  Returns false when it gave up.
__device__ __forceinline__ bool mbarWait(uint64_t *bar, uint32_t parity, volatile int *abortFlag,
                                         unsigned long long limitNs) {
  if (mbarTryWait(bar, parity)) return true;
  const unsigned long long t0 = timerNs();
  unsigned spins = 0;
  for (;;) {
    if (mbarTryWait(bar, parity)) return true;
    if ((++spins & 255u) == 0) {
      if (*abortFlag) return false;
      if (timerNs() - t0 > limitNs) { *abortFlag = 1; return false; }
    }
  }
}

// ---- TMA ----------------------------------------------------------------------------
// 2-D tile load, no multicast; completes `bytes` on the mbarrier.
__device__ __forceinline__ void tmaLoad2d(void *smemDst, const CUtensorMap *map, int c0, int c1, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smemAddr(smemDst)),
      "l"(map), "r"(c0), "r"(c1), "r"(smemAddr(bar))
      : "memory");
}
__device__ __forceinline__ void prefetchTensorMap(const CUtensorMap *map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void fenceProxyAsync() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ---- TMEM ---------------------------------------------------------------------------
// Whole-warp calls.  The base address lands in *smemResult.
__device__ __forceinline__ void tmemAlloc(uint32_t *smemResult, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(smemResult)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmemRelinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemDealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void fenceBeforeSync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fenceAfterSync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- MMA ----------------------------------------------------------------------------
// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t smemDescSw128(const void *tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smemAddr(tile) & 0x3FFFFu) >> 4); // start address
  d |= (uint64_t)1 << 16;                            // leading byte offset (unused with swizzle)
  d |= (uint64_t)(1024 >> 4) << 32;                  // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                            // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                            // 128-byte swizzle
  return d;
}
// Instruction descriptor: bf16 x bf16 -> fp32, both operands K-major, tile M x N.
__host__ __device__ constexpr uint32_t instrDescBf16(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread.
__device__ __forceinline__ void mmaBf16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmemD),
      "l"(descA), "l"(descB), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
// The mbarrier receives one arrival when all MMAs issued so far by this thread are done.
__device__ __forceinline__ void mmaCommit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smemAddr(bar))
               : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane (warp w reads lanes 32*(w%4)..).
__device__ __forceinline__ void tmemLoad32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmemLoadWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- CTA pairs (cta_group::2): two CTAs of a cluster share one 256-row MMA -----------
__device__ __forceinline__ uint32_t clusterCtaRank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void clusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared variable in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapToCta(uint32_t localSmemAddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(localSmemAddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbarArriveCluster(uint32_t clusterAddr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
// Tile load into THIS CTA's shared memory whose bytes are counted on an mbarrier that may
// live in the partner CTA (given as a shared::cluster address).  No multicast.
__device__ __forceinline__ void tmaLoad2dPair(void *smemDst, const CUtensorMap *map, int c0, int c1,
                                              uint32_t barClusterAddr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smemAddr(smemDst)),
      "l"(map), "r"(c0), "r"(c1), "r"(barClusterAddr)
      : "memory");
}
__device__ __forceinline__ void tmemAllocPair(uint32_t *smemResult, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(smemResult)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmemRelinquishPair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmemDeallocPair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D (128 rows in each CTA's TMEM) (+)= A (128 rows from each CTA) * B^T (N/2 rows from each CTA)
__device__ __forceinline__ void mmaBf16Pair(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc,
                                            bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmemD),
      "l"(descA), "l"(descB), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
// One arrival on the mbarrier at the same offset in every CTA named by ctaMask.
__device__ __forceinline__ void mmaCommitPair(uint64_t *bar, uint16_t ctaMask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          smemAddr(bar)),
      "h"(ctaMask)
      : "memory");
}

} // namespace tc
} // namespace fcx
