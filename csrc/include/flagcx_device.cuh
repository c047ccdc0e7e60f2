/*
 * flagcx_device.cuh -- device-side API: communicator and memory handles, teams,
 * cooperative groups, barriers, peer/multicast pointers and one-sided
 * put/get/signal/counter primitives, all over NVLink peer mappings.
 *
 * The vocabulary (flagcxDevComm, flagcxDevMem, flagcxTeam, flagcxCoop*,
 * flagcxDevBarrier, flagcxGet*Pointer, flagcxSymPtr, flagcxDevNet with
 * put/get/signal/putValue/waitSignal/counters/shadows) follows the FlagCX device
 * API (flagcx/adaptor/include/device_api/flagcx_device_core.h in the FlagCX
 * project).  The mechanism does not: there is no device-to-host FIFO and no
 * proxy thread.  Every primitive is a handful of loads/stores on peer-mapped
 * memory with explicit release/acquire at system scope, and every wait is
 * bounded: it gives up after devComm.timeoutNs (or when the host raises the abort
 * flag), records who it was waiting for in the host-visible status block and
 * returns false, so a missing peer becomes an error code rather than a hung GPU.
 *
 * All structs are plain data and are passed to kernels by value.
 */
#ifndef FLAGCX_DEVICE_CUH_
#define FLAGCX_DEVICE_CUH_

#include <stdint.h>
#include <cuda_runtime.h>

#define FLAGCX_MAX_RANKS 8           /* ranks of one NVLink domain */
#define FLAGCX_COLL_BARRIER_SLOTS 256 /* slots [0,256): the library's own kernels */
#define FLAGCX_USER_BARRIER_SLOTS 256 /* slots [256,512): flagcxDevBarrier users */
#define FLAGCX_BARRIER_SLOTS (FLAGCX_COLL_BARRIER_SLOTS + FLAGCX_USER_BARRIER_SLOTS)
#define FLAGCX_MAX_SIGNALS 1024
#define FLAGCX_MAX_COUNTERS 256
/* signals [512, 512+320): arrival counters of the multicast barrier (flagcxDevBarrierNvls),
 * 256 for the library's kernels (one per CTA slot) and 64 for users */
#define FLAGCX_NVLS_BARRIER_SIGNAL_BASE 512
#define FLAGCX_NVLS_USER_BARRIER_SLOTS 64

#define FLAGCX_DEVICE_CTA_COUNT 32
#define FLAGCX_DEVICE_THREADS_PER_CTA 512

/* error codes written to flagcxDevStatus.code */
#define FLAGCX_DEV_OK 0u
#define FLAGCX_DEV_TIMEOUT 1u
#define FLAGCX_DEV_ABORTED 2u
#define FLAGCX_DEV_BOUNDS 3u

/* where a wait gave up (flagcxDevStatus.where) */
#define FLAGCX_DEV_AT_BARRIER 1u
#define FLAGCX_DEV_AT_SIGNAL 2u
#define FLAGCX_DEV_AT_COUNTER 3u
#define FLAGCX_DEV_AT_KERNEL 4u

/* Lives in pinned host memory mapped into the device: the host reads it
 * without any CUDA call, device code writes the first error only. */
struct flagcxDevStatus {
  unsigned int abortFlag; /* host -> device: give up all waits */
  unsigned int code;      /* device -> host: first error */
  unsigned int peer;
  unsigned int where;
  unsigned long long detail; /* value waited for / offending offset */
  unsigned long long errCount;
};

struct flagcxDevComm {
  int rank, nRanks;
  int intraRank, intraSize;
  /* barrierInbox[p] is rank p's inbox as mapped here: [slot][sender] u64 */
  unsigned long long *barrierInbox[FLAGCX_MAX_RANKS];
  /* signalPad[p] is rank p's signal array as mapped here */
  unsigned long long *signalPad[FLAGCX_MAX_RANKS];
  unsigned long long *barrierEpoch; /* local, one per slot */
  unsigned long long *signalShadow; /* local, one per signal */
  unsigned long long *counters;     /* local, one per counter */
  unsigned long long *mcSignalPad;  /* multicast alias of the signal pads, or NULL */
  flagcxDevStatus *status;
  unsigned long long timeoutNs;
  int nSignals, nCounters;
  int nvlsBarrier; /* 1: the library's kernels meet through the multicast barrier */
  int reserved;
};

struct flagcxDevMem {
  char *peer[FLAGCX_MAX_RANKS]; /* peer[r]: rank r's buffer as mapped here */
  char *mc;                     /* multicast alias, or NULL */
  size_t size;
  int rank, nRanks;
};

/* ---- teams: {nRanks, rank, stride} subsets of the world ----------------- */
struct flagcxTeam {
  int nRanks, rank, stride;
};

__host__ __device__ inline flagcxTeam flagcxMakeTeam(int n, int r, int s) {
  flagcxTeam t; t.nRanks = n; t.rank = r; t.stride = s; return t;
}
__host__ __device__ inline flagcxTeam flagcxTeamWorld(const flagcxDevComm &c) {
  return flagcxMakeTeam(c.nRanks, c.rank, 1);
}
__host__ __device__ inline flagcxTeam flagcxTeamIntra(const flagcxDevComm &c) {
  return flagcxMakeTeam(c.intraSize, c.intraRank, 1);
}
__host__ __device__ inline flagcxTeam flagcxTeamInter(const flagcxDevComm &c) {
  return flagcxMakeTeam(c.nRanks / c.intraSize, c.rank / c.intraSize, c.intraSize);
}
/* world rank of member `r` of `team` */
__host__ __device__ inline int flagcxTeamRankToWorld(const flagcxDevComm &c, flagcxTeam team, int r) {
  return c.rank + (r - team.rank) * team.stride;
}
__host__ __device__ inline int flagcxTeamRankToIntra(const flagcxDevComm &c, flagcxTeam team, int r) {
  return c.intraRank + (r - team.rank) * team.stride;
}
/* is member bPeer of team b also a member of team a / which one */
__host__ __device__ inline bool flagcxTeamRankIsMember(flagcxTeam a, flagcxTeam b, int bPeer) {
  int w = (bPeer - b.rank) * b.stride;
  int ar = a.rank + w / a.stride;
  return w % a.stride == 0 && ar >= 0 && ar < a.nRanks;
}
__host__ __device__ inline int flagcxTeamRankToTeam(flagcxTeam a, flagcxTeam b, int bPeer) {
  return a.rank + ((bPeer - b.rank) * b.stride) / a.stride;
}
__host__ __device__ inline flagcxTeam flagcxTeamInnerFactor(flagcxTeam parent, int inner) {
  return flagcxMakeTeam(inner, parent.rank % inner, parent.stride);
}
__host__ __device__ inline flagcxTeam flagcxTeamOuterFactor(flagcxTeam parent, int inner) {
  return flagcxMakeTeam(parent.nRanks / inner, parent.rank / inner, parent.stride * inner);
}

#ifdef __CUDACC__

/* ---- memory-order primitives --------------------------------------------- */
namespace fcxdev {

__device__ __forceinline__ unsigned long long ldAcquireSys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ldRelaxedSys(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void stReleaseSys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void stRelaxedSys(unsigned long long *p, unsigned long long v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void redAddReleaseSys(unsigned long long *p, unsigned long long v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void fenceSys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}
__device__ __forceinline__ unsigned long long globalTimerNs() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned int ldVolatileU32(const unsigned int *p) {
  unsigned int v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

/* First error wins; later ones are only counted. */
__device__ __forceinline__ void reportError(flagcxDevStatus *st, unsigned int code, unsigned int where,
                                            unsigned int peer, unsigned long long detail) {
  if (!st) return;
  if (atomicCAS_system(&st->code, FLAGCX_DEV_OK, code) == FLAGCX_DEV_OK) {
    st->peer = peer;
    st->where = where;
    st->detail = detail;
  }
  atomicAdd_system(&st->errCount, 1ull);
  __threadfence_system();
}

/* Spin until *p >= want.  Returns false after timeoutNs or on abort. */
__device__ __forceinline__ bool waitGe(const flagcxDevComm &c, const unsigned long long *p,
                                       unsigned long long want, unsigned int where, unsigned int peer) {
  if (ldAcquireSys(p) >= want) return true;
  const unsigned long long t0 = globalTimerNs();
  unsigned int spins = 0, ns = 20;
  for (;;) {
    if (ldAcquireSys(p) >= want) return true;
    __nanosleep(ns);
    if (ns < 400) ns += ns >> 1;
    if ((++spins & 63u) == 0) {
      if (c.status && ldVolatileU32(&c.status->abortFlag)) {
        reportError(c.status, FLAGCX_DEV_ABORTED, where, peer, want);
        return false;
      }
      if (globalTimerNs() - t0 > c.timeoutNs) {
        reportError(c.status, FLAGCX_DEV_TIMEOUT, where, peer, want);
        return false;
      }
    }
  }
}

} // namespace fcxdev

/* ---- cooperative groups ---------------------------------------------------- */
struct flagcxCoopThread {
  __device__ int threadRank() const { return 0; }
  __device__ int size() const { return 1; }
  __device__ void sync() const {}
};
struct flagcxCoopWarp {
  __device__ int threadRank() const { return threadIdx.x & 31; }
  __device__ int size() const { return 32; }
  __device__ void sync() const { __syncwarp(); }
};
template <int N>
struct flagcxCoopTile { /* N consecutive lanes of a warp, N a power of two <= 32 */
  __device__ int threadRank() const { return threadIdx.x & (N - 1); }
  __device__ int size() const { return N; }
  __device__ unsigned mask() const {
    unsigned lane = threadIdx.x & 31;
    unsigned base = lane & ~(unsigned)(N - 1);
    return (N == 32 ? 0xffffffffu : ((1u << N) - 1u)) << base;
  }
  __device__ void sync() const { __syncwarp(mask()); }
};
struct flagcxCoopBlock {
  __device__ int threadRank() const {
    return threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
  }
  __device__ int size() const { return blockDim.x * blockDim.y * blockDim.z; }
  __device__ void sync() const { __syncthreads(); }
};
/* All threads of a thread-block cluster (a single block when launched without
 * cluster dimensions). */
struct flagcxCoopCluster {
  __device__ static unsigned ctaRank() {
    unsigned r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
  }
  __device__ static unsigned nCtas() {
    unsigned r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r;
  }
  __device__ int threadRank() const {
    return (int)(ctaRank() * blockDim.x * blockDim.y * blockDim.z) + flagcxCoopBlock().threadRank();
  }
  __device__ int size() const { return (int)(nCtas() * blockDim.x * blockDim.y * blockDim.z); }
  __device__ void sync() const {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
};

/* ---- pointers ------------------------------------------------------------------ */
__device__ __forceinline__ void *flagcxGetPeerPointer(const flagcxDevMem &m, size_t off, int worldPeer) {
  return (worldPeer >= 0 && worldPeer < m.nRanks && m.peer[worldPeer]) ? m.peer[worldPeer] + off : nullptr;
}
__device__ __forceinline__ void *flagcxGetPeerPointer(const flagcxDevComm &c, const flagcxDevMem &m,
                                                      size_t off, flagcxTeam team, int teamPeer) {
  return flagcxGetPeerPointer(m, off, flagcxTeamRankToWorld(c, team, teamPeer));
}
__device__ __forceinline__ void *flagcxGetLocalPointer(const flagcxDevMem &m, size_t off) {
  return m.peer[m.rank] + off;
}
__device__ __forceinline__ void *flagcxGetIntraPointer(const flagcxDevMem &m, size_t off, int intraPeer) {
  return flagcxGetPeerPointer(m, off, intraPeer); /* one NVLink domain: intra rank == world rank */
}
__device__ __forceinline__ void *flagcxGetMulticastPointer(const flagcxDevMem &m, size_t off) {
  return m.mc ? m.mc + off : nullptr;
}

/* A typed offset into a symmetric buffer: the same flagcxSymPtr names the same
 * element in every rank's copy. */
template <typename T>
struct flagcxSymPtr {
  flagcxDevMem mem;
  size_t byteOff;
  __device__ flagcxSymPtr() : mem(), byteOff(0) {}
  __device__ flagcxSymPtr(const flagcxDevMem &m, size_t off) : mem(m), byteOff(off) {}
  __device__ T *localPtr() const { return (T *)flagcxGetLocalPointer(mem, byteOff); }
  __device__ T *peerPtr(int worldPeer) const { return (T *)flagcxGetPeerPointer(mem, byteOff, worldPeer); }
  __device__ T *multicastPtr() const { return (T *)flagcxGetMulticastPointer(mem, byteOff); }
  __device__ flagcxSymPtr operator+(ptrdiff_t n) const { return flagcxSymPtr(mem, byteOff + n * sizeof(T)); }
  __device__ flagcxSymPtr operator-(ptrdiff_t n) const { return flagcxSymPtr(mem, byteOff - n * sizeof(T)); }
  __device__ flagcxSymPtr &operator+=(ptrdiff_t n) { byteOff += n * sizeof(T); return *this; }
  __device__ ptrdiff_t operator-(const flagcxSymPtr &o) const {
    return ((ptrdiff_t)byteOff - (ptrdiff_t)o.byteOff) / (ptrdiff_t)sizeof(T);
  }
  __device__ bool operator==(const flagcxSymPtr &o) const {
    return byteOff == o.byteOff && mem.peer[mem.rank] == o.mem.peer[o.mem.rank];
  }
  template <typename U>
  __device__ flagcxSymPtr<U> cast() const { return flagcxSymPtr<U>(mem, byteOff); }
};

/* ---- barrier across the ranks of one NVLink domain --------------------------------
 * Slot `index` has, on every rank, one inbox word per sender.  arrive() publishes
 * epoch+1 into every peer's inbox with release semantics; wait() spins (bounded)
 * until every peer's word in the local inbox reached it.  All threads of the
 * group must call; the result is uniform across the group (block groups only). */
struct flagcxDevBarrierIntra {
  const flagcxDevComm &c;
  int slot;
  unsigned long long epoch;
  __device__ flagcxDevBarrierIntra(const flagcxDevComm &comm, int index)
      : c(comm), slot(index), epoch(0) {}

  template <typename Coop>
  __device__ void arrive(Coop g) {
    g.sync(); /* the group's earlier writes happen-before the flag */
    epoch = c.barrierEpoch[slot] + 1;
    int t = g.threadRank();
    if (t < c.nRanks && t != c.rank) {
      fcxdev::fenceSys();
      fcxdev::stReleaseSys(c.barrierInbox[t] + (size_t)slot * FLAGCX_MAX_RANKS + c.rank, epoch);
    }
  }
  template <typename Coop>
  __device__ bool wait(Coop g) {
    int t = g.threadRank();
    bool ok = true;
    if (t < c.nRanks && t != c.rank)
      ok = fcxdev::waitGe(c, c.barrierInbox[c.rank] + (size_t)slot * FLAGCX_MAX_RANKS + t, epoch,
                          FLAGCX_DEV_AT_BARRIER, (unsigned)t);
    /* __syncthreads_or both joins the group and makes the verdict uniform */
    int bad = __syncthreads_or(ok ? 0 : 1);
    if (g.threadRank() == 0) c.barrierEpoch[slot] = epoch;
    return !bad;
  }
  template <typename Coop>
  __device__ bool sync(Coop g) { arrive(g); return wait(g); }
};
/* One NVLink domain: the world barrier is the intra barrier. */
typedef flagcxDevBarrierIntra flagcxDevBarrierWorld;

/* ---- the same barrier through the NVLink switch ------------------------------------
 * Needs the communicator's multicast binding (comm.mcSignalPad != NULL).  Arriving is ONE
 * multimem.red: the switch adds 1 to the slot's counter in every rank's memory at once,
 * instead of one store per peer; a rank waits until its own copy has grown by nRanks.
 * Slot `index` < 256 + FLAGCX_NVLS_USER_BARRIER_SLOTS; slots from 256 on are for users.
 * The number of completed rounds lives in the slot's signal shadow.  Block groups only. */
struct flagcxDevBarrierNvls {
  const flagcxDevComm &c;
  int sig;
  __device__ flagcxDevBarrierNvls(const flagcxDevComm &comm, int index)
      : c(comm), sig(FLAGCX_NVLS_BARRIER_SIGNAL_BASE + index) {}
  template <typename Coop>
  __device__ bool sync(Coop g) {
    g.sync(); /* the group's earlier writes happen-before the arrival */
    bool ok = true;
    if (g.threadRank() == 0) {
      const unsigned long long target = c.signalShadow[sig] + (unsigned long long)c.nRanks;
      fcxdev::fenceSys();
      asm volatile("multimem.red.release.sys.global.add.u64 [%0], %1;" ::"l"(c.mcSignalPad + sig), "l"(1ull) : "memory");
      ok = fcxdev::waitGe(c, c.signalPad[c.rank] + sig, target, FLAGCX_DEV_AT_BARRIER, 0xffffffffu);
      c.signalShadow[sig] = target;
    }
    int bad = __syncthreads_or(ok ? 0 : 1);
    return !bad;
  }
};

/* ---- one-sided operations ------------------------------------------------------------ */
struct flagcxDevNet_None {};
struct flagcxDevNet_SignalInc { int signal; };
struct flagcxDevNet_SignalAdd { int signal; unsigned long long value; };
struct flagcxDevNet_CounterInc { int counter; };

namespace fcxdev {
/* Group-cooperative copy, widest aligned access first. */
template <typename Coop>
__device__ __forceinline__ void coopCopy(Coop g, void *dst, const void *src, size_t bytes) {
  const int t = g.threadRank(), n = g.size();
  char *d = (char *)dst;
  const char *s = (const char *)src;
  if ((((uintptr_t)d | (uintptr_t)s) & 15) == 0) {
    size_t nv = bytes >> 4;
    for (size_t i = t; i < nv; i += n) ((uint4 *)d)[i] = ((const uint4 *)s)[i];
    size_t done = nv << 4;
    for (size_t i = done + t; i < bytes; i += n) d[i] = s[i];
  } else if ((((uintptr_t)d | (uintptr_t)s) & 3) == 0) {
    size_t nv = bytes >> 2;
    for (size_t i = t; i < nv; i += n) ((uint32_t *)d)[i] = ((const uint32_t *)s)[i];
    size_t done = nv << 2;
    for (size_t i = done + t; i < bytes; i += n) d[i] = s[i];
  } else {
    for (size_t i = t; i < bytes; i += n) d[i] = s[i];
  }
}
} // namespace fcxdev

struct flagcxDevNet {
  const flagcxDevComm &c;
  __device__ explicit flagcxDevNet(const flagcxDevComm &comm) : c(comm) {}

  __device__ void remote(int peer, flagcxDevNet_None) const {}
  __device__ void remote(int peer, flagcxDevNet_SignalInc a) const {
    fcxdev::redAddReleaseSys(c.signalPad[peer] + a.signal, 1ull);
  }
  __device__ void remote(int peer, flagcxDevNet_SignalAdd a) const {
    fcxdev::redAddReleaseSys(c.signalPad[peer] + a.signal, a.value);
  }
  __device__ void local(flagcxDevNet_None) const {}
  __device__ void local(flagcxDevNet_CounterInc a) const {
    atomicAdd(c.counters + a.counter, 1ull);
  }

  /* Copy bytes from the local copy of src into peer's copy of dst, then apply the
   * remote action on the peer (ordered after the data) and the local action. */
  template <typename RemoteAction, typename LocalAction, typename Coop>
  __device__ void put(int peer, const flagcxDevMem &dst, size_t dstOff, const flagcxDevMem &src,
                      size_t srcOff, size_t bytes, RemoteAction ra, LocalAction la, Coop g) const {
    fcxdev::coopCopy(g, dst.peer[peer] + dstOff, src.peer[src.rank] + srcOff, bytes);
    g.sync();
    if (g.threadRank() == 0) {
      fcxdev::fenceSys();
      remote(peer, ra);
      local(la);
    }
  }
  /* Copy bytes from peer's copy of src into the local copy of dst. */
  template <typename Coop>
  __device__ void get(int peer, const flagcxDevMem &src, size_t srcOff, const flagcxDevMem &dst,
                      size_t dstOff, size_t bytes, Coop g) const {
    fcxdev::coopCopy(g, dst.peer[dst.rank] + dstOff, src.peer[peer] + srcOff, bytes);
    g.sync();
  }
  /* Store one 64-bit value into peer's copy of dst (8-byte aligned offset). */
  template <typename RemoteAction, typename Coop>
  __device__ void putValue(int peer, const flagcxDevMem &dst, size_t dstOff, unsigned long long v,
                           RemoteAction ra, Coop g) const {
    if (g.threadRank() == 0) {
      fcxdev::stRelaxedSys((unsigned long long *)(dst.peer[peer] + dstOff), v);
      fcxdev::fenceSys();
      remote(peer, ra);
    }
  }
  template <typename RemoteAction, typename Coop>
  __device__ void signal(int peer, RemoteAction ra, Coop g) const {
    g.sync();
    if (g.threadRank() == 0) { fcxdev::fenceSys(); remote(peer, ra); }
  }

  __device__ unsigned long long readSignal(int sig) const {
    return fcxdev::ldAcquireSys(c.signalPad[c.rank] + sig);
  }
  /* Wait until local signal `sig` >= least.  Uniform result across the group. */
  template <typename Coop>
  __device__ bool waitSignal(int sig, unsigned long long least, Coop g) const {
    bool ok = true;
    if (g.threadRank() == 0)
      ok = fcxdev::waitGe(c, c.signalPad[c.rank] + sig, least, FLAGCX_DEV_AT_SIGNAL, 0xffffffffu);
    return shareVerdict(ok, g);
  }
  /* Shadows remember how far a signal has been consumed, so a kernel can wait for
   * "delta more than last time" without host bookkeeping. */
  __device__ unsigned long long readShadow(int sig) const { return c.signalShadow[sig]; }
  template <typename Coop>
  __device__ bool waitSignalMeetShadow(int sig, unsigned long long delta, Coop g) const {
    unsigned long long target = c.signalShadow[sig] + delta;
    bool ok = waitSignal(sig, target, g);
    return ok;
  }
  template <typename Coop>
  __device__ bool waitSignalFollowShadow(int sig, unsigned long long delta, Coop g) const {
    unsigned long long target = c.signalShadow[sig] + delta;
    bool ok = waitSignal(sig, target, g);
    g.sync();
    if (ok && g.threadRank() == 0) c.signalShadow[sig] = target;
    g.sync();
    return ok;
  }
  __device__ void resetSignal(int sig) const {
    fcxdev::stRelaxedSys(c.signalPad[c.rank] + sig, 0ull);
    c.signalShadow[sig] = 0;
  }
  __device__ unsigned long long readCounter(int ctr) const {
    return *(volatile unsigned long long *)(c.counters + ctr);
  }
  template <typename Coop>
  __device__ bool waitCounter(int ctr, unsigned long long least, Coop g) const {
    bool ok = true;
    if (g.threadRank() == 0)
      ok = fcxdev::waitGe(c, c.counters + ctr, least, FLAGCX_DEV_AT_COUNTER, 0xffffffffu);
    return shareVerdict(ok, g);
  }
  __device__ void resetCounter(int ctr) const { c.counters[ctr] = 0; }
  /* Stores to peer memory are complete once a system fence has been passed;
   * flush exists so code written against a network-backed put keeps working. */
  template <typename Coop>
  __device__ void flush(Coop g) const { fcxdev::fenceSys(); g.sync(); }

 private:
  __device__ bool shareVerdict(bool ok, flagcxCoopBlock) const { return !__syncthreads_or(ok ? 0 : 1); }
  __device__ bool shareVerdict(bool ok, flagcxCoopWarp) const { return __all_sync(0xffffffffu, ok); }
  template <int N>
  __device__ bool shareVerdict(bool ok, flagcxCoopTile<N> g) const { return __all_sync(g.mask(), ok); }
  __device__ bool shareVerdict(bool ok, flagcxCoopThread) const { return ok; }
};

#endif /* __CUDACC__ */
#endif /* FLAGCX_DEVICE_CUH_ */
