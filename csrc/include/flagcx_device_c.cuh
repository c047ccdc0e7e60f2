/*
 * flagcx_device_c.cuh -- the device API with C linkage: every operation of
 * flagcx_device.cuh as an `extern "C" __device__` function that takes only opaque
 * pointers and scalars, so that code generators and foreign front ends (anything that
 * emits calls by symbol name rather than instantiating C++ templates) can use it.
 *
 * Names and parameter lists follow the "unified one-sided IR" of the FlagCX project
 * (bindings/ir/flagcx_device_unified_ir.h:47-330 there): flagcxDevPut and its five
 * completion-action variants, flagcxDevGet, flagcxDevPutValue (+2), flagcxDevSignalInc /
 * Add, flagcxDevWaitSignal / WaitCounter, flagcxDevReadSignal / ReadCounter,
 * flagcxDevFlush, ResetSignal / ResetCounter, IncreaseSignalShadow,
 * WaitSignalMeetShadow, and the barrier trio.  The implementation is this library's:
 * one NVLink domain, so there is no transport dispatch -- a put is a group-cooperative
 * copy into the peer's mapping followed by a system fence and the completion action.
 *
 * `comm` points to a flagcxDevComm, `dst` / `src` to flagcxDevMem structs (device or
 * constant memory).  teamKind selects how `peer` is numbered (intra / inter / world;
 * identical on one NVLink domain with intraSize == nRanks).  coopKind says which
 * threads call together: FLAGCX_COOP_THREAD, _WARP or _BLOCK.  contextId, scope and
 * order are accepted for source compatibility: every action here is ordered at system
 * scope with release (remote actions) or acquire (waits) semantics, the strongest the
 * callers can ask for.  Waits are bounded like everywhere in this library; a wait that
 * gives up is recorded in the communicator's status block.
 *
 * Include this header in exactly one translation unit of a device link (the functions
 * are definitions, not inline).
 */
#ifndef FLAGCX_DEVICE_C_CUH_
#define FLAGCX_DEVICE_C_CUH_

#include "flagcx_device.cuh"

typedef enum { FLAGCX_COOP_THREAD = 0, FLAGCX_COOP_WARP = 1, FLAGCX_COOP_BLOCK = 2 } flagcxDevCoopKind_t;
typedef enum { FLAGCX_TEAM_INTRA = 0, FLAGCX_TEAM_INTER = 1, FLAGCX_TEAM_WORLD = 2 } flagcxDevTeamKind_t;
typedef enum {
  FLAGCX_MEMORY_ORDER_RELAXED = 0,
  FLAGCX_MEMORY_ORDER_ACQUIRE = 1,
  FLAGCX_MEMORY_ORDER_RELEASE = 2,
  FLAGCX_MEMORY_ORDER_ACQ_REL = 3,
  FLAGCX_MEMORY_ORDER_SEQ_CST = 4
} flagcxDevMemoryOrder_t;
typedef enum {
  FLAGCX_MEMORY_SCOPE_SYSTEM = 0,
  FLAGCX_MEMORY_SCOPE_DEVICE = 1,
  FLAGCX_MEMORY_SCOPE_BLOCK = 2,
  FLAGCX_MEMORY_SCOPE_THREAD = 3
} flagcxDevMemoryScope_t;
typedef uint32_t flagcxDevSignal_t;
typedef uint32_t flagcxDevCounter_t;
typedef uint32_t flagcxDevContext_t;

#ifdef __CUDACC__

namespace fcxdev_c {

__device__ __forceinline__ const flagcxDevComm &commOf(const void *p) { return *(const flagcxDevComm *)p; }
__device__ __forceinline__ const flagcxDevMem &memOf(const void *p) { return *(const flagcxDevMem *)p; }

/* world rank of `peer` numbered within the team of that kind */
__device__ __forceinline__ int worldPeer(const flagcxDevComm &c, flagcxDevTeamKind_t kind, int peer) {
  flagcxTeam t = kind == FLAGCX_TEAM_INTRA ? flagcxTeamIntra(c) : kind == FLAGCX_TEAM_INTER ? flagcxTeamInter(c)
                                                                                           : flagcxTeamWorld(c);
  return flagcxTeamRankToWorld(c, t, peer);
}

/* Runs f(group) with the cooperative group the caller named. */
template <typename F>
__device__ __forceinline__ void withCoop(flagcxDevCoopKind_t kind, F f) {
  if (kind == FLAGCX_COOP_BLOCK) f(flagcxCoopBlock());
  else if (kind == FLAGCX_COOP_WARP) f(flagcxCoopWarp());
  else f(flagcxCoopThread());
}

/* The one put behind all six entry points: sigMode 0 none, 1 increment, 2 add. */
__device__ __forceinline__ void put(const void *comm, const void *dst, size_t dstOff, const void *src, size_t srcOff,
                                    size_t bytes, flagcxDevTeamKind_t team, int peer, flagcxDevCoopKind_t coop,
                                    int sigMode, flagcxDevSignal_t sig, unsigned long long sigValue, bool count,
                                    flagcxDevCounter_t ctr) {
  const flagcxDevComm &c = commOf(comm);
  const int wp = worldPeer(c, team, peer);
  flagcxDevNet net(c);
  withCoop(coop, [&](auto g) {
    fcxdev::coopCopy(g, memOf(dst).peer[wp] + dstOff, memOf(src).peer[memOf(src).rank] + srcOff, bytes);
    g.sync();
    if (g.threadRank() == 0) {
      fcxdev::fenceSys();
      if (sigMode == 1) net.remote(wp, flagcxDevNet_SignalInc{(int)sig});
      else if (sigMode == 2) net.remote(wp, flagcxDevNet_SignalAdd{(int)sig, sigValue});
      if (count) net.local(flagcxDevNet_CounterInc{(int)ctr});
    }
  });
}

} // namespace fcxdev_c

#define FCX_C_DEV extern "C" __device__

/* ---- put (6) ---------------------------------------------------------------------------- */
FCX_C_DEV void flagcxDevPut(const void *comm, const void *dst, size_t dstOffset, const void *src, size_t srcOffset,
                            size_t bytes, flagcxDevTeamKind_t teamKind, int peer, flagcxDevContext_t,
                            flagcxDevCoopKind_t coopKind, flagcxDevMemoryScope_t, flagcxDevMemoryOrder_t) {
  fcxdev_c::put(comm, dst, dstOffset, src, srcOffset, bytes, teamKind, peer, coopKind, 0, 0, 0, false, 0);
}
FCX_C_DEV void flagcxDevPut_RSigInc(const void *comm, const void *dst, size_t dstOffset, const void *src,
                                    size_t srcOffset, size_t bytes, flagcxDevTeamKind_t teamKind, int peer,
                                    flagcxDevContext_t, flagcxDevCoopKind_t coopKind, flagcxDevMemoryScope_t,
                                    flagcxDevMemoryOrder_t, flagcxDevSignal_t remoteSignal) {
  fcxdev_c::put(comm, dst, dstOffset, src, srcOffset, bytes, teamKind, peer, coopKind, 1, remoteSignal, 0, false, 0);
}
FCX_C_DEV void flagcxDevPut_RSigAdd(const void *comm, const void *dst, size_t dstOffset, const void *src,
                                    size_t srcOffset, size_t bytes, flagcxDevTeamKind_t teamKind, int peer,
                                    flagcxDevContext_t, flagcxDevCoopKind_t coopKind, flagcxDevMemoryScope_t,
                                    flagcxDevMemoryOrder_t, flagcxDevSignal_t remoteSignal, uint64_t signalValue) {
  fcxdev_c::put(comm, dst, dstOffset, src, srcOffset, bytes, teamKind, peer, coopKind, 2, remoteSignal, signalValue,
                false, 0);
}
FCX_C_DEV void flagcxDevPut_LCtrInc(const void *comm, const void *dst, size_t dstOffset, const void *src,
                                    size_t srcOffset, size_t bytes, flagcxDevTeamKind_t teamKind, int peer,
                                    flagcxDevContext_t, flagcxDevCoopKind_t coopKind, flagcxDevMemoryScope_t,
                                    flagcxDevMemoryOrder_t, flagcxDevCounter_t localCounter) {
  fcxdev_c::put(comm, dst, dstOffset, src, srcOffset, bytes, teamKind, peer, coopKind, 0, 0, 0, true, localCounter);
}
FCX_C_DEV void flagcxDevPut_RSigInc_LCtrInc(const void *comm, const void *dst, size_t dstOffset, const void *src,
                                            size_t srcOffset, size_t bytes, flagcxDevTeamKind_t teamKind, int peer,
                                            flagcxDevContext_t, flagcxDevCoopKind_t coopKind, flagcxDevMemoryScope_t,
                                            flagcxDevMemoryOrder_t, flagcxDevSignal_t remoteSignal,
                                            flagcxDevCounter_t localCounter) {
  fcxdev_c::put(comm, dst, dstOffset, src, srcOffset, bytes, teamKind, peer, coopKind, 1, remoteSignal, 0, true,
                localCounter);
}
FCX_C_DEV void flagcxDevPut_RSigAdd_LCtrInc(const void *comm, const void *dst, size_t dstOffset, const void *src,
                                            size_t srcOffset, size_t bytes, flagcxDevTeamKind_t teamKind, int peer,
                                            flagcxDevContext_t, flagcxDevCoopKind_t coopKind, flagcxDevMemoryScope_t,
                                            flagcxDevMemoryOrder_t, flagcxDevSignal_t remoteSignal, uint64_t signalValue,
                                            flagcxDevCounter_t localCounter) {
  fcxdev_c::put(comm, dst, dstOffset, src, srcOffset, bytes, teamKind, peer, coopKind, 2, remoteSignal, signalValue, true,
                localCounter);
}

/* ---- get -------------------------------------------------------------------------------- */
FCX_C_DEV void flagcxDevGet(const void *comm, const void *src, size_t srcOffset, const void *dst, size_t dstOffset,
                            size_t bytes, flagcxDevTeamKind_t teamKind, int peer, flagcxDevContext_t,
                            flagcxDevCoopKind_t coopKind, flagcxDevMemoryScope_t, flagcxDevMemoryOrder_t) {
  const flagcxDevComm &c = fcxdev_c::commOf(comm);
  const int wp = fcxdev_c::worldPeer(c, teamKind, peer);
  flagcxDevNet net(c);
  fcxdev_c::withCoop(coopKind, [&](auto g) {
    net.get(wp, fcxdev_c::memOf(src), srcOffset, fcxdev_c::memOf(dst), dstOffset, bytes, g);
  });
}

/* ---- putValue (3) ------------------------------------------------------------------------- */
FCX_C_DEV void flagcxDevPutValue(const void *comm, const void *dst, size_t dstOffset, uint64_t value,
                                 flagcxDevTeamKind_t teamKind, int peer, flagcxDevContext_t, flagcxDevCoopKind_t coopKind,
                                 flagcxDevMemoryScope_t, flagcxDevMemoryOrder_t) {
  const flagcxDevComm &c = fcxdev_c::commOf(comm);
  const int wp = fcxdev_c::worldPeer(c, teamKind, peer);
  flagcxDevNet net(c);
  fcxdev_c::withCoop(coopKind, [&](auto g) { net.putValue(wp, fcxdev_c::memOf(dst), dstOffset, value, flagcxDevNet_None{}, g); });
}
FCX_C_DEV void flagcxDevPutValue_RSigInc(const void *comm, const void *dst, size_t dstOffset, uint64_t value,
                                         flagcxDevTeamKind_t teamKind, int peer, flagcxDevContext_t,
                                         flagcxDevCoopKind_t coopKind, flagcxDevMemoryScope_t, flagcxDevMemoryOrder_t,
                                         flagcxDevSignal_t remoteSignal) {
  const flagcxDevComm &c = fcxdev_c::commOf(comm);
  const int wp = fcxdev_c::worldPeer(c, teamKind, peer);
  flagcxDevNet net(c);
  fcxdev_c::withCoop(coopKind, [&](auto g) {
    net.putValue(wp, fcxdev_c::memOf(dst), dstOffset, value, flagcxDevNet_SignalInc{(int)remoteSignal}, g);
  });
}
FCX_C_DEV void flagcxDevPutValue_RSigAdd(const void *comm, const void *dst, size_t dstOffset, uint64_t value,
                                         flagcxDevTeamKind_t teamKind, int peer, flagcxDevContext_t,
                                         flagcxDevCoopKind_t coopKind, flagcxDevMemoryScope_t, flagcxDevMemoryOrder_t,
                                         flagcxDevSignal_t remoteSignal, uint64_t signalValue) {
  const flagcxDevComm &c = fcxdev_c::commOf(comm);
  const int wp = fcxdev_c::worldPeer(c, teamKind, peer);
  flagcxDevNet net(c);
  fcxdev_c::withCoop(coopKind, [&](auto g) {
    net.putValue(wp, fcxdev_c::memOf(dst), dstOffset, value, flagcxDevNet_SignalAdd{(int)remoteSignal, signalValue}, g);
  });
}

/* ---- signal (2) ----------------------------------------------------------------------------- */
FCX_C_DEV void flagcxDevSignalInc(const void *comm, flagcxDevTeamKind_t teamKind, int peer, flagcxDevSignal_t signal,
                                  flagcxDevContext_t, flagcxDevCoopKind_t coopKind, flagcxDevMemoryScope_t) {
  const flagcxDevComm &c = fcxdev_c::commOf(comm);
  const int wp = fcxdev_c::worldPeer(c, teamKind, peer);
  flagcxDevNet net(c);
  fcxdev_c::withCoop(coopKind, [&](auto g) { net.signal(wp, flagcxDevNet_SignalInc{(int)signal}, g); });
}
FCX_C_DEV void flagcxDevSignalAdd(const void *comm, flagcxDevTeamKind_t teamKind, int peer, flagcxDevSignal_t signal,
                                  uint64_t value, flagcxDevContext_t, flagcxDevCoopKind_t coopKind,
                                  flagcxDevMemoryScope_t) {
  const flagcxDevComm &c = fcxdev_c::commOf(comm);
  const int wp = fcxdev_c::worldPeer(c, teamKind, peer);
  flagcxDevNet net(c);
  fcxdev_c::withCoop(coopKind, [&](auto g) { net.signal(wp, flagcxDevNet_SignalAdd{(int)signal, value}, g); });
}

/* ---- wait (2): `bits` 32 compares the low word only -------------------------------------------- */
FCX_C_DEV void flagcxDevWaitSignal(const void *comm, flagcxDevSignal_t signal, uint64_t least, int bits,
                                   flagcxDevContext_t, flagcxDevCoopKind_t coopKind, flagcxDevMemoryOrder_t) {
  flagcxDevNet net(fcxdev_c::commOf(comm));
  if (bits == 32) least &= 0xffffffffull;
  fcxdev_c::withCoop(coopKind, [&](auto g) { net.waitSignal((int)signal, least, g); });
}
FCX_C_DEV void flagcxDevWaitCounter(const void *comm, flagcxDevCounter_t counter, uint64_t least, int bits,
                                    flagcxDevContext_t, flagcxDevCoopKind_t coopKind, flagcxDevMemoryOrder_t) {
  flagcxDevNet net(fcxdev_c::commOf(comm));
  if (bits == 32) least &= 0xffffffffull;
  fcxdev_c::withCoop(coopKind, [&](auto g) { net.waitCounter((int)counter, least, g); });
}

/* ---- read (2) ----------------------------------------------------------------------------------- */
FCX_C_DEV uint64_t flagcxDevReadSignal(const void *comm, flagcxDevSignal_t signal, int bits, flagcxDevContext_t,
                                       flagcxDevMemoryOrder_t) {
  uint64_t v = flagcxDevNet(fcxdev_c::commOf(comm)).readSignal((int)signal);
  return bits == 32 ? (v & 0xffffffffull) : v;
}
FCX_C_DEV uint64_t flagcxDevReadCounter(const void *comm, flagcxDevCounter_t counter, int bits, flagcxDevContext_t,
                                        flagcxDevMemoryOrder_t) {
  uint64_t v = flagcxDevNet(fcxdev_c::commOf(comm)).readCounter((int)counter);
  return bits == 32 ? (v & 0xffffffffull) : v;
}

/* ---- flush / reset / shadow (5) --------------------------------------------------------------------- */
FCX_C_DEV void flagcxDevFlush(const void *comm, flagcxDevContext_t, flagcxDevCoopKind_t coopKind, flagcxDevMemoryOrder_t) {
  flagcxDevNet net(fcxdev_c::commOf(comm));
  fcxdev_c::withCoop(coopKind, [&](auto g) { net.flush(g); });
}
FCX_C_DEV void flagcxDevResetSignal(const void *comm, flagcxDevContext_t, flagcxDevSignal_t slot) {
  flagcxDevNet(fcxdev_c::commOf(comm)).resetSignal((int)slot);
}
FCX_C_DEV void flagcxDevResetCounter(const void *comm, flagcxDevContext_t, flagcxDevCounter_t slot) {
  flagcxDevNet(fcxdev_c::commOf(comm)).resetCounter((int)slot);
}
FCX_C_DEV void flagcxDevIncreaseSignalShadow(const void *comm, flagcxDevContext_t, flagcxDevSignal_t slot,
                                             uint64_t delta) {
  fcxdev_c::commOf(comm).signalShadow[slot] += delta;
}
/* Waits until the signal has reached its shadow (raise the shadow first with
 * flagcxDevIncreaseSignalShadow by what is expected to arrive). */
FCX_C_DEV void flagcxDevWaitSignalMeetShadow(const void *comm, flagcxDevContext_t, flagcxDevSignal_t slot, int bits,
                                             flagcxDevCoopKind_t coopKind, flagcxDevMemoryOrder_t) {
  flagcxDevNet net(fcxdev_c::commOf(comm));
  fcxdev_c::withCoop(coopKind, [&](auto g) {
    g.sync();
    uint64_t target = net.readShadow((int)slot);
    if (bits == 32) target &= 0xffffffffull;
    net.waitSignal((int)slot, target, g);
  });
}

/* ---- barrier (3): block-cooperative; `index` is the barrier slot among the user slots ------------------ */
FCX_C_DEV void flagcxDevBarrierSync(const void *comm, flagcxDevTeamKind_t, uint32_t index, flagcxDevContext_t,
                                    flagcxDevCoopKind_t, flagcxDevMemoryOrder_t, flagcxDevMemoryScope_t) {
  flagcxDevBarrierIntra bar(fcxdev_c::commOf(comm), FLAGCX_COLL_BARRIER_SLOTS + (int)(index % FLAGCX_USER_BARRIER_SLOTS));
  bar.sync(flagcxCoopBlock());
}
/* Split form.  The epoch that ties an arrive to its wait lives in the slot's local
 * epoch word, so the pair must run in the same block, arrive first. */
FCX_C_DEV void flagcxDevBarrierArrive(const void *comm, flagcxDevTeamKind_t, uint32_t index, flagcxDevContext_t,
                                      flagcxDevCoopKind_t, flagcxDevMemoryOrder_t, flagcxDevMemoryScope_t) {
  flagcxDevBarrierIntra bar(fcxdev_c::commOf(comm), FLAGCX_COLL_BARRIER_SLOTS + (int)(index % FLAGCX_USER_BARRIER_SLOTS));
  bar.arrive(flagcxCoopBlock());
}
FCX_C_DEV void flagcxDevBarrierWait(const void *comm, flagcxDevTeamKind_t, uint32_t index, flagcxDevContext_t,
                                    flagcxDevCoopKind_t, flagcxDevMemoryOrder_t, flagcxDevMemoryScope_t) {
  const flagcxDevComm &c = fcxdev_c::commOf(comm);
  const int slot = FLAGCX_COLL_BARRIER_SLOTS + (int)(index % FLAGCX_USER_BARRIER_SLOTS);
  flagcxDevBarrierIntra bar(c, slot);
  bar.epoch = c.barrierEpoch[slot] + 1; /* the epoch the matching arrive published */
  bar.wait(flagcxCoopBlock());
}

#undef FCX_C_DEV
#endif /* __CUDACC__ */
#endif /* FLAGCX_DEVICE_C_CUH_ */
