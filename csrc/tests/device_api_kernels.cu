// device_api_kernels.cu -- conformance kernels for the device API (flagcx_device.cuh).
//
// Built as a separate test library.  Every kernel is launched cooperatively with
// gridDim.y = number of ranks of an emulated world; block (0, r) plays rank r with its
// own flagcxDevComm / flagcxDevMem.  The host test prepares the buffers and checks them.
// The scenarios follow the FlagCX device-API test kernels (test/kernel/nvidia/
// device_api.cu:332-1298 in the FlagCX project): pointers, barrier, put with signal,
// counters, putValue, shadows, get, cooperative-group flavours, teams, resets, and a
// wait that runs out.
#include <cuda_runtime.h>

#include "flagcx_device.cuh"
#include "flagcx_device_c.cuh"

namespace {

struct TestArgs {
  const flagcxDevComm *comms;
  const flagcxDevMem *mems; // one registered buffer of u64 per rank
  unsigned long long *results; // [nRanks][64] scratch for verdicts
  int nWords;                // u64 words in each registered buffer
  int iterations;
};

__device__ unsigned long long *resultOf(const TestArgs &a, int rank) { return a.results + (size_t)rank * 64; }

// 1. pointer functions and SymPtr: every rank writes its id into slot `rank` of every peer.
__global__ void kPointers(TestArgs a) {
  const flagcxDevComm &c = a.comms[blockIdx.y];
  const flagcxDevMem &m = a.mems[blockIdx.y];
  flagcxCoopBlock blk;
  flagcxDevBarrierIntra bar(c, FLAGCX_COLL_BARRIER_SLOTS + 0);
  bool ok = bar.sync(blk);
  flagcxSymPtr<unsigned long long> sp(m, 0);
  if (threadIdx.x < c.nRanks) {
    int p = threadIdx.x;
    unsigned long long *viaPeer = (unsigned long long *)flagcxGetPeerPointer(m, 0, p);
    unsigned long long *viaIntra = (unsigned long long *)flagcxGetIntraPointer(m, 0, p);
    unsigned long long *viaTeam = (unsigned long long *)flagcxGetPeerPointer(c, m, 0, flagcxTeamWorld(c), p);
    unsigned long long *viaSym = (sp + c.rank).peerPtr(p);
    bool same = viaPeer == viaIntra && viaPeer == viaTeam && viaSym == viaPeer + c.rank;
    if (p == c.rank) same = same && viaPeer == (unsigned long long *)flagcxGetLocalPointer(m, 0) && sp.localPtr() == viaPeer;
    viaSym[0] = same ? 1000 + c.rank : 0xdead;
  }
  ok = bar.sync(blk) && ok;
  if (threadIdx.x == 0) resultOf(a, c.rank)[0] = ok;
}

// 2. barrier: a token travels round the ring, one hop per barrier.
__global__ void kBarrierRing(TestArgs a) {
  const flagcxDevComm &c = a.comms[blockIdx.y];
  const flagcxDevMem &m = a.mems[blockIdx.y];
  flagcxCoopBlock blk;
  flagcxDevBarrierIntra bar(c, FLAGCX_COLL_BARRIER_SLOTS + 1);
  unsigned long long *mine = (unsigned long long *)flagcxGetLocalPointer(m, 0);
  bool ok = true;
  if (threadIdx.x == 0) mine[0] = c.rank == 0 ? 1 : 0;
  ok = bar.sync(blk) && ok;
  for (int it = 0; it < a.iterations; ++it) {
    unsigned long long v = 0;
    int prev = (c.rank + c.nRanks - 1) % c.nRanks;
    if (threadIdx.x == 0) v = fcxdev::ldRelaxedSys((unsigned long long *)flagcxGetPeerPointer(m, 0, prev));
    ok = bar.sync(blk) && ok; // everyone has read before anyone writes
    if (threadIdx.x == 0) mine[0] = v ? v + 1 : 0;
    ok = bar.sync(blk) && ok;
  }
  if (threadIdx.x == 0) resultOf(a, c.rank)[0] = ok;
}

// 3. put + SignalInc + CounterInc, waitSignal, waitCounter: block of words to the next rank.
__global__ void kPutSignal(TestArgs a) {
  const flagcxDevComm &c = a.comms[blockIdx.y];
  const flagcxDevMem &m = a.mems[blockIdx.y];
  flagcxCoopBlock blk;
  flagcxDevNet net(c);
  const int half = a.nWords / 2;
  unsigned long long *mine = (unsigned long long *)flagcxGetLocalPointer(m, 0);
  for (int i = threadIdx.x; i < half; i += blockDim.x) mine[i] = (unsigned long long)c.rank * 100000 + i;
  blk.sync();
  int next = (c.rank + 1) % c.nRanks;
  // source: first half of my buffer; destination: second half of the next rank's buffer
  net.put(next, m, (size_t)half * 8, m, 0, (size_t)half * 8, flagcxDevNet_SignalInc{5}, flagcxDevNet_CounterInc{2}, blk);
  bool ok = net.waitSignal(5, (unsigned long long)a.iterations, blk); // iterations = how many puts so far
  ok = net.waitCounter(2, (unsigned long long)a.iterations, blk) && ok;
  if (threadIdx.x == 0) {
    resultOf(a, c.rank)[0] = ok;
    resultOf(a, c.rank)[1] = net.readSignal(5);
    resultOf(a, c.rank)[2] = net.readCounter(2);
  }
}

// 4. putValue + SignalAdd, shadows: two rounds of "wait for 3 more than last time".
__global__ void kPutValueShadow(TestArgs a) {
  const flagcxDevComm &c = a.comms[blockIdx.y];
  const flagcxDevMem &m = a.mems[blockIdx.y];
  flagcxCoopBlock blk;
  flagcxDevNet net(c);
  int next = (c.rank + 1) % c.nRanks;
  bool ok = true;
  for (int round = 0; round < 2; ++round) {
    net.putValue(next, m, 8 * (size_t)(10 + round), 7000 + (unsigned long long)c.rank * 10 + round,
                 flagcxDevNet_SignalAdd{6, 3}, blk);
    ok = net.waitSignalMeetShadow(6, 3, blk) && ok;       // does not move the shadow
    ok = net.waitSignalFollowShadow(6, 3, blk) && ok;     // moves it by 3
  }
  if (threadIdx.x == 0) {
    resultOf(a, c.rank)[0] = ok;
    resultOf(a, c.rank)[1] = net.readShadow(6);
  }
}

// 5. get: pull the previous rank's first words into my second half, warp-cooperative.
__global__ void kGetWarp(TestArgs a) {
  const flagcxDevComm &c = a.comms[blockIdx.y];
  const flagcxDevMem &m = a.mems[blockIdx.y];
  flagcxCoopBlock blk;
  flagcxDevBarrierIntra bar(c, FLAGCX_COLL_BARRIER_SLOTS + 2);
  const int half = a.nWords / 2;
  unsigned long long *mine = (unsigned long long *)flagcxGetLocalPointer(m, 0);
  for (int i = threadIdx.x; i < half; i += blockDim.x) mine[i] = (unsigned long long)c.rank * 100000 + 50000 + i;
  bool ok = bar.sync(blk);
  flagcxDevNet net(c);
  int prev = (c.rank + c.nRanks - 1) % c.nRanks;
  if (threadIdx.x < 32) net.get(prev, m, 0, m, (size_t)half * 8, (size_t)half * 8, flagcxCoopWarp());
  ok = bar.sync(blk) && ok;
  if (threadIdx.x == 0) resultOf(a, c.rank)[0] = ok;
}

// 6. cooperative-group flavours: sizes and ranks, and a tile-level signal.
__global__ void kCoops(TestArgs a) {
  const flagcxDevComm &c = a.comms[blockIdx.y];
  flagcxDevNet net(c);
  unsigned long long bad = 0;
  flagcxCoopThread th;
  flagcxCoopWarp wp;
  flagcxCoopTile<8> t8;
  flagcxCoopBlock blk;
  flagcxCoopCluster cl;
  bad |= th.size() != 1 || th.threadRank() != 0;
  bad |= wp.size() != 32 || wp.threadRank() != (int)(threadIdx.x & 31);
  bad |= t8.size() != 8 || t8.threadRank() != (int)(threadIdx.x & 7);
  bad |= blk.size() != (int)blockDim.x || blk.threadRank() != (int)threadIdx.x;
  bad |= cl.size() != (int)blockDim.x; // launched without cluster dimensions
  unsigned lane = threadIdx.x & 31;
  unsigned want = 0xffu << (lane & ~7u);
  bad |= t8.mask() != want;
  t8.sync();
  wp.sync();
  // one tile of 8 threads signals the next rank; a single thread waits for it
  int next = (c.rank + 1) % c.nRanks;
  if (threadIdx.x < 8) net.signal(next, flagcxDevNet_SignalInc{9}, t8);
  bool ok = true;
  if (threadIdx.x == 0) ok = net.waitSignal(9, (unsigned long long)a.iterations, th);
  int anyBad = __syncthreads_or((int)bad);
  if (threadIdx.x == 0) { resultOf(a, c.rank)[0] = ok && !anyBad; }
}

// 7. teams on the device (the same functions are host-callable and tested there too)
__global__ void kTeams(TestArgs a) {
  const flagcxDevComm &c = a.comms[blockIdx.y];
  if (threadIdx.x != 0) return;
  flagcxTeam w = flagcxTeamWorld(c), in = flagcxTeamIntra(c), out = flagcxTeamInter(c);
  bool ok = w.nRanks == c.nRanks && w.rank == c.rank && in.nRanks == c.intraSize && out.nRanks == c.nRanks / c.intraSize;
  for (int p = 0; p < w.nRanks; ++p) ok = ok && flagcxTeamRankToWorld(c, w, p) == p && flagcxTeamRankToIntra(c, in, p) == p;
  if (c.nRanks % 2 == 0) {
    flagcxTeam inner = flagcxTeamInnerFactor(w, 2), outer = flagcxTeamOuterFactor(w, 2);
    ok = ok && inner.nRanks == 2 && inner.rank == c.rank % 2 && outer.nRanks == c.nRanks / 2 && outer.stride == 2;
    // my pair partner is a member of the inner team, ranks two apart are members of the outer team
    ok = ok && flagcxTeamRankIsMember(inner, w, c.rank ^ 1);
    ok = ok && flagcxTeamRankToTeam(outer, w, c.rank) == c.rank / 2;
    if (c.rank + 2 < c.nRanks) ok = ok && flagcxTeamRankToTeam(outer, w, c.rank + 2) == c.rank / 2 + 1;
  }
  resultOf(a, c.rank)[0] = ok;
}

// 8. reset: signals, shadows and counters go back to zero.
__global__ void kReset(TestArgs a) {
  const flagcxDevComm &c = a.comms[blockIdx.y];
  if (threadIdx.x != 0) return;
  flagcxDevNet net(c);
  net.resetSignal(5); net.resetSignal(6); net.resetSignal(9);
  net.resetCounter(2);
  resultOf(a, c.rank)[0] = net.readSignal(5) == 0 && net.readSignal(6) == 0 && net.readShadow(6) == 0 &&
                           net.readCounter(2) == 0;
}

// 9. a wait nobody satisfies gives up after the communicator's limit and says so.
__global__ void kWaitTimesOut(TestArgs a) {
  const flagcxDevComm &c = a.comms[blockIdx.y];
  flagcxDevNet net(c);
  bool ok = net.waitSignal(11, 1, flagcxCoopBlock());
  if (threadIdx.x == 0) resultOf(a, c.rank)[0] = ok ? 1 : 0;
}

// 10. the C-linkage wrappers (flagcx_device_c.cuh): the same ring exchange as scenario 3
// through flagcxDevPut_RSigAdd_LCtrInc / flagcxDevWaitSignal, a flagcxDevGet back, a
// flagcxDevPutValue_RSigInc, shadows and the barrier, addressed only by opaque pointers.
__global__ void kCWrappers(TestArgs a) {
  const void *comm = &a.comms[blockIdx.y];
  const void *mem = &a.mems[blockIdx.y];
  const flagcxDevComm &c = a.comms[blockIdx.y];
  const int half = a.nWords / 2, n = c.nRanks;
  const int next = (c.rank + 1) % n, prev = (c.rank + n - 1) % n;
  const flagcxDevSignal_t sigData = 20, sigValue = 21;
  const flagcxDevCounter_t ctr = 7;
  unsigned long long *mine = (unsigned long long *)flagcxGetLocalPointer(a.mems[blockIdx.y], 0);
  bool ok = true;
  if (threadIdx.x == 0) {
    flagcxDevResetSignal(comm, 0, sigData);
    flagcxDevResetSignal(comm, 0, sigValue);
    flagcxDevResetCounter(comm, 0, ctr);
  }
  for (int i = threadIdx.x; i < half; i += blockDim.x) mine[i] = (unsigned long long)c.rank * 100000 + i;
  for (int i = half + threadIdx.x; i < a.nWords; i += blockDim.x) mine[i] = 0;
  flagcxDevBarrierSync(comm, FLAGCX_TEAM_WORLD, 9, 0, FLAGCX_COOP_BLOCK, FLAGCX_MEMORY_ORDER_ACQ_REL, FLAGCX_MEMORY_SCOPE_SYSTEM);
  // first quarter to the next rank's second half, signal += 5, local counter += 1
  const size_t q = (size_t)(half / 2) * 8;
  flagcxDevPut_RSigAdd_LCtrInc(comm, mem, (size_t)half * 8, mem, 0, q, FLAGCX_TEAM_WORLD, next, 0, FLAGCX_COOP_BLOCK,
                               FLAGCX_MEMORY_SCOPE_SYSTEM, FLAGCX_MEMORY_ORDER_RELEASE, sigData, 5, ctr);
  flagcxDevWaitSignal(comm, sigData, 5, 64, 0, FLAGCX_COOP_BLOCK, FLAGCX_MEMORY_ORDER_ACQUIRE);
  flagcxDevWaitCounter(comm, ctr, 1, 64, 0, FLAGCX_COOP_BLOCK, FLAGCX_MEMORY_ORDER_ACQUIRE);
  for (int i = threadIdx.x; i < half / 2; i += blockDim.x)
    ok = ok && mine[half + i] == (unsigned long long)prev * 100000 + i;
  ok = ok && flagcxDevReadSignal(comm, sigData, 64, 0, FLAGCX_MEMORY_ORDER_ACQUIRE) == 5 &&
       flagcxDevReadCounter(comm, ctr, 64, 0, FLAGCX_MEMORY_ORDER_ACQUIRE) == 1;
  // warp 0 fetches the second quarter of the previous rank's first half, all but its last
  // word: the buffer's last word is the target of the putValue below
  if (threadIdx.x < 32)
    flagcxDevGet(comm, mem, q, mem, (size_t)half * 8 + q, q - 8, FLAGCX_TEAM_INTRA, prev, 0, FLAGCX_COOP_WARP,
                 FLAGCX_MEMORY_SCOPE_SYSTEM, FLAGCX_MEMORY_ORDER_ACQUIRE);
  __syncthreads();
  for (int i = threadIdx.x; i < half / 2 - 1; i += blockDim.x)
    ok = ok && mine[half + half / 2 + i] == (unsigned long long)prev * 100000 + half / 2 + i;
  // one thread writes a value into the next rank's last word and raises a signal; the
  // receiver waits for "one more than its shadow"
  if (threadIdx.x == 0) {
    flagcxDevIncreaseSignalShadow(comm, 0, sigValue, 1);
    flagcxDevPutValue_RSigInc(comm, mem, (size_t)(a.nWords - 1) * 8, 0xabc000ull + c.rank, FLAGCX_TEAM_WORLD, next, 0,
                              FLAGCX_COOP_THREAD, FLAGCX_MEMORY_SCOPE_SYSTEM, FLAGCX_MEMORY_ORDER_RELEASE, sigValue);
    flagcxDevWaitSignalMeetShadow(comm, 0, sigValue, 64, FLAGCX_COOP_THREAD, FLAGCX_MEMORY_ORDER_ACQUIRE);
    ok = ok && fcxdev::ldRelaxedSys(mine + a.nWords - 1) == 0xabc000ull + prev;
  }
  flagcxDevFlush(comm, 0, FLAGCX_COOP_BLOCK, FLAGCX_MEMORY_ORDER_RELEASE);
  // split barrier: nobody leaves before everyone has checked
  flagcxDevBarrierArrive(comm, FLAGCX_TEAM_WORLD, 9, 0, FLAGCX_COOP_BLOCK, FLAGCX_MEMORY_ORDER_RELEASE, FLAGCX_MEMORY_SCOPE_SYSTEM);
  flagcxDevBarrierWait(comm, FLAGCX_TEAM_WORLD, 9, 0, FLAGCX_COOP_BLOCK, FLAGCX_MEMORY_ORDER_ACQUIRE, FLAGCX_MEMORY_SCOPE_SYSTEM);
  int good = __syncthreads_and(ok ? 1 : 0);
  if (threadIdx.x == 0) resultOf(a, c.rank)[0] = good;
}

} // namespace

extern "C" int fcxDevTestSizes(int *devCommBytes, int *devMemBytes) {
  *devCommBytes = (int)sizeof(flagcxDevComm);
  *devMemBytes = (int)sizeof(flagcxDevMem);
  return 0;
}

// Host-callable team algebra (same inline functions as on the device).
extern "C" int fcxDevTestTeamsHost() {
  flagcxDevComm c{};
  c.rank = 5; c.nRanks = 8; c.intraRank = 1; c.intraSize = 4;
  flagcxTeam w = flagcxTeamWorld(c), in = flagcxTeamIntra(c), out = flagcxTeamInter(c);
  bool ok = w.nRanks == 8 && in.nRanks == 4 && in.rank == 1 && out.nRanks == 2 && out.rank == 1 && out.stride == 4;
  ok = ok && flagcxTeamRankToWorld(c, in, 3) == 7 && flagcxTeamRankToWorld(c, out, 0) == 1;
  ok = ok && flagcxTeamRankIsMember(in, w, 6) && !flagcxTeamRankIsMember(in, w, 3);
  ok = ok && flagcxTeamRankToTeam(in, w, 6) == 2;
  flagcxTeam inner = flagcxTeamInnerFactor(w, 4), outer = flagcxTeamOuterFactor(w, 4);
  ok = ok && inner.nRanks == 4 && inner.rank == 1 && outer.nRanks == 2 && outer.rank == 1 && outer.stride == 4;
  return ok ? 0 : 1;
}

extern "C" int fcxDevTestLaunch(int which, const void *dComms, const void *dMems, unsigned long long *dResults,
                                int nRanks, int nWords, int iterations, void *stream) {
  TestArgs a{(const flagcxDevComm *)dComms, (const flagcxDevMem *)dMems, dResults, nWords, iterations};
  void *params[] = {&a};
  const void *fn = nullptr;
  switch (which) {
    case 1: fn = (const void *)kPointers; break;
    case 2: fn = (const void *)kBarrierRing; break;
    case 3: fn = (const void *)kPutSignal; break;
    case 4: fn = (const void *)kPutValueShadow; break;
    case 5: fn = (const void *)kGetWarp; break;
    case 6: fn = (const void *)kCoops; break;
    case 7: fn = (const void *)kTeams; break;
    case 8: fn = (const void *)kReset; break;
    case 9: fn = (const void *)kWaitTimesOut; break;
    case 10: fn = (const void *)kCWrappers; break;
    default: return (int)cudaErrorInvalidValue;
  }
  return (int)cudaLaunchCooperativeKernel(fn, dim3(1, nRanks), dim3(256), params, 0, (cudaStream_t)stream);
}
