// api_onesided.cc -- the extern "C" surface, part 2: the one-sided host API (register,
// put / get / signal / counters) between ranks of one NVLink domain.  Same calls as
// flagcxOneSide* / flagcxPut / flagcxGet / flagcxPutSignal / flagcxWaitSignal of the FlagCX
// project (flagcx/flagcx.cc), which go through a net adaptor there; here a put is a copy
// kernel into the peer's mapped window and a signal is a remote atomic.
#include <algorithm>

#include "../kernels/launch.h"
#include "api_internal.h"

using namespace fcx;

extern "C" {

// ---------------------------------------------------------------------------
// one-sided host API (ranks of one NVLink domain)
// ---------------------------------------------------------------------------
static int hostSignalIndex(int srcRank) { return FLAGCX_MAX_SIGNALS - FLAGCX_MAX_RANKS + srcRank; }

flagcxResult_t flagcxOneSideRegister(flagcxComm_t comm, void *buff, size_t size) {
  FCX_COMMCHECK(comm);
  if (!comm->devicePath) return flagcxNotSupported;
  Window *w = comm->windows.find(buff, size);
  const bool created = w == nullptr;
  if (!w) {
    if (comm->emu) FCXCHECK(emuWindowRegister(comm, buff, size, FLAGCX_WIN_COLL_SYMMETRIC, &w));
    else FCXCHECK(windowRegister(comm, buff, size, FLAGCX_WIN_COLL_SYMMETRIC, &w));
  }
  comm->oneSideData.push_back(w);
  comm->oneSideOwned.push_back(created ? 1 : 0);
  return flagcxSuccess;
}

// Collective: forgets every memory region of flagcxOneSideRegister (indices start at 0
// again) and unmaps the windows that call created.  Declared in
// flagcx_kernel_internal.h in the FlagCX project.
flagcxResult_t flagcxOneSideDeregister(flagcxComm_t comm) {
  FCX_COMMCHECK(comm);
  if (!comm->devicePath) return flagcxNotSupported;
  flagcxResult_t first = flagcxSuccess;
  for (size_t i = 0; i < comm->oneSideData.size(); ++i) {
    if (!comm->oneSideOwned[i]) continue;
    flagcxResult_t r = flagcxCommWindowDeregister(comm, (flagcxWindow_t)comm->oneSideData[i], flagcxMemCCL);
    if (r != flagcxSuccess && first == flagcxSuccess) first = r;
  }
  comm->oneSideData.clear();
  comm->oneSideOwned.clear();
  return first;
}
flagcxResult_t flagcxOneSideSignalDeregister(flagcxComm_t comm) {
  FCX_COMMCHECK(comm);
  if (!comm->devicePath) return flagcxNotSupported;
  flagcxResult_t r = flagcxSuccess;
  if (comm->oneSideSignalWin) r = flagcxCommWindowDeregister(comm, (flagcxWindow_t)comm->oneSideSignalWin, flagcxMemCCL);
  comm->oneSideSignalWin = nullptr;
  return r;
}
flagcxResult_t flagcxOneSideSignalRegister(const flagcxComm_t comm, void *buff, size_t size, int) {
  FCX_COMMCHECK(comm);
  if (!comm->devicePath) return flagcxNotSupported;
  Window *w = nullptr;
  if (comm->emu) FCXCHECK(emuWindowRegister(comm, buff, size, FLAGCX_WIN_COLL_SYMMETRIC, &w));
  else FCXCHECK(windowRegister(comm, buff, size, FLAGCX_WIN_COLL_SYMMETRIC, &w));
  comm->oneSideSignalWin = w;
  return flagcxSuccess;
}
// NVLink puts need no bounce buffer; the calls are accepted so callers keep working.
flagcxResult_t flagcxOneSideStagingRegister(const flagcxComm_t comm, void *, size_t) {
  FCX_COMMCHECK(comm);
  return flagcxSuccess;
}
flagcxResult_t flagcxOneSideStagingDeregister(const flagcxComm_t comm) {
  FCX_COMMCHECK(comm);
  return flagcxSuccess;
}

static flagcxResult_t rmaCopy(flagcxComm *c, bool isPut, int peer, size_t srcOff, size_t dstOff, size_t size,
                              int srcMr, int dstMr) {
  if (!c->devicePath) return flagcxNotSupported;
  FCX_ARGCHECK(peer >= 0 && peer < c->nranks && srcMr >= 0 && dstMr >= 0 && srcMr < (int)c->oneSideData.size() &&
                   dstMr < (int)c->oneSideData.size(),
               "put/get: bad peer or memory-region index");
  Window *sw = c->oneSideData[srcMr], *dw = c->oneSideData[dstMr];
  FCX_ARGCHECK(srcOff + size <= sw->size && dstOff + size <= dw->size, "put/get: range outside the registered region");
  // put: local src -> peer's dst.  get: peer's src -> local dst.
  const char *src = (const char *)(isPut ? sw->peer[c->rank] : sw->peer[peer]) + srcOff;
  char *dst = (char *)(isPut ? dw->peer[peer] : dw->peer[c->rank]) + dstOff;
  cudaError_t e = launchPutSignal(c->internalStream, dst, src, size, nullptr, 0, c->putArrival, 8);
  if (e != cudaSuccess) { FCX_WARN("put/get launch failed: %s", cudaGetErrorString(e)); return flagcxUnhandledDeviceError; }
  c->rmaIssued++;
  // completion counter the host can read without touching the stream
  void *dptr = nullptr;
  FCX_CUDACHECK(cudaHostGetDevicePointer(&dptr, (void *)c->rmaCounter, 0));
  return cu::streamWriteValue64(c->internalStream, dptr, c->rmaIssued);
}

flagcxResult_t flagcxPut(flagcxComm_t comm, int peer, size_t srcOffset, size_t dstOffset, size_t size, int srcMrIdx,
                         int dstMrIdx) {
  FCX_COMMCHECK(comm);
  return rmaCopy(comm, true, peer, srcOffset, dstOffset, size, srcMrIdx, dstMrIdx);
}
flagcxResult_t flagcxGet(flagcxComm_t comm, int peer, size_t srcOffset, size_t dstOffset, size_t size, int srcMrIdx,
                         int dstMrIdx) {
  FCX_COMMCHECK(comm);
  return rmaCopy(comm, false, peer, srcOffset, dstOffset, size, srcMrIdx, dstMrIdx);
}
flagcxResult_t flagcxBatchPut(flagcxComm_t comm, int peer, const size_t *srcOffsets, const size_t *dstOffsets,
                              const size_t *sizes, const int *srcMrIdxs, const int *dstMrIdxs, size_t count) {
  FCX_COMMCHECK(comm);
  for (size_t i = 0; i < count; ++i)
    FCXCHECK(rmaCopy(comm, true, peer, srcOffsets[i], dstOffsets[i], sizes[i], srcMrIdxs[i], dstMrIdxs[i]));
  return flagcxSuccess;
}
flagcxResult_t flagcxReadCounter(flagcxComm_t comm, uint64_t *count) {
  FCX_COMMCHECK(comm);
  if (!comm->rmaCounter || !count) return flagcxNotSupported;
  *count = *comm->rmaCounter;
  return flagcxSuccess;
}
flagcxResult_t flagcxWaitCounter(flagcxComm_t comm, uint64_t target) {
  FCX_COMMCHECK(comm);
  if (!comm->rmaCounter) return flagcxNotSupported;
  uint64_t deadline = nowNs() + comm->dev.timeoutNs;
  while (*comm->rmaCounter < target) {
    if (nowNs() > deadline) { FCX_WARN("flagcxWaitCounter: %llu not reached in time", (unsigned long long)target); return flagcxRemoteError; }
    sched_yield();
  }
  return flagcxSuccess;
}

flagcxResult_t flagcxPutSignal(const void *localbuff, size_t count, flagcxDataType_t datatype, int peer,
                               flagcxWindow_t peerWin, size_t peerWinOffset, unsigned int, flagcxComm_t comm,
                               flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  if (!comm->devicePath) return flagcxNotSupported;
  Window *w = (Window *)peerWin;
  size_t bytes = count * getFlagcxDataTypeSize(datatype);
  FCX_ARGCHECK(w && peer >= 0 && peer < comm->nranks && peerWinOffset + bytes <= w->size, "putSignal: bad argument");
  unsigned long long *sig = comm->dev.signalPad[peer] + hostSignalIndex(comm->rank);
  int ctas = (int)std::max<size_t>(1, std::min<size_t>(bytes >> 16, 32));
  cudaError_t e = launchPutSignal(rawStream(stream), (char *)w->peer[peer] + peerWinOffset, localbuff, bytes, sig, 1,
                                  comm->putArrival, ctas);
  if (e != cudaSuccess) { FCX_WARN("putSignal launch failed: %s", cudaGetErrorString(e)); return flagcxUnhandledDeviceError; }
  comm->signalSent[peer]++;
  return flagcxSuccess;
}

flagcxResult_t flagcxSignal(int peer, unsigned int, flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  if (!comm->devicePath) return flagcxNotSupported;
  FCX_ARGCHECK(peer >= 0 && peer < comm->nranks, "signal: bad peer");
  unsigned long long *sig = comm->dev.signalPad[peer] + hostSignalIndex(comm->rank);
  cudaError_t e = launchPutSignal(rawStream(stream), nullptr, nullptr, 0, sig, 1, comm->putArrival, 1);
  if (e != cudaSuccess) return flagcxUnhandledDeviceError;
  comm->signalSent[peer]++;
  return flagcxSuccess;
}

flagcxResult_t flagcxWaitSignal(int nDesc, const flagcxWaitSignalDesc_t *descs, flagcxComm_t comm,
                                flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  if (!comm->devicePath) return flagcxNotSupported;
  for (int i = 0; i < nDesc; ++i) {
    int peer = descs[i].peer;
    FCX_ARGCHECK(peer >= 0 && peer < comm->nranks, "waitSignal: bad peer");
    comm->signalSeen[peer] += descs[i].opCnt;
    const unsigned long long *sig = comm->dev.signalPad[comm->rank] + hostSignalIndex(peer);
    cudaError_t e = launchWaitSignal(rawStream(stream), comm->dev, sig, comm->signalSeen[peer], (unsigned)peer);
    if (e != cudaSuccess) return flagcxUnhandledDeviceError;
  }
  return flagcxSuccess;
}

} // extern "C"
