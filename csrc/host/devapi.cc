// devapi.cc -- host half of the device API (handles for user kernels) and the
// runtime function table of flagcx.h (flagcxDeviceHandle).
//
// Counterparts in the FlagCX project: flagcx/adaptor/flagcx_device.cc:25-197
// (DevComm/DevMem create, destroy, device pointers) and the handle table filled at
// flagcx/flagcx.cc:75-130.  On a host without a GPU the table drives a "host
// device": malloc/memcpy, streams that run nothing asynchronously and events that
// are always complete, so portable caller code keeps working.
#include <chrono>

#include "comm.h"
#include "flagcx_kernel.h"

using namespace fcx;

struct flagcxDevCommInternal {
  flagcxComm *comm;
  flagcxDevComm dev;
  void *devCopy;
};
struct flagcxDevMemInternal {
  flagcxComm *comm;
  flagcxDevMem mem;
  void *devCopy;
  Window *ownedWindow;
};
struct flagcxIpcMemHandle {
  cudaIpcMemHandle_t base;
};

namespace fcx {
flagcxResult_t emuWindowRegister(flagcxComm *c, void *buff, size_t size, int flags, Window **out);
}

extern "C" {

flagcxResult_t flagcxDevCommCreate(flagcxComm_t comm, const flagcxDevCommRequirements *reqs, flagcxDevComm_t *out) {
  if (!commValid(comm) || !out) return flagcxInvalidArgument;
  if (!comm->devicePath) { FCX_WARN("device API needs the NVLink device path"); return flagcxNotSupported; }
  if (reqs) {
    int bars = std::max(reqs->barrierCount, reqs->intraBarrierCount);
    if (bars > FLAGCX_USER_BARRIER_SLOTS || reqs->interSignalCount > FLAGCX_MAX_SIGNALS - FLAGCX_MAX_RANKS ||
        reqs->interCounterCount > FLAGCX_MAX_COUNTERS) {
      FCX_WARN("device communicator requirements exceed the fixed pads (%d barriers, %d signals, %d counters)",
               FLAGCX_USER_BARRIER_SLOTS, FLAGCX_MAX_SIGNALS - FLAGCX_MAX_RANKS, FLAGCX_MAX_COUNTERS);
      return flagcxInvalidArgument;
    }
    if (reqs->intraMulticast && !(comm->internalWin && comm->internalWin->mc)) {
      FCX_WARN("multicast requested but this communicator has none (FLAGCX_NVLS_ENABLE=1 and hardware support needed)");
      return flagcxNotSupported;
    }
  }
  auto *d = new flagcxDevCommInternal{comm, comm->dev, nullptr};
  *out = d;
  return flagcxSuccess;
}

flagcxResult_t flagcxDevCommDestroy(flagcxComm_t, flagcxDevComm_t d) {
  if (!d) return flagcxSuccess;
  if (d->devCopy) cudaFree(d->devCopy);
  delete d;
  return flagcxSuccess;
}

flagcxResult_t flagcxDevMemCreate(flagcxComm_t comm, void *buff, size_t size, flagcxWindow_t win, flagcxDevMem_t *out) {
  if (!commValid(comm) || !out || !buff) return flagcxInvalidArgument;
  if (!comm->devicePath) return flagcxNotSupported;
  Window *w = (Window *)win;
  Window *owned = nullptr;
  if (!w) w = comm->windows.find(buff, size);
  if (!w) {
    if (comm->emu) FCXCHECK(emuWindowRegister(comm, buff, size, FLAGCX_WIN_DEFAULT, &w));
    else FCXCHECK(windowRegister(comm, buff, size, FLAGCX_WIN_DEFAULT, &w));
    owned = w;
  }
  if ((char *)buff < (char *)w->local || (char *)buff + size > (char *)w->local + w->size) {
    FCX_WARN("flagcxDevMemCreate: buffer is not inside the window");
    return flagcxInvalidArgument;
  }
  size_t off = (char *)buff - (char *)w->local;
  auto *m = new flagcxDevMemInternal{comm, {}, nullptr, owned};
  memset(&m->mem, 0, sizeof m->mem);
  for (int p = 0; p < comm->nranks; ++p) m->mem.peer[p] = w->peer[p] ? (char *)w->peer[p] + off : nullptr;
  m->mem.mc = w->mc ? (char *)w->mc + off : nullptr;
  m->mem.size = size;
  m->mem.rank = comm->rank;
  m->mem.nRanks = comm->nranks;
  *out = m;
  return flagcxSuccess;
}

flagcxResult_t flagcxDevMemDestroy(flagcxComm_t comm, flagcxDevMem_t m) {
  if (!m) return flagcxSuccess;
  if (m->devCopy) cudaFree(m->devCopy);
  if (m->ownedWindow && commValid(comm)) windowDeregister(comm, m->ownedWindow);
  delete m;
  return flagcxSuccess;
}

flagcxResult_t flagcxDevCommGetStruct(flagcxDevComm_t d, void *out, size_t outBytes) {
  if (!d || !out || outBytes < sizeof(flagcxDevComm)) return flagcxInvalidArgument;
  d->dev.timeoutNs = d->comm->dev.timeoutNs; // follow flagcxCommSetWaitTimeoutMs
  memcpy(out, &d->dev, sizeof(flagcxDevComm));
  return flagcxSuccess;
}
flagcxResult_t flagcxDevMemGetStruct(flagcxDevMem_t m, void *out, size_t outBytes) {
  if (!m || !out || outBytes < sizeof(flagcxDevMem)) return flagcxInvalidArgument;
  memcpy(out, &m->mem, sizeof(flagcxDevMem));
  return flagcxSuccess;
}

flagcxResult_t flagcxDevCommGetDevicePtr(flagcxDevComm_t d, void **devPtr) {
  if (!d || !devPtr) return flagcxInvalidArgument;
  if (!d->devCopy) {
    FCX_CUDACHECK(cudaMalloc(&d->devCopy, sizeof(flagcxDevComm)));
    FCX_CUDACHECK(cudaMemcpy(d->devCopy, &d->dev, sizeof(flagcxDevComm), cudaMemcpyHostToDevice));
  }
  *devPtr = d->devCopy;
  return flagcxSuccess;
}
flagcxResult_t flagcxDevCommFreeDevicePtr(flagcxDevComm_t d) {
  if (d && d->devCopy) { cudaFree(d->devCopy); d->devCopy = nullptr; }
  return flagcxSuccess;
}
flagcxResult_t flagcxDevMemGetDevicePtr(flagcxDevMem_t m, void **devPtr) {
  if (!m || !devPtr) return flagcxInvalidArgument;
  if (!m->devCopy) {
    FCX_CUDACHECK(cudaMalloc(&m->devCopy, sizeof(flagcxDevMem)));
    FCX_CUDACHECK(cudaMemcpy(m->devCopy, &m->mem, sizeof(flagcxDevMem), cudaMemcpyHostToDevice));
  }
  *devPtr = m->devCopy;
  return flagcxSuccess;
}
flagcxResult_t flagcxDevMemFreeDevicePtr(flagcxDevMem_t m) {
  if (m && m->devCopy) { cudaFree(m->devCopy); m->devCopy = nullptr; }
  return flagcxSuccess;
}

flagcxResult_t flagcxCommQueryProperties(flagcxComm_t comm, flagcxCommProperties_t *props) {
  if (!commValid(comm) || !props) return flagcxInvalidArgument;
  props->rank = comm->rank;
  props->nRanks = comm->nranks;
  props->deviceId = comm->cudaDev;
  props->vendorDeviceApiSupport = false;
  props->multicastSupport = comm->internalWin && comm->internalWin->mc;
  props->netType = flagcxNetTypeNone;
  return flagcxSuccess;
}

} // extern "C"

// ---------------------------------------------------------------------------
// runtime function table
// ---------------------------------------------------------------------------
namespace {

bool gpu() { return cu::available(); }

#define DH_CUDA(call)                                                         \
  do {                                                                        \
    cudaError_t e__ = (call);                                                 \
    if (e__ != cudaSuccess) {                                                 \
      FCX_WARN("CUDA failure '%s'", cudaGetErrorString(e__));                 \
      return flagcxUnhandledDeviceError;                                      \
    }                                                                         \
  } while (0)

flagcxResult_t dhSync() { if (gpu()) DH_CUDA(cudaDeviceSynchronize()); return flagcxSuccess; }

flagcxResult_t dhMemcpy(void *dst, void *src, size_t size, flagcxMemcpyType_t type, flagcxStream_t s) {
  if (!gpu()) { memmove(dst, src, size); return flagcxSuccess; }
  cudaMemcpyKind k = type == flagcxMemcpyHostToDevice   ? cudaMemcpyHostToDevice
                     : type == flagcxMemcpyDeviceToHost ? cudaMemcpyDeviceToHost
                                                        : cudaMemcpyDeviceToDevice;
  if (s) DH_CUDA(cudaMemcpyAsync(dst, src, size, k, s->base));
  else DH_CUDA(cudaMemcpy(dst, src, size, k));
  return flagcxSuccess;
}
flagcxResult_t dhMemset(void *ptr, int value, size_t size, flagcxMemType_t type, flagcxStream_t s) {
  if (!gpu() || type == flagcxMemHost) { memset(ptr, value, size); return flagcxSuccess; }
  if (s) DH_CUDA(cudaMemsetAsync(ptr, value, size, s->base));
  else DH_CUDA(cudaMemset(ptr, value, size));
  return flagcxSuccess;
}
flagcxResult_t dhMalloc(void **ptr, size_t size, flagcxMemType_t type, flagcxStream_t) {
  if (!gpu()) {
    *ptr = nullptr;
    return posix_memalign(ptr, 256, size ? size : 1) == 0 ? flagcxSuccess : flagcxSystemError;
  }
  if (type == flagcxMemHost) DH_CUDA(cudaHostAlloc(ptr, size, cudaHostAllocMapped));
  else if (type == flagcxMemManaged) DH_CUDA(cudaMallocManaged(ptr, size));
  else DH_CUDA(cudaMalloc(ptr, size));
  return flagcxSuccess;
}
flagcxResult_t dhFree(void *ptr, flagcxMemType_t type, flagcxStream_t) {
  if (!ptr) return flagcxSuccess;
  if (!gpu()) { free(ptr); return flagcxSuccess; }
  if (type == flagcxMemHost) DH_CUDA(cudaFreeHost(ptr));
  else DH_CUDA(cudaFree(ptr));
  return flagcxSuccess;
}
flagcxResult_t dhSetDevice(int dev) { if (gpu()) DH_CUDA(cudaSetDevice(dev)); return flagcxSuccess; }
flagcxResult_t dhGetDevice(int *dev) {
  *dev = 0;
  if (gpu()) DH_CUDA(cudaGetDevice(dev));
  return flagcxSuccess;
}
flagcxResult_t dhGetDeviceCount(int *count) {
  *count = gpu() ? cu::deviceCount() : 1; // the host device
  return flagcxSuccess;
}
flagcxResult_t dhGetVendor(char *vendor) { strcpy(vendor, gpu() ? "NVIDIA" : "HOST"); return flagcxSuccess; }
flagcxResult_t dhHostGetDevicePointer(void **pDevice, void *pHost) {
  if (!gpu()) { *pDevice = pHost; return flagcxSuccess; }
  DH_CUDA(cudaHostGetDevicePointer(pDevice, pHost, 0));
  return flagcxSuccess;
}
flagcxResult_t dhStreamCreate(flagcxStream_t *s) {
  *s = new flagcxStream{nullptr};
  if (gpu()) DH_CUDA(cudaStreamCreateWithFlags(&(*s)->base, cudaStreamNonBlocking));
  return flagcxSuccess;
}
flagcxResult_t dhStreamDestroy(flagcxStream_t s) {
  if (!s) return flagcxSuccess;
  if (gpu() && s->base) cudaStreamDestroy(s->base);
  delete s;
  return flagcxSuccess;
}
// Wraps an existing cudaStream_t (passed by address) without taking ownership.
flagcxResult_t dhStreamCopy(flagcxStream_t *newStream, void *oldStream) {
  *newStream = new flagcxStream{oldStream ? *(cudaStream_t *)oldStream : nullptr};
  return flagcxSuccess;
}
flagcxResult_t dhStreamFree(flagcxStream_t s) { delete s; return flagcxSuccess; }
flagcxResult_t dhStreamSync(flagcxStream_t s) {
  if (gpu()) DH_CUDA(cudaStreamSynchronize(s ? s->base : nullptr));
  return flagcxSuccess;
}
flagcxResult_t dhStreamQuery(flagcxStream_t s) {
  if (!gpu()) return flagcxSuccess;
  cudaError_t e = cudaStreamQuery(s ? s->base : nullptr);
  if (e == cudaSuccess) return flagcxSuccess;
  if (e == cudaErrorNotReady) return flagcxInProgress;
  return flagcxUnhandledDeviceError;
}
flagcxResult_t dhStreamWaitEvent(flagcxStream_t s, flagcxEvent_t e) {
  if (gpu()) DH_CUDA(cudaStreamWaitEvent(s ? s->base : nullptr, e->base, 0));
  return flagcxSuccess;
}

// host device: an event remembers when it was recorded so elapsed time works
struct HostEvent { flagcxEvent ev; std::chrono::steady_clock::time_point t; };

flagcxResult_t dhEventCreate(flagcxEvent_t *e, flagcxEventType_t type) {
  if (!gpu()) { auto *h = new HostEvent(); h->ev.base = nullptr; *e = &h->ev; return flagcxSuccess; }
  *e = new flagcxEvent{nullptr};
  DH_CUDA(cudaEventCreateWithFlags(&(*e)->base, type == flagcxEventDisableTiming ? cudaEventDisableTiming : cudaEventDefault));
  return flagcxSuccess;
}
flagcxResult_t dhEventDestroy(flagcxEvent_t e) {
  if (!e) return flagcxSuccess;
  if (!gpu()) { delete (HostEvent *)e; return flagcxSuccess; }
  cudaEventDestroy(e->base);
  delete e;
  return flagcxSuccess;
}
flagcxResult_t dhEventRecord(flagcxEvent_t e, flagcxStream_t s) {
  if (!gpu()) { ((HostEvent *)e)->t = std::chrono::steady_clock::now(); return flagcxSuccess; }
  DH_CUDA(cudaEventRecord(e->base, s ? s->base : nullptr));
  return flagcxSuccess;
}
flagcxResult_t dhEventSync(flagcxEvent_t e) {
  if (gpu()) DH_CUDA(cudaEventSynchronize(e->base));
  return flagcxSuccess;
}
flagcxResult_t dhEventQuery(flagcxEvent_t e) {
  if (!gpu()) return flagcxSuccess;
  cudaError_t r = cudaEventQuery(e->base);
  return r == cudaSuccess ? flagcxSuccess : r == cudaErrorNotReady ? flagcxInProgress : flagcxUnhandledDeviceError;
}
flagcxResult_t dhEventElapsed(float *ms, flagcxEvent_t a, flagcxEvent_t b) {
  if (!gpu()) {
    *ms = std::chrono::duration<float, std::milli>(((HostEvent *)b)->t - ((HostEvent *)a)->t).count();
    return flagcxSuccess;
  }
  DH_CUDA(cudaEventElapsedTime(ms, a->base, b->base));
  return flagcxSuccess;
}
flagcxResult_t dhIpcCreate(flagcxIpcMemHandle_t *h, size_t *size) {
  *h = new flagcxIpcMemHandle();
  if (size) *size = sizeof(cudaIpcMemHandle_t);
  return flagcxSuccess;
}
flagcxResult_t dhIpcGet(flagcxIpcMemHandle_t h, void *devPtr) {
  if (!gpu()) return flagcxNotSupported;
  DH_CUDA(cudaIpcGetMemHandle(&h->base, devPtr));
  return flagcxSuccess;
}
flagcxResult_t dhIpcOpen(flagcxIpcMemHandle_t h, void **devPtr) {
  if (!gpu()) return flagcxNotSupported;
  DH_CUDA(cudaIpcOpenMemHandle(devPtr, h->base, cudaIpcMemLazyEnablePeerAccess));
  return flagcxSuccess;
}
flagcxResult_t dhIpcClose(void *devPtr) {
  if (!gpu()) return flagcxNotSupported;
  DH_CUDA(cudaIpcCloseMemHandle(devPtr));
  return flagcxSuccess;
}
flagcxResult_t dhIpcFree(flagcxIpcMemHandle_t h) { delete h; return flagcxSuccess; }

} // namespace

extern "C" {

flagcxResult_t flagcxDeviceHandleInit(flagcxDeviceHandle_t *out) {
  if (!out) return flagcxInvalidArgument;
  logInit();
  auto *h = new flagcxDeviceHandle();
  h->deviceSynchronize = dhSync;
  h->deviceMemcpy = dhMemcpy;
  h->deviceMemset = dhMemset;
  h->deviceMalloc = dhMalloc;
  h->deviceFree = dhFree;
  h->setDevice = dhSetDevice;
  h->getDevice = dhGetDevice;
  h->getDeviceCount = dhGetDeviceCount;
  h->getVendor = dhGetVendor;
  h->hostGetDevicePointer = dhHostGetDevicePointer;
  h->streamCreate = dhStreamCreate;
  h->streamDestroy = dhStreamDestroy;
  h->streamCopy = dhStreamCopy;
  h->streamFree = dhStreamFree;
  h->streamSynchronize = dhStreamSync;
  h->streamQuery = dhStreamQuery;
  h->streamWaitEvent = dhStreamWaitEvent;
  h->eventCreate = dhEventCreate;
  h->eventDestroy = dhEventDestroy;
  h->eventRecord = dhEventRecord;
  h->eventSynchronize = dhEventSync;
  h->eventQuery = dhEventQuery;
  h->eventElapsedTime = dhEventElapsed;
  h->ipcMemHandleCreate = dhIpcCreate;
  h->ipcMemHandleGet = dhIpcGet;
  h->ipcMemHandleOpen = dhIpcOpen;
  h->ipcMemHandleClose = dhIpcClose;
  h->ipcMemHandleFree = dhIpcFree;
  *out = h;
  return flagcxSuccess;
}

flagcxResult_t flagcxDeviceHandleFree(flagcxDeviceHandle_t h) {
  delete h;
  return flagcxSuccess;
}

flagcxResult_t flagcxHandleInit(flagcxHandlerGroup_t *handler) {
  if (!handler) return flagcxInvalidArgument;
  auto *g = new flagcxHandlerGroup();
  g->uniqueId = new flagcxUniqueId();
  memset(g->uniqueId, 0, sizeof(flagcxUniqueId));
  g->comm = nullptr;
  flagcxResult_t r = flagcxDeviceHandleInit(&g->devHandle);
  if (r != flagcxSuccess) { delete g->uniqueId; delete g; return r; }
  *handler = g;
  return flagcxSuccess;
}

flagcxResult_t flagcxHandleFree(flagcxHandlerGroup_t g) {
  if (!g) return flagcxSuccess;
  flagcxDeviceHandleFree(g->devHandle);
  delete g->uniqueId;
  delete g;
  return flagcxSuccess;
}

} // extern "C"
