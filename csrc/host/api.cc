// api.cc -- the extern "C" surface, part 1: communicator life cycle, memory, windows,
// collectives and grouping (the one-sided host API is in api_onesided.cc, the extension
// entry points of flagcx_ext.h in api_ext.cc).
//
// A collective call takes one of three routes:
//   device  buffers are on the GPU and the communicator has the NVLink device
//           path: one kernel (device_coll.cc);
//   host    buffers are host memory: socket collectives (cpu_coll.cc);
//   staged  buffers are on the GPU but the ranks cannot reach each other over
//           NVLink (different machines, FLAGCX_P2P_DISABLE=1): copy to pinned
//           host memory, run the host collective, copy back -- what FlagCX calls
//           its host runner (flagcx/runner/host_runner.cc:236-289).
#include <algorithm>
#include <mutex>

#include "../kernels/launch.h"
#include "api_internal.h"
#include "tuner.h"

using namespace fcx;

namespace {

enum Route { kRouteDevice, kRouteHost, kRouteStaged };

Route routeFor(flagcxComm *c, const void *a, const void *b) {
  if (c->emu) return kRouteDevice;
  const void *probe = a ? a : b;
  int dev = -1;
  cu::PtrKind k = cu::available() ? cu::classify(probe, &dev) : cu::kPtrHost;
  if (k == cu::kPtrHost) return kRouteHost;
  return c->devicePath ? kRouteDevice : kRouteStaged;
}

} // namespace

namespace fcx {
flagcxResult_t ensureHostNet(flagcxComm *c) {
  if (c->hostNet) return flagcxSuccess;
  if (!c->bootstrap) return flagcxNotSupported;
  c->hostNet.reset(new HostNet());
  FCXCHECK(c->hostNet->init(c->bootstrap.get()));
  c->cpu.net = c->hostNet.get();
  return flagcxSuccess;
}
} // namespace fcx

namespace {

flagcxResult_t hostStage(flagcxComm *c, size_t bytes, char **out) {
  if (c->hostStageBytes < bytes) {
    if (c->hostStage) cudaFreeHost(c->hostStage);
    c->hostStage = nullptr;
    size_t want = alignUp(std::max(bytes, (size_t)1 << 20), 1 << 20);
    FCX_CUDACHECK(cudaHostAlloc(&c->hostStage, want, cudaHostAllocDefault));
    c->hostStageBytes = want;
  }
  *out = (char *)c->hostStage;
  return flagcxSuccess;
}

// Runs `fn(sendHost, recvHost)` on pinned copies of device buffers.
template <typename Fn>
flagcxResult_t stagedCall(flagcxComm *c, const void *send, size_t sendBytes, void *recv, size_t recvBytes,
                          cudaStream_t stream, Fn fn) {
  char *stage;
  size_t sOff = 0, rOff = alignUp(sendBytes, 256);
  FCXCHECK(hostStage(c, rOff + recvBytes, &stage));
  if (send && sendBytes) FCX_CUDACHECK(cudaMemcpyAsync(stage + sOff, send, sendBytes, cudaMemcpyDeviceToHost, stream));
  FCX_CUDACHECK(cudaStreamSynchronize(stream));
  FCXCHECK(ensureHostNet(c));
  FCXCHECK(fn(stage + sOff, stage + rOff));
  if (recv && recvBytes) {
    FCX_CUDACHECK(cudaMemcpyAsync(recv, stage + rOff, recvBytes, cudaMemcpyHostToDevice, stream));
    FCX_CUDACHECK(cudaStreamSynchronize(stream));
  }
  return flagcxSuccess;
}

std::mutex gApiMu;

} // namespace

extern "C" {

// ---------------------------------------------------------------------------
// versions, errors
// ---------------------------------------------------------------------------
flagcxResult_t flagcxGetVersion(int *version) {
  if (!version) return flagcxInvalidArgument;
  *version = FLAGCX_VERSION_CODE;
  return flagcxSuccess;
}

const char *flagcxGetErrorString(flagcxResult_t r) {
  switch (r) {
    case flagcxSuccess: return "no error";
    case flagcxUnhandledDeviceError: return "unhandled device (CUDA) error";
    case flagcxSystemError: return "unhandled system error (socket, file, timeout)";
    case flagcxInternalError: return "internal error";
    case flagcxInvalidArgument: return "invalid argument";
    case flagcxInvalidUsage: return "invalid usage";
    case flagcxRemoteError: return "remote process exited, network error, or a device-side wait timed out";
    case flagcxInProgress: return "operation in progress";
    case flagcxUnhandledCCLError: return "unhandled collective library error";
    case flagcxNotSupported: return "not supported";
    default: return "unknown result code";
  }
}

const char *flagcxGetLastError(flagcxComm_t comm) {
  if (commValid(comm) && !comm->lastError.empty()) return comm->lastError.c_str();
  return lastErrorText();
}

flagcxResult_t flagcxCommGetAsyncError(flagcxComm_t comm, flagcxResult_t *asyncError) {
  FCX_COMMCHECK(comm);
  if (!asyncError) return flagcxInvalidArgument;
  *asyncError = commCheckDevice(comm);
  return flagcxSuccess;
}

// ---------------------------------------------------------------------------
// life cycle
// ---------------------------------------------------------------------------
flagcxResult_t flagcxGetUniqueId(flagcxUniqueId_t uniqueId) {
  if (!uniqueId) return flagcxInvalidArgument;
  logInit();
  return bootstrapCreateId(uniqueId);
}

flagcxResult_t flagcxCommInitRank(flagcxComm_t *comm, int nranks, flagcxUniqueId_t commId, int rank) {
  if (!comm || !commId) return flagcxInvalidArgument;
  *comm = nullptr;
  FCXCHECK(commCreate(comm, nranks, *commId, rank));
  if (int64_t cap = readParam("TRACE", 0)) (*comm)->trace.enable((int)std::min<int64_t>(cap, 1 << 20));
  // FLAGCX_USE_TUNER=1 (name kept from the FlagCX project): measure at init unless a
  // table was loaded from FLAGCX_TUNE_FILE; rank 0 then writes the table there.
  flagcxComm *c = *comm;
  if (readParam("USE_TUNER", 0) != 0 && c->devicePath && !c->emu && c->tuner && nranks > 1 && c->tuner->table.empty()) {
    const size_t lo = (size_t)std::max<int64_t>(1024, readParam("TUNER_MIN_BYTES", 64 << 10));
    const size_t hi = (size_t)std::max<int64_t>((int64_t)lo, readParam("TUNER_MAX_BYTES", 64 << 20));
    for (flagcxCommOp_t op : {flagcxCommOpAllReduce, flagcxCommOpAllGather, flagcxCommOpReduceScatter, flagcxCommOpAlltoAll}) {
      flagcxResult_t r = c->tuner->tune(c, op, flagcxBfloat16, lo, hi, 5);
      if (r != flagcxSuccess) { FCX_WARN("FLAGCX_USE_TUNER: tuning %s failed (%d); heuristics stay in force", commOpName(op), (int)r); break; }
    }
    if (const char *f = getEnv("FLAGCX_TUNE_FILE"))
      if (rank == 0 && !c->tuner->table.empty()) c->tuner->save(f);
  }
  return flagcxSuccess;
}

flagcxResult_t flagcxCommFinalize(flagcxComm_t comm) {
  FCX_COMMCHECK(comm);
  if (comm->devicePath) {
    cudaSetDevice(comm->cudaDev);
    FCX_CUDACHECK(cudaDeviceSynchronize());
  }
  comm->finalized = true;
  return commCheckDevice(comm);
}

flagcxResult_t flagcxCommDestroy(flagcxComm_t comm) {
  FCX_COMMCHECK(comm);
  if (comm->trace.on()) {
    if (const char *f = getEnv("FLAGCX_TRACE_FILE")) { // %r -> rank
      std::string path(f);
      size_t at = path.find("%r");
      if (at != std::string::npos) path.replace(at, 2, std::to_string(comm->rank));
      comm->trace.dump(comm, path.c_str());
    }
    comm->trace.enable(0); // events go before the context does
  }
  return commDestroy(comm);
}

flagcxResult_t flagcxCommAbort(flagcxComm_t comm) {
  FCX_COMMCHECK(comm);
  comm->aborted = true;
  if (comm->status) {
    // every bounded wait polls this word
    __atomic_store_n(&comm->status->abortFlag, 1u, __ATOMIC_SEQ_CST);
    if (comm->devicePath) { cudaSetDevice(comm->cudaDev); cudaDeviceSynchronize(); }
  }
  comm->asyncError.store(flagcxInvalidUsage);
  if (comm->emu) return flagcxSuccess; // the world is torn down by flagcxEmuWorldDestroy
  return commDestroy(comm);
}

// Suspend drains the device and parks the communicator; collectives issued while
// suspended are refused.  Resume lifts that.  Neither moves state between ranks.
flagcxResult_t flagcxCommSuspend(flagcxComm_t comm) {
  FCX_COMMCHECK(comm);
  if (comm->devicePath) { cudaSetDevice(comm->cudaDev); FCX_CUDACHECK(cudaDeviceSynchronize()); }
  comm->finalized = true;
  return flagcxSuccess;
}
flagcxResult_t flagcxCommResume(flagcxComm_t comm) {
  FCX_COMMCHECK(comm);
  comm->finalized = false;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommCount(const flagcxComm_t comm, int *count) {
  FCX_COMMCHECK(comm);
  *count = comm->nranks;
  return flagcxSuccess;
}
flagcxResult_t flagcxCommGetDeviceNumber(const flagcxComm_t comm, int *device) {
  FCX_COMMCHECK(comm);
  *device = comm->cudaDev;
  return flagcxSuccess;
}
flagcxResult_t flagcxCommUserRank(const flagcxComm_t comm, int *rank) {
  FCX_COMMCHECK(comm);
  *rank = comm->rank;
  return flagcxSuccess;
}
flagcxResult_t flagcxIsHomoComm(flagcxComm_t comm, int *isHomo) {
  FCX_COMMCHECK(comm);
  *isHomo = 1; // one vendor, one code path
  return flagcxSuccess;
}

// ---------------------------------------------------------------------------
// memory
// ---------------------------------------------------------------------------
flagcxResult_t flagcxMemAlloc(void **ptr, size_t size, flagcxMemAllocator_t) {
  if (!ptr) return flagcxInvalidArgument;
  *ptr = nullptr;
  if (!cu::available()) {
    void *p = nullptr;
    if (posix_memalign(&p, 4096, alignUp(size ? size : 1, 4096)) != 0) return flagcxSystemError;
    *ptr = p;
    return flagcxSuccess;
  }
  int dev = 0;
  FCX_CUDACHECK(cudaGetDevice(&dev));
  if (cu::vmmSupported(dev) && readParam("VMM_ENABLE", 1) != 0) {
    cu::VmmBlock b;
    FCXCHECK(cu::vmmAlloc(size, dev, &b));
    *ptr = b.ptr;
    return flagcxSuccess;
  }
  FCX_CUDACHECK(cudaMalloc(ptr, size ? size : 1));
  return flagcxSuccess;
}

flagcxResult_t flagcxMemFree(void *ptr, flagcxMemAllocator_t) {
  if (!ptr) return flagcxSuccess;
  if (!cu::available()) { free(ptr); return flagcxSuccess; }
  if (const cu::VmmBlock *b = cu::vmmLookup(ptr)) {
    if (b->ptr != ptr) return flagcxInvalidArgument;
    cu::VmmBlock copy = *b;
    return cu::vmmFree(&copy);
  }
  FCX_CUDACHECK(cudaFree(ptr));
  return flagcxSuccess;
}

// Local (non-collective) registration: exports the allocation to the peers ahead of its
// first use, which a collective would otherwise do on the fly (reg_cache.h).  Memory that
// cannot be exported is accepted too; collectives then copy through a stand-in.
struct RegHandle { void *buf; size_t size; };

flagcxResult_t flagcxCommRegister(const flagcxComm_t comm, void *buff, size_t size, void **handle,
                                  flagcxMemAllocator_t) {
  FCX_COMMCHECK(comm);
  if (!buff || !handle) return flagcxInvalidArgument;
  if (comm->exportUserBuffers && comm->reg && !comm->windows.find(buff, size ? size : 1)) {
    void *va[FLAGCX_MAX_RANKS];
    comm->reg->lookup(buff, size ? size : 1, va);
  }
  *handle = new RegHandle{buff, size};
  return flagcxSuccess;
}
flagcxResult_t flagcxCommDeregister(const flagcxComm_t comm, void *handle, flagcxMemAllocator_t) {
  FCX_COMMCHECK(comm);
  RegHandle *h = (RegHandle *)handle;
  if (h && comm->reg) {
    // nobody may still be reading the allocation through its mappings
    if (comm->devicePath) { cudaSetDevice(comm->cudaDev); cudaDeviceSynchronize(); }
    comm->reg->forget(h->buf);
  }
  delete h;
  return flagcxSuccess;
}

} // extern "C"

namespace fcx {
flagcxResult_t emuWindowRegister(flagcxComm *c, void *buff, size_t size, int flags, Window **out);
}

extern "C" {

flagcxResult_t flagcxCommWindowRegister(flagcxComm_t comm, void *buff, size_t size, flagcxWindow_t *win, int winFlags,
                                        flagcxMemAllocator_t) {
  FCX_COMMCHECK(comm);
  if (!buff || !win || size == 0) return flagcxInvalidArgument;
  Window *w = nullptr;
  if (comm->emu) FCXCHECK(emuWindowRegister(comm, buff, size, winFlags, &w));
  else FCXCHECK(windowRegister(comm, buff, size, winFlags, &w));
  *win = (flagcxWindow_t)w;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommWindowDeregister(flagcxComm_t comm, flagcxWindow_t win, flagcxMemAllocator_t) {
  FCX_COMMCHECK(comm);
  if (!win) return flagcxSuccess;
  if (!comm->emu && comm->bootstrap) {
    // peers unmap together: nobody may still be reading this rank's memory
    if (comm->devicePath) { cudaSetDevice(comm->cudaDev); cudaDeviceSynchronize(); }
    FCXCHECK(comm->bootstrap->barrier());
  }
  return windowDeregister(comm, (Window *)win);
}

flagcxResult_t flagcxWindowGetPeerPointer(flagcxWindow_t win, int peer, size_t offset, void **ptr) {
  Window *w = (Window *)win;
  if (!w || !ptr || peer < 0 || peer >= FLAGCX_MAX_RANKS || !w->peer[peer] || offset > w->size) return flagcxInvalidArgument;
  *ptr = (char *)w->peer[peer] + offset;
  return flagcxSuccess;
}
flagcxResult_t flagcxWindowGetMulticastPointer(flagcxWindow_t win, size_t offset, void **ptr) {
  Window *w = (Window *)win;
  if (!w || !ptr) return flagcxInvalidArgument;
  *ptr = w->mc ? (char *)w->mc + offset : nullptr;
  return w->mc ? flagcxSuccess : flagcxNotSupported;
}

// ---------------------------------------------------------------------------
// collectives
// ---------------------------------------------------------------------------
} // extern "C"

namespace fcx {
flagcxResult_t checkUsable(flagcxComm *c) {
  if (c->finalized) { FCX_WARN("communicator was finalized or suspended"); return flagcxInvalidUsage; }
  int e = c->asyncError.load();
  return e == flagcxSuccess ? flagcxSuccess : (flagcxResult_t)e;
}
} // namespace fcx

extern "C" {

static flagcxResult_t runCollective(flagcxComm *c, DeviceCollRequest &rq, size_t sendBytes, size_t recvBytes,
                                    flagcxStream_t stream) {
  FCXCHECK(checkUsable(c));
  FCX_TRACE(SUB_CALL, "%s count %zu %s rank %d", commOpName(rq.op), rq.count, dtypeName(rq.dtype), c->rank);
  Route route = routeFor(c, rq.send, rq.recv);
  // trace record and NVTX range around whatever route the call takes
  struct Scope {
    flagcxComm *c;
    int slot;
    cudaStream_t s;
    ~Scope() { c->trace.end(c, slot, s); nvtxPop(); }
  };
  nvtxPush(commOpName(rq.op));
  Scope scope{c, c->trace.begin(c, rq.op, std::max(sendBytes, recvBytes),
                                route == kRouteDevice ? 0 : route == kRouteHost ? 1 : 2, rawStream(stream)),
              rawStream(stream)};
  if (route == kRouteDevice) return deviceCollective(c, rq, rawStream(stream));
  auto host = [&](const void *s, void *r) -> flagcxResult_t {
    CpuColl &cc = c->cpu;
    switch (rq.op) {
      case flagcxCommOpAllReduce: return cc.allReduce(s, r, rq.count, rq.dtype, rq.redOp);
      case flagcxCommOpReduceScatter: return cc.reduceScatter(s, r, rq.count, rq.dtype, rq.redOp);
      case flagcxCommOpAllGather: return cc.allGather(s, r, rq.count, rq.dtype);
      case flagcxCommOpBroadcast: return cc.broadcast(s, r, rq.count, rq.dtype, rq.root);
      case flagcxCommOpReduce: return cc.reduce(s, r, rq.count, rq.dtype, rq.redOp, rq.root);
      case flagcxCommOpGather: return cc.gather(s, r, rq.count, rq.dtype, rq.root);
      case flagcxCommOpScatter: return cc.scatter(s, r, rq.count, rq.dtype, rq.root);
      case flagcxCommOpAlltoAll: return cc.allToAll(s, r, rq.count, rq.dtype);
      case flagcxCommOpAlltoAllv:
        return cc.allToAllv(s, rq.sendCounts, rq.sendDispls, r, rq.recvCounts, rq.recvDispls, rq.dtype);
      default: return flagcxInternalError;
    }
  };
  c->stats[rq.op].calls++;
  c->stats[rq.op].bytes += std::max(sendBytes, recvBytes);
  if (route == kRouteHost) {
    FCXCHECK(ensureHostNet(c));
    return host(rq.send, rq.recv);
  }
  // ranks in several NVLink domains: two-level route for the operations that have one
  if (c->intra && rq.op == flagcxCommOpAllReduce)
    return hierAllReduce(c, rq.send, rq.recv, rq.count, rq.dtype, rq.redOp, rawStream(stream));
  if (c->intra && rq.op == flagcxCommOpAllGather)
    return hierAllGather(c, rq.send, rq.recv, rq.count, rq.dtype, rawStream(stream));
  // in-place device calls must see the input in the receive staging too
  return stagedCall(c, rq.send, sendBytes, rq.recv, recvBytes, rawStream(stream), [&](char *s, char *r) {
    return host(s, r);
  });
}

flagcxResult_t flagcxAllReduce(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype,
                               flagcxRedOp_t op, flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  size_t es = getFlagcxDataTypeSize(datatype);
  FCX_ARGCHECK(es && sendbuff && recvbuff && (int)op >= 0 && op < flagcxNumRedOps, "allreduce: bad argument");
  DeviceCollRequest rq{flagcxCommOpAllReduce, sendbuff, recvbuff, count, datatype, op, 0};
  return runCollective(comm, rq, count * es, count * es, stream);
}

flagcxResult_t flagcxReduceScatter(const void *sendbuff, void *recvbuff, size_t recvcount, flagcxDataType_t datatype,
                                   flagcxRedOp_t op, flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  size_t es = getFlagcxDataTypeSize(datatype);
  FCX_ARGCHECK(es && sendbuff && recvbuff && (int)op >= 0 && op < flagcxNumRedOps, "reducescatter: bad argument");
  DeviceCollRequest rq{flagcxCommOpReduceScatter, sendbuff, recvbuff, recvcount, datatype, op, 0};
  return runCollective(comm, rq, recvcount * es * comm->nranks, recvcount * es, stream);
}

flagcxResult_t flagcxAllGather(const void *sendbuff, void *recvbuff, size_t sendcount, flagcxDataType_t datatype,
                               flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  size_t es = getFlagcxDataTypeSize(datatype);
  FCX_ARGCHECK(es && sendbuff && recvbuff, "allgather: bad argument");
  DeviceCollRequest rq{flagcxCommOpAllGather, sendbuff, recvbuff, sendcount, datatype, flagcxSum, 0};
  return runCollective(comm, rq, sendcount * es, sendcount * es * comm->nranks, stream);
}

flagcxResult_t flagcxBroadcast(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, int root,
                               flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  size_t es = getFlagcxDataTypeSize(datatype);
  FCX_ARGCHECK(es && recvbuff && root >= 0 && root < comm->nranks, "broadcast: bad argument");
  DeviceCollRequest rq{flagcxCommOpBroadcast, sendbuff, recvbuff, count, datatype, flagcxSum, root};
  return runCollective(comm, rq, comm->rank == root ? count * es : 0, count * es, stream);
}

flagcxResult_t flagcxReduce(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype,
                            flagcxRedOp_t op, int root, flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  size_t es = getFlagcxDataTypeSize(datatype);
  FCX_ARGCHECK(es && sendbuff && root >= 0 && root < comm->nranks && (int)op >= 0 && op < flagcxNumRedOps,
               "reduce: bad argument");
  DeviceCollRequest rq{flagcxCommOpReduce, sendbuff, recvbuff, count, datatype, op, root};
  return runCollective(comm, rq, count * es, comm->rank == root ? count * es : 0, stream);
}

flagcxResult_t flagcxGather(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, int root,
                            flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  size_t es = getFlagcxDataTypeSize(datatype);
  FCX_ARGCHECK(es && sendbuff && root >= 0 && root < comm->nranks, "gather: bad argument");
  DeviceCollRequest rq{flagcxCommOpGather, sendbuff, recvbuff, count, datatype, flagcxSum, root};
  return runCollective(comm, rq, count * es, comm->rank == root ? count * es * comm->nranks : 0, stream);
}

flagcxResult_t flagcxScatter(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, int root,
                             flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  size_t es = getFlagcxDataTypeSize(datatype);
  FCX_ARGCHECK(es && recvbuff && root >= 0 && root < comm->nranks, "scatter: bad argument");
  DeviceCollRequest rq{flagcxCommOpScatter, sendbuff, recvbuff, count, datatype, flagcxSum, root};
  return runCollective(comm, rq, comm->rank == root ? count * es * comm->nranks : 0, count * es, stream);
}

flagcxResult_t flagcxAlltoAll(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype,
                              flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  size_t es = getFlagcxDataTypeSize(datatype);
  FCX_ARGCHECK(es && sendbuff && recvbuff && sendbuff != recvbuff, "alltoall: bad argument (in-place is not supported)");
  DeviceCollRequest rq{flagcxCommOpAlltoAll, sendbuff, recvbuff, count, datatype, flagcxSum, 0};
  return runCollective(comm, rq, count * es * comm->nranks, count * es * comm->nranks, stream);
}

flagcxResult_t flagcxAlltoAllv(const void *sendbuff, size_t *sendcounts, size_t *sdispls, void *recvbuff,
                               size_t *recvcounts, size_t *rdispls, flagcxDataType_t datatype, flagcxComm_t comm,
                               flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  size_t es = getFlagcxDataTypeSize(datatype);
  FCX_ARGCHECK(es && sendcounts && sdispls && recvcounts && rdispls && sendbuff != recvbuff, "alltoallv: bad argument");
  size_t sb = 0, rb = 0;
  for (int p = 0; p < comm->nranks; ++p) {
    sb = std::max(sb, (sdispls[p] + sendcounts[p]) * es);
    rb = std::max(rb, (rdispls[p] + recvcounts[p]) * es);
  }
  DeviceCollRequest rq{flagcxCommOpAlltoAllv, sendbuff, recvbuff, 0, datatype, flagcxSum, 0};
  rq.sendCounts = sendcounts;
  rq.sendDispls = sdispls;
  rq.recvCounts = recvcounts;
  rq.recvDispls = rdispls;
  return runCollective(comm, rq, sb, rb, stream);
}

flagcxResult_t flagcxBarrier(flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  FCXCHECK(checkUsable(comm));
  if (comm->devicePath) {
    FCXCHECK(deviceBarrier(comm, rawStream(stream)));
    if (comm->emu) return flagcxSuccess;
    // same contract as the FlagCX barrier: the host returns after the stream drained
    FCX_CUDACHECK(cudaStreamSynchronize(rawStream(stream)));
    return commCheckDevice(comm);
  }
  if (cu::available() && stream) FCX_CUDACHECK(cudaStreamSynchronize(rawStream(stream)));
  return comm->bootstrap->barrier();
}

// ---------------------------------------------------------------------------
// point-to-point and groups
// ---------------------------------------------------------------------------
struct HostP2p { bool isSend; int peer; void *buf; size_t bytes; };
static thread_local std::vector<HostP2p> tlsHostOps;

static flagcxResult_t flushGroup(flagcxComm *c) {
  flagcxResult_t r = flagcxSuccess;
  if (!c->groupOps.empty()) r = deviceGroupLaunch(c);
  if (!tlsHostOps.empty()) {
    std::vector<HostNet::Op> ops;
    // self transfers first: match sends to receives in order
    std::vector<HostP2p> selfS, selfR;
    for (auto &o : tlsHostOps) {
      if (o.peer == c->rank) (o.isSend ? selfS : selfR).push_back(o);
      else ops.push_back({o.isSend, o.peer, o.buf, o.bytes});
    }
    tlsHostOps.clear();
    for (size_t i = 0; i < std::min(selfS.size(), selfR.size()); ++i)
      memmove(selfR[i].buf, selfS[i].buf, std::min(selfS[i].bytes, selfR[i].bytes));
    if (!ops.empty()) {
      flagcxResult_t hr = ensureHostNet(c);
      if (hr == flagcxSuccess) hr = c->hostNet->run(ops);
      if (r == flagcxSuccess) r = hr;
    }
  }
  return r;
}

static flagcxResult_t p2pCall(bool isSend, void *buf, size_t count, flagcxDataType_t dt, int peer, flagcxComm *c,
                              flagcxStream_t stream) {
  FCXCHECK(checkUsable(c));
  size_t es = getFlagcxDataTypeSize(dt);
  FCX_ARGCHECK(es && peer >= 0 && peer < c->nranks, "send/recv: bad argument");
  size_t bytes = count * es;
  Route route = routeFor(c, buf, nullptr);
  if (route == kRouteDevice) {
    c->groupOps.push_back({isSend, peer, buf, bytes, rawStream(stream)});
  } else if (route == kRouteHost) {
    tlsHostOps.push_back({isSend, peer, buf, bytes});
  } else {
    // staged: device buffer over sockets; runs immediately
    char *stage;
    FCXCHECK(hostStage(c, bytes, &stage));
    FCXCHECK(ensureHostNet(c));
    if (isSend) {
      FCX_CUDACHECK(cudaMemcpyAsync(stage, buf, bytes, cudaMemcpyDeviceToHost, rawStream(stream)));
      FCX_CUDACHECK(cudaStreamSynchronize(rawStream(stream)));
      return c->hostNet->run({{true, peer, stage, bytes}});
    }
    FCX_CUDACHECK(cudaStreamSynchronize(rawStream(stream)));
    FCXCHECK(c->hostNet->run({{false, peer, stage, bytes}}));
    FCX_CUDACHECK(cudaMemcpyAsync(buf, stage, bytes, cudaMemcpyHostToDevice, rawStream(stream)));
    FCX_CUDACHECK(cudaStreamSynchronize(rawStream(stream)));
    return flagcxSuccess;
  }
  c->stats[isSend ? flagcxCommOpSend : flagcxCommOpRecv].bytes += bytes;
  if (c->groupDepth == 0) return flushGroup(c);
  return flagcxSuccess;
}

flagcxResult_t flagcxSend(const void *sendbuff, size_t count, flagcxDataType_t datatype, int peer, flagcxComm_t comm,
                          flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  return p2pCall(true, const_cast<void *>(sendbuff), count, datatype, peer, comm, stream);
}
flagcxResult_t flagcxRecv(void *recvbuff, size_t count, flagcxDataType_t datatype, int peer, flagcxComm_t comm,
                          flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  return p2pCall(false, recvbuff, count, datatype, peer, comm, stream);
}

flagcxResult_t flagcxGroupStart(flagcxComm_t comm) {
  FCX_COMMCHECK(comm);
  comm->groupDepth++;
  return flagcxSuccess;
}
flagcxResult_t flagcxGroupEnd(flagcxComm_t comm) {
  FCX_COMMCHECK(comm);
  if (comm->groupDepth <= 0) { FCX_WARN("flagcxGroupEnd without flagcxGroupStart"); return flagcxInvalidUsage; }
  if (--comm->groupDepth > 0) return flagcxSuccess;
  return flushGroup(comm);
}

} // extern "C"
