// api_ext.cc -- the extern "C" surface, part 3: the entry points of flagcx_ext.h (fused
// and algorithm-selecting collectives, tuner, trace, statistics, user-buffer export
// control, the emulated world for single-GPU tests).
#include <algorithm>

#include "../kernels/launch.h"
#include "api_internal.h"
#include "tuner.h"

using namespace fcx;

extern "C" {

// ---------------------------------------------------------------------------
// extensions
// ---------------------------------------------------------------------------
// Device collective of the extension entry points, with the same trace record and NVTX range
// that the FlagCX-compatible entry points get.
static flagcxResult_t tracedDeviceCollective(flagcxComm *c, const DeviceCollRequest &rq, size_t bytes, flagcxStream_t stream) {
  nvtxPush(commOpName(rq.op));
  const int slot = c->trace.begin(c, rq.op, bytes, 0, rawStream(stream));
  flagcxResult_t r = deviceCollective(c, rq, rawStream(stream));
  c->trace.end(c, slot, rawStream(stream));
  nvtxPop();
  return r;
}

flagcxResult_t flagcxAllReduceFused(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype,
                                    flagcxRedOp_t op, const flagcxFusedOpts_t *opts, flagcxComm_t comm,
                                    flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  FCXCHECK(checkUsable(comm));
  if (!comm->devicePath) return flagcxNotSupported;
  DeviceCollRequest rq{flagcxCommOpAllReduce, sendbuff, recvbuff, count, datatype, op, 0};
  if (opts) {
    rq.scale = opts->scale;
    rq.outDtype = opts->outDtype;
    rq.residual = opts->residual;
    rq.algo = opts->algo;
    rq.nCtas = opts->nCtas > 0 ? opts->nCtas : -1;
  }
  return tracedDeviceCollective(comm, rq, count * getFlagcxDataTypeSize(datatype), stream);
}

flagcxResult_t flagcxReduceScatterFused(const void *sendbuff, void *recvbuff, size_t recvcount,
                                        flagcxDataType_t datatype, flagcxRedOp_t op, const flagcxFusedOpts_t *opts,
                                        flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  FCXCHECK(checkUsable(comm));
  if (!comm->devicePath) return flagcxNotSupported;
  DeviceCollRequest rq{flagcxCommOpReduceScatter, sendbuff, recvbuff, recvcount, datatype, op, 0};
  if (opts) {
    rq.scale = opts->scale;
    rq.outDtype = opts->outDtype;
    rq.residual = opts->residual;
    rq.algo = opts->algo;
    rq.nCtas = opts->nCtas > 0 ? opts->nCtas : -1;
  }
  return tracedDeviceCollective(comm, rq, recvcount * getFlagcxDataTypeSize(datatype) * comm->nranks, stream);
}

flagcxResult_t flagcxAllGatherEx(const void *sendbuff, void *recvbuff, size_t sendcount, flagcxDataType_t datatype,
                                 int algo, int nCtas, flagcxComm_t comm, flagcxStream_t stream) {
  FCX_COMMCHECK(comm);
  FCXCHECK(checkUsable(comm));
  if (!comm->devicePath) return flagcxNotSupported;
  DeviceCollRequest rq{flagcxCommOpAllGather, sendbuff, recvbuff, sendcount, datatype, flagcxSum, 0};
  rq.algo = algo;
  rq.nCtas = nCtas > 0 ? nCtas : -1;
  return tracedDeviceCollective(comm, rq, sendcount * getFlagcxDataTypeSize(datatype) * comm->nranks, stream);
}

flagcxResult_t flagcxTunerTune(flagcxComm_t comm, flagcxCommOp_t op, flagcxDataType_t dtype, size_t minBytes,
                               size_t maxBytes, int iters) {
  FCX_COMMCHECK(comm);
  if (!comm->tuner) return flagcxNotSupported;
  return comm->tuner->tune(comm, op, dtype, minBytes, maxBytes, iters);
}
flagcxResult_t flagcxTunerSave(flagcxComm_t comm, const char *path) {
  FCX_COMMCHECK(comm);
  if (!comm->tuner || !path) return flagcxNotSupported;
  return comm->tuner->save(path);
}
flagcxResult_t flagcxTunerLoad(flagcxComm_t comm, const char *path) {
  FCX_COMMCHECK(comm);
  if (!comm->tuner || !path) return flagcxNotSupported;
  return comm->tuner->load(path);
}
flagcxResult_t flagcxTunerQuery(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, int registered, int *algo,
                                int *nCtas) {
  FCX_COMMCHECK(comm);
  if (!comm->tuner) return flagcxNotSupported;
  TuneChoice ch = comm->tuner->choose(op, bytes, comm->nranks, registered != 0, comm->nvls);
  if (algo) *algo = ch.algo;
  if (nCtas) *nCtas = ch.nCtas;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommTraceEnable(flagcxComm_t comm, int capacity) {
  FCX_COMMCHECK(comm);
  if (capacity < 0 || capacity > (1 << 20)) return flagcxInvalidArgument;
  comm->trace.enable(capacity);
  return flagcxSuccess;
}

flagcxResult_t flagcxCommTraceDump(flagcxComm_t comm, const char *path) {
  FCX_COMMCHECK(comm);
  if (!comm->trace.on()) return flagcxInvalidUsage;
  return comm->trace.dump(comm, path);
}

flagcxResult_t flagcxCommGetStats(flagcxComm_t comm, flagcxCommOp_t op, flagcxOpStats_t *out) {
  FCX_COMMCHECK(comm);
  if (!out || (int)op < 0 || op >= flagcxNumCommOps) return flagcxInvalidArgument;
  const OpStats &s = comm->stats[op];
  out->calls = s.calls;
  out->bytes = s.bytes;
  out->lastAlgo = s.lastAlgo;
  out->lastCtas = s.lastCtas;
  out->lastMs = s.lastMs;
  return flagcxSuccess;
}
flagcxResult_t flagcxCommUserBufferStats(flagcxComm_t comm, flagcxUserBufferStats_t *out) {
  FCX_COMMCHECK(comm);
  if (!out) return flagcxInvalidArgument;
  memset(out, 0, sizeof *out);
  out->enabled = comm->exportUserBuffers ? 1 : 0;
  if (comm->reg) {
    RegCache::Counters k = comm->reg->counters();
    out->hits = k.hits;
    out->exports = k.exports;
    out->refused = k.refused;
    out->stale = k.stale;
    out->peerOpened = k.opened;
    out->peerClosed = k.closed;
  }
  return flagcxSuccess;
}
flagcxResult_t flagcxCommSetAutoExport(flagcxComm_t comm, int on) {
  FCX_COMMCHECK(comm);
  comm->autoExport = on != 0 && comm->exportUserBuffers;
  return flagcxSuccess;
}
flagcxResult_t flagcxCommForgetUserBuffer(flagcxComm_t comm, const void *ptr) {
  FCX_COMMCHECK(comm);
  if (comm->reg && ptr) comm->reg->forget(ptr);
  return flagcxSuccess;
}
flagcxResult_t flagcxCommIsDevicePath(flagcxComm_t comm, int *yes) {
  FCX_COMMCHECK(comm);
  *yes = comm->devicePath ? 1 : 0;
  return flagcxSuccess;
}
flagcxResult_t flagcxCommHasMulticast(flagcxComm_t comm, int *yes) {
  FCX_COMMCHECK(comm);
  *yes = (comm->internalWin && comm->internalWin->mc) ? 1 : 0;
  return flagcxSuccess;
}
flagcxResult_t flagcxCommSetWaitTimeoutMs(flagcxComm_t comm, int ms) {
  FCX_COMMCHECK(comm);
  comm->dev.timeoutNs = (unsigned long long)std::max(ms, 1) * 1000000ull;
  return flagcxSuccess;
}

flagcxResult_t flagcxEmuWorldCreate(int nranks, int device, flagcxComm_t *comms) {
  if (!comms) return flagcxInvalidArgument;
  return emuWorldCreate(nranks, device, comms);
}
flagcxResult_t flagcxEmuWorldDestroy(flagcxComm_t anyRank) {
  FCX_COMMCHECK(anyRank);
  return emuWorldDestroy(anyRank);
}

flagcxResult_t flagcxHostReduce(void *dst, const void *src, size_t count, flagcxDataType_t dtype, flagcxRedOp_t op) {
  return hostReduce(dst, src, count, dtype, op);
}

} // extern "C"
