// nccl_shim.cc -- a libnccl stand-in that forwards the NCCL API to this library.
//
//   make -C csrc nccl-shim
//   LD_PRELOAD=<dir>/libnccl_flagcx_shim.so  <program written against NCCL>
//
// Preloaded, its symbols win over libnccl.so.2, so a program that calls ncclAllReduce
// runs the NVLink kernels (or, with host buffers, the socket path) of libflagcx.  Same
// role as plugin/nccl/src/nccl_wrapper.cc in the FlagCX project.  NCCL's types are
// redeclared here with the values of its public ABI (result codes, data types and
// reduction operators happen to number exactly like flagcx.h's), so nccl.h is not
// needed to build.  Covered: version, unique id, communicator life cycle and queries,
// the five collectives, send/recv, groups, memory allocation and registration.  Not
// covered (ncclInvalidUsage): ncclCommInitAll, ncclCommSplit, custom reduction operators.
#include <stdint.h>
#include <string.h>

#include <vector>

#include "flagcx.h"

extern "C" {

typedef int ncclResult_t; // ncclSuccess 0 ... ncclInProgress 7: same numbering as flagcxResult_t
typedef int ncclDataType_t;
typedef int ncclRedOp_t;
typedef struct flagcxComm *ncclComm_t; // opaque to the caller
typedef struct CUstream_st *cudaStream_t;
#define NCCL_UNIQUE_ID_BYTES 128
typedef struct { char internal[NCCL_UNIQUE_ID_BYTES]; } ncclUniqueId;

enum { ncclSuccessV = 0, ncclInternalErrorV = 3, ncclInvalidArgumentV = 4, ncclInvalidUsageV = 5 };
enum { kNcclNumTypes = 10 /* int8 ... bfloat16; fp8 types are refused */, kNcclNumOps = 5 };

} // extern "C"

namespace {

// Layout of the library's stream handle (one member: the CUDA stream).
struct StreamBox {
  cudaStream_t base;
};

inline flagcxStream_t box(StreamBox *b) { return reinterpret_cast<flagcxStream_t>(b); }

// NCCL's groups are per thread and name no communicator; this library's are per
// communicator.  Inside an NCCL group every communicator that gets a send or a receive
// has its own group opened, and ncclGroupEnd closes them all.
thread_local int tlsGroupDepth = 0;
thread_local std::vector<flagcxComm_t> tlsGroupComms;

inline flagcxResult_t joinGroup(flagcxComm_t comm) {
  if (tlsGroupDepth == 0) return flagcxSuccess;
  for (flagcxComm_t c : tlsGroupComms)
    if (c == comm) return flagcxSuccess;
  flagcxResult_t r = flagcxGroupStart(comm);
  if (r == flagcxSuccess) tlsGroupComms.push_back(comm);
  return r;
}

inline bool typeOk(ncclDataType_t t) { return t >= 0 && t < kNcclNumTypes; }
inline bool opOk(ncclRedOp_t o) { return o >= 0 && o < kNcclNumOps; }

} // namespace

extern "C" {

ncclResult_t ncclGetVersion(int *version) {
  if (!version) return ncclInvalidArgumentV;
  *version = 22809; // the NCCL API level this shim answers for (2.28.9)
  return ncclSuccessV;
}

ncclResult_t ncclGetUniqueId(ncclUniqueId *id) {
  if (!id) return ncclInvalidArgumentV;
  flagcxUniqueId full;
  memset(&full, 0, sizeof full);
  flagcxResult_t r = flagcxGetUniqueId(&full);
  if (r != flagcxSuccess) return (ncclResult_t)r;
  // the bootstrap address lives in the first bytes; the rest of the 256 must be unused
  for (size_t i = NCCL_UNIQUE_ID_BYTES; i < sizeof full.internal; ++i)
    if (full.internal[i]) return ncclInternalErrorV;
  memcpy(id->internal, full.internal, NCCL_UNIQUE_ID_BYTES);
  return ncclSuccessV;
}

ncclResult_t ncclCommInitRank(ncclComm_t *comm, int nranks, ncclUniqueId commId, int rank) {
  if (!comm) return ncclInvalidArgumentV;
  flagcxUniqueId full;
  memset(&full, 0, sizeof full);
  memcpy(full.internal, commId.internal, NCCL_UNIQUE_ID_BYTES);
  return (ncclResult_t)flagcxCommInitRank(comm, nranks, &full, rank);
}

// The configuration (blocking mode, CTA limits, ...) has no counterpart here.
ncclResult_t ncclCommInitRankConfig(ncclComm_t *comm, int nranks, ncclUniqueId commId, int rank, void *) {
  return ncclCommInitRank(comm, nranks, commId, rank);
}

ncclResult_t ncclCommInitAll(ncclComm_t *, int, const int *) { return ncclInvalidUsageV; } // one process per GPU
ncclResult_t ncclCommSplit(ncclComm_t, int, int, ncclComm_t *, void *) { return ncclInvalidUsageV; }

ncclResult_t ncclCommFinalize(ncclComm_t comm) { return (ncclResult_t)flagcxCommFinalize(comm); }
ncclResult_t ncclCommDestroy(ncclComm_t comm) { return (ncclResult_t)flagcxCommDestroy(comm); }
ncclResult_t ncclCommAbort(ncclComm_t comm) { return (ncclResult_t)flagcxCommAbort(comm); }
ncclResult_t ncclCommCount(const ncclComm_t comm, int *count) { return (ncclResult_t)flagcxCommCount(comm, count); }
ncclResult_t ncclCommUserRank(const ncclComm_t comm, int *rank) { return (ncclResult_t)flagcxCommUserRank(comm, rank); }
ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int *device) {
  return (ncclResult_t)flagcxCommGetDeviceNumber(comm, device);
}
ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t *asyncError) {
  flagcxResult_t e = flagcxSuccess;
  flagcxResult_t r = flagcxCommGetAsyncError(comm, &e);
  if (asyncError) *asyncError = (ncclResult_t)e;
  return (ncclResult_t)r;
}
const char *ncclGetErrorString(ncclResult_t result) { return flagcxGetErrorString((flagcxResult_t)result); }
const char *ncclGetLastError(ncclComm_t comm) { return flagcxGetLastError(comm); }

ncclResult_t ncclMemAlloc(void **ptr, size_t size) { return (ncclResult_t)flagcxMemAlloc(ptr, size, flagcxMemCCL); }
ncclResult_t ncclMemFree(void *ptr) { return (ncclResult_t)flagcxMemFree(ptr, flagcxMemCCL); }
ncclResult_t ncclCommRegister(const ncclComm_t comm, void *buff, size_t size, void **handle) {
  return (ncclResult_t)flagcxCommRegister(comm, buff, size, handle, flagcxMemCCL);
}
ncclResult_t ncclCommDeregister(const ncclComm_t comm, void *handle) {
  return (ncclResult_t)flagcxCommDeregister(comm, handle, flagcxMemCCL);
}

ncclResult_t ncclAllReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                           ncclComm_t comm, cudaStream_t stream) {
  if (!typeOk(datatype) || !opOk(op)) return ncclInvalidArgumentV;
  StreamBox s{stream};
  return (ncclResult_t)flagcxAllReduce(sendbuff, recvbuff, count, (flagcxDataType_t)datatype, (flagcxRedOp_t)op, comm,
                                       box(&s));
}

ncclResult_t ncclBroadcast(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, int root,
                           ncclComm_t comm, cudaStream_t stream) {
  if (!typeOk(datatype)) return ncclInvalidArgumentV;
  StreamBox s{stream};
  return (ncclResult_t)flagcxBroadcast(sendbuff, recvbuff, count, (flagcxDataType_t)datatype, root, comm, box(&s));
}

ncclResult_t ncclBcast(void *buff, size_t count, ncclDataType_t datatype, int root, ncclComm_t comm,
                       cudaStream_t stream) {
  return ncclBroadcast(buff, buff, count, datatype, root, comm, stream);
}

ncclResult_t ncclReduce(const void *sendbuff, void *recvbuff, size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                        int root, ncclComm_t comm, cudaStream_t stream) {
  if (!typeOk(datatype) || !opOk(op)) return ncclInvalidArgumentV;
  StreamBox s{stream};
  return (ncclResult_t)flagcxReduce(sendbuff, recvbuff, count, (flagcxDataType_t)datatype, (flagcxRedOp_t)op, root,
                                    comm, box(&s));
}

ncclResult_t ncclAllGather(const void *sendbuff, void *recvbuff, size_t sendcount, ncclDataType_t datatype,
                           ncclComm_t comm, cudaStream_t stream) {
  if (!typeOk(datatype)) return ncclInvalidArgumentV;
  StreamBox s{stream};
  return (ncclResult_t)flagcxAllGather(sendbuff, recvbuff, sendcount, (flagcxDataType_t)datatype, comm, box(&s));
}

ncclResult_t ncclReduceScatter(const void *sendbuff, void *recvbuff, size_t recvcount, ncclDataType_t datatype,
                               ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
  if (!typeOk(datatype) || !opOk(op)) return ncclInvalidArgumentV;
  StreamBox s{stream};
  return (ncclResult_t)flagcxReduceScatter(sendbuff, recvbuff, recvcount, (flagcxDataType_t)datatype,
                                           (flagcxRedOp_t)op, comm, box(&s));
}

ncclResult_t ncclSend(const void *sendbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm,
                      cudaStream_t stream) {
  if (!typeOk(datatype)) return ncclInvalidArgumentV;
  StreamBox s{stream};
  if (flagcxResult_t r = joinGroup(comm)) return (ncclResult_t)r;
  return (ncclResult_t)flagcxSend(sendbuff, count, (flagcxDataType_t)datatype, peer, comm, box(&s));
}

ncclResult_t ncclRecv(void *recvbuff, size_t count, ncclDataType_t datatype, int peer, ncclComm_t comm,
                      cudaStream_t stream) {
  if (!typeOk(datatype)) return ncclInvalidArgumentV;
  StreamBox s{stream};
  if (flagcxResult_t r = joinGroup(comm)) return (ncclResult_t)r;
  return (ncclResult_t)flagcxRecv(recvbuff, count, (flagcxDataType_t)datatype, peer, comm, box(&s));
}

ncclResult_t ncclGroupStart() {
  ++tlsGroupDepth;
  return ncclSuccessV;
}
ncclResult_t ncclGroupEnd() {
  if (tlsGroupDepth <= 0) return ncclInvalidUsageV;
  if (--tlsGroupDepth > 0) return ncclSuccessV;
  ncclResult_t first = ncclSuccessV;
  for (flagcxComm_t c : tlsGroupComms) {
    flagcxResult_t r = flagcxGroupEnd(c);
    if (r != flagcxSuccess && first == ncclSuccessV) first = (ncclResult_t)r;
  }
  tlsGroupComms.clear();
  return first;
}

ncclResult_t ncclRedOpCreatePreMulSum(ncclRedOp_t *, void *, ncclDataType_t, int, ncclComm_t) { return ncclInvalidUsageV; }
ncclResult_t ncclRedOpDestroy(ncclRedOp_t, ncclComm_t) { return ncclInvalidUsageV; }

} // extern "C"
