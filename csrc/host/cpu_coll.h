// cpu_coll.h -- collectives on host memory over the network adaptor.
//
// This is the path taken for host pointers, on hosts without a GPU, and as the
// staged fallback for device buffers whose ranks cannot reach each other over
// NVLink (different machines, or FLAGCX_P2P_DISABLE=1).  It covers what the
// FlagCX project does with its bootstrap CCL adaptor and host runner
// (flagcx/adaptor/ccl/bootstrap_adaptor.cc, flagcx/service/bootstrap.cc:787-1286,
// flagcx/runner/host_runner.cc): ring reduce-scatter / all-gather / all-reduce,
// tree broadcast and reduce, rooted gather/scatter, pairwise all-to-all(v) and
// point-to-point, for all ten element types and five reductions.
#pragma once
#include <vector>

#include <memory>

#include "bootstrap.h"
#include "flagcx_net.h"
#include "shm.h"

namespace fcx {

// Pairwise message layer: lazily opened adaptor connections to each peer.
class HostNet {
 public:
  ~HostNet() { close(); }
  flagcxResult_t init(Bootstrap *bs);
  void close();
  int rank() const { return bs_->rank(); }
  int nranks() const { return bs_->nranks(); }

  struct Op {
    bool isSend;
    int peer;
    void *data;
    size_t bytes;
  };
  // Posts every op, then drives them all to completion (deadline: the socket
  // timeout without any byte moving).  Ops towards one peer complete in order.
  flagcxResult_t run(const std::vector<Op> &ops);
  flagcxResult_t sendRecv(int sendPeer, const void *sbuf, size_t sbytes, int recvPeer, void *rbuf,
                          size_t rbytes);

 private:
  flagcxResult_t sendComm(int peer, void **c);
  flagcxResult_t recvComm(int peer, void **c);
  Bootstrap *bs_ = nullptr;
  const flagcxNetAdaptor_v1 *net_ = nullptr;
  void *listen_ = nullptr;
  std::vector<char> handles_; // nranks * FLAGCX_NET_HANDLE_BYTES
  std::vector<void *> send_, recv_;
  // Ranks of this machine talk through shared-memory rings instead (FLAGCX_HOST_SHM=0
  // or a net plugin switches that off; all ranks must have got their rings).
  bool shm_ = false;
  std::vector<std::unique_ptr<ShmRing>> shmSend_, shmRecv_; // per peer, null: use the adaptor
  std::vector<int> pids_;
  flagcxResult_t initShm();
};

// Element-wise dst = dst (op) src on host memory; used by the collectives and
// exported for unit tests.
flagcxResult_t hostReduce(void *dst, const void *src, size_t count, flagcxDataType_t dt,
                          flagcxRedOp_t op);
// dst[i] /= n (integer division for integer types); completes flagcxAvg.
flagcxResult_t hostDivide(void *dst, size_t count, flagcxDataType_t dt, int n);

struct CpuColl {
  HostNet *net;
  flagcxResult_t allReduce(const void *send, void *recv, size_t count, flagcxDataType_t dt,
                           flagcxRedOp_t op);
  flagcxResult_t reduceScatter(const void *send, void *recv, size_t recvCount,
                               flagcxDataType_t dt, flagcxRedOp_t op);
  flagcxResult_t allGather(const void *send, void *recv, size_t sendCount, flagcxDataType_t dt);
  flagcxResult_t broadcast(const void *send, void *recv, size_t count, flagcxDataType_t dt,
                           int root);
  flagcxResult_t reduce(const void *send, void *recv, size_t count, flagcxDataType_t dt,
                        flagcxRedOp_t op, int root);
  flagcxResult_t gather(const void *send, void *recv, size_t count, flagcxDataType_t dt, int root);
  flagcxResult_t scatter(const void *send, void *recv, size_t count, flagcxDataType_t dt,
                         int root);
  flagcxResult_t allToAll(const void *send, void *recv, size_t count, flagcxDataType_t dt);
  flagcxResult_t allToAllv(const void *send, const size_t *scounts, const size_t *sdispls,
                           void *recv, const size_t *rcounts, const size_t *rdispls,
                           flagcxDataType_t dt);
};

// bf16 / fp16 <-> float on the host (round to nearest even).
float bf16ToFloat(uint16_t v);
uint16_t floatToBf16(float f);
float halfToFloat(uint16_t v);
uint16_t floatToHalf(float f);

} // namespace fcx
