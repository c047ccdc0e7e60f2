// trace.h -- per-communicator ring of collective records (operation, bytes, chosen
// algorithm, host time, device time from a pair of CUDA events) that can be written out
// as JSON, and optional NVTX ranges around every call.  Takes the place of the
// event-record ring that the FlagCX project keeps for its tuner
// (flagcx/service/include/timer.h:102-150, flagcx/core/flagcx_tuner.cc:743-813).
#pragma once
#include <cuda_runtime.h>

#include <mutex>
#include <string>
#include <vector>

#include "flagcx.h"

struct flagcxComm;

namespace fcx {

struct TraceRecord {
  uint64_t seq = 0;
  int op = 0;
  size_t bytes = 0;
  int algo = -1, nCtas = 0;
  int route = 0; // 0 device kernels, 1 host sockets, 2 device buffers staged over sockets
  uint64_t hostStartNs = 0, hostEndNs = 0;
  cudaEvent_t e0 = nullptr, e1 = nullptr; // recorded on the caller's stream (device route)
  bool timed = false;
  float deviceMs = 0.f; // filled by resolve()
};

class Trace {
 public:
  ~Trace();
  // capacity 0 switches tracing off and drops the records
  void enable(int capacity);
  bool on() const { return capacity_ > 0; }
  // Opens a record; returns its slot or -1 when tracing is off.
  int begin(flagcxComm *c, flagcxCommOp_t op, size_t bytes, int route, cudaStream_t stream);
  void end(flagcxComm *c, int slot, cudaStream_t stream);
  // Reads the device times of all finished records (synchronises their events).
  void resolve(flagcxComm *c);
  flagcxResult_t dump(flagcxComm *c, const char *path);

 private:
  std::mutex mu_;
  int capacity_ = 0;
  uint64_t next_ = 0;
  std::vector<TraceRecord> ring_;
};

// NVTX range around a call when FLAGCX_NVTX=1 (a no-op unless a tool is attached).
void nvtxPush(const char *name);
void nvtxPop();

} // namespace fcx
