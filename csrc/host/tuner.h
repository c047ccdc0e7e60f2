// tuner.h -- picks the algorithm and CTA count of each device collective from
// measured time.
//
// FlagCX's tuner (flagcx/core/flagcx_tuner.cc in the FlagCX project) searches NCCL
// environment settings by re-creating NCCL communicators.  Here the search space
// is this library's own algorithms x CTA counts; candidates are timed with CUDA
// events (max over ranks), the winner per (operation, size bucket, registered or
// staged) is kept with 5 % hysteresis against the built-in heuristic, and the
// table can be saved to / loaded from JSON (FLAGCX_TUNE_FILE) so a job can skip
// tuning.
#pragma once
#include <map>
#include <string>

#include "flagcx.h"
#include "flagcx_ext.h"

struct flagcxComm;

namespace fcx {

struct TuneChoice {
  int algo = FLAGCX_ALGO_AUTO;
  int nCtas = 0;
  float usec = 0.f;     // measured time of this choice (0: heuristic, never measured)
  float bestUsec = 0.f; // fastest candidate measured for the bucket (the choice may be the
                        // heuristic's when that is within 5 % of it)
};

struct Tuner {
  flagcxResult_t init(flagcxComm *c);
  // registered: 1 when the buffers need no staging.  nvlsOk: multimem usable for
  // this call.  Always returns a concrete algorithm and CTA count.
  // elemSize: bytes per element for the reducing operations (a table may hold different
  // winners for 2- and 4-byte types: the adds per byte differ), 0 for pure copies or "any".
  // A lookup falls back to the size-agnostic entry, then to any entry of the bucket.
  TuneChoice choose(flagcxCommOp_t op, size_t bytes, int nranks, bool registered, bool nvlsOk, int elemSize = 0) const;
  TuneChoice heuristic(flagcxCommOp_t op, size_t bytes, int nranks, bool registered, bool nvlsOk) const;
  flagcxResult_t tune(flagcxComm *c, flagcxCommOp_t op, flagcxDataType_t dtype, size_t minBytes,
                      size_t maxBytes, int iters);
  flagcxResult_t save(const char *path) const;
  flagcxResult_t load(const char *path);
  std::string toJson() const;
  flagcxResult_t fromJson(const std::string &text);

  static int bucketOf(size_t bytes); // ceil(log2(bytes))
  // key = elemSize * 100000 + op * 1000 + bucket * 2 + registered
  std::map<int, TuneChoice> table;
  int maxCtas = 32;
  int forcedAlgo = FLAGCX_ALGO_AUTO; // FLAGCX_ALGO
  int forcedCtas = 0;                // FLAGCX_NCTAS
  // largest messages the heuristic sends down the barrier-free LL path
  // (FLAGCX_LL_MAX_BYTES, FLAGCX_LL_ALLGATHER_MAX_BYTES; 0 switches it off)
  size_t llMaxAllReduce = 0, llMaxAllGather = 0;
};

} // namespace fcx
