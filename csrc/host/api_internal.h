// api_internal.h -- what the translation units of the extern "C" surface share.
#pragma once
#include "comm.h"
#include "flagcx_ext.h"

#define FCX_COMMCHECK(comm)                                                   \
  do {                                                                        \
    if (!fcx::commValid(comm)) {                                              \
      FCX_WARN("%s: invalid communicator handle", __func__);                  \
      return flagcxInvalidArgument;                                           \
    }                                                                         \
  } while (0)

namespace fcx {

inline cudaStream_t rawStream(flagcxStream_t s) { return s ? s->base : nullptr; }

// flagcxInvalidUsage after finalize / suspend, the recorded asynchronous error otherwise.
flagcxResult_t checkUsable(flagcxComm *c);

} // namespace fcx
