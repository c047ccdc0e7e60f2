// launch.h -- host-callable launchers of the collective kernels.
#pragma once
#include <cuda_runtime.h>

#include "coll_args.h"

namespace fcx {

struct LaunchCtx {
  const flagcxDevComm *comm = nullptr; // host copy, passed to the kernel by value
  cudaStream_t stream = nullptr;
  int nCtas = 1;
  int nThreads = FLAGCX_DEVICE_THREADS_PER_CTA;
  // Emulated world (several ranks of one process on one GPU): one cooperative
  // launch with gridDim.y = emuRanks; the per-rank blocks live in device memory.
  int emuRanks = 0;
  const flagcxDevComm *emuComms = nullptr;
  const CollArgs *emuArgs = nullptr;
  const P2pArgs *emuP2p = nullptr;
  const void *emuBlob = nullptr; // per-rank argument blocks of the other kernel families
  bool emuBulk = false;          // some emulated rank takes a bulk-copy path: the launch needs the shared-memory ring
};

struct MoeArgs;
cudaError_t launchMoeDispatch(const LaunchCtx &lc, const MoeArgs &a);
cudaError_t launchMoeCombine(const LaunchCtx &lc, const MoeArgs &a, bool pull);

cudaError_t launchReduceKernel(const LaunchCtx &lc, const CollArgs &a, int nRanks);
cudaError_t launchCopyKernel(const LaunchCtx &lc, const CollArgs &a);
cudaError_t launchP2pKernel(const LaunchCtx &lc, const P2pArgs &a);
cudaError_t launchNvlsKernel(const LaunchCtx &lc, const CollArgs &a);
cudaError_t launchLlKernel(const LaunchCtx &lc, const CollArgs &a);
// One-sided host API (onesided.cu).  `arrival` is a zero-initialised device word the
// CTAs of one put count themselves in; puts on one stream may share it.
cudaError_t launchPutSignal(cudaStream_t s, void *dst, const void *src, size_t bytes, unsigned long long *peerSignal,
                            unsigned long long addValue, unsigned int *arrival, int nCtas);
cudaError_t launchWaitSignal(cudaStream_t s, const flagcxDevComm &c, const unsigned long long *sig,
                             unsigned long long want, unsigned int peer);
// Upper bound on grid size (x * y) for the cooperative emulated-world launch.
int maxCoresidentCtas(int nThreads);

} // namespace fcx
