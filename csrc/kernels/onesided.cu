// onesided.cu -- stream-ordered one-sided operations of the host API: put with
// signal, bare signal, and a bounded wait for signals.
//
// FlagCX implements these with a proxy thread that posts RDMA writes and atomics,
// or for ranks of one node with cudaMemcpyAsync plus cuStreamWriteValue64
// (flagcx/core/flagcx_hetero.cc:1339-1519 in the FlagCX project).  Here a put is one
// kernel: all CTAs copy into the peer's mapping with 16-byte stores, the CTA that
// finishes last publishes the signal with release semantics.  Waiting is a kernel
// too, so that it can give up after the communicator's time limit instead of
// blocking the stream forever.
#include <cuda_runtime.h>

#include "launch.h"
#include "prims.cuh"

namespace fcx {
namespace {

__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    putSignalKernel(char *dst, const char *src, size_t bytes, unsigned long long *peerSignal,
                    unsigned long long addValue, unsigned int *arrival) {
  size_t ub, ue;
  ctaShare((bytes + 15) >> 4, blockIdx.x, gridDim.x, &ub, &ue);
  size_t bb = ub << 4, be = (ue << 4) < bytes ? (ue << 4) : bytes;
  ctaCopy(dst, src, bb, be);
  __syncthreads();
  if (threadIdx.x == 0) {
    fcxdev::fenceSys();
    // last CTA to arrive signals; the counter wraps back to zero for the next put
    unsigned int prev = atomicInc(arrival, gridDim.x - 1);
    if (prev == gridDim.x - 1 && peerSignal) {
      fcxdev::fenceSys();
      fcxdev::redAddReleaseSys(peerSignal, addValue);
    }
  }
}

__global__ void waitSignalKernel(const flagcxDevComm c, const unsigned long long *sig, unsigned long long want,
                                 unsigned int peer) {
  if (threadIdx.x == 0) fcxdev::waitGe(c, sig, want, FLAGCX_DEV_AT_SIGNAL, peer);
}

} // namespace

cudaError_t launchPutSignal(cudaStream_t s, void *dst, const void *src, size_t bytes, unsigned long long *peerSignal,
                            unsigned long long addValue, unsigned int *arrival, int nCtas) {
  if (bytes == 0 && !peerSignal) return cudaSuccess;
  if (nCtas < 1) nCtas = 1;
  putSignalKernel<<<nCtas, FLAGCX_DEVICE_THREADS_PER_CTA, 0, s>>>((char *)dst, (const char *)src, bytes, peerSignal,
                                                                  addValue, arrival);
  return cudaGetLastError();
}

cudaError_t launchWaitSignal(cudaStream_t s, const flagcxDevComm &c, const unsigned long long *sig,
                             unsigned long long want, unsigned int peer) {
  waitSignalKernel<<<1, 32, 0, s>>>(c, sig, want, peer);
  return cudaGetLastError();
}

} // namespace fcx
