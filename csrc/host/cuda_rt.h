// cuda_rt.h -- the CUDA device layer: driver entry points resolved at run time
// (so the library also loads on hosts without a driver), virtual-memory
// allocations that can be exported to other processes as file descriptors,
// NVLink multicast objects, legacy IPC handles, and pointer classification.
//
// Covers the CUDA half of the FlagCX device adaptor
// (flagcx/adaptor/device/cuda_adaptor.cc:114-217 VMM alloc, :576-678 export and
// flat map, :691-880 multicast) with a single CUDA-only implementation.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "base.h"

namespace fcx {
namespace cu {

// True when a driver is present and at least one GPU is visible.
bool available();
int deviceCount();
const char *drvErrorString(CUresult r);

#define FCX_CUDACHECK(call)                                                    \
  do {                                                                         \
    cudaError_t e__ = (call);                                                  \
    if (e__ != cudaSuccess) {                                                  \
      FCX_WARN("CUDA failure %s:%d '%s'", __FILE__, __LINE__,                  \
               cudaGetErrorString(e__));                                       \
      return flagcxUnhandledDeviceError;                                       \
    }                                                                          \
  } while (0)

#define FCX_CUCHECK(call)                                                      \
  do {                                                                         \
    CUresult e__ = (call);                                                     \
    if (e__ != CUDA_SUCCESS) {                                                 \
      FCX_WARN("CUDA driver failure %s:%d '%s'", __FILE__, __LINE__,           \
               ::fcx::cu::drvErrorString(e__));                                \
      return flagcxUnhandledDeviceError;                                       \
    }                                                                          \
  } while (0)

// One physical allocation mapped into this process.
struct VmmBlock {
  void *ptr = nullptr;
  size_t size = 0; // multiple of the granularity
  CUmemGenericAllocationHandle handle = 0;
  int dev = -1;
  bool imported = false;
};

bool vmmSupported(int dev);
size_t vmmGranularity(int dev);
// Allocates `size` bytes (rounded up) of device memory on `dev`, exportable as a
// POSIX file descriptor, mapped read/write for `dev`.
flagcxResult_t vmmAlloc(size_t size, int dev, VmmBlock *out);
flagcxResult_t vmmFree(VmmBlock *b);
flagcxResult_t vmmExportFd(const VmmBlock &b, int *fd);
// Maps another process's allocation (received as fd) for device `dev`.
flagcxResult_t vmmImportFd(int fd, size_t size, int dev, VmmBlock *out);
// The block a pointer obtained from vmmAlloc lies in (nullptr if unknown).
const VmmBlock *vmmLookup(const void *p);

// NVLink multicast (NVLS).
struct McObject {
  CUmemGenericAllocationHandle handle = 0;
  void *ptr = nullptr; // multicast VA mapped for this device
  size_t size = 0;
  int dev = -1;
  bool bound = false;
};
bool mcSupported(int dev);
size_t mcGranularity(int nDevices, size_t size);
flagcxResult_t mcCreate(int nDevices, size_t size, McObject *out);
flagcxResult_t mcExportFd(const McObject &m, int *fd);
flagcxResult_t mcImportFd(int fd, size_t size, McObject *out);
flagcxResult_t mcAddDevice(McObject *m, int dev);
// Binds the whole of `mem` at offset 0 and maps the multicast VA.  All devices
// must have been added (by every rank) before the first bind.
flagcxResult_t mcBindAndMap(McObject *m, const VmmBlock &mem);
// Unmaps and unbinds; safe to call twice.
flagcxResult_t mcRelease(McObject *m);

// Pointer classification.
enum PtrKind { kPtrHost = 0, kPtrDevice = 1, kPtrManaged = 2 };
PtrKind classify(const void *p, int *dev);
// Base and size of the driver allocation containing p.
flagcxResult_t addressRange(const void *p, void **base, size_t *size);
// The same plus the driver's id of that allocation, which is never handed out twice:
// tells a freed-and-reallocated address from the allocation seen before.
flagcxResult_t allocationInfo(const void *p, void **base, size_t *size, uint64_t *id);

// Tensor map for TMA tile loads of a row-major bf16 matrix [rows, cols] (cols
// contiguous), box of boxRows x boxCols elements, 128-byte swizzle.  boxCols * 2 must
// be 128; base 16-byte aligned; cols * 2 a multiple of 16.
flagcxResult_t tensorMap2dBf16(CUtensorMap *out, const void *base, uint64_t rows, uint64_t cols, uint32_t boxRows,
                               uint32_t boxCols);

// Stream-ordered 64-bit write / wait on device memory.
flagcxResult_t streamWriteValue64(cudaStream_t s, void *addr, uint64_t v);
flagcxResult_t streamWaitValueGeq64(cudaStream_t s, void *addr, uint64_t v);

} // namespace cu
} // namespace fcx
