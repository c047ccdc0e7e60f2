// cuda_rt.cc -- see cuda_rt.h.
#include "cuda_rt.h"

#include <unistd.h>

#include <map>
#include <mutex>

namespace fcx {
namespace cu {
namespace {

// Driver API entry points, resolved through the runtime so that the library has
// no link-time dependency on libcuda.
struct Driver {
  bool ok = false;
  int ndev = 0;
#define FCX_DRV(name) decltype(&::name) p_##name = nullptr;
  FCX_DRV(cuGetErrorString)
  FCX_DRV(cuDeviceGet)
  FCX_DRV(cuDeviceGetAttribute)
  FCX_DRV(cuMemCreate)
  FCX_DRV(cuMemRelease)
  FCX_DRV(cuMemAddressReserve)
  FCX_DRV(cuMemAddressFree)
  FCX_DRV(cuMemMap)
  FCX_DRV(cuMemUnmap)
  FCX_DRV(cuMemSetAccess)
  FCX_DRV(cuMemGetAllocationGranularity)
  FCX_DRV(cuMemExportToShareableHandle)
  FCX_DRV(cuMemImportFromShareableHandle)
  FCX_DRV(cuMemGetAddressRange)
  FCX_DRV(cuPointerGetAttribute)
  FCX_DRV(cuMulticastCreate)
  FCX_DRV(cuMulticastAddDevice)
  FCX_DRV(cuMulticastBindMem)
  FCX_DRV(cuMulticastUnbind)
  FCX_DRV(cuMulticastGetGranularity)
  FCX_DRV(cuStreamWriteValue64)
  FCX_DRV(cuStreamWaitValue64)
  FCX_DRV(cuTensorMapEncodeTiled)
#undef FCX_DRV
};

Driver *driver() {
  static Driver d;
  static std::once_flag once;
  std::call_once(once, [] {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      return;
    }
    d.ndev = n;
    bool all = true;
    auto load = [&](const char *name, void **fn, bool required) {
      cudaDriverEntryPointQueryResult st;
      if (cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &st) != cudaSuccess ||
          st != cudaDriverEntryPointSuccess || !*fn) {
        cudaGetLastError();
        *fn = nullptr;
        if (required) { all = false; FCX_WARN("CUDA driver lacks %s", name); }
      }
    };
#define FCX_LOAD(name, req) load(#name, (void **)&d.p_##name, req);
    FCX_LOAD(cuGetErrorString, true)
    FCX_LOAD(cuDeviceGet, true)
    FCX_LOAD(cuDeviceGetAttribute, true)
    FCX_LOAD(cuMemCreate, true)
    FCX_LOAD(cuMemRelease, true)
    FCX_LOAD(cuMemAddressReserve, true)
    FCX_LOAD(cuMemAddressFree, true)
    FCX_LOAD(cuMemMap, true)
    FCX_LOAD(cuMemUnmap, true)
    FCX_LOAD(cuMemSetAccess, true)
    FCX_LOAD(cuMemGetAllocationGranularity, true)
    FCX_LOAD(cuMemExportToShareableHandle, true)
    FCX_LOAD(cuMemImportFromShareableHandle, true)
    FCX_LOAD(cuMemGetAddressRange, true)
    FCX_LOAD(cuPointerGetAttribute, true)
    FCX_LOAD(cuMulticastCreate, false)
    FCX_LOAD(cuMulticastAddDevice, false)
    FCX_LOAD(cuMulticastBindMem, false)
    FCX_LOAD(cuMulticastUnbind, false)
    FCX_LOAD(cuMulticastGetGranularity, false)
    FCX_LOAD(cuStreamWriteValue64, true)
    FCX_LOAD(cuStreamWaitValue64, true)
    FCX_LOAD(cuTensorMapEncodeTiled, false)
#undef FCX_LOAD
    d.ok = all;
  });
  return &d;
}

std::mutex gBlocksMu;
std::map<uintptr_t, VmmBlock> gBlocks; // blocks created by vmmAlloc, keyed by base

CUmemAllocationProp allocProp(int dev) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = dev;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  return prop;
}

flagcxResult_t mapHandle(CUmemGenericAllocationHandle h, size_t size, size_t align, int dev, void **out) {
  Driver *d = driver();
  CUdeviceptr va = 0;
  FCX_CUCHECK(d->p_cuMemAddressReserve(&va, size, align, 0, 0));
  CUresult r = d->p_cuMemMap(va, size, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    d->p_cuMemAddressFree(va, size);
    FCX_WARN("cuMemMap failed: %s", drvErrorString(r));
    return flagcxUnhandledDeviceError;
  }
  CUmemAccessDesc acc = {};
  acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  acc.location.id = dev;
  acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = d->p_cuMemSetAccess(va, size, &acc, 1);
  if (r != CUDA_SUCCESS) {
    d->p_cuMemUnmap(va, size);
    d->p_cuMemAddressFree(va, size);
    FCX_WARN("cuMemSetAccess failed: %s", drvErrorString(r));
    return flagcxUnhandledDeviceError;
  }
  *out = (void *)va;
  return flagcxSuccess;
}

} // namespace

bool available() { return driver()->ok; }
int deviceCount() { return driver()->ndev; }

const char *drvErrorString(CUresult r) {
  const char *s = nullptr;
  Driver *d = driver();
  if (d->p_cuGetErrorString && d->p_cuGetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "unknown driver error";
}

bool vmmSupported(int dev) {
  Driver *d = driver();
  if (!d->ok) return false;
  CUdevice cd;
  int v = 0;
  if (d->p_cuDeviceGet(&cd, dev) != CUDA_SUCCESS) return false;
  if (d->p_cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, cd) != CUDA_SUCCESS || !v)
    return false;
  if (d->p_cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cd) != CUDA_SUCCESS)
    return false;
  return v != 0;
}

size_t vmmGranularity(int dev) {
  Driver *d = driver();
  if (!d->ok) return 2u << 20;
  CUmemAllocationProp prop = allocProp(dev);
  size_t g = 0;
  if (d->p_cuMemGetAllocationGranularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0)
    g = 2u << 20;
  return g;
}

flagcxResult_t vmmAlloc(size_t size, int dev, VmmBlock *out) {
  Driver *d = driver();
  if (!d->ok) return flagcxNotSupported;
  // The context must exist before driver-level allocation.
  FCX_CUDACHECK(cudaSetDevice(dev));
  FCX_CUDACHECK(cudaFree(0));
  size_t gran = vmmGranularity(dev);
  size_t sz = alignUp(size ? size : 1, gran);
  CUmemAllocationProp prop = allocProp(dev);
  VmmBlock b;
  FCX_CUCHECK(d->p_cuMemCreate(&b.handle, sz, &prop, 0));
  flagcxResult_t r = mapHandle(b.handle, sz, gran, dev, &b.ptr);
  if (r != flagcxSuccess) { d->p_cuMemRelease(b.handle); return r; }
  b.size = sz;
  b.dev = dev;
  {
    std::lock_guard<std::mutex> g(gBlocksMu);
    gBlocks[(uintptr_t)b.ptr] = b;
  }
  *out = b;
  FCX_TRACE(SUB_ALLOC, "vmmAlloc %zu bytes at %p on device %d", sz, b.ptr, dev);
  return flagcxSuccess;
}

flagcxResult_t vmmFree(VmmBlock *b) {
  Driver *d = driver();
  if (!b->ptr) return flagcxSuccess;
  if (!b->imported) {
    std::lock_guard<std::mutex> g(gBlocksMu);
    gBlocks.erase((uintptr_t)b->ptr);
  }
  FCX_CUCHECK(d->p_cuMemUnmap((CUdeviceptr)b->ptr, b->size));
  FCX_CUCHECK(d->p_cuMemAddressFree((CUdeviceptr)b->ptr, b->size));
  FCX_CUCHECK(d->p_cuMemRelease(b->handle));
  b->ptr = nullptr;
  return flagcxSuccess;
}

flagcxResult_t vmmExportFd(const VmmBlock &b, int *fd) {
  Driver *d = driver();
  int f = -1;
  FCX_CUCHECK(d->p_cuMemExportToShareableHandle(&f, b.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *fd = f;
  return flagcxSuccess;
}

flagcxResult_t vmmImportFd(int fd, size_t size, int dev, VmmBlock *out) {
  Driver *d = driver();
  VmmBlock b;
  FCX_CUCHECK(d->p_cuMemImportFromShareableHandle(&b.handle, (void *)(uintptr_t)fd,
                                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  flagcxResult_t r = mapHandle(b.handle, size, vmmGranularity(dev), dev, &b.ptr);
  if (r != flagcxSuccess) { d->p_cuMemRelease(b.handle); return r; }
  b.size = size;
  b.dev = dev;
  b.imported = true;
  *out = b;
  return flagcxSuccess;
}

const VmmBlock *vmmLookup(const void *p) {
  std::lock_guard<std::mutex> g(gBlocksMu);
  auto it = gBlocks.upper_bound((uintptr_t)p);
  if (it == gBlocks.begin()) return nullptr;
  --it;
  if ((uintptr_t)p < it->first + it->second.size) return &it->second;
  return nullptr;
}

// ---------------------------------------------------------------------------
bool mcSupported(int dev) {
  Driver *d = driver();
  if (!d->ok || !d->p_cuMulticastCreate) return false;
  CUdevice cd;
  int v = 0;
  if (d->p_cuDeviceGet(&cd, dev) != CUDA_SUCCESS) return false;
  if (d->p_cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd) != CUDA_SUCCESS) return false;
  return v != 0;
}

static CUmulticastObjectProp mcProp(int nDevices, size_t size) {
  CUmulticastObjectProp p = {};
  p.numDevices = nDevices;
  p.size = size;
  p.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  p.flags = 0;
  return p;
}

size_t mcGranularity(int nDevices, size_t size) {
  Driver *d = driver();
  CUmulticastObjectProp p = mcProp(nDevices, size);
  size_t g = 0;
  if (!d->p_cuMulticastGetGranularity ||
      d->p_cuMulticastGetGranularity(&g, &p, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || g == 0)
    g = 2u << 20;
  return g;
}

flagcxResult_t mcCreate(int nDevices, size_t size, McObject *out) {
  Driver *d = driver();
  if (!d->p_cuMulticastCreate) return flagcxNotSupported;
  CUmulticastObjectProp p = mcProp(nDevices, size);
  FCX_CUCHECK(d->p_cuMulticastCreate(&out->handle, &p));
  out->size = size;
  return flagcxSuccess;
}

flagcxResult_t mcExportFd(const McObject &m, int *fd) {
  Driver *d = driver();
  int f = -1;
  FCX_CUCHECK(d->p_cuMemExportToShareableHandle(&f, m.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
  *fd = f;
  return flagcxSuccess;
}

flagcxResult_t mcImportFd(int fd, size_t size, McObject *out) {
  Driver *d = driver();
  FCX_CUCHECK(d->p_cuMemImportFromShareableHandle(&out->handle, (void *)(uintptr_t)fd,
                                                  CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
  out->size = size;
  return flagcxSuccess;
}

flagcxResult_t mcAddDevice(McObject *m, int dev) {
  Driver *d = driver();
  CUdevice cd;
  FCX_CUCHECK(d->p_cuDeviceGet(&cd, dev));
  FCX_CUCHECK(d->p_cuMulticastAddDevice(m->handle, cd));
  m->dev = dev;
  return flagcxSuccess;
}

flagcxResult_t mcBindAndMap(McObject *m, const VmmBlock &mem) {
  Driver *d = driver();
  FCX_CUCHECK(d->p_cuMulticastBindMem(m->handle, 0, mem.handle, 0, m->size, 0));
  m->bound = true;
  flagcxResult_t r = mapHandle(m->handle, m->size, mcGranularity(2, m->size), m->dev, &m->ptr);
  if (r != flagcxSuccess) { mcRelease(m); return r; }
  return flagcxSuccess;
}

flagcxResult_t mcRelease(McObject *m) {
  Driver *d = driver();
  if (m->ptr) {
    d->p_cuMemUnmap((CUdeviceptr)m->ptr, m->size);
    d->p_cuMemAddressFree((CUdeviceptr)m->ptr, m->size);
    m->ptr = nullptr;
  }
  if (m->bound) {
    CUdevice cd;
    if (d->p_cuDeviceGet(&cd, m->dev) == CUDA_SUCCESS) d->p_cuMulticastUnbind(m->handle, cd, 0, m->size);
    m->bound = false;
  }
  if (m->handle) {
    d->p_cuMemRelease(m->handle);
    m->handle = 0;
  }
  return flagcxSuccess;
}

// ---------------------------------------------------------------------------
PtrKind classify(const void *p, int *dev) {
  if (dev) *dev = -1;
  if (!p || !driver()->ok) return kPtrHost;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return kPtrHost;
  }
  if (attr.type == cudaMemoryTypeDevice) { if (dev) *dev = attr.device; return kPtrDevice; }
  if (attr.type == cudaMemoryTypeManaged) { if (dev) *dev = attr.device; return kPtrManaged; }
  return kPtrHost;
}

flagcxResult_t addressRange(const void *p, void **base, size_t *size) {
  Driver *d = driver();
  if (!d->ok) return flagcxNotSupported;
  CUdeviceptr b = 0;
  size_t s = 0;
  FCX_CUCHECK(d->p_cuMemGetAddressRange(&b, &s, (CUdeviceptr)p));
  *base = (void *)b;
  *size = s;
  return flagcxSuccess;
}

flagcxResult_t allocationInfo(const void *p, void **base, size_t *size, uint64_t *id) {
  Driver *d = driver();
  if (!d->ok) return flagcxNotSupported;
  CUdeviceptr b = 0;
  size_t s = 0;
  // quiet on failure: callers probe pointers that may not be device allocations
  if (d->p_cuMemGetAddressRange(&b, &s, (CUdeviceptr)p) != CUDA_SUCCESS) return flagcxInvalidArgument;
  unsigned long long bid = 0;
  if (d->p_cuPointerGetAttribute(&bid, CU_POINTER_ATTRIBUTE_BUFFER_ID, b) != CUDA_SUCCESS) return flagcxInvalidArgument;
  *base = (void *)b;
  *size = s;
  *id = bid;
  return flagcxSuccess;
}

flagcxResult_t tensorMap2dBf16(CUtensorMap *out, const void *base, uint64_t rows, uint64_t cols, uint32_t boxRows,
                               uint32_t boxCols) {
  Driver *d = driver();
  if (!d->p_cuTensorMapEncodeTiled) return flagcxNotSupported;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {boxCols, boxRows};
  cuuint32_t estr[2] = {1, 1};
  FCX_CUCHECK(d->p_cuTensorMapEncodeTiled(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides,
                                          box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE));
  return flagcxSuccess;
}

flagcxResult_t streamWriteValue64(cudaStream_t s, void *addr, uint64_t v) {
  FCX_CUCHECK(driver()->p_cuStreamWriteValue64((CUstream)s, (CUdeviceptr)addr, v, CU_STREAM_WRITE_VALUE_DEFAULT));
  return flagcxSuccess;
}

flagcxResult_t streamWaitValueGeq64(cudaStream_t s, void *addr, uint64_t v) {
  FCX_CUCHECK(driver()->p_cuStreamWaitValue64((CUstream)s, (CUdeviceptr)addr, v, CU_STREAM_WAIT_VALUE_GEQ));
  return flagcxSuccess;
}

} // namespace cu
} // namespace fcx
