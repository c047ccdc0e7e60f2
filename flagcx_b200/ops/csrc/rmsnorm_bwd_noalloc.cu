// rmsnorm_bwd_noalloc.cu -- see rmsnorm_bwd_noalloc.h for the contract.
//
// Same arithmetic as the regular RMSNorm backward of this package: CTA b walks rows
// b, b+grid, ...; each thread owns fixed columns, so the weight-gradient partial
// sums stay in registers across rows and are written once per CTA.  The difference
// is where those partial sums go (a fixed device array of this file instead of a
// freshly allocated tensor) and who reduces them (a second small kernel here
// instead of a framework reduction that allocates its result).
#include "rmsnorm_bwd_noalloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include <atomic>

namespace {

using bf16 = __nv_bfloat16;

constexpr int kThreads = 512;
constexpr int kMaxPacksPerThread = FLAGCX_NOALLOC_RMSNORM_MAX_HIDDEN / 8 / kThreads; // 2
constexpr int kMaxDevices = 64;

// Scratch for the per-CTA partial weight gradients: [MAX_CTAS][MAX_HIDDEN] floats.
// In host code this name is only a handle for cudaGetSymbolAddress; device code may
// use it directly, but the kernels below take the looked-up pointer so that they can
// be read (and tested) like the allocating variant.
static __device__ __align__(256) float gPartialScratch[FLAGCX_NOALLOC_RMSNORM_MAX_CTAS * FLAGCX_NOALLOC_RMSNORM_MAX_HIDDEN];

// Device address of gPartialScratch per device, filled on the first call there.  Atomic:
// two host threads may make that first call at once; both look the address up and store
// the same value.
std::atomic<float *> gScratchAddr[kMaxDevices];

__device__ __forceinline__ float warpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float blockSum(float v, float *red) {
  v = warpSum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) t = warpSum(t);
  if (threadIdx.x == 0) red[0] = t;
  __syncthreads();
  return red[0];
}

struct Pack8 {
  uint4 raw;
  __device__ float get(int i) const { return __bfloat162float(((const bf16 *)&raw)[i]); }
  __device__ void set(int i, float v) { ((bf16 *)&raw)[i] = __float2bfloat16_rn(v); }
};

// dx = rstd * (g*w - x * rstd^2 * mean(g*w*x)); partial[b][:] = sum over this CTA's rows of g*x*rstd
__global__ void __launch_bounds__(kThreads)
    bwdKernel(const bf16 *__restrict__ g, const bf16 *__restrict__ x, const bf16 *__restrict__ w,
              const float *__restrict__ rstdIn, bf16 *__restrict__ dx, float *__restrict__ partial, long rows, int H) {
  __shared__ float red[32];
  const int nPacks = H / 8;
  float acc[kMaxPacksPerThread][8];
  Pack8 pw[kMaxPacksPerThread];
#pragma unroll
  for (int k = 0; k < kMaxPacksPerThread; ++k) {
    int p = threadIdx.x + k * kThreads;
    if (p < nPacks) pw[k].raw = ((const uint4 *)w)[p];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[k][i] = 0.f;
  }
  for (long row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4 *gr = (const uint4 *)(g + row * H), *xr = (const uint4 *)(x + row * H);
    const float rstd = rstdIn[row];
    Pack8 pg[kMaxPacksPerThread], px[kMaxPacksPerThread];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxPacksPerThread; ++k) {
      int p = threadIdx.x + k * kThreads;
      if (p < nPacks) {
        pg[k].raw = gr[p];
        px[k].raw = xr[p];
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += pg[k].get(i) * pw[k].get(i) * px[k].get(i);
      }
    }
    dot = blockSum(dot, red);
    const float c = dot * rstd * rstd / H;
    uint4 *dxr = (uint4 *)(dx + row * H);
#pragma unroll
    for (int k = 0; k < kMaxPacksPerThread; ++k) {
      int p = threadIdx.x + k * kThreads;
      if (p < nPacks) {
        Pack8 po;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float gv = pg[k].get(i), xv = px[k].get(i);
          po.set(i, rstd * (gv * pw[k].get(i) - xv * c));
          acc[k][i] += gv * xv * rstd;
        }
        dxr[p] = po.raw;
      }
    }
  }
  // every CTA of the grid writes its whole row of the scratch, including zeros when
  // it had no rows: the reduction below never reads a slot left over from an earlier call
  float *out = partial + (size_t)blockIdx.x * H;
#pragma unroll
  for (int k = 0; k < kMaxPacksPerThread; ++k) {
    int p = threadIdx.x + k * kThreads;
    if (p < nPacks) {
      *(float4 *)(out + p * 8) = make_float4(acc[k][0], acc[k][1], acc[k][2], acc[k][3]);
      *(float4 *)(out + p * 8 + 4) = make_float4(acc[k][4], acc[k][5], acc[k][6], acc[k][7]);
    }
  }
}

// dw[c] = sum over CTAs of partial[b][c], rounded to bf16 once.
__global__ void reduceKernel(const float *__restrict__ partial, bf16 *__restrict__ dw, int ctas, int H) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int b = 0; b < ctas; ++b) s += partial[(size_t)b * H + c];
  dw[c] = __float2bfloat16_rn(s);
}

} // namespace

extern "C" int flagcxRmsnormBwdNoAlloc(const void *g, const void *x, const void *w, const float *rstd, void *dx,
                                       void *dw, long rows, int hidden, void *stream) {
  if (!g || !x || !w || !rstd || !dx || !dw || rows < 0 || hidden <= 0) {
    fprintf(stderr, "flagcxRmsnormBwdNoAlloc: null pointer or negative size\n");
    return (int)cudaErrorInvalidValue;
  }
  if (hidden % 8 != 0 || hidden > FLAGCX_NOALLOC_RMSNORM_MAX_HIDDEN) {
    fprintf(stderr,
            "flagcxRmsnormBwdNoAlloc: hidden size %d is not supported (multiple of 8, at most %d: the scratch "
            "array of this entry point has a fixed size)\n",
            hidden, FLAGCX_NOALLOC_RMSNORM_MAX_HIDDEN);
    return (int)cudaErrorInvalidValue;
  }
  if ((((size_t)g | (size_t)x | (size_t)w | (size_t)dx) & 15) != 0) {
    fprintf(stderr, "flagcxRmsnormBwdNoAlloc: g, x, w and dx must be 16-byte aligned\n");
    return (int)cudaErrorInvalidValue;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  cudaStream_t s = (cudaStream_t)stream;
  if (s) {
    // the scratch address used below belongs to the current device: the stream must too
    int sdev = -1;
    e = cudaStreamGetDevice(s, &sdev);
    if (e != cudaSuccess) return (int)e;
    if (sdev != dev) {
      fprintf(stderr, "flagcxRmsnormBwdNoAlloc: the stream belongs to device %d but device %d is current\n", sdev, dev);
      return (int)cudaErrorInvalidValue;
    }
  }
  float *scratch = gScratchAddr[dev].load(std::memory_order_acquire);
  if (!scratch) {
    // once per device, with that device current: the array's name is a host-side
    // stand-in, the kernels need its device address
    e = cudaGetSymbolAddress((void **)&scratch, gPartialScratch);
    if (e != cudaSuccess) {
      fprintf(stderr, "flagcxRmsnormBwdNoAlloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return (int)e;
    }
    gScratchAddr[dev].store(scratch, std::memory_order_release);
  }
  int ctas = rows < FLAGCX_NOALLOC_RMSNORM_MAX_CTAS ? (int)rows : FLAGCX_NOALLOC_RMSNORM_MAX_CTAS;
  if (ctas < 1) ctas = 1;
  bwdKernel<<<ctas, kThreads, 0, s>>>((const bf16 *)g, (const bf16 *)x, (const bf16 *)w, rstd, (bf16 *)dx, scratch, rows,
                                      hidden);
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  reduceKernel<<<(hidden + 255) / 256, 256, 0, s>>>(scratch, (bf16 *)dw, ctas, hidden);
  return (int)cudaGetLastError();
}
