// fused_elementwise.cu -- the memory-bound model kernels that sit between the GEMMs
// of a Llama-shaped decoder: RMSNorm (forward, backward), rotary embedding
// (in place, forward/backward by sign), SwiGLU (forward, backward), softmax
// cross-entropy with the gradient written in place of the logits, and a flat
// AdamW step.  All are sm_100a kernels with 16-byte accesses and fp32 math; each
// reads its operands once and writes its results once.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAException.h>
#include <c10/cuda/CUDAGuard.h>
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <torch/extension.h>

#include <algorithm>
#include <cstdlib>

namespace cg = cooperative_groups;

namespace {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float warpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warpMax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide reductions through shared memory; `red` holds 32 floats.
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
__device__ __forceinline__ float blockMax(float v, float *red) {
  v = warpMax(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : -INFINITY;
  if (threadIdx.x < 32) t = warpMax(t);
  if (threadIdx.x == 0) red[0] = t;
  __syncthreads();
  return red[0];
}

__device__ __forceinline__ uint32_t sharedAddr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Waits for a phase of an mbarrier for at most about one second.
__device__ __forceinline__ bool mbarWaitBounded(uint64_t *bar, uint32_t parity) {
  unsigned long long t0 = 0;
  for (uint32_t it = 0;; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(sharedAddr(bar)), "r"(parity)
        : "memory");
    if (done) return true;
    if ((it & 63) == 63) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > 1000000000ull) return false;
    }
  }
}

// One bulk asynchronous copy global -> this CTA's shared memory, counted on an mbarrier.
// Both addresses and the size are multiples of 16 bytes.
__device__ __forceinline__ void bulkLoad(void *dstShared, const void *src, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   sharedAddr(dstShared)),
               "l"(src), "r"(bytes), "r"(sharedAddr(bar))
               : "memory");
}
__device__ __forceinline__ void mbarInit(uint64_t *bar) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sharedAddr(bar)) : "memory");
}
__device__ __forceinline__ void mbarExpect(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(sharedAddr(bar)), "r"(bytes) : "memory");
}

struct Pack8 {
  uint4 raw;
  __device__ float get(int i) const { return __bfloat162float(((const bf16 *)&raw)[i]); }
  __device__ void set(int i, float v) { ((bf16 *)&raw)[i] = __float2bfloat16_rn(v); }
};

// ---------------------------------------------------------------------------
// RMSNorm: y = x * rstd * w,  rstd = rsqrt(mean(x^2) + eps).  One CTA per row,
// H a multiple of 8; a thread owns packs t, t+blockDim, ...
// ---------------------------------------------------------------------------
template <int MAXP>
__global__ void rmsnormFwd(const bf16 *__restrict__ x, const bf16 *__restrict__ w, bf16 *__restrict__ y,
                           float *__restrict__ rstdOut, int H, float eps) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const uint4 *xr = (const uint4 *)(x + row * H);
  const int nPacks = H / 8;
  Pack8 px[MAXP];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < MAXP; ++k) {
    int p = threadIdx.x + k * blockDim.x;
    if (p < nPacks) {
      px[k].raw = xr[p];
#pragma unroll
      for (int i = 0; i < 8; ++i) { float v = px[k].get(i); ss += v * v; }
    }
  }
  ss = blockSum(ss, red);
  const float rstd = rsqrtf(ss / H + eps);
  if (threadIdx.x == 0) rstdOut[row] = rstd;
  uint4 *yr = (uint4 *)(y + row * H);
#pragma unroll
  for (int k = 0; k < MAXP; ++k) {
    int p = threadIdx.x + k * blockDim.x;
    if (p < nPacks) {
      Pack8 pw, po;
      pw.raw = ((const uint4 *)w)[p];
#pragma unroll
      for (int i = 0; i < 8; ++i) po.set(i, px[k].get(i) * rstd * pw.get(i));
      yr[p] = po.raw;
    }
  }
}

// The same for H <= 4096 with one WARP per row: a lane keeps its share of the row in
// registers (PPL packs of 8), the sum of squares needs shuffles only, and a CTA of eight
// warps has eight rows in flight with no block-wide barrier.
template <int PPL>
__global__ void __launch_bounds__(256)
rmsnormFwdWarp(const bf16 *__restrict__ x, const bf16 *__restrict__ w, bf16 *__restrict__ y, float *__restrict__ rstdOut,
               long rows, int H, float eps) {
  const int lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int nPacks = H / 8;
  const uint4 *xr = (const uint4 *)(x + row * H);
  Pack8 px[PPL];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PPL; ++k) {
    const int p = lane + k * 32;
    if (p < nPacks) {
      px[k].raw = xr[p];
#pragma unroll
      for (int i = 0; i < 8; ++i) { float v = px[k].get(i); ss += v * v; }
    }
  }
  ss = warpSum(ss);
  const float rstd = rsqrtf(ss / H + eps);
  if (lane == 0) rstdOut[row] = rstd;
  uint4 *yr = (uint4 *)(y + row * H);
#pragma unroll
  for (int k = 0; k < PPL; ++k) {
    const int p = lane + k * 32;
    if (p < nPacks) {
      Pack8 pw, po;
      pw.raw = ((const uint4 *)w)[p];
#pragma unroll
      for (int i = 0; i < 8; ++i) po.set(i, px[k].get(i) * rstd * pw.get(i));
      yr[p] = po.raw;
    }
  }
}

// Backward: dx = rstd * (g*w - x * rstd^2 * mean(g*w*x)); the weight gradient is summed
// per CTA in fp32 (thread t owns the same columns for all of its CTA's rows) and the
// partials are added up by columnSumToBf16.
//
// The backward with the rows brought in by the copy engine.  Each persistent CTA owns a
// ring of `stages` slots in shared memory; one thread keeps the ring full with bulk
// asynchronous copies of (g row, x row) that complete on one mbarrier per slot, so several
// rows per CTA are in flight while the 512 threads reduce and write the current one.
constexpr int kNormBwdThreads = 512, kNormBwdMaxStages = 8;

template <int MAXP>
__global__ void __launch_bounds__(kNormBwdThreads)
rmsnormBwdPipelined(const bf16 *__restrict__ g, const bf16 *__restrict__ x, const bf16 *__restrict__ w,
                    const float *__restrict__ rstdIn, const bf16 *__restrict__ addIn, bf16 *__restrict__ dx,
                    float *__restrict__ dwPartial, int rows, int H, int stages) {
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ float red[32];
  __shared__ __align__(8) uint64_t full[kNormBwdMaxStages];
  const int nPacks = H / 8;
  const uint32_t rowBytes = (uint32_t)H * 2u;
  // a slot holds the g row, the x row and, when a gradient of the same shape is to be added
  // to dx (the residual branch around the norm), that gradient's row
  const uint32_t slotBytes = (addIn ? 3u : 2u) * rowBytes;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) mbarInit(&full[s]);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  auto issue = [&](int k) { // thread 0: the row of iteration k into slot k % stages
    const size_t row = blockIdx.x + (size_t)k * gridDim.x;
    if (row >= (size_t)rows) return;
    const int s = k % stages;
    unsigned char *dst = ring + (size_t)s * slotBytes;
    mbarExpect(&full[s], slotBytes);
    bulkLoad(dst, g + row * H, rowBytes, &full[s]);
    bulkLoad(dst + rowBytes, x + row * H, rowBytes, &full[s]);
    if (addIn) bulkLoad(dst + 2 * rowBytes, addIn + row * H, rowBytes, &full[s]);
  };
  if (threadIdx.x == 0)
    for (int k = 0; k < stages; ++k) issue(k);

  float dwAcc[MAXP][8];
  Pack8 pw[MAXP];
#pragma unroll
  for (int k = 0; k < MAXP; ++k) {
    int p = threadIdx.x + k * blockDim.x;
    if (p < nPacks) pw[k].raw = ((const uint4 *)w)[p];
#pragma unroll
    for (int i = 0; i < 8; ++i) dwAcc[k][i] = 0.f;
  }
  bool ok = true;
  int it = 0;
  for (size_t row = blockIdx.x; row < (size_t)rows; row += gridDim.x, ++it) {
    const int s = it % stages;
    const float rstd = rstdIn[row];
    // Every thread goes on through the same barriers whatever its wait returned; a wait
    // that ran out marks this CTA's weight-gradient partial as NaN.
    if (ok) ok = mbarWaitBounded(&full[s], (uint32_t)(it / stages) & 1u);
    const uint4 *gs = (const uint4 *)(ring + (size_t)s * slotBytes), *xs = gs + nPacks, *as = xs + nPacks;
    Pack8 pg[MAXP], px[MAXP], pa[MAXP];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < MAXP; ++k) {
      int p = threadIdx.x + k * blockDim.x;
      if (p < nPacks) {
        pg[k].raw = gs[p];
        px[k].raw = xs[p];
        if (addIn) pa[k].raw = as[p];
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += pg[k].get(i) * pw[k].get(i) * px[k].get(i);
      }
    }
    dot = blockSum(dot, red); // all threads have read the slot once its barriers are passed
    if (threadIdx.x == 0) issue(it + stages);
    const float c = dot * rstd * rstd / H;
    uint4 *dxr = (uint4 *)(dx + row * H);
#pragma unroll
    for (int k = 0; k < MAXP; ++k) {
      int p = threadIdx.x + k * blockDim.x;
      if (p < nPacks) {
        Pack8 po;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float gv = pg[k].get(i), xv = px[k].get(i);
          float d = rstd * (gv * pw[k].get(i) - xv * c);
          if (addIn) d += pa[k].get(i);
          po.set(i, d);
          dwAcc[k][i] += gv * xv * rstd;
        }
        dxr[p] = po.raw;
      }
    }
  }
  float *out = dwPartial + (size_t)blockIdx.x * H;
  const float bad = ok ? 0.f : NAN;
#pragma unroll
  for (int k = 0; k < MAXP; ++k) {
    int p = threadIdx.x + k * blockDim.x;
    if (p < nPacks) {
      *(float4 *)(out + p * 8) = make_float4(dwAcc[k][0] + bad, dwAcc[k][1] + bad, dwAcc[k][2] + bad, dwAcc[k][3] + bad);
      *(float4 *)(out + p * 8 + 4) = make_float4(dwAcc[k][4] + bad, dwAcc[k][5] + bad, dwAcc[k][6] + bad, dwAcc[k][7] + bad);
    }
  }
}

// dw[c] = sum over the CTAs' partials, in a fixed order, rounded to bf16 once.
// Block (32, 32): 32 neighbouring columns, 32 lanes over the rows.
__global__ void columnSumToBf16(const float *__restrict__ partial, bf16 *__restrict__ dw, int R, int H) {
  __shared__ float tile[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float acc = 0.f;
  if (c < H)
    for (int r = threadIdx.y; r < R; r += 32) acc += partial[(size_t)r * H + c];
  tile[threadIdx.y][threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.y == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) t += tile[i][threadIdx.x];
    dw[c] = __float2bfloat16_rn(t);
  }
}

// ---------------------------------------------------------------------------
// Rotary embedding, in place, half-split layout: for a head of dimension D,
// (x[i], x[i+D/2]) is rotated by angle pos * theta^(-2i/D).  sign=-1 is the backward.
// x: [tokens, heads, D]; one thread per pair of 8-element packs.
// ---------------------------------------------------------------------------
__global__ void ropeKernel(bf16 *__restrict__ x, const int *__restrict__ positions, int tokens, int heads, int D,
                           float logTheta, float sign) {
  const int half = D / 2, packsPerHalf = half / 8;
  const size_t total = (size_t)tokens * heads * packsPerHalf;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    int pk = idx % packsPerHalf;
    size_t th = idx / packsPerHalf;
    int tok = th / heads;
    float pos = positions ? (float)positions[tok] : (float)tok;
    bf16 *base = x + th * D;
    Pack8 a, b, oa, ob;
    a.raw = *(uint4 *)(base + pk * 8);
    b.raw = *(uint4 *)(base + half + pk * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      int d = pk * 8 + i;
      float inv = __expf(-logTheta * (2.0f * d / D));
      float s, c;
      sincosf(pos * inv, &s, &c);
      s *= sign;
      float x1 = a.get(i), x2 = b.get(i);
      oa.set(i, x1 * c - x2 * s);
      ob.set(i, x2 * c + x1 * s);
    }
    *(uint4 *)(base + pk * 8) = oa.raw;
    *(uint4 *)(base + half + pk * 8) = ob.raw;
  }
}

// The same rotation applied to a fused projection [tokens, totalHeads, D] whose first
// ropeHeads heads (queries, then keys) are rotated and whose other heads (values) are
// copied through: one pass that reads src once and writes dst once, so the model needs no
// separate q / k copies before or after the rotation.
__global__ void ropeFusedQkv(const bf16 *__restrict__ src, bf16 *__restrict__ dst, int tokens, int ropeHeads,
                             int totalHeads, int D, float logTheta, float sign) {
  const int half = D / 2, packsPerHalf = half / 8;
  const size_t total = (size_t)tokens * totalHeads * packsPerHalf;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int pk = idx % packsPerHalf;
    const size_t th = idx / packsPerHalf;
    const int head = th % totalHeads;
    const int tok = th / totalHeads;
    const bf16 *in = src + th * D;
    bf16 *out = dst + th * D;
    Pack8 a, b, oa, ob;
    a.raw = *(const uint4 *)(in + pk * 8);
    b.raw = *(const uint4 *)(in + half + pk * 8);
    if (head < ropeHeads) {
      const float pos = (float)tok;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int d = pk * 8 + i;
        const float inv = __expf(-logTheta * (2.0f * d / D));
        float s, c;
        sincosf(pos * inv, &s, &c);
        s *= sign;
        const float x1 = a.get(i), x2 = b.get(i);
        oa.set(i, x1 * c - x2 * s);
        ob.set(i, x2 * c + x1 * s);
      }
    } else {
      oa = a;
      ob = b;
    }
    *(uint4 *)(out + pk * 8) = oa.raw;
    *(uint4 *)(out + half + pk * 8) = ob.raw;
  }
}

// ---------------------------------------------------------------------------
// SwiGLU on a fused projection ab = [a | b] of shape [T, 2F]: out = silu(a) * b.
// ---------------------------------------------------------------------------
__global__ void swigluFwd(const bf16 *__restrict__ ab, bf16 *__restrict__ out, size_t T, int F) {
  const int packs = F / 8;
  const size_t total = T * packs;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    size_t t = idx / packs;
    int p = idx % packs;
    Pack8 a, b, o;
    a.raw = *(const uint4 *)(ab + t * 2 * F + p * 8);
    b.raw = *(const uint4 *)(ab + t * 2 * F + F + p * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float av = a.get(i);
      o.set(i, av / (1.f + __expf(-av)) * b.get(i));
    }
    *(uint4 *)(out + t * F + p * 8) = o.raw;
  }
}

__global__ void swigluBwd(const bf16 *__restrict__ g, const bf16 *__restrict__ ab, bf16 *__restrict__ dab, size_t T,
                          int F) {
  const int packs = F / 8;
  const size_t total = T * packs;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    size_t t = idx / packs;
    int p = idx % packs;
    Pack8 a, b, gg, da, db;
    a.raw = *(const uint4 *)(ab + t * 2 * F + p * 8);
    b.raw = *(const uint4 *)(ab + t * 2 * F + F + p * 8);
    gg.raw = *(const uint4 *)(g + t * F + p * 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float av = a.get(i), bv = b.get(i), gv = gg.get(i);
      float sig = 1.f / (1.f + __expf(-av));
      float silu = av * sig;
      da.set(i, gv * bv * (sig + silu * (1.f - sig)));
      db.set(i, gv * silu);
    }
    *(uint4 *)(dab + t * 2 * F + p * 8) = da.raw;
    *(uint4 *)(dab + t * 2 * F + F + p * 8) = db.raw;
  }
}

// ---------------------------------------------------------------------------
// Softmax cross-entropy, one CTA per row.  Writes the per-row loss and overwrites
// the logits with gradScale * (softmax - onehot): the [T, V] tensor is read three
// times out of L2 and written once; no fp32 copy of the logits is ever made.
// ---------------------------------------------------------------------------
__global__ void crossEntropyFwdBwd(bf16 *__restrict__ logits, const long *__restrict__ targets,
                                   float *__restrict__ loss, int V, float gradScale) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  bf16 *lr = logits + row * V;
  const int packs = V / 8; // V a multiple of 8
  float mx = -INFINITY;
  for (int p = threadIdx.x; p < packs; p += blockDim.x) {
    Pack8 v;
    v.raw = ((const uint4 *)lr)[p];
#pragma unroll
    for (int i = 0; i < 8; ++i) mx = fmaxf(mx, v.get(i));
  }
  mx = blockMax(mx, red);
  float sum = 0.f;
  for (int p = threadIdx.x; p < packs; p += blockDim.x) {
    Pack8 v;
    v.raw = ((const uint4 *)lr)[p];
#pragma unroll
    for (int i = 0; i < 8; ++i) sum += __expf(v.get(i) - mx);
  }
  sum = blockSum(sum, red);
  const long tgt = targets[row];
  const float lse = mx + __logf(sum);
  if (threadIdx.x == 0) loss[row] = lse - __bfloat162float(lr[tgt]);
  __syncthreads(); // the target logit was read before anybody overwrites it
  const float inv = 1.f / sum;
  for (int p = threadIdx.x; p < packs; p += blockDim.x) {
    Pack8 v, o;
    v.raw = ((const uint4 *)lr)[p];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float pr = __expf(v.get(i) - mx) * inv;
      if ((long)p * 8 + i == tgt) pr -= 1.f;
      o.set(i, pr * gradScale);
    }
    ((uint4 *)lr)[p] = o.raw;
  }
}

// ---------------------------------------------------------------------------
// The same operation with the row held on chip.  A thread-block cluster of C CTAs
// owns one row; each CTA brings its 1/C of the row into shared memory with one
// bulk asynchronous copy, finds its own maximum and sum of exponentials (the
// exponentials replace the logits in shared memory, as bf16), trades (max, sum)
// with the other CTAs of the cluster through distributed shared memory, scales
// its exponentials into gradients and sends them back with one bulk store.  The
// [T, V] tensor crosses L2/HBM once in each direction and every element costs one
// exponential instead of two.
// ---------------------------------------------------------------------------
constexpr int kCeMaxThreads = 1024;
constexpr uint32_t kCeBulkPiece = 32768;

__global__ void __launch_bounds__(kCeMaxThreads)
crossEntropyCluster(bf16 *__restrict__ logits, const long *__restrict__ targets, float *__restrict__ loss, int V,
                    float gradScale, int packsPerCta) {
  extern __shared__ __align__(128) unsigned char ceRow[];
  __shared__ float red[32];
  __shared__ float stat[2];
  __shared__ __align__(8) uint64_t bar;
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned C = cluster.num_blocks(), cr = cluster.block_rank();
  const size_t row = blockIdx.x / C;
  const int packs = V / 8, p0 = (int)cr * packsPerCta;
  const int n = max(0, min(packsPerCta, packs - p0));
  unsigned char *gRow = (unsigned char *)(logits + row * V + (size_t)p0 * 8);
  uint4 *buf = (uint4 *)ceRow;
  const uint32_t bytes = (uint32_t)n * 16u;

  if (threadIdx.x == 0) {
    mbarInit(&bar);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  bool ok = true;
  if (n > 0) {
    if (threadIdx.x == 0) {
      mbarExpect(&bar, bytes);
      for (uint32_t off = 0; off < bytes; off += kCeBulkPiece) bulkLoad(ceRow + off, gRow + off, min(kCeBulkPiece, bytes - off), &bar);
    }
    ok = mbarWaitBounded(&bar, 0);
  }

  const long tLocal = targets[row] - (long)p0 * 8; // index of the target inside this CTA's part, if it is here
  const bool own = tLocal >= 0 && tLocal < (long)n * 8;
  const float tgtLogit = own ? __bfloat162float(((const bf16 *)ceRow)[tLocal]) : 0.f;
  // maximum: on packed bf16 pairs, no conversion
  __nv_bfloat162 m2 = __float2bfloat162_rn(-INFINITY);
  for (int p = threadIdx.x; p < n; p += (int)blockDim.x) {
    const uint4 v = buf[p];
    const __nv_bfloat162 *h = (const __nv_bfloat162 *)&v;
    m2 = __hmax2(m2, __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3])));
  }
  float mx = fmaxf(__low2float(m2), __high2float(m2));
  mx = blockMax(mx, red); // its barriers also order the read of the target logit before the overwrite below
  // exponentials: 2^(v*log2e - mx*log2e), one FMA and one MUFU each
  constexpr float kLog2e = 1.4426950408889634f;
  const float mxs = mx * kLog2e;
  float sum = 0.f;
  for (int p = threadIdx.x; p < n; p += (int)blockDim.x) {
    const uint4 v = buf[p];
    uint4 e;
    const __nv_bfloat162 *h = (const __nv_bfloat162 *)&v;
    __nv_bfloat162 *eo = (__nv_bfloat162 *)&e;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h[i]);
      const float e0 = exp2f(fmaf(f.x, kLog2e, -mxs)), e1 = exp2f(fmaf(f.y, kLog2e, -mxs));
      sum += e0 + e1;
      eo[i] = __floats2bfloat162_rn(e0, e1);
    }
    buf[p] = e;
  }
  sum = blockSum(sum, red);
  if (threadIdx.x == 0) {
    stat[0] = mx;
    stat[1] = ok ? sum : NAN; // a copy that never arrived poisons the whole row's loss and gradient
  }
  cluster.sync();
  float M = -INFINITY, S = 0.f;
  for (unsigned r = 0; r < C; ++r) M = fmaxf(M, cluster.map_shared_rank(stat, r)[0]);
  for (unsigned r = 0; r < C; ++r) {
    const float *rs = cluster.map_shared_rank(stat, r);
    const float si = rs[1];
    if (si != 0.f) S += si * __expf(rs[0] - M);
  }
  if (own && threadIdx.x == 0) loss[row] = M + __logf(S) - tgtLogit;
  const float f = n > 0 ? __expf(mx - M) / S * gradScale : 0.f;
  for (int p = threadIdx.x; p < n; p += (int)blockDim.x) {
    const uint4 e = buf[p];
    uint4 o;
    const __nv_bfloat162 *h = (const __nv_bfloat162 *)&e;
    __nv_bfloat162 *oo = (__nv_bfloat162 *)&o;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 v = __bfloat1622float2(h[i]);
      oo[i] = __floats2bfloat162_rn(v.x * f, v.y * f);
    }
    buf[p] = o;
  }
  // the one element that is softmax - 1, redone in fp32 by the thread that wrote its pack
  if (own && threadIdx.x == (int)((tLocal >> 3) % blockDim.x))
    ((bf16 *)ceRow)[tLocal] = __float2bfloat16_rn(exp2f(fmaf(tgtLogit, kLog2e, -mxs)) * f - gradScale);
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the stores above, before the engine reads them
  __syncthreads();
  if (threadIdx.x == 0 && n > 0 && ok) {
    for (uint32_t off = 0; off < bytes; off += kCeBulkPiece) {
      const uint32_t sz = min(kCeBulkPiece, bytes - off);
      asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gRow + off),
                   "r"(sharedAddr(ceRow + off)), "r"(sz)
                   : "memory");
    }
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
  }
  cluster.sync(); // no CTA leaves while another may still read its (max, sum)
}

// ---------------------------------------------------------------------------
// AdamW on flat bf16 tensors (parameters, gradients, both moments), fp32 math.
// ---------------------------------------------------------------------------
__global__ void adamwFlat(bf16 *__restrict__ p, const bf16 *__restrict__ g, bf16 *__restrict__ m, bf16 *__restrict__ v,
                          size_t n, float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2) {
  const size_t packs = n / 8;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < packs; idx += (size_t)gridDim.x * blockDim.x) {
    Pack8 pp, pg, pm, pv;
    pp.raw = ((const uint4 *)p)[idx];
    pg.raw = ((const uint4 *)g)[idx];
    pm.raw = ((const uint4 *)m)[idx];
    pv.raw = ((const uint4 *)v)[idx];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float gv = pg.get(i), mv = pm.get(i), vv = pv.get(i), pw = pp.get(i);
      mv = beta1 * mv + (1.f - beta1) * gv;
      vv = beta2 * vv + (1.f - beta2) * gv * gv;
      float upd = (mv / bc1) / (sqrtf(vv / bc2) + eps);
      pw = pw * (1.f - lr * wd) - lr * upd;
      pp.set(i, pw); pm.set(i, mv); pv.set(i, vv);
    }
    ((uint4 *)p)[idx] = pp.raw;
    ((uint4 *)m)[idx] = pm.raw;
    ((uint4 *)v)[idx] = pv.raw;
  }
  // tail (n not a multiple of 8)
  size_t tail = packs * 8 + blockIdx.x * (size_t)blockDim.x + threadIdx.x;
  if (tail < n) {
    float gv = __bfloat162float(g[tail]), mv = __bfloat162float(m[tail]), vv = __bfloat162float(v[tail]);
    float pw = __bfloat162float(p[tail]);
    mv = beta1 * mv + (1.f - beta1) * gv;
    vv = beta2 * vv + (1.f - beta2) * gv * gv;
    pw = pw * (1.f - lr * wd) - lr * (mv / bc1) / (sqrtf(vv / bc2) + eps);
    p[tail] = __float2bfloat16_rn(pw);
    m[tail] = __float2bfloat16_rn(mv);
    v[tail] = __float2bfloat16_rn(vv);
  }
}

// ---------------------------------------------------------------------------
// host wrappers
// ---------------------------------------------------------------------------
void checkBf16(const at::Tensor &t, const char *name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous(), name,
              " must be a contiguous CUDA bfloat16 tensor");
  TORCH_CHECK(((uintptr_t)t.data_ptr() & 15) == 0, name, " must be 16-byte aligned");
}

int gridFor(size_t items, int threads, int perSm = 8) {
  int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  size_t want = (items + threads - 1) / threads;
  return (int)std::max<size_t>(1, std::min<size_t>(want, (size_t)sms * perSm));
}

std::vector<at::Tensor> rmsnorm_fwd(const at::Tensor &x, const at::Tensor &w, double eps) {
  checkBf16(x, "x");
  checkBf16(w, "weight");
  const int H = (int)x.size(-1);
  TORCH_CHECK(H % 8 == 0 && H <= 8 * 512 * 4 && w.numel() == H, "rmsnorm: hidden size must be a multiple of 8, at most 16384");
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.numel() / H;
  auto y = at::empty_like(x);
  auto rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  auto stream = at::cuda::getCurrentCUDAStream();
  const int threads = 512, packs = H / 8;
  const int maxp = (packs + threads - 1) / threads;
  auto launch = [&](auto tag) {
    rmsnormFwd<decltype(tag)::value><<<(unsigned)rows, threads, 0, stream>>>(
        (const bf16 *)x.data_ptr(), (const bf16 *)w.data_ptr(), (bf16 *)y.data_ptr(), rstd.data_ptr<float>(), H, (float)eps);
  };
  auto launchWarp = [&](auto tag) { // one warp per row, eight rows per CTA
    rmsnormFwdWarp<decltype(tag)::value><<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(
        (const bf16 *)x.data_ptr(), (const bf16 *)w.data_ptr(), (bf16 *)y.data_ptr(), rstd.data_ptr<float>(), (long)rows, H,
        (float)eps);
  };
  if (rows > 0) {
    if (packs <= 32 * 4) launchWarp(std::integral_constant<int, 4>());
    else if (packs <= 32 * 8) launchWarp(std::integral_constant<int, 8>());
    else if (packs <= 32 * 16) launchWarp(std::integral_constant<int, 16>());
    else if (maxp <= 1) launch(std::integral_constant<int, 1>());
    else if (maxp <= 2) launch(std::integral_constant<int, 2>());
    else launch(std::integral_constant<int, 4>());
    C10_CUDA_KERNEL_LAUNCH_CHECK();
  }
  return {y, rstd};
}

// `add`, when given, has x's shape and is added to dx inside the kernel (the gradient that
// reaches x through a residual connection around the norm).
std::vector<at::Tensor> rmsnorm_bwd(const at::Tensor &g, const at::Tensor &x, const at::Tensor &w,
                                    const at::Tensor &rstd, const c10::optional<at::Tensor> &add) {
  checkBf16(g, "grad");
  if (add.has_value()) {
    checkBf16(*add, "add");
    TORCH_CHECK(add->numel() == x.numel(), "rmsnorm_bwd: `add` must have x's shape");
  }
  checkBf16(x, "x");
  checkBf16(w, "weight");
  const int H = (int)x.size(-1);
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.numel() / H;
  auto dx = at::empty_like(x);
  TORCH_CHECK(H % 8 == 0 && H <= 8 * 512 * 4 && w.numel() == H, "rmsnorm: hidden size must be a multiple of 8, at most 16384");
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int ctas = (int)std::max<int64_t>(1, std::min<int64_t>(rows, sms * 2));
  auto partial = at::empty({ctas, H}, x.options().dtype(at::kFloat));
  auto dw = at::empty({H}, x.options());
  auto stream = at::cuda::getCurrentCUDAStream();
  const int packs = H / 8;
  const int maxp = (packs + kNormBwdThreads - 1) / kNormBwdThreads;
  // ring of (g row, x row) slots: about 96 KiB per CTA so that two CTAs share an SM
  const size_t slot = (size_t)H * (add.has_value() ? 6 : 4);
  const int stages = (int)std::max<size_t>(2, std::min<size_t>(kNormBwdMaxStages, ((size_t)96 << 10) / slot));
  const size_t smem = slot * stages;
  auto launch = [&](auto tag) {
    auto kern = rmsnormBwdPipelined<decltype(tag)::value>;
    C10_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<ctas, kNormBwdThreads, smem, stream>>>((const bf16 *)g.data_ptr(), (const bf16 *)x.data_ptr(),
                                                  (const bf16 *)w.data_ptr(), rstd.data_ptr<float>(),
                                                  add.has_value() ? (const bf16 *)add->data_ptr() : nullptr,
                                                  (bf16 *)dx.data_ptr(), partial.data_ptr<float>(), (int)rows, H, stages);
  };
  if (rows == 0) {
    dw.zero_();
    return {dx, dw};
  }
  TORCH_CHECK(smem <= ((size_t)200 << 10), "rmsnorm_bwd: hidden size too large for the shared-memory ring");
  if (maxp <= 1) launch(std::integral_constant<int, 1>());
  else if (maxp <= 2) launch(std::integral_constant<int, 2>());
  else launch(std::integral_constant<int, 4>());
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  columnSumToBf16<<<(H + 31) / 32, dim3(32, 32), 0, stream>>>(partial.data_ptr<float>(), (bf16 *)dw.data_ptr(), ctas, H);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return {dx, dw};
}

void rope_inplace(at::Tensor &x, const c10::optional<at::Tensor> &positions, double theta, bool backward) {
  checkBf16(x, "x");
  TORCH_CHECK(x.dim() >= 3, "rope: expected [..., heads, head_dim]");
  const int D = (int)x.size(-1), heads = (int)x.size(-2);
  TORCH_CHECK(D % 16 == 0, "rope: head_dim must be a multiple of 16");
  const int64_t tokens = x.numel() / ((int64_t)D * heads);
  const int *pos = nullptr;
  if (positions.has_value()) {
    TORCH_CHECK(positions->scalar_type() == at::kInt && positions->numel() == tokens && positions->is_cuda(), "rope: bad positions");
    pos = positions->data_ptr<int>();
  }
  const c10::cuda::CUDAGuard guard(x.device());
  size_t items = (size_t)tokens * heads * (D / 16);
  ropeKernel<<<gridFor(items, 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (bf16 *)x.data_ptr(), pos, (int)tokens, heads, D, logf((float)theta), backward ? -1.f : 1.f);
}

// qkv: [tokens, (ropeHeads + otherHeads) * D]; returns a new tensor of the same shape.
at::Tensor rope_fused_qkv(const at::Tensor &qkv, int64_t ropeHeads, int64_t totalHeads, int64_t D, double theta,
                          bool backward) {
  checkBf16(qkv, "qkv");
  TORCH_CHECK(D % 16 == 0 && qkv.size(-1) == totalHeads * D && ropeHeads <= totalHeads, "rope_fused_qkv: bad shape");
  const int64_t tokens = qkv.numel() / (totalHeads * D);
  const c10::cuda::CUDAGuard guard(qkv.device());
  auto out = at::empty_like(qkv);
  if (qkv.numel() == 0) return out;
  size_t items = (size_t)tokens * totalHeads * (D / 16);
  ropeFusedQkv<<<gridFor(items, 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const bf16 *)qkv.data_ptr(), (bf16 *)out.data_ptr(), (int)tokens, (int)ropeHeads, (int)totalHeads, (int)D,
      logf((float)theta), backward ? -1.f : 1.f);
  C10_CUDA_KERNEL_LAUNCH_CHECK();
  return out;
}

at::Tensor swiglu_fwd(const at::Tensor &ab) {
  checkBf16(ab, "ab");
  const int F = (int)ab.size(-1) / 2;
  TORCH_CHECK(F % 8 == 0, "swiglu: width must be a multiple of 8");
  const c10::cuda::CUDAGuard guard(ab.device());
  auto sizes = ab.sizes().vec();
  sizes.back() = F;
  auto out = at::empty(sizes, ab.options());
  size_t T = ab.numel() / (2 * (size_t)F);
  swigluFwd<<<gridFor(T * (F / 8), 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>((const bf16 *)ab.data_ptr(),
                                                                                    (bf16 *)out.data_ptr(), T, F);
  return out;
}

at::Tensor swiglu_bwd(const at::Tensor &g, const at::Tensor &ab) {
  checkBf16(g, "grad");
  checkBf16(ab, "ab");
  const int F = (int)ab.size(-1) / 2;
  const c10::cuda::CUDAGuard guard(ab.device());
  auto dab = at::empty_like(ab);
  size_t T = ab.numel() / (2 * (size_t)F);
  swigluBwd<<<gridFor(T * (F / 8), 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (const bf16 *)g.data_ptr(), (const bf16 *)ab.data_ptr(), (bf16 *)dab.data_ptr(), T, F);
  return dab;
}

// Returns per-row losses; `logits` now holds gradScale * dLoss/dlogits.
at::Tensor cross_entropy_fwd_bwd_(at::Tensor &logits, const at::Tensor &targets, double gradScale) {
  checkBf16(logits, "logits");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous(), "targets must be int64 CUDA");
  const int V = (int)logits.size(-1);
  TORCH_CHECK(V % 8 == 0, "cross-entropy: vocabulary must be a multiple of 8");
  const int64_t rows = logits.numel() / V;
  TORCH_CHECK(targets.numel() == rows, "cross-entropy: one target per row");
  const c10::cuda::CUDAGuard guard(logits.device());
  auto loss = at::empty({rows}, logits.options().dtype(at::kFloat));
  if (rows == 0) return loss;
  auto stream = at::cuda::getCurrentCUDAStream();
  // Smallest cluster whose per-CTA part of a row fits beside two other CTAs on the SM
  // (72 KiB each); failing that, one CTA per SM with up to 200 KiB; failing that, the
  // kernel that streams the row three times.
  const int packs = V / 8;
  int cluster = 0, per = 0;
  static const size_t partKb = std::getenv("FLAGCX_OPS_CE_PART_KB") ? (size_t)atoi(std::getenv("FLAGCX_OPS_CE_PART_KB")) : 72;
  for (size_t limit : {partKb << 10, (size_t)200 << 10}) {
    for (int c : {1, 2, 4, 8}) {
      per = (packs + c - 1) / c;
      if ((size_t)per * 16 <= limit) { cluster = c; break; }
    }
    if (cluster) break;
  }
  static const bool forceStreaming = std::getenv("FLAGCX_OPS_CE_STREAMING") && atoi(std::getenv("FLAGCX_OPS_CE_STREAMING")) != 0;
  if (!cluster || forceStreaming || rows * cluster > 0x7fffffffLL) {
    crossEntropyFwdBwd<<<(unsigned)rows, 1024, 0, stream>>>((bf16 *)logits.data_ptr(), targets.data_ptr<long>(),
                                                            loss.data_ptr<float>(), V, (float)gradScale);
    C10_CUDA_KERNEL_LAUNCH_CHECK();
    return loss;
  }
  const size_t smem = (size_t)per * 16;
  C10_CUDA_CHECK(cudaFuncSetAttribute(crossEntropyCluster, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(rows * cluster));
  static const int ceThreads = std::getenv("FLAGCX_OPS_CE_THREADS") ? std::min(kCeMaxThreads, std::max(32, atoi(std::getenv("FLAGCX_OPS_CE_THREADS")) / 32 * 32)) : 256;
  cfg.blockDim = dim3(ceThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  C10_CUDA_CHECK(cudaLaunchKernelEx(&cfg, crossEntropyCluster, (bf16 *)logits.data_ptr(), (const long *)targets.data_ptr<long>(),
                                    loss.data_ptr<float>(), V, (float)gradScale, per));
  return loss;
}

void adamw_flat_(at::Tensor &p, const at::Tensor &g, at::Tensor &m, at::Tensor &v, double lr, double beta1, double beta2,
                 double eps, double wd, int64_t step) {
  checkBf16(p, "param");
  checkBf16(g, "grad");
  checkBf16(m, "exp_avg");
  checkBf16(v, "exp_avg_sq");
  TORCH_CHECK(p.numel() == g.numel() && p.numel() == m.numel() && p.numel() == v.numel(), "adamw: size mismatch");
  const c10::cuda::CUDAGuard guard(p.device());
  const size_t n = p.numel();
  if (n == 0) return;
  float bc1 = 1.f - (float)std::pow(beta1, (double)step), bc2 = 1.f - (float)std::pow(beta2, (double)step);
  adamwFlat<<<gridFor(n / 8 + 8, 256), 256, 0, at::cuda::getCurrentCUDAStream()>>>(
      (bf16 *)p.data_ptr(), (const bf16 *)g.data_ptr(), (bf16 *)m.data_ptr(), (bf16 *)v.data_ptr(), n, (float)lr,
      (float)beta1, (float)beta2, (float)eps, (float)wd, bc1, bc2);
}

} // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("g"), py::arg("x"), py::arg("w"), py::arg("rstd"), py::arg("add") = py::none());
  m.def("rope_inplace", &rope_inplace);
  m.def("rope_fused_qkv", &rope_fused_qkv);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("cross_entropy_fwd_bwd_", &cross_entropy_fwd_bwd_);
  m.def("adamw_flat_", &adamw_flat_);
}
