// fused_elementwise.cu -- the memory-bound model kernels that sit between the GEMMs
// of a Llama-shaped decoder: RMSNorm (forward, backward), rotary embedding
// (in place, forward/backward by sign), SwiGLU (forward, backward), softmax
// cross-entropy with the gradient written in place of the logits, and a flat
// AdamW step.  All are sm_100a kernels with 16-byte accesses and fp32 math; each
// reads its operands once and writes its results once.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_bf16.h>
#include <torch/extension.h>

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

// dx = rstd * (g*w - x * rstd^2 * mean(g*w*x));  dw partial per CTA (fp32).
// CTA b handles rows b, b+grid, ...; thread t owns the same columns for all rows.
template <int MAXP>
__global__ void rmsnormBwd(const bf16 *__restrict__ g, const bf16 *__restrict__ x, const bf16 *__restrict__ w,
                           const float *__restrict__ rstdIn, bf16 *__restrict__ dx, float *__restrict__ dwPartial,
                           int rows, int H) {
  __shared__ float red[32];
  const int nPacks = H / 8;
  float dwAcc[MAXP][8];
  Pack8 pw[MAXP];
#pragma unroll
  for (int k = 0; k < MAXP; ++k) {
    int p = threadIdx.x + k * blockDim.x;
    if (p < nPacks) pw[k].raw = ((const uint4 *)w)[p];
#pragma unroll
    for (int i = 0; i < 8; ++i) dwAcc[k][i] = 0.f;
  }
  for (size_t row = blockIdx.x; row < (size_t)rows; row += gridDim.x) {
    const uint4 *gr = (const uint4 *)(g + row * H), *xr = (const uint4 *)(x + row * H);
    const float rstd = rstdIn[row];
    Pack8 pg[MAXP], px[MAXP];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < MAXP; ++k) {
      int p = threadIdx.x + k * blockDim.x;
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
    for (int k = 0; k < MAXP; ++k) {
      int p = threadIdx.x + k * blockDim.x;
      if (p < nPacks) {
        Pack8 po;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float gv = pg[k].get(i), xv = px[k].get(i);
          po.set(i, rstd * (gv * pw[k].get(i) - xv * c));
          dwAcc[k][i] += gv * xv * rstd;
        }
        dxr[p] = po.raw;
      }
    }
  }
  float *out = dwPartial + (size_t)blockIdx.x * H;
#pragma unroll
  for (int k = 0; k < MAXP; ++k) {
    int p = threadIdx.x + k * blockDim.x;
    if (p < nPacks) {
      *(float4 *)(out + p * 8) = make_float4(dwAcc[k][0], dwAcc[k][1], dwAcc[k][2], dwAcc[k][3]);
      *(float4 *)(out + p * 8 + 4) = make_float4(dwAcc[k][4], dwAcc[k][5], dwAcc[k][6], dwAcc[k][7]);
    }
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
  if (rows > 0) {
    if (maxp <= 1) launch(std::integral_constant<int, 1>());
    else if (maxp <= 2) launch(std::integral_constant<int, 2>());
    else launch(std::integral_constant<int, 4>());
  }
  return {y, rstd};
}

std::vector<at::Tensor> rmsnorm_bwd(const at::Tensor &g, const at::Tensor &x, const at::Tensor &w,
                                    const at::Tensor &rstd) {
  checkBf16(g, "grad");
  checkBf16(x, "x");
  checkBf16(w, "weight");
  const int H = (int)x.size(-1);
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.numel() / H;
  auto dx = at::empty_like(x);
  const int sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  const int ctas = (int)std::max<int64_t>(1, std::min<int64_t>(rows, sms * 2));
  auto partial = at::empty({ctas, H}, x.options().dtype(at::kFloat));
  auto stream = at::cuda::getCurrentCUDAStream();
  const int threads = 512, packs = H / 8;
  const int maxp = (packs + threads - 1) / threads;
  auto launch = [&](auto tag) {
    rmsnormBwd<decltype(tag)::value><<<ctas, threads, 0, stream>>>(
        (const bf16 *)g.data_ptr(), (const bf16 *)x.data_ptr(), (const bf16 *)w.data_ptr(), rstd.data_ptr<float>(),
        (bf16 *)dx.data_ptr(), partial.data_ptr<float>(), (int)rows, H);
  };
  if (maxp <= 1) launch(std::integral_constant<int, 1>());
  else if (maxp <= 2) launch(std::integral_constant<int, 2>());
  else launch(std::integral_constant<int, 4>());
  auto dw = partial.sum(0).to(at::kBFloat16);
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
  if (rows > 0)
    crossEntropyFwdBwd<<<(unsigned)rows, 1024, 0, at::cuda::getCurrentCUDAStream()>>>(
        (bf16 *)logits.data_ptr(), targets.data_ptr<long>(), loss.data_ptr<float>(), V, (float)gradScale);
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
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rope_inplace", &rope_inplace);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("cross_entropy_fwd_bwd_", &cross_entropy_fwd_bwd_);
  m.def("adamw_flat_", &adamw_flat_);
}
