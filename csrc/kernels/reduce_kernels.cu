// reduce_kernels.cu -- the reducing collectives: one-shot and two-shot all-reduce (with
// the casting variant), reduce-scatter, reduce to a root, and the ring flavours.
//
// Every collective of the device path is ONE kernel launch per rank.  The kernel
// reads and writes the other ranks' buffers directly through their NVLink peer
// mappings; ranks meet only at per-CTA barriers made of release/acquire flags in
// peer memory (flagcx_device.cuh).  The adjacent element-wise work -- scaling
// (average, 1/world), bf16<->fp32 conversion of the result, a residual add -- is
// applied to the accumulator in registers before the single store.
//
// These kernels take the place of the FlagCX custom all-reduce kernels
// (flagcx/adaptor/kernel/nvidia/custom_allreduce.cu:337-467 in the FlagCX project:
// one-shot peer reduce, NVLS one-shot and NVLS two-shot) and of the reducing NCCL calls of
// its NCCL adaptor (flagcx/adaptor/ccl/nccl_adaptor.cc:228-382).  Differences:
// 16-byte accesses, fp32 accumulation in a fixed rank order (all ranks get
// bit-identical results), no staging copy when the buffers are reachable, no
// size cap, all reductions and element types, and waits that give up with an
// error status instead of spinning forever.
#include "coll_common.cuh"

namespace fcx {
namespace {

// ---------------------------------------------------------------------------
// reduce family
// ---------------------------------------------------------------------------
template <typename T, int OP, int NR>
struct Reducer {
  using Acc = typename Elem<T>::Acc;
  static constexpr int N = 16 / (int)sizeof(T);

  // Reduces the 16-byte pack at byte offset `off` of every rank's input, always in
  // rank order 0..n-1 so that every rank computes bit-identical sums.
  static __device__ __forceinline__ void loadReduce(const CollArgs &a, int nRanks, size_t off, Acc (&acc)[N]) {
    uint4 v[FLAGCX_MAX_RANKS];
    if (NR > 0) {
#pragma unroll
      for (int p = 0; p < NR; ++p) v[p] = ldSys16(a.in[p] + off);
    } else {
#pragma unroll
      for (int p = 0; p < FLAGCX_MAX_RANKS; ++p)
        if (p < nRanks) v[p] = ldSys16(a.in[p] + off);
    }
    const T *e0 = (const T *)&v[0];
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = toAcc<T>(e0[i]);
#pragma unroll
    for (int p = 1; p < (NR > 0 ? NR : FLAGCX_MAX_RANKS); ++p) {
      if (NR > 0 || p < nRanks) {
        const T *e = (const T *)&v[p];
#pragma unroll
        for (int i = 0; i < N; ++i) acc[i] = combine<OP, Acc>(acc[i], toAcc<T>(e[i]), a.redOp);
      }
    }
  }

  // Applies the epilogue and stores one pack at element index `e` (relative to
  // each destination base) to nDst destinations.
  static __device__ __forceinline__ void storePack(const CollArgs &a, char *const *dst, int nDst, size_t e,
                                                   Acc (&acc)[N]) {
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = finish<Acc>(acc[i], a.scale, a.divisor);
    if constexpr (sizeof(T) == 2) {
      if (a.outMode == kOutFloat) { // 8 x 16-bit in, 8 x fp32 out
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = (float)acc[i];
        if (a.residual) {
          const float *r = (const float *)a.residual + e;
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] += r[i];
        }
        for (int d = 0; d < nDst; ++d) {
          float *o = (float *)dst[d] + e;
          st16(o, *(uint4 *)&f[0]);
          st16(o + 4, *(uint4 *)&f[4]);
        }
        return;
      }
    }
    if constexpr (sizeof(T) == 4) {
      if (a.outMode == kOutBf16) { // 4 x fp32 in, 4 x bf16 out
        __align__(8) __nv_bfloat16 h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float x = (float)acc[i];
          if (a.residual) x += __bfloat162float(((const __nv_bfloat16 *)a.residual)[e + i]);
          h[i] = __float2bfloat16_rn(x);
        }
        for (int d = 0; d < nDst; ++d) *(uint2 *)((__nv_bfloat16 *)dst[d] + e) = *(uint2 *)h;
        return;
      }
    }
    uint4 o;
    T *oe = (T *)&o;
    if (a.residual) {
      uint4 rv = ldLocal16((const T *)a.residual + e);
      const T *re = (const T *)&rv;
#pragma unroll
      for (int i = 0; i < N; ++i) oe[i] = fromAcc<T>(acc[i] + toAcc<T>(re[i]));
    } else {
#pragma unroll
      for (int i = 0; i < N; ++i) oe[i] = fromAcc<T>(acc[i]);
    }
    for (int d = 0; d < nDst; ++d) st16((T *)dst[d] + e, o);
  }

  static __device__ __forceinline__ void storeOne(const CollArgs &a, char *const *dst, int nDst, size_t e, Acc v) {
    v = finish<Acc>(v, a.scale, a.divisor);
    for (int d = 0; d < nDst; ++d) {
      if (a.outMode == kOutFloat && sizeof(T) == 2) {
        float x = (float)v;
        if (a.residual) x += ((const float *)a.residual)[e];
        ((float *)dst[d])[e] = x;
      } else if (a.outMode == kOutBf16 && sizeof(T) == 4) {
        float x = (float)v;
        if (a.residual) x += __bfloat162float(((const __nv_bfloat16 *)a.residual)[e]);
        ((__nv_bfloat16 *)dst[d])[e] = __float2bfloat16_rn(x);
      } else {
        Acc x = v;
        if (a.residual) x = x + toAcc<T>(((const T *)a.residual)[e]);
        ((T *)dst[d])[e] = fromAcc<T>(x);
      }
    }
  }

  // Reduces elements [sb, se) of the inputs (indices into in[p]) and stores them at
  // element index (i - sb + dstBase) of each destination.  The CTA takes its share
  // of the range in 16-byte units.
  static __device__ void slice(const CollArgs &a, int nRanks, size_t sb, size_t se, char *const *dst, int nDst,
                               size_t dstBase, int b, int g) {
    if (se <= sb) return;
    const size_t elems = se - sb;
    const size_t outSize = a.outMode == kOutFloat ? 4 : (a.outMode == kOutBf16 ? 2 : sizeof(T));
    bool vec = ((sb * sizeof(T)) & 15) == 0 && ((dstBase * outSize) & 15) == 0;
    for (int p = 0; p < nRanks; ++p) vec &= (((uintptr_t)a.in[p]) & 15) == 0;
    for (int d = 0; d < nDst; ++d) vec &= (((uintptr_t)dst[d]) & 15) == 0;
    if (a.residual) vec &= (((uintptr_t)a.residual) & 15) == 0;
    size_t ub, ue;
    ctaShare((elems * sizeof(T) + 15) >> 4, b, g, &ub, &ue);
    size_t eb = ub * N, ee = ue * N < elems ? ue * N : elems; // this CTA's elements, relative to sb
    if (vec) {
      const size_t fullEnd = ee / N * N; // whole packs only
      const size_t stride = (size_t)blockDim.x * N;
      size_t e = eb + (size_t)threadIdx.x * N;
      if constexpr (NR > 0) {
        // NVLink loads take microseconds: keep 16 of them in flight per thread
        constexpr int U = 16 / NR;
        for (; e + (U - 1) * stride < fullEnd; e += U * stride) {
          uint4 v[U][NR];
#pragma unroll
          for (int u = 0; u < U; ++u)
#pragma unroll
            for (int p = 0; p < NR; ++p) v[u][p] = ldSys16(a.in[p] + (sb + e + u * stride) * sizeof(T));
#pragma unroll
          for (int u = 0; u < U; ++u) {
            Acc acc[N];
            const T *e0 = (const T *)&v[u][0];
#pragma unroll
            for (int i = 0; i < N; ++i) acc[i] = toAcc<T>(e0[i]);
#pragma unroll
            for (int p = 1; p < NR; ++p) {
              const T *ep = (const T *)&v[u][p];
#pragma unroll
              for (int i = 0; i < N; ++i) acc[i] = combine<OP, Acc>(acc[i], toAcc<T>(ep[i]), a.redOp);
            }
            storePack(a, dst, nDst, dstBase + e + u * stride, acc);
          }
        }
      }
      for (; e < fullEnd; e += stride) {
        Acc acc[N];
        loadReduce(a, nRanks, (sb + e) * sizeof(T), acc);
        storePack(a, dst, nDst, dstBase + e, acc);
      }
      eb = fullEnd > eb ? fullEnd : eb;
    }
    for (size_t e = eb + threadIdx.x; e < ee; e += blockDim.x) {
      Acc acc = toAcc<T>(ldSysElem((const T *)a.in[0] + sb + e));
      for (int p = 1; p < nRanks; ++p)
        acc = combine<OP, Acc>(acc, toAcc<T>(ldSysElem((const T *)a.in[p] + sb + e)), a.redOp);
      storeOne(a, dst, nDst, dstBase + e, acc);
    }
  }

  // The same reduction with the inputs brought in by the bulk-copy engine: one thread
  // asks for a piece (16 bytes per thread) of every rank's input at once, peers
  // included, into one stage of the shared-memory ring; all threads then reduce
  // out of shared memory.  Needs NR > 0, 16-byte aligned inputs and whole packs.
  // Loads are plain bulk copies: none is multicast.  Returns false after a timeout.
  static __device__ bool sliceBulk(const flagcxDevComm &c, const CollArgs &a, size_t sb, size_t se, char *const *dst,
                                   int nDst, size_t dstBase, int b, int g) {
    constexpr int R = NR > 0 ? NR : 1;
    __shared__ __align__(8) uint64_t full[kBulkMaxStages], empty[kBulkMaxStages];
    __shared__ int abortS;
    const int nt = blockDim.x, tid = threadIdx.x;
    const uint32_t pieceBytes = (uint32_t)nt * 16u, stageBytes = pieceBytes * R;
    int stages = (int)(kBulkRingBytes / stageBytes);
    if (stages > kBulkMaxStages) stages = kBulkMaxStages;
    const int ahead = stages - 1;
    size_t ub, ue;
    ctaShare((se - sb) * sizeof(T) >> 4, b, g, &ub, &ue);
    const size_t nPieces = (ue - ub + nt - 1) / nt;
    const uint32_t ring = smem32(bulkRing);
    if (tid == 0) {
      abortS = 0;
      for (int s = 0; s < stages; ++s) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem32(&full[s])) : "memory");
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem32(&empty[s])), "r"(nt >> 5) : "memory");
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async;" ::: "memory"); // a copy-in by this CTA's threads precedes the engine's reads
    __syncthreads();

    auto issue = [&](size_t j) {
      const int s = (int)(j % stages);
      const size_t first = ub + j * nt;
      const uint32_t sz = (uint32_t)((ue - first) < (size_t)nt ? (ue - first) : (size_t)nt) * 16u;
      const uint32_t bar = smem32(&full[s]);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(sz * R) : "memory");
      for (int k = 0; k < R; ++k) {
        int p = c.rank + 1 + k; // peers first, each rank starting with a different one
        if (p >= R) p -= R;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         ring + s * stageBytes + p * pieceBytes),
                     "l"(a.in[p] + sb * sizeof(T) + (first << 4)), "r"(sz), "r"(bar)
                     : "memory");
      }
    };

    if (tid == 0)
      for (size_t j = 0; j < nPieces && j < (size_t)ahead; ++j) issue(j);
    bool ok = true;
    for (size_t i = 0; i < nPieces; ++i) {
      if (tid == 0 && i + ahead < nPieces) {
        const size_t j = i + ahead;
        if (j >= (size_t)stages) ok = mbarWaitBounded(c, &empty[j % stages], (uint32_t)(j / stages - 1) & 1u, &abortS);
        if (ok) issue(j);
      }
      const int s = (int)(i % stages);
      if (ok) ok = mbarWaitBounded(c, &full[s], (uint32_t)(i / stages) & 1u, &abortS);
      if (!ok) break;
      const size_t pack = ub + i * nt + tid;
      if (pack < ue) {
        const uint4 *stage = (const uint4 *)(bulkRing + (size_t)s * stageBytes);
        uint4 v[R];
#pragma unroll
        for (int p = 0; p < R; ++p) v[p] = stage[p * nt + tid];
        Acc acc[N];
        const T *e0 = (const T *)&v[0];
#pragma unroll
        for (int i2 = 0; i2 < N; ++i2) acc[i2] = toAcc<T>(e0[i2]);
#pragma unroll
        for (int p = 1; p < R; ++p) {
          const T *ep = (const T *)&v[p];
#pragma unroll
          for (int i2 = 0; i2 < N; ++i2) acc[i2] = combine<OP, Acc>(acc[i2], toAcc<T>(ep[i2]), a.redOp);
        }
        storePack(a, dst, nDst, dstBase + pack * N, acc);
      }
      __syncwarp();
      if ((tid & 31) == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem32(&empty[s])) : "memory");
    }
    if (!ok && tid == 0) fcxdev::reportError(c.status, FLAGCX_DEV_TIMEOUT, FLAGCX_DEV_AT_KERNEL, (unsigned)b, 0);
    return !__syncthreads_or(ok ? 0 : 1);
  }
};

// Second phase of the casting two-shot all-reduce: `elems` 16-bit values of a reduced
// slice (local or a peer's scratch) become fp32 in the local output, plus an optional
// fp32 residual.  The CTA takes the share of the slice that the same CTA of the
// slice's owner produced (same partition as Reducer::slice).
template <typename T>
__device__ void widenSlice(const T *src, float *dst, size_t elems, const float *residual, int b, int g) {
  constexpr int N = 8;
  size_t ub, ue;
  ctaShare((elems * sizeof(T) + 15) >> 4, b, g, &ub, &ue);
  const size_t eb = ub * N, ee = ue * N < elems ? ue * N : elems;
  if (eb >= ee) return;
  const bool vec = ((((uintptr_t)src) | ((uintptr_t)dst) | ((uintptr_t)residual)) & 15) == 0;
  size_t done = eb;
  if (vec) {
    const size_t fullEnd = ee / N * N, stride = (size_t)blockDim.x * N;
    auto emit = [&](size_t e, uint4 v) {
      const T *h = (const T *)&v;
      float f[N];
#pragma unroll
      for (int i = 0; i < N; ++i) f[i] = toAcc<T>(h[i]);
      if (residual) {
        uint4 r0 = ldLocal16(residual + e), r1 = ldLocal16(residual + e + 4);
        const float *ra = (const float *)&r0, *rb = (const float *)&r1;
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[i] += ra[i]; f[4 + i] += rb[i]; }
      }
      st16(dst + e, *(uint4 *)&f[0]);
      st16(dst + e + 4, *(uint4 *)&f[4]);
    };
    size_t e = eb + (size_t)threadIdx.x * N;
    for (; e + 3 * stride < fullEnd; e += 4 * stride) {
      uint4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = ldSys16(src + e + u * stride);
#pragma unroll
      for (int u = 0; u < 4; ++u) emit(e + u * stride, v[u]);
    }
    for (; e < fullEnd; e += stride) emit(e, ldSys16(src + e));
    done = fullEnd > eb ? fullEnd : eb;
  }
  for (size_t e = done + threadIdx.x; e < ee; e += blockDim.x) {
    float x = toAcc<T>(ldSysElem(src + e));
    if (residual) x += residual[e];
    dst[e] = x;
  }
}

// One hop of a ring reduction: dst[i] = x[i] (op) y[i] over this CTA's share of `elems`
// elements (y may be null: a plain copy), accumulating in the wider type.  `last` applies
// the scale / integer division of the epilogue.  dst may be peer memory.
template <typename T, int OP>
__device__ void ringCombine(const CollArgs &a, T *dst, const T *x, const T *y, size_t elems, bool last, int b, int g) {
  using Acc = typename Elem<T>::Acc;
  constexpr int N = 16 / (int)sizeof(T);
  size_t ub, ue;
  ctaShare((elems * sizeof(T) + 15) >> 4, b, g, &ub, &ue);
  const size_t eb = ub * N, ee = ue * N < elems ? ue * N : elems;
  if (eb >= ee) return;
  const bool vec = ((((uintptr_t)dst) | ((uintptr_t)x) | ((uintptr_t)y)) & 15) == 0;
  size_t done = eb;
  if (vec) {
    const size_t fullEnd = ee / N * N, stride = (size_t)blockDim.x * N;
    auto emit = [&](size_t e, uint4 vx, uint4 vy) {
      const T *px = (const T *)&vx, *py = (const T *)&vy;
      uint4 o;
      T *po = (T *)&o;
#pragma unroll
      for (int i = 0; i < N; ++i) {
        Acc v = toAcc<T>(px[i]);
        if (y) v = combine<OP, Acc>(v, toAcc<T>(py[i]), a.redOp);
        if (last) v = finish<Acc>(v, a.scale, a.divisor);
        po[i] = fromAcc<T>(v);
      }
      st16(dst + e, o);
    };
    size_t e = eb + (size_t)threadIdx.x * N;
    for (; e + 3 * stride < fullEnd; e += 4 * stride) {
      uint4 vx[4], vy[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        vx[u] = ldSys16(x + e + u * stride);
        vy[u] = y ? ldSys16(y + e + u * stride) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) emit(e + u * stride, vx[u], vy[u]);
    }
    for (; e < fullEnd; e += stride) emit(e, ldSys16(x + e), y ? ldSys16(y + e) : make_uint4(0, 0, 0, 0));
    done = fullEnd > eb ? fullEnd : eb;
  }
  for (size_t e = done + threadIdx.x; e < ee; e += blockDim.x) {
    Acc v = toAcc<T>(ldSysElem(x + e));
    if (y) v = combine<OP, Acc>(v, toAcc<T>(ldSysElem(y + e)), a.redOp);
    if (last) v = finish<Acc>(v, a.scale, a.divisor);
    dst[e] = fromAcc<T>(v);
  }
}

// Ring reduce-scatter over blocks [blockBegin(i), blockBegin(i) + blockLen(i)) of the
// inputs; rank r ends up with the complete block r in `result` (n-1 hops, each adding the
// sender's own contribution to the partial sum it received).  Returns false after a
// timed-out wait.
template <typename T, int OP>
__device__ bool ringReduceScatter(const flagcxDevComm &c, const CollArgs &a, size_t blockElems, size_t totalElems,
                                  T *result, int b, int g) {
  const int rank = c.rank, n = c.nRanks, next = (rank + 1) % n, prev = (rank + n - 1) % n;
  const T *own = (const T *)a.in[rank];
  auto begin = [&](int i) { size_t s = blockElems * (size_t)i; return s < totalElems ? s : totalElems; };
  auto len = [&](int i) { size_t s = begin(i); return s + blockElems < totalElems ? blockElems : totalElems - s; };
  T *mine = (T *)a.aux[rank], *theirs = (T *)a.aux[next];
  for (int s = 0; s < n - 1; ++s) {
    int ci = rank - s - 1; while (ci < 0) ci += n;
    ringCombine<T, OP>(a, theirs + (size_t)s * a.ringSlotElems, own + begin(ci),
                       s > 0 ? mine + (size_t)(s - 1) * a.ringSlotElems : (const T *)nullptr, len(ci), false, b, g);
    ctaRaiseFlag(a.ringNext + b, a.ringBase + s + 1);
    if (!ctaWaitFlag(c, a.ringMine + b, a.ringBase + s + 1, (unsigned)prev)) return false;
  }
  ringCombine<T, OP>(a, result, own + begin(rank), n > 1 ? mine + (size_t)(n - 2) * a.ringSlotElems : (const T *)nullptr,
                     len(rank), true, b, g);
  return true;
}

template <typename T, int OP, int NR>
__device__ void reduceBody(const flagcxDevComm &c, CollArgs &a) {
  const int b = blockIdx.x, g = gridDim.x, rank = c.rank, n = c.nRanks;
  using R = Reducer<T, OP, NR>;

  copyIn(a, rank, b, g);
  publishPointers(c, a, b);
  if (a.flags & kFlagBeginBarrier)
    if (!ctaBarrier(c, b)) return;
  learnPointers(c, a, b);
  const bool bulk = NR > 0 && a.bulkStage && learntPointersAligned(c, a);
  {
    const size_t outEs = a.outMode == kOutFloat ? 4 : (a.outMode == kOutBf16 ? 2 : sizeof(T));
    const size_t inEnd = a.kind == kReduceScatter ? a.inStride * (size_t)(n - 1) + a.count * sizeof(T)
                       : a.kind == kReduceScatterRing ? a.count * sizeof(T) * (size_t)n
                                                      : a.count * sizeof(T);
    (void)outEs;
    (void)inEnd;
    FCX_BOUNDS(c, inEnd, a.inBytes, 1);
    FCX_BOUNDS(c, a.count * outEs, a.outBytes, 2);
    if (a.kind == kReduceScatterRing || a.kind == kAllReduceRing) {
      const size_t blockElems = a.kind == kReduceScatterRing ? a.count : sliceElems(a.count, n, sizeof(T));
      (void)blockElems;
      FCX_BOUNDS(c, blockElems, a.ringSlotElems, 3);
    }
  }

  char *local[1] = {a.out[rank]};
  switch (a.kind) {
    case kAllReduceOneShot:
      R::slice(a, n, 0, a.count, local, 1, 0, b, g);
      break;
    case kAllReduceTwoShot: {
      size_t s = sliceElems(a.count, n, sizeof(T));
      size_t sb = s * rank < a.count ? s * rank : a.count;
      size_t se = sb + s < a.count ? sb + s : a.count;
      if (bulk) {
        if (!R::sliceBulk(c, a, sb, se, a.out, n, sb, b, g)) return;
      } else {
        R::slice(a, n, sb, se, a.out, n, sb, b, g);
      }
      break;
    }
    case kReduceScatter: {
      size_t sb = a.inStride / sizeof(T) * rank;
      if (bulk) {
        if (!R::sliceBulk(c, a, sb, sb + a.count, local, 1, 0, b, g)) return;
      } else {
        R::slice(a, n, sb, sb + a.count, local, 1, 0, b, g);
      }
      break;
    }
    case kReduceToRoot:
      if (rank == a.root) R::slice(a, n, 0, a.count, local, 1, 0, b, g);
      break;
    case kReduceScatterRing:
      if (!ringReduceScatter<T, OP>(c, a, a.count, a.count * (size_t)n, (T *)a.out[rank], b, g)) return;
      break;
    case kAllReduceRing: {
      // reduce-scatter into this rank's block of its own output, then pass the finished
      // blocks round the ring: after step s a rank holds blocks rank, rank-1, .., rank-s-1
      const size_t s = sliceElems(a.count, n, sizeof(T));
      auto begin = [&](int i) { size_t x = s * (size_t)i; return x < a.count ? x : a.count; };
      auto len = [&](int i) { size_t x = begin(i); return x + s < a.count ? s : a.count - x; };
      T *myOut = (T *)a.out[rank];
      if (!ringReduceScatter<T, OP>(c, a, s, a.count, myOut + begin(rank), b, g)) return;
      const int next = (rank + 1) % n, prev = (rank + n - 1) % n;
      for (int st = 0; st < n - 1; ++st) {
        int bi = rank - st; while (bi < 0) bi += n;
        ringCombine<T, OP>(a, (T *)a.out[next] + begin(bi), myOut + begin(bi), (const T *)nullptr, len(bi), false, b, g);
        ctaRaiseFlag(a.ringNext + b, a.ringBase + (n - 1) + st + 1);
        if (!ctaWaitFlag(c, a.ringMine + b, a.ringBase + (n - 1) + st + 1, (unsigned)prev)) return;
      }
      break;
    }
    case kAllReduceTwoShotCast: {
      // 16-bit inputs, fp32 result.  Sending fp32 to every peer would double the NVLink
      // bytes, so each rank rounds its reduced (and scaled) slice once to the input type
      // into its own scratch, and every rank then pulls all slices and widens them while
      // writing its output: the same bytes cross NVLink as in the plain all-reduce, and
      // all ranks end up with identical values.
      if constexpr (sizeof(T) == 2) {
        const size_t s = sliceElems(a.count, n, sizeof(T));
        const size_t sb = s * rank < a.count ? s * rank : a.count;
        const size_t se = sb + s < a.count ? sb + s : a.count;
        const char *residual = a.residual;
        __syncthreads();
        if (threadIdx.x == 0) { a.outMode = kOutSame; a.residual = nullptr; }
        __syncthreads();
        char *scratch[1] = {a.aux[rank]};
        if (bulk) {
          if (!R::sliceBulk(c, a, sb, se, scratch, 1, 0, b, g)) return;
        } else {
          R::slice(a, n, sb, se, scratch, 1, 0, b, g);
        }
        if (!ctaBarrier(c, b)) return;
        for (int k = 0; k < n; ++k) {
          int p = rank + k; if (p >= n) p -= n;
          const size_t pb = s * p < a.count ? s * p : a.count;
          const size_t pe = pb + s < a.count ? pb + s : a.count;
          widenSlice<T>((const T *)a.aux[p], (float *)a.out[rank] + pb, pe - pb,
                        residual ? (const float *)residual + pb : nullptr, b, g);
        }
      }
      break;
    }
    default: break;
  }

  if (a.flags & kFlagEndBarrier)
    if (!ctaBarrier(c, b)) return;
  copyOut(a, rank, b, g);
}

template <typename T, int OP, int NR>
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    reduceKernel(const __grid_constant__ flagcxDevComm c, const __grid_constant__ CollArgs a) {
  reduceBody<T, OP, NR>(c, stageArgs(a));
}

// Emulated world: one cooperative launch, blockIdx.y plays the rank.
template <typename T, int OP, int NR>
__global__ void __launch_bounds__(FLAGCX_DEVICE_THREADS_PER_CTA)
    reduceKernelEmu(const flagcxDevComm *cs, const CollArgs *as) {
  reduceBody<T, OP, NR>(cs[blockIdx.y], stageArgs(as[blockIdx.y]));
}

// ---------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------
template <typename T, int OP, int NR>
cudaError_t launchReduceT(const LaunchCtx &lc, const CollArgs &a) {
  dim3 grid(lc.nCtas, lc.emuRanks > 0 ? lc.emuRanks : 1), block(lc.nThreads);
  if (lc.emuRanks > 0) {
    void *params[] = {(void *)&lc.emuComms, (void *)&lc.emuArgs};
    size_t emuSmem = 0;
    if (NR > 0 && lc.emuBulk) {
      emuSmem = kBulkRingBytes;
      static bool emuConfigured = false; // one per instantiation
      if (!emuConfigured) {
        cudaError_t e = cudaFuncSetAttribute(reduceKernelEmu<T, OP, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)emuSmem);
        if (e != cudaSuccess) return e;
        emuConfigured = true;
      }
    }
    return cudaLaunchCooperativeKernel((const void *)reduceKernelEmu<T, OP, NR>, grid, block, params, emuSmem,
                                       lc.stream);
  }
  size_t smem = 0;
  if (NR > 0 && a.bulkStage) {
    smem = kBulkRingBytes;
    static bool configured = false; // one per instantiation
    if (!configured) {
      cudaError_t e = cudaFuncSetAttribute(reduceKernel<T, OP, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return e;
      configured = true;
    }
  }
  reduceKernel<T, OP, NR><<<grid, block, smem, lc.stream>>>(*lc.comm, a);
  return cudaGetLastError();
}

template <typename T>
cudaError_t launchReduceHot(const LaunchCtx &lc, const CollArgs &a, int nRanks) {
  // sum (and average, which is sum with a scale) at the common world sizes get the
  // fully unrolled instantiation; everything else takes the generic one
  if (a.redOp == kOpSum) {
    switch (nRanks) {
      case 2: return launchReduceT<T, kOpSum, 2>(lc, a);
      case 4: return launchReduceT<T, kOpSum, 4>(lc, a);
      case 8: return launchReduceT<T, kOpSum, 8>(lc, a);
      default: break;
    }
  }
  return launchReduceT<T, kOpRuntime, 0>(lc, a);
}

} // namespace

cudaError_t launchReduceKernel(const LaunchCtx &lc, const CollArgs &a, int nRanks) {
  switch ((flagcxDataType_t)a.dtype) {
    case flagcxFloat32: return launchReduceHot<float>(lc, a, nRanks);
    case flagcxBfloat16: return launchReduceHot<__nv_bfloat16>(lc, a, nRanks);
    case flagcxFloat16: return launchReduceHot<__half>(lc, a, nRanks);
    case flagcxFloat64: return launchReduceT<double, kOpRuntime, 0>(lc, a);
    case flagcxInt8: return launchReduceT<signed char, kOpRuntime, 0>(lc, a);
    case flagcxUint8: return launchReduceT<unsigned char, kOpRuntime, 0>(lc, a);
    case flagcxInt32: return launchReduceT<int, kOpRuntime, 0>(lc, a);
    case flagcxUint32: return launchReduceT<unsigned int, kOpRuntime, 0>(lc, a);
    case flagcxInt64: return launchReduceT<long long, kOpRuntime, 0>(lc, a);
    case flagcxUint64: return launchReduceT<unsigned long long, kOpRuntime, 0>(lc, a);
    default: return cudaErrorInvalidValue;
  }
}

// Upper bound on CTAs per SM for the cooperative emulated-world launch of this family.
int reduceEmuOccupancy(int nThreads) {
  int occ = 0;
  cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, (const void *)reduceKernelEmu<double, kOpRuntime, 0>, nThreads, 0);
  return occ;
}

} // namespace fcx
