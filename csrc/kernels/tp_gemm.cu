// tp_gemm.cu -- bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, fp32
// accumulators in tensor memory, operands brought into shared memory by TMA) with the
// tensor-parallel collective fused into the same kernel:
//
//   mode kPlain           D[M,N] = A[M,K] * B[N,K]^T
//   mode kAllGatherGemm   column-parallel layer: A is sequence-sharded over the ranks.
//                         A few CTAs push this rank's shard, 128 rows at a time, into
//                         every peer's gather buffer over NVLink and raise a flag per
//                         chunk; the GEMM CTAs start with the local rows and take up a
//                         remote row block as soon as its flag is up, loading it by TMA
//                         from LOCAL memory (no TMA ever reads a peer, no multicast).
//   mode kGemmReduceScatter  row-parallel layer: every output tile is a partial sum.
//                         The epilogue converts the accumulator tile and stores it
//                         straight into the owning rank's partial buffer (remote owners
//                         first), counts it in on that rank, and each rank finally sums
//                         the partial slices of its own rows in fp32.
//
// One persistent CTA per SM, 192 threads: warp 0 issues TMA, warp 1 issues MMA, warps
// 2-5 run the epilogue (one TMEM lane quarter each).  Tile 128 x 256 x 64, four
// shared-memory stages, two accumulator buffers in TMEM so that the epilogue of one tile
// overlaps the main loop of the next.  Every wait (mbarrier, flag, counter) is bounded:
// on a timeout the CTA raises an abort flag, reports through the status block, lets its
// other warps fall out of their loops, frees its TMEM and returns.
//
// The FlagCX project contains no GEMM; the comparison target is NCCL all-gather /
// reduce-scatter followed or preceded by a cuBLAS GEMM.
#include <cuda_bf16.h>

#include "launch.h"
#include "prims.cuh"
#include "tcgen05.cuh"
#include "tp_gemm_args.h"

namespace fcx {
namespace {

using bf16 = __nv_bfloat16;
using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int kThreads = 192;
constexpr uint32_t kStageBytes = (BM + BN) * BK * 2;
constexpr uint32_t kTmemCols = 512;
constexpr unsigned long long kWaitLimitNs = 4000000000ull; // 4 s

struct __align__(1024) Smem {
  bf16 a[STAGES][BM * BK];
  bf16 b[STAGES][BN * BK];
  uint64_t full[STAGES], empty[STAGES], tmemFull[2], tmemEmpty[2];
  uint32_t tmemBase;
  int abortFlag;
};

// Which row block (of 128 rows) a CTA's i-th tile covers: remote-owned blocks are
// rotated so that every rank starts with different peers / with its own rows.
__device__ __forceinline__ void tileCoords(const TpGemmArgs &a, int rank, int tile, int tilesN, int *tm, int *tn) {
  int rb = tile / tilesN;
  *tn = tile % tilesN;
  const int blocks = a.M / BM;
  if (a.mode == kAllGatherGemm) rb = (rb + rank * (a.rowsPerRank / BM)) % blocks;           // own rows first
  else if (a.mode == kGemmReduceScatter) rb = (rb + (rank + 1) * (a.rowsPerRank / BM)) % blocks; // own rows last
  *tm = rb;
}

__device__ __forceinline__ bool waitFlagGe(const flagcxDevComm &c, const unsigned long long *flag,
                                           unsigned long long want, volatile int *abortFlag, unsigned peer) {
  if (fcxdev::ldAcquireSys(flag) >= want) return true;
  const unsigned long long t0 = timerNs();
  unsigned spins = 0;
  for (;;) {
    if (fcxdev::ldAcquireSys(flag) >= want) return true;
    __nanosleep(100);
    if ((++spins & 63u) == 0) {
      if (*abortFlag) return false;
      if (timerNs() - t0 > c.timeoutNs || (c.status && fcxdev::ldVolatileU32(&c.status->abortFlag))) {
        *abortFlag = 1;
        fcxdev::reportError(c.status, FLAGCX_DEV_TIMEOUT, FLAGCX_DEV_AT_SIGNAL, peer, want);
        return false;
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
    tpGemmKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const flagcxDevComm c, const TpGemmArgs a) {
  extern __shared__ uint8_t rawSmem[];
  Smem &s = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(rawSmem) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = c.rank, n = c.nRanks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbarInit(&s.full[i], 1); mbarInit(&s.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbarInit(&s.tmemFull[i], 1); mbarInit(&s.tmemEmpty[i], 4); }
    s.abortFlag = 0;
    mbarInitFence();
    prefetchTensorMap(&tmA);
    prefetchTensorMap(&tmB);
  }
  if (warp == 1) {
    tmemAlloc(&s.tmemBase, kTmemCols);
    tmemRelinquish();
  }
  fenceBeforeSync();
  __syncthreads();
  fenceAfterSync();
  const uint32_t tmemBase = s.tmemBase;
  volatile int *abortFlag = &s.abortFlag;

  // All ranks are inside this call (so all of them left the previous one) before any
  // peer memory of this call is written.
  bool alive = true;
  if (a.mode != kPlain && n > 1) {
    flagcxDevBarrierIntra bar(c, blockIdx.x);
    alive = bar.sync(flagcxCoopBlock());
  }

  const int nGemmCtas = gridDim.x - a.nPushCtas;
  const int tilesN = a.N / BN;
  const int nTiles = (a.M / BM) * tilesN;
  const int kBlocks = a.K / BK;

  if (!alive) {
    // fall through to the common exit
  } else if ((int)blockIdx.x >= nGemmCtas) {
    // ---- pusher CTAs (all-gather mode): my shard -> every peer, chunk by chunk ----
    const int j = blockIdx.x - nGemmCtas;
    const int chunks = a.rowsPerRank / BM;
    const size_t chunkBytes = (size_t)BM * a.K * 2;
    const char *src = (const char *)(a.gathered[rank] + (size_t)rank * a.rowsPerRank * a.K);
    for (int ch = j; ch < chunks && !*abortFlag; ch += a.nPushCtas) {
      for (int k = 1; k < n; ++k) {
        int p = rank + k; if (p >= n) p -= n;
        char *dst = (char *)(a.gathered[p] + (size_t)rank * a.rowsPerRank * a.K) + ch * chunkBytes;
        ctaCopy(dst, src + ch * chunkBytes, 0, chunkBytes);
        __syncthreads();
        if (threadIdx.x == 0) {
          fcxdev::fenceSys();
          fcxdev::stReleaseSys(a.chunkFlags[p] + (size_t)rank * chunks + ch, a.epoch);
        }
      }
    }
  } else if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < nTiles && ok; tile += nGemmCtas) {
        int tm, tn;
        tileCoords(a, rank, tile, tilesN, &tm, &tn);
        if (a.mode == kAllGatherGemm && n > 1) {
          const int chunks = a.rowsPerRank / BM;
          const int owner = tm / chunks;
          if (owner != rank) {
            ok = waitFlagGe(c, a.chunkFlags[rank] + (size_t)owner * chunks + tm % chunks, a.epoch, abortFlag, owner);
            fenceProxyAsync(); // the rows were written by a peer's stores; TMA reads them next
            if (!ok) break;
          }
        }
        for (int kb = 0; kb < kBlocks; ++kb) {
          if (!mbarWait(&s.empty[stage], phase ^ 1, abortFlag, kWaitLimitNs)) { ok = false; break; }
          mbarExpectTx(&s.full[stage], kStageBytes);
          tmaLoad2d(s.a[stage], &tmA, kb * BK, tm * BM, &s.full[stage]);
          tmaLoad2d(s.b[stage], &tmB, kb * BK, tn * BN, &s.full[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      constexpr uint32_t idesc = instrDescBf16(BM, BN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, accPhase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < nTiles && ok; tile += nGemmCtas) {
        if (!mbarWait(&s.tmemEmpty[acc], accPhase ^ 1, abortFlag, kWaitLimitNs)) break;
        fenceAfterSync();
        for (int kb = 0; kb < kBlocks; ++kb) {
          if (!mbarWait(&s.full[stage], phase, abortFlag, kWaitLimitNs)) { ok = false; break; }
          fenceAfterSync();
          const uint64_t da = smemDescSw128(s.a[stage]), db = smemDescSw128(s.b[stage]);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) // 16 bf16 = 32 bytes along K inside the swizzled row
            mmaBf16(tmemBase + acc * BN, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0);
          mmaCommit(&s.empty[stage]); // stage may be refilled once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mmaCommit(&s.tmemFull[acc]);
        if (++acc == 2) { acc = 0; accPhase ^= 1; }
      }
    }
  } else {
    // ---- epilogue: warps 2..5, TMEM lane quarter = warp % 4 ----
    const int q = warp & 3;
    int acc = 0;
    uint32_t accPhase = 0;
    for (int tile = blockIdx.x; tile < nTiles; tile += nGemmCtas) {
      int tm, tn;
      tileCoords(a, rank, tile, tilesN, &tm, &tn);
      if (!mbarWait(&s.tmemFull[acc], accPhase, abortFlag, kWaitLimitNs)) break;
      fenceAfterSync();
      const int rowInTile = q * 32 + lane;
      const size_t grow = (size_t)tm * BM + rowInTile;
      bf16 *drow;
      int owner = rank;
      if (a.mode == kGemmReduceScatter) {
        owner = (int)(grow / a.rowsPerRank);
        drow = a.partial[owner] + ((size_t)rank * a.rowsPerRank + (grow - (size_t)owner * a.rowsPerRank)) * a.N;
      } else {
        drow = a.D + grow * a.N;
      }
      drow += (size_t)tn * BN;
#pragma unroll 1
      for (int cb = 0; cb < BN / 32; ++cb) {
        uint32_t r[32];
        tmemLoad32(tmemBase + ((uint32_t)(q * 32) << 16) + acc * BN + cb * 32, r);
        tmemLoadWait();
        uint4 o[4];
        bf16 *ob = (bf16 *)o;
#pragma unroll
        for (int i = 0; i < 32; ++i) ob[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
#pragma unroll
        for (int i = 0; i < 4; ++i) st16((uint4 *)(drow + cb * 32) + i, o[i]);
      }
      fenceBeforeSync();
      __syncwarp();
      if (lane == 0) mbarArrive(&s.tmemEmpty[acc]);
      if (a.mode == kGemmReduceScatter) {
        // count the tile in on its owner once all four epilogue warps have stored it
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          fcxdev::fenceSys();
          const int rbLocal = (int)((grow - (size_t)owner * a.rowsPerRank) / BM);
          fcxdev::redAddReleaseSys(a.rowFlags[owner] + rbLocal, 1ull);
        }
      }
      if (++acc == 2) { acc = 0; accPhase ^= 1; }
    }
  }

  __syncthreads();
  if (a.mode == kGemmReduceScatter && !*abortFlag && alive) {
    // ---- reduce my rows: sum the n partial slices in fp32, one bf16 store ----
    const int rbs = a.rowsPerRank / BM;
    const unsigned long long want = a.epoch * (unsigned long long)(n * tilesN);
    const size_t sliceElems = (size_t)a.rowsPerRank * a.N;
    // every CTA takes a share of every row block, so the whole GPU streams the slices
    for (int rb = 0; rb < rbs; ++rb) {
      bool ok = true;
      if (threadIdx.x == 0) ok = waitFlagGe(c, a.rowFlags[rank] + rb, want, abortFlag, 0xffffffffu);
      if (__syncthreads_or(ok ? 0 : 1)) break;
      const size_t base = (size_t)rb * BM * a.N, packs = (size_t)BM * a.N / 8;
      for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < packs; i += (size_t)gridDim.x * kThreads) {
        float accv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int sidx = 0; sidx < n; ++sidx) {
          uint4 v = ldSys16(a.partial[rank] + sidx * sliceElems + base + i * 8);
          const bf16 *e = (const bf16 *)&v;
#pragma unroll
          for (int t = 0; t < 8; ++t) accv[t] += __bfloat162float(e[t]);
        }
        uint4 o;
        bf16 *oe = (bf16 *)&o;
#pragma unroll
        for (int t = 0; t < 8; ++t) oe[t] = __float2bfloat16_rn(accv[t]);
        st16(a.out + base + i * 8, o);
      }
    }
  }
  if (threadIdx.x == 0 && *abortFlag)
    fcxdev::reportError(c.status, FLAGCX_DEV_TIMEOUT, FLAGCX_DEV_AT_KERNEL, (unsigned)blockIdx.x, 0);
  __syncthreads();
  if (warp == 1) tmemDealloc(tmemBase, kTmemCols);
}

} // namespace

size_t tpGemmSmemBytes() { return sizeof(Smem) + 1024; }

cudaError_t launchTpGemm(cudaStream_t stream, const CUtensorMap &tmA, const CUtensorMap &tmB, const flagcxDevComm &c,
                         const TpGemmArgs &a, int nCtas) {
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(tpGemmKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tpGemmSmemBytes());
    if (e != cudaSuccess) return e;
    configured = true;
  }
  tpGemmKernel<<<nCtas, kThreads, tpGemmSmemBytes(), stream>>>(tmA, tmB, c, a);
  return cudaGetLastError();
}

} // namespace fcx
