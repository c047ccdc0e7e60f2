// tp_gemm.cu -- bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, fp32
// accumulators in tensor memory, operands brought into shared memory by TMA) with the
// tensor-parallel collective fused into the same kernel:
//
//   mode kPlain           D[M,N] = A[M,K] * B[N,K]^T
//   mode kAllGatherGemm   column-parallel layer: A is sequence-sharded over the ranks.
//                         Two spare warps of EVERY CTA push this rank's shard, 64 KiB
//                         at a time, into every peer's gather buffer over NVLink and
//                         count each piece in on the destination; the GEMM starts with
//                         the local rows and takes up a remote 128-row block as soon as
//                         all of its pieces are counted in, loading it by TMA from LOCAL
//                         memory (no TMA ever reads a peer, no multicast).
//   mode kGemmReduceScatter  row-parallel layer: every output tile is a partial sum.
//                         The epilogue converts the accumulator tile, transposes it
//                         through shared memory so that every store instruction writes
//                         whole 128-byte lines, and stores it straight into the owning
//                         rank's partial buffer (remote owners first) and counts it in
//                         on that rank.  A rank's own rows come last: their epilogue
//                         waits for the peers' counts, adds the peers' partial tiles
//                         (local memory by then) in fp32 and stores the final rows --
//                         there is no separate reduction pass.
//
// Two flavours of the same kernel.  PAIR=false: every CTA owns a 128 x 256 tile
// (cta_group::1).  PAIR=true: the two CTAs of a cluster share a 256 x 256 tile
// (cta_group::2): each loads its own 128 rows of A and 128 of the 256 rows of B, the
// leader CTA issues one MMA that reads both CTAs' shared memory and writes 128
// accumulator rows into each CTA's TMEM -- a third less operand traffic per flop.
//
// One persistent CTA per SM, 256 threads: warp 0 issues TMA, warp 1 issues MMA, warps
// 2-5 run the epilogue (one TMEM lane quarter each), warps 6-7 push (all-gather mode).
// K step 64, four (single CTA) or six (pair) shared-memory stages, two accumulator
// buffers in TMEM so that the epilogue of one tile overlaps the main loop of the next.
// Tiles are walked in compact groups (see tileCoords) for L2 reuse.  Every wait
// (mbarrier, flag, counter) is bounded: on a timeout the CTA raises an abort flag,
// reports through the status block, lets its other warps fall out of their loops, frees
// its TMEM and returns.
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

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kThreads = 256;
constexpr uint32_t kTmemCols = 512;
constexpr unsigned long long kWaitLimitNs = 4000000000ull; // 4 s
constexpr int kEpiCols = 64;                                // columns staged per epilogue step

template <bool PAIR>
struct __align__(1024) Smem {
  static constexpr int STAGES = PAIR ? 6 : 4;
  static constexpr int BROWS = PAIR ? BN / 2 : BN; // rows of B this CTA loads per stage
  bf16 a[STAGES][BM * BK];
  bf16 b[STAGES][BROWS * BK];
  uint4 epi[4][32 * kEpiCols * 2 / 16]; // per epilogue warp: 32 rows x 64 bf16, 16-byte chunks swizzled
  uint64_t full[STAGES], empty[STAGES], tmemFull[2], tmemEmpty[2];
  uint32_t tmemBase;
  int abortFlag;
};

// Which tile the grid's i-th scheduling slot covers.  Rank by rank (remote-owned row
// blocks rotated so that every rank starts with its own rows / with a different
// peer's), and inside one rank's rows in groups of `groupRows` row blocks that are
// walked column by column: the tiles in flight at any moment then form a compact
// rectangle (about 8 x 9 tiles of 256 x 256) instead of a one-tile-high stripe, so the
// rows of A and B that they share are fetched from HBM once and hit in L2 afterwards.
__device__ __forceinline__ void tileCoords(const TpGemmArgs &a, int rank, int tile, int tilesN, int TM, int *tm, int *tn) {
  const int blocks = a.M / TM, bpr = a.rowsPerRank / TM, tilesPerRank = bpr * tilesN;
  const int r = tile / tilesPerRank, w = tile - r * tilesPerRank;
  const int perGroup = a.groupRows * tilesN;
  const int g = w / perGroup, wg = w - g * perGroup;
  const int gsize = min(a.groupRows, bpr - g * a.groupRows);
  *tn = wg / gsize;
  int rb = r * bpr + g * a.groupRows + (wg - *tn * gsize);
  if (a.mode == kAllGatherGemm) rb = (rb + rank * bpr) % blocks;                 // own rows first
  else if (a.mode == kGemmReduceScatter) rb = (rb + (rank + 1) * bpr) % blocks; // own rows last
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

template <bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
    tpGemmKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const flagcxDevComm c, const TpGemmArgs a) {
  extern __shared__ uint8_t rawSmem[];
  using SmemT = Smem<PAIR>;
  constexpr int STAGES = SmemT::STAGES;
  constexpr uint32_t kStageBytes = ((PAIR ? 2 * BM : BM) + BN) * BK * 2; // per stage; a pair loads 256 rows of A
  SmemT &s = *reinterpret_cast<SmemT *>((reinterpret_cast<uintptr_t>(rawSmem) + 1023) & ~(uintptr_t)1023);
  const uint32_t ctaRank = PAIR ? clusterCtaRank() : 0; // position inside the CTA pair
  const bool leader = ctaRank == 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = c.rank, n = c.nRanks;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbarInit(&s.full[i], 1); mbarInit(&s.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbarInit(&s.tmemFull[i], 1); mbarInit(&s.tmemEmpty[i], PAIR ? 8 : 4); }
    s.abortFlag = 0;
    mbarInitFence();
    prefetchTensorMap(&tmA);
    prefetchTensorMap(&tmB);
  }
  if (warp == 1) {
    if (PAIR) { tmemAllocPair(&s.tmemBase, kTmemCols); tmemRelinquishPair(); }
    else { tmemAlloc(&s.tmemBase, kTmemCols); tmemRelinquish(); }
  }
  fenceBeforeSync();
  __syncthreads();
  if (PAIR) clusterSync(); // the partner's barriers exist before anything is signalled on them
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

  const int G = gridDim.x;
  // a scheduling unit is a CTA (128-row tiles) or a CTA pair (256-row tiles)
  const int unit = PAIR ? blockIdx.x / 2 : blockIdx.x, units = PAIR ? G / 2 : G;
  const int TM = PAIR ? 2 * BM : BM;
  const int tilesN = a.N / BN;
  const int nTiles = (a.M / TM) * tilesN;
  const int kBlocks = a.K / BK;

  if (!alive) {
    // fall through to the common exit
  } else if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = unit; tile < nTiles && ok; tile += units) {
        int tm, tn;
        tileCoords(a, rank, tile, tilesN, TM, &tm, &tn);
        const int arow = tm * TM + (int)ctaRank * BM; // first row of A this CTA loads
        if (a.mode == kAllGatherGemm && n > 1) {
          const int chunks = a.rowsPerRank / BM;
          const int owner = arow / a.rowsPerRank;
          if (owner != rank) {
            ok = waitFlagGe(c, a.chunkFlags[rank] + (size_t)owner * chunks + (arow / BM) % chunks,
                            a.epoch * (unsigned long long)a.piecesPerChunk, abortFlag, owner);
            fenceProxyAsync(); // the rows were written by a peer's stores; TMA reads them next
            if (!ok) break;
          }
        }
        for (int kb = 0; kb < kBlocks; ++kb) {
          if (!mbarWait(&s.empty[stage], phase ^ 1, abortFlag, kWaitLimitNs)) { ok = false; break; }
          if (PAIR) {
            // both CTAs' loads are counted on the leader's barrier, which the MMA waits on
            if (leader) mbarExpectTx(&s.full[stage], kStageBytes);
            const uint32_t bar = mapToCta(smemAddr(&s.full[stage]), 0);
            tmaLoad2dPair(s.a[stage], &tmA, kb * BK, arow, bar);
            tmaLoad2dPair(s.b[stage], &tmB, kb * BK, tn * BN + (int)ctaRank * (BN / 2), bar);
          } else {
            mbarExpectTx(&s.full[stage], kStageBytes);
            tmaLoad2d(s.a[stage], &tmA, kb * BK, arow, &s.full[stage]);
            tmaLoad2d(s.b[stage], &tmB, kb * BK, tn * BN, &s.full[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = instrDescBf16(PAIR ? 2 * BM : BM, BN);
      int stage = 0, acc = 0;
      uint32_t phase = 0, accPhase = 0;
      bool ok = true;
      for (int tile = unit; tile < nTiles && ok; tile += units) {
        if (!mbarWait(&s.tmemEmpty[acc], accPhase ^ 1, abortFlag, kWaitLimitNs)) break;
        fenceAfterSync();
        for (int kb = 0; kb < kBlocks; ++kb) {
          if (!mbarWait(&s.full[stage], phase, abortFlag, kWaitLimitNs)) { ok = false; break; }
          fenceAfterSync();
          const uint64_t da = smemDescSw128(s.a[stage]), db = smemDescSw128(s.b[stage]);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) { // 16 bf16 = 32 bytes along K inside the swizzled row
            if (PAIR) mmaBf16Pair(tmemBase + acc * BN, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0);
            else mmaBf16(tmemBase + acc * BN, da + 2 * k4, db + 2 * k4, idesc, (kb | k4) != 0);
          }
          // the stage may be refilled (in both CTAs) once these MMAs have read it
          if (PAIR) mmaCommitPair(&s.empty[stage], 3); else mmaCommit(&s.empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (PAIR) mmaCommitPair(&s.tmemFull[acc], 3); else mmaCommit(&s.tmemFull[acc]);
        if (++acc == 2) { acc = 0; accPhase ^= 1; }
      }
    }
  } else if (warp < 6) {
    // ---- epilogue: warps 2..5, TMEM lane quarter = warp % 4 ----
    const int q = warp & 3;
    uint4 *stg = s.epi[warp - 2];
    int acc = 0;
    uint32_t accPhase = 0;
    for (int tile = unit; tile < nTiles; tile += units) {
      int tm, tn;
      tileCoords(a, rank, tile, tilesN, TM, &tm, &tn);
      if (!mbarWait(&s.tmemFull[acc], accPhase, abortFlag, kWaitLimitNs)) break;
      fenceAfterSync();
      // rows q*32 .. q*32+31 of the tile belong to this warp; all of them have one owner
      const size_t growBase = (size_t)tm * TM + ctaRank * BM + q * 32;
      bf16 *dbase;
      int owner = rank;
      const bf16 *others = nullptr; // reduce-scatter, own rows: slice 0 of the partial sums of these rows
      if (a.mode == kGemmReduceScatter) {
        owner = (int)(growBase / a.rowsPerRank);
        const size_t rowLocal = growBase - (size_t)owner * a.rowsPerRank;
        if (owner != rank) {
          dbase = a.partial[owner] + ((size_t)rank * a.rowsPerRank + rowLocal) * a.N;
        } else {
          // My own rows come last in the tile order, when the peers' partial sums of them
          // have (nearly) all landed here: wait for the row block's counter, then add
          // them to the accumulator tile on its way out and store the final rows.
          dbase = a.out + rowLocal * a.N;
          if (n > 1) {
            bool ok = true;
            if (lane == 0)
              ok = waitFlagGe(c, a.rowFlags[rank] + rowLocal / BM,
                              a.epoch * (unsigned long long)((n - 1) * tilesN), abortFlag, 0xffffffffu);
            if (!__shfl_sync(0xffffffffu, (int)ok, 0)) break;
            others = a.partial[rank] + rowLocal * a.N + (size_t)tn * BN;
          }
        }
      } else {
        dbase = a.D + growBase * a.N;
      }
      dbase += (size_t)tn * BN;
      const size_t sliceElems = (size_t)a.rowsPerRank * a.N;
#pragma unroll 1
      for (int cb = 0; cb < BN / kEpiCols; ++cb) {
        // this thread's row, 64 fp32 columns -> 64 bf16 = eight 16-byte chunks, swizzled into the staging
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmemLoad32(tmemBase + ((uint32_t)(q * 32) << 16) + acc * BN + cb * kEpiCols + h * 32, r);
          tmemLoadWait();
          uint4 o[4];
          bf16 *ob = (bf16 *)o;
#pragma unroll
          for (int i = 0; i < 32; ++i) ob[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
#pragma unroll
          for (int i = 0; i < 4; ++i) stg[lane * 8 + ((h * 4 + i) ^ (lane & 7))] = o[i];
        }
        __syncwarp();
        // read back transposed: one instruction stores four rows x 128 contiguous bytes
        if (others == nullptr) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int row = k * 4 + (lane >> 3), ch = lane & 7;
            uint4 v = stg[row * 8 + (ch ^ (row & 7))];
            st16((uint4 *)(dbase + (size_t)row * a.N + cb * kEpiCols) + ch, v);
          }
        } else {
#pragma unroll 2
          for (int k = 0; k < 8; ++k) {
            const int row = k * 4 + (lane >> 3), ch = lane & 7;
            const bf16 *src = others + (size_t)row * a.N + cb * kEpiCols + ch * 8;
            uint4 p[FLAGCX_MAX_RANKS];
#pragma unroll
            for (int sidx = 0; sidx < FLAGCX_MAX_RANKS; ++sidx)
              if (sidx < n && sidx != rank) p[sidx] = ldSys16(src + (size_t)sidx * sliceElems);
            uint4 v = stg[row * 8 + (ch ^ (row & 7))];
            float accv[8];
            const bf16 *ve = (const bf16 *)&v;
#pragma unroll
            for (int t = 0; t < 8; ++t) accv[t] = __bfloat162float(ve[t]);
            // fixed rank order except that this rank's own term comes first
#pragma unroll
            for (int sidx = 0; sidx < FLAGCX_MAX_RANKS; ++sidx)
              if (sidx < n && sidx != rank) {
                const bf16 *e = (const bf16 *)&p[sidx];
#pragma unroll
                for (int t = 0; t < 8; ++t) accv[t] += __bfloat162float(e[t]);
              }
            bf16 *oe = (bf16 *)&v;
#pragma unroll
            for (int t = 0; t < 8; ++t) oe[t] = __float2bfloat16_rn(accv[t]);
            st16((uint4 *)(dbase + (size_t)row * a.N + cb * kEpiCols) + ch, v);
          }
        }
        __syncwarp();
      }
      fenceBeforeSync();
      __syncwarp();
      if (lane == 0) {
        // the accumulator buffer is free again: tell the CTA that issues the MMAs
        if (PAIR && !leader) mbarArriveCluster(mapToCta(smemAddr(&s.tmemEmpty[acc]), 0));
        else mbarArrive(&s.tmemEmpty[acc]);
      }
      if (a.mode == kGemmReduceScatter && owner != rank) {
        // count the tile in on its owner once all four epilogue warps have stored it
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          fcxdev::fenceSys();
          const int rbLocal = (int)(((size_t)tm * TM + ctaRank * BM - (size_t)owner * a.rowsPerRank) / BM);
          fcxdev::redAddReleaseSys(a.rowFlags[owner] + rbLocal, 1ull);
        }
      }
      if (++acc == 2) { acc = 0; accPhase ^= 1; }
    }
  } else if (a.mode == kAllGatherGemm && n > 1) {
    // ---- pusher warps 6..7: my shard -> every peer, piece by piece, chunk 0 first ----
    const int t = threadIdx.x - 192; // 0..63
    const int chunks = a.rowsPerRank / BM;
    const size_t chunkBytes = (size_t)BM * a.K * 2;
    const size_t pieceBytes = chunkBytes / a.piecesPerChunk;
    const size_t shardOff = (size_t)rank * a.rowsPerRank * a.K * 2;
    const char *src = (const char *)a.gathered[rank] + shardOff;
    const int itemsPerChunk = (n - 1) * a.piecesPerChunk;
    const int items = chunks * itemsPerChunk;
    for (int u = blockIdx.x; u < items && !*abortFlag; u += G) {
      const int ch = u / itemsPerChunk, rem = u % itemsPerChunk;
      const int piece = rem / (n - 1);
      int p = rank + 1 + rem % (n - 1);
      if (p >= n) p -= n;
      const size_t off = ch * chunkBytes + piece * pieceBytes;
      const uint4 *sv = (const uint4 *)(src + off);
      uint4 *dv = (uint4 *)((char *)a.gathered[p] + shardOff + off);
      const size_t nv = pieceBytes >> 4;
      size_t i = t;
      for (; i + 7 * 64 < nv; i += 8 * 64) {
        uint4 r[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) r[k] = ldLocal16(sv + i + k * 64);
#pragma unroll
        for (int k = 0; k < 8; ++k) st16(dv + i + k * 64, r[k]);
      }
      for (; i < nv; i += 64) st16(dv + i, ldLocal16(sv + i));
      asm volatile("bar.sync 2, 64;" ::: "memory");
      if (t == 0) {
        fcxdev::fenceSys();
        fcxdev::redAddReleaseSys(a.chunkFlags[p] + (size_t)rank * chunks + ch, 1ull);
      }
    }
  }

  __syncthreads();
  if (threadIdx.x == 0 && *abortFlag)
    fcxdev::reportError(c.status, FLAGCX_DEV_TIMEOUT, FLAGCX_DEV_AT_KERNEL, (unsigned)blockIdx.x, 0);
  __syncthreads();
  if (PAIR) clusterSync(); // neither CTA leaves while its partner may still signal it
  if (warp == 1) {
    if (PAIR) tmemDeallocPair(tmemBase, kTmemCols); else tmemDealloc(tmemBase, kTmemCols);
  }
}

} // namespace

size_t tpGemmSmemBytes(bool pair) { return (pair ? sizeof(Smem<true>) : sizeof(Smem<false>)) + 1024; }

// pair: use CTA pairs (cluster of two, 256 x 256 tiles); needs an even grid and M a
// multiple of 256 (per rank in the fused modes).
cudaError_t launchTpGemm(cudaStream_t stream, const CUtensorMap &tmA, const CUtensorMap &tmB, const flagcxDevComm &c,
                         const TpGemmArgs &a, int nCtas, bool pair) {
  static bool configured[2] = {false, false};
  const void *fn = pair ? (const void *)tpGemmKernel<true> : (const void *)tpGemmKernel<false>;
  if (!configured[pair]) {
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tpGemmSmemBytes(pair));
    if (e != cudaSuccess) return e;
    configured[pair] = true;
  }
  if (!pair) {
    tpGemmKernel<false><<<nCtas, kThreads, tpGemmSmemBytes(false), stream>>>(tmA, tmB, c, a);
    return cudaGetLastError();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(nCtas & ~1);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = tpGemmSmemBytes(true);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, tpGemmKernel<true>, tmA, tmB, c, a);
}

} // namespace fcx
