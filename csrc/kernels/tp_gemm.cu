// tp_gemm.cu -- bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, fp32
// accumulators in tensor memory, operands brought into shared memory by TMA) with the
// tensor-parallel collective fused into the same kernel:
//
//   mode kPlain           D[M,N] = A[M,K] * B[N,K]^T
//   mode kAllGatherGemm   column-parallel layer: A is sequence-sharded over the ranks.
//                         One thread of EVERY CTA drives the bulk-copy engine: 4 KiB
//                         pieces of this rank's shard pass through a small shared-memory
//                         ring into every peer's gather buffer over NVLink and are
//                         counted in on the destination; the GEMM starts with
//                         the local rows and takes up a remote 128-row block as soon as
//                         all of its pieces are counted in, loading it by TMA from LOCAL
//                         memory (no TMA ever reads a peer, no multicast).
//   mode kGemmReduceScatter  row-parallel layer: every output tile is a partial sum.
//                         The epilogue converts the accumulator tile into a swizzled
//                         shared-memory staging and sends it by TMA tile stores straight
//                         into the owning rank's partial buffer (remote owners first),
//                         then counts it in on that rank.  (Per-thread stores to a peer
//                         ran at a fifth of the link rate with the few threads an
//                         epilogue has.)  A rank's own rows come last: their epilogue
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
// 2-5 run the epilogue (one TMEM lane quarter each), warp 6 pushes (all-gather mode).
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
constexpr int kFlagStride = 16; // counters sit one per 128-byte line (see tp_gemm_args.h)
constexpr int kEpiCols = 64;                                // columns staged per epilogue step
constexpr int kRing = 4, kRingAhead = 2;                    // all-gather pusher: ring stages, loads in flight
constexpr uint32_t kPieceBytes = 4096;                      // bytes per ring stage; 4 x 4 KiB = sizeof(Smem::extra)

template <bool PAIR>
struct __align__(1024) Smem {
  static constexpr int STAGES = PAIR ? 6 : 4;
  static constexpr int BROWS = PAIR ? BN / 2 : BN; // rows of B this CTA loads per stage
  bf16 a[STAGES][BM * BK];
  bf16 b[STAGES][BROWS * BK];
  uint4 epi[4][32 * kEpiCols * 2 / 16]; // per epilogue warp: 32 rows x 64 bf16, 16-byte chunks swizzled
  // reduce-scatter mode: second staging buffer of every epilogue warp (TMA stores read
  // one while the warp fills the other); all-gather mode: the pusher's ring of pieces
  uint4 extra[4 * 32 * kEpiCols * 2 / 16];
  uint64_t full[STAGES], empty[STAGES], tmemFull[2], tmemEmpty[2], ringFull[kRing];
  uint32_t tmemBase;
  int abortFlag;
};

// ---- bulk-copy engine helpers (no load here names a peer, none is multicast) ----
__device__ __forceinline__ void bulkLoad(void *smemDst, const void *gsrc, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smemAddr(smemDst)),
               "l"(gsrc), "r"(bytes), "r"(smemAddr(bar))
               : "memory");
}
__device__ __forceinline__ void bulkStore(void *gdst, const void *smemSrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smemAddr(smemSrc)), "r"(bytes)
               : "memory");
}
// 2D tile store through a tensor map (box 64 columns x 32 rows, 128-byte swizzle)
__device__ __forceinline__ void tmaStore2d(const CUtensorMap *map, const void *smemSrc, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(c0), "r"(c1),
               "r"(smemAddr(smemSrc))
               : "memory");
}
__device__ __forceinline__ void bulkCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulkWaitRead() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
template <int N>
__device__ __forceinline__ void bulkWaitDone() { asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fenceProxyAsyncSmem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void redAddRelaxedSys(unsigned long long *p, unsigned long long v) {
  asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// Which tile the grid's i-th scheduling slot covers.  The row blocks are taken in an
// order that suits the mode (below), cut into runs of one rank's worth, and inside a
// run in groups of `groupRows` row blocks that are
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
  if (a.mode == kAllGatherGemm) {
    // own rows first; then the peers' rows in the order in which the pushers deliver
    // them: block 0 of every peer, block 1 of every peer, ...
    if (rb < bpr) {
      rb += rank * bpr;
    } else {
      const int peers = blocks / bpr - 1, j = rb - bpr;
      const int blk = j / peers, src = (rank + 1 + j % peers) % (peers + 1);
      rb = src * bpr + blk;
    }
  } else if (a.mode == kGemmReduceScatter) {
    rb = (rb + (rank + 1) * bpr) % blocks; // own rows last
  }
  *tm = rb;
}

__device__ __forceinline__ bool waitFlagGe(const flagcxDevComm &c, const unsigned long long *flag,
                                           unsigned long long want, volatile int *abortFlag, unsigned peer) {
  // Poll with relaxed loads and fence once at the end: a stream of acquire loads from
  // one warp made every system-scope fence of the CTA's other warps (the pusher's,
  // the epilogue's) take about a hundred microseconds.
  if (fcxdev::ldRelaxedSys(flag) >= want) { fcxdev::fenceSys(); return true; }
  const unsigned long long t0 = timerNs();
  unsigned spins = 0, ns = 100;
  for (;;) {
    if (fcxdev::ldRelaxedSys(flag) >= want) { fcxdev::fenceSys(); return true; }
    // back off: every poll is an L2 access on the line the peers' atomics must reach
    __nanosleep(ns);
    if (ns < 1600) ns *= 2;
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
                 const __grid_constant__ TpStoreMaps sm, const flagcxDevComm c, const TpGemmArgs a) {
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
    for (int i = 0; i < kRing; ++i) mbarInit(&s.ringFull[i], 1);
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
            ok = waitFlagGe(c, a.chunkFlags[rank] + kFlagStride * ((size_t)owner * chunks + (arow / BM) % chunks),
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
      bool tmaOut = false;          // reduce-scatter, a peer's rows: the tile leaves by TMA stores
      int tmaRow = 0;
      if (a.mode == kGemmReduceScatter) {
        owner = (int)(growBase / a.rowsPerRank);
        const size_t rowLocal = growBase - (size_t)owner * a.rowsPerRank;
        if (owner != rank) {
          // Per-thread stores to a peer are limited by the stores each thread may have
          // in flight; the copy engine is not.  Row of the owner's stacked partial buffer:
          tmaOut = true;
          tmaRow = rank * a.rowsPerRank + (int)rowLocal;
          dbase = a.partial[owner] + ((size_t)rank * a.rowsPerRank + rowLocal) * a.N;
        } else {
          // My own rows come last in the tile order, when the peers' partial sums of them
          // have (nearly) all landed here: wait for the row block's counter, then add
          // them to the accumulator tile on its way out and store the final rows.
          dbase = a.out + rowLocal * a.N;
          if (n > 1) {
            bool ok = true;
            if (lane == 0)
              ok = waitFlagGe(c, a.rowFlags[rank] + kFlagStride * (rowLocal / BM),
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
        // TMA stores alternate between the warp's two staging buffers; a buffer is
        // rewritten only after the engine has read its previous contents out
        uint4 *buf = (tmaOut && (cb & 1)) ? s.extra + (warp - 2) * (32 * kEpiCols * 2 / 16) : stg;
        if (lane == 0) {
          if (tmaOut) bulkWaitRead<1>(); else bulkWaitRead<0>();
        }
        __syncwarp();
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
          for (int i = 0; i < 4; ++i) buf[lane * 8 + ((h * 4 + i) ^ (lane & 7))] = o[i];
        }
        if (tmaOut) {
          // the staging layout is the tensor map's 128-byte swizzle: one store moves the 32 x 64 box
          fenceProxyAsyncSmem();
          __syncwarp();
          if (lane == 0) {
            tmaStore2d(&sm.m[owner], buf, tn * BN + cb * kEpiCols, tmaRow);
            bulkCommit();
          }
          continue;
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
        // Count the tile in on its owner once all four epilogue warps' stores are complete:
        // ONE remote atomic per tile, at once.  (Counting in one tile later, per warp, was
        // tried: with more than two ranks the counts a rank still held while it waited for
        // its own rows closed a circular wait, and with that fixed the four atomics per tile
        // on lines the owner's CTAs poll cost more than the deferral saved: 704 against
        // 426-497 us at 8 ranks.)
        if (lane == 0) { bulkWaitDone<0>(); fenceProxyAsync(); }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          fcxdev::fenceSys();
          const int rbLocal = (int)(((size_t)tm * TM + ctaRank * BM - (size_t)owner * a.rowsPerRank) / BM);
          fcxdev::redAddReleaseSys(a.rowFlags[owner] + kFlagStride * rbLocal, 1ull);
        }
      }
      if (++acc == 2) { acc = 0; accPhase ^= 1; }
    }
  } else if (warp == 6 && a.mode == kAllGatherGemm && n > 1) {
    // ---- pusher: one thread drives the copy engine.  My shard goes out in 4 KiB
    // pieces, chunk 0 first: bulk load into a ring stage, one bulk store per peer
    // from that stage, and once a piece's stores are complete it is counted in on
    // every peer.  The pieces of one chunk are spread over all CTAs. ----
    if (lane == 0) {
      const int chunks = a.rowsPerRank / BM;
      const size_t shardBytes = (size_t)a.rowsPerRank * a.K * 2;
      const size_t shardOff = (size_t)rank * shardBytes;
      const char *src = (const char *)a.gathered[rank] + shardOff;
      const long long nPieces = (long long)(shardBytes / kPieceBytes);
      const long long cnt = blockIdx.x < nPieces ? (nPieces - blockIdx.x + G - 1) / G : 0;
      char *ring = (char *)s.extra;
      auto pieceOf = [&](long long i) { return (size_t)blockIdx.x + (size_t)i * G; };
      auto issueLoad = [&](long long i) {
        const int st = (int)(i % kRing);
        mbarExpectTx(&s.ringFull[st], kPieceBytes);
        bulkLoad(ring + st * kPieceBytes, src + pieceOf(i) * kPieceBytes, kPieceBytes, &s.ringFull[st]);
      };
      // Completed pieces are counted in on the peers once per chunk (this CTA's pieces
      // of one chunk are consecutive): one fence and one atomic per peer and chunk.
      long long pendChunk = -1;
      unsigned long long pendCount = 0;
      auto flush = [&]() {
        if (pendCount == 0) return;
        fenceProxyAsync();
        fcxdev::fenceSys();
        for (int k = 1; k < n; ++k) {
          int p = rank + k; if (p >= n) p -= n;
          redAddRelaxedSys(a.chunkFlags[p] + kFlagStride * ((size_t)rank * chunks + pendChunk), pendCount);
        }
        pendCount = 0;
      };
      auto countIn = [&](long long i) {
        const long long ch = (long long)(pieceOf(i) / a.piecesPerChunk);
        if (ch != pendChunk) { flush(); pendChunk = ch; }
        ++pendCount;
      };
      for (long long i = 0; i < cnt && i < kRingAhead; ++i) issueLoad(i);
      long long i = 0;
      for (; i < cnt && !*abortFlag; ++i) {
        // stage of piece i+ahead = stage of piece i+ahead-ring, complete since the last iteration's wait
        if (i + kRingAhead < cnt) issueLoad(i + kRingAhead);
        const int st = (int)(i % kRing);
        if (!mbarWait(&s.ringFull[st], (uint32_t)(i / kRing) & 1u, abortFlag, kWaitLimitNs)) break;
        const size_t off = shardOff + pieceOf(i) * kPieceBytes;
        for (int k = 1; k < n; ++k) {
          int p = rank + k; if (p >= n) p -= n;
          bulkStore((char *)a.gathered[p] + off, ring + st * kPieceBytes, kPieceBytes);
        }
        bulkCommit();
        if (i >= 1) { bulkWaitDone<1>(); countIn(i - 1); }
      }
      bulkWaitDone<0>();
      if (i == cnt && cnt > 0) countIn(cnt - 1);
      flush();
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
cudaError_t launchTpGemm(cudaStream_t stream, const CUtensorMap &tmA, const CUtensorMap &tmB, const TpStoreMaps *maps,
                         const flagcxDevComm &c, const TpGemmArgs &a, int nCtas, bool pair) {
  static const TpStoreMaps noMaps = {};
  const TpStoreMaps &sm = maps ? *maps : noMaps;
  static bool configured[2] = {false, false};
  const void *fn = pair ? (const void *)tpGemmKernel<true> : (const void *)tpGemmKernel<false>;
  if (!configured[pair]) {
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)tpGemmSmemBytes(pair));
    if (e != cudaSuccess) return e;
    configured[pair] = true;
  }
  if (!pair) {
    tpGemmKernel<false><<<nCtas, kThreads, tpGemmSmemBytes(false), stream>>>(tmA, tmB, sm, c, a);
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
  return cudaLaunchKernelEx(&cfg, tpGemmKernel<true>, tmA, tmB, sm, c, a);
}

} // namespace fcx
