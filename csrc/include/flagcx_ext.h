/*
 * flagcx_ext.h -- entry points beyond the FlagCX-compatible surface of flagcx.h:
 * collectives with a fused epilogue, explicit algorithm choice, the tuner,
 * per-operation statistics, and the emulated world used to run multi-rank
 * kernels on a single GPU.
 */
#ifndef FLAGCX_EXT_H_
#define FLAGCX_EXT_H_
#include "flagcx.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Algorithms of the device path.  FLAGCX_ALGO_AUTO lets the tuner decide. */
typedef enum {
  FLAGCX_ALGO_AUTO = -1,
  FLAGCX_ALGO_ONESHOT = 0,      /* allreduce: every rank reduces all data from all peers */
  FLAGCX_ALGO_TWOSHOT = 1,      /* allreduce: reduce own slice, write it to all peers */
  FLAGCX_ALGO_NVLS_ONESHOT = 2, /* allreduce: multimem.ld_reduce everything */
  FLAGCX_ALGO_NVLS_TWOSHOT = 3, /* allreduce: multimem.ld_reduce own slice + multimem.st */
  FLAGCX_ALGO_PUSH = 4,         /* allgather/broadcast/alltoall: write into the peers' outputs */
  FLAGCX_ALGO_PULL = 5,         /* reduce-scatter/allgather/...: read from the peers' inputs */
  FLAGCX_ALGO_NVLS = 6,         /* reduce-scatter: multimem.ld_reduce; allgather: multimem.st */
  FLAGCX_ALGO_LL = 7,           /* allreduce/allgather of small messages: data+flag stores, no barrier */
  FLAGCX_ALGO_RING = 8,         /* allreduce/reduce-scatter/allgather in n-1 neighbour-to-neighbour steps */
  FLAGCX_ALGO_COPY_ENGINE = 9,  /* the data crosses NVLink on the DMA copy engines, between two one-CTA barrier
                                   kernels: allgather into a window; reduce-scatter of any buffers (peer copies
                                   into the staging area, then a reduce over local memory only) */
  FLAGCX_ALGO_COUNT = 10
} flagcxAlgo_t;

/* Optional work fused into the store of a reducing collective. */
typedef struct {
  float scale;               /* result multiplier; 1.0f for none (flagcxAvg already implies 1/nranks) */
  flagcxDataType_t outDtype; /* flagcxNumTypes: same as input; flagcxFloat32 for 16-bit inputs;
                                flagcxBfloat16 for fp32 inputs */
  const void *residual;      /* added to the result (in the output type), or NULL */
  int algo;                  /* flagcxAlgo_t or FLAGCX_ALGO_AUTO */
  int nCtas;                 /* <=0: automatic */
} flagcxFusedOpts_t;

#define FLAGCX_FUSED_OPTS_INITIALIZER {1.0f, flagcxNumTypes, NULL, FLAGCX_ALGO_AUTO, 0}

flagcxResult_t flagcxAllReduceFused(const void *sendbuff, void *recvbuff, size_t count,
                                    flagcxDataType_t datatype, flagcxRedOp_t op,
                                    const flagcxFusedOpts_t *opts, flagcxComm_t comm,
                                    flagcxStream_t stream);
flagcxResult_t flagcxReduceScatterFused(const void *sendbuff, void *recvbuff, size_t recvcount,
                                        flagcxDataType_t datatype, flagcxRedOp_t op,
                                        const flagcxFusedOpts_t *opts, flagcxComm_t comm,
                                        flagcxStream_t stream);
/* Non-reducing collectives with an explicit algorithm / CTA count. */
flagcxResult_t flagcxAllGatherEx(const void *sendbuff, void *recvbuff, size_t sendcount,
                                 flagcxDataType_t datatype, int algo, int nCtas, flagcxComm_t comm,
                                 flagcxStream_t stream);

/* ---- tuner ------------------------------------------------------------------ */
/* Collective.  Measures every applicable (algorithm, CTA count) for `op` over the
 * sizes minBytes..maxBytes (powers of two) on registered scratch buffers, keeps the
 * fastest per size (max over ranks, CUDA events), and agrees on it across ranks. */
flagcxResult_t flagcxTunerTune(flagcxComm_t comm, flagcxCommOp_t op, flagcxDataType_t dtype,
                               size_t minBytes, size_t maxBytes, int iters);
flagcxResult_t flagcxTunerSave(flagcxComm_t comm, const char *path);
flagcxResult_t flagcxTunerLoad(flagcxComm_t comm, const char *path);
/* What the tuner would pick. */
flagcxResult_t flagcxTunerQuery(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, int registered,
                                int *algo, int *nCtas);

/* ---- statistics ----------------------------------------------------------------- */
typedef struct {
  uint64_t calls;
  uint64_t bytes;
  int lastAlgo;
  int lastCtas;
  float lastMs; /* device time of the last profiled call (0 when profiling is off) */
} flagcxOpStats_t;
flagcxResult_t flagcxCommGetStats(flagcxComm_t comm, flagcxCommOp_t op, flagcxOpStats_t *out);
/* Trace: a ring of the last `capacity` collective calls of this communicator (operation,
 * bytes, route, algorithm, CTAs, host time, device time between two CUDA events on the
 * caller's stream).  capacity 0 switches it off.  FLAGCX_TRACE=<capacity> enables it at
 * init; FLAGCX_TRACE_FILE=<path, %r = rank> writes it at flagcxCommDestroy.  Dump
 * synchronises the recorded events, fills flagcxOpStats_t.lastMs and writes JSON.
 * FLAGCX_NVTX=1 additionally opens an NVTX range around every collective. */
flagcxResult_t flagcxCommTraceEnable(flagcxComm_t comm, int capacity);
flagcxResult_t flagcxCommTraceDump(flagcxComm_t comm, const char *path);
/* User buffers outside registered windows (ordinary cudaMalloc memory, e.g. PyTorch
 * tensors) are exported to the peers the first time a collective meets them, one-sidedly
 * and without staging copies afterwards; flagcxCommRegister does the same ahead of time.
 * Counters of this rank: lookups served from the cache, allocations exported, allocations
 * that could not be exported (they go through an exportable stand-in), stale entries
 * replaced after the address was freed and reused, allocations of peers mapped / unmapped
 * here.  enabled is 0 when FLAGCX_USER_BUFFER_EXPORT=0 or the service could not start. */
typedef struct {
  int enabled;
  uint64_t hits, exports, refused, stale, peerOpened, peerClosed;
} flagcxUserBufferStats_t;
flagcxResult_t flagcxCommUserBufferStats(flagcxComm_t comm, flagcxUserBufferStats_t *out);
/* Not collective.  Has every peer unmap the exported allocation that contains ptr (nothing
 * happens if there is none).  Call it before the allocation is freed: an allocation must
 * not be freed while another process still has it mapped.  Allocator integrations call
 * this from their "segment is about to be released" hook (the torch backend does); no
 * collective of any rank may still be using the memory. */
flagcxResult_t flagcxCommForgetUserBuffer(flagcxComm_t comm, const void *ptr);
/* By default only buffers registered with flagcxCommRegister (by every rank) are exported;
 * other device buffers are staged.  on != 0 exports every device buffer a collective meets.
 * The caller then guarantees that flagcxCommForgetUserBuffer (or flagcxCommDeregister) runs
 * before any such allocation is freed -- typically from an allocator hook.  Every rank must
 * make the same choice before its next collective.  FLAGCX_USER_BUFFER_EXPORT=2 has the same
 * effect from the environment; =0 switches the mechanism off altogether. */
flagcxResult_t flagcxCommSetAutoExport(flagcxComm_t comm, int on);
/* 1 when collectives on device buffers run as NVLink kernels, 0 on the socket path. */
flagcxResult_t flagcxCommIsDevicePath(flagcxComm_t comm, int *yes);
flagcxResult_t flagcxCommHasMulticast(flagcxComm_t comm, int *yes);
/* Sets the bound of every device-side wait of this communicator. */
flagcxResult_t flagcxCommSetWaitTimeoutMs(flagcxComm_t comm, int ms);
/* Peer-mapped address of `offset` within a registered window as seen from this rank. */
flagcxResult_t flagcxWindowGetPeerPointer(flagcxWindow_t win, int peer, size_t offset, void **ptr);
flagcxResult_t flagcxWindowGetMulticastPointer(flagcxWindow_t win, size_t offset, void **ptr);

/* ---- one-sided API: release --------------------------------------------------------------
 * Collective.  flagcxOneSideDeregister forgets all memory regions of flagcxOneSideRegister
 * (region indices start at 0 again) and unmaps the windows those calls created;
 * flagcxOneSideSignalDeregister releases the signal buffer's window. */
flagcxResult_t flagcxOneSideDeregister(flagcxComm_t comm);
flagcxResult_t flagcxOneSideSignalDeregister(flagcxComm_t comm);

/* ---- emulated world ----------------------------------------------------------------
 * nranks communicators inside one process on one GPU.  A collective call on one
 * of them is parked until all of them have made the matching call; the last call
 * launches ONE cooperative kernel in which blockIdx.y plays the rank, so the
 * multi-rank protocols (barriers, peer loads/stores) run unchanged on a single
 * GPU.  Buffers of emulated ranks see each other without registration. */
flagcxResult_t flagcxEmuWorldCreate(int nranks, int device, flagcxComm_t *comms);
flagcxResult_t flagcxEmuWorldDestroy(flagcxComm_t anyRank);

/* ---- expert-parallel (MoE) dispatch / combine ------------------------------------------
 * Create is collective: it allocates, on every rank, a peer-mapped receive buffer and an
 * expert-output buffer of capacityRows x hidden bf16 each.  Experts are spread evenly:
 * rank r owns experts [r*E/n, (r+1)*E/n).
 *
 * Dispatch copies every (token, chosen expert) row to the owning rank, grouped by
 * expert; afterwards the rows of local expert e are recvRows[offsets[e] .. offsets[e+1]).
 * The caller runs its experts over those rows and writes the results to the same rows of
 * expertOutRows.  Combine then produces out[t] = sum_k weights[t,k] * expertOut(t,k).
 * A dispatch whose rows exceed capacityRows on some rank is reported through
 * flagcxCommGetAsyncError (flagcxInvalidArgument); nothing is written out of bounds. */
typedef struct flagcxMoe *flagcxMoe_t;
flagcxResult_t flagcxMoeCreate(flagcxComm_t comm, int maxTokens, int hidden, int topk, int nExperts,
                               size_t capacityRows, flagcxMoe_t *moe);
flagcxResult_t flagcxMoeDestroy(flagcxMoe_t moe);
flagcxResult_t flagcxMoeGetBuffers(flagcxMoe_t moe, void **recvRows, void **expertOutRows, int **expertOffsets);
flagcxResult_t flagcxMoeDispatch(flagcxMoe_t moe, const void *x, const int *topkIdx, int nTokens,
                                 flagcxStream_t stream);
flagcxResult_t flagcxMoeCombine(flagcxMoe_t moe, const float *topkWeights, void *out, int nTokens,
                                flagcxStream_t stream);

/* ---- tensor-core GEMM and fused tensor-parallel layers ---------------------------------
 * All matrices are bf16, row-major with K contiguous: D[M,N] = A[M,K] * B[N,K]^T, fp32
 * accumulation on the tcgen05 tensor cores.  M %% 128 == 0, N %% 256 == 0, K %% 64 == 0. */
flagcxResult_t flagcxGemmBf16(const void *A, const void *B, void *D, int M, int N, int K, flagcxStream_t stream);

/* mode 1, all-gather -> GEMM (column-parallel): the activation matrix [M,K] is split by
 * rows over the ranks.  Each rank writes its [M/n, K] shard at the address returned by
 * flagcxTpGemmGetShard and calls flagcxTpAllGatherGemm with its weight slice B[N,K]; one
 * kernel moves the shards between the ranks and computes D[M,N], starting with the local
 * rows and taking up remote rows as they arrive.
 * mode 2, GEMM -> reduce-scatter (row-parallel): each rank holds A[M,K] and B[N,K] for its
 * slice of K; one kernel computes the partial products, delivers every tile to the rank
 * that owns its rows and sums the partials there: out[M/n, N].
 * Create/Destroy are collective. */
typedef struct flagcxTpGemm *flagcxTpGemm_t;
flagcxResult_t flagcxTpGemmCreate(flagcxComm_t comm, int mode, int M, int N, int K, flagcxTpGemm_t *handle);
flagcxResult_t flagcxTpGemmDestroy(flagcxTpGemm_t handle);
flagcxResult_t flagcxTpGemmGetShard(flagcxTpGemm_t handle, void **localShard);
flagcxResult_t flagcxTpAllGatherGemm(flagcxTpGemm_t handle, const void *B, void *D, flagcxStream_t stream);
flagcxResult_t flagcxTpGemmReduceScatter(flagcxTpGemm_t handle, const void *A, const void *B, void *out,
                                         flagcxStream_t stream);

/* Host-side element-wise reduction used by the socket path (exposed for tests). */
flagcxResult_t flagcxHostReduce(void *dst, const void *src, size_t count, flagcxDataType_t dtype,
                                flagcxRedOp_t op);

#ifdef __cplusplus
}
#endif
#endif
