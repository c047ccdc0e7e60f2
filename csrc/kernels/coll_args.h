// coll_args.h -- argument blocks shared by the host launcher and the collective
// kernels.  Plain data, passed to the kernels by value.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "flagcx_device.cuh"

namespace fcx {

// What a launch computes.  Every collective kernel has the same skeleton:
//   [copy user input into the peer-visible staging]  -> barrier ->
//   main phase (peer loads and/or peer stores)       -> barrier ->
//   [copy staged output to the user buffer]
enum CollKind : int {
  kAllReduceOneShot = 0, // every rank reduces everything from all peers
  kAllReduceTwoShot,     // reduce own slice from all peers, write it to all peers
  kReduceScatter,        // reduce own block from all peers into the local output
  kReduceToRoot,         // root reduces everything from all peers
  kAllGatherPush,        // write own block into every peer's output
  kAllGatherPull,        // read every peer's block into the local output
  kBroadcastPush,        // root writes to every peer's output
  kBroadcastPull,        // everyone reads from the root's input
  kGatherPull,           // root reads every peer's input
  kScatterPull,          // everyone reads its block of the root's input
  kAllToAllPush,         // write block p of the input into peer p's output block `rank`
  kAllToAllPull,         // read block `rank` of peer p's input into output block p
  kAllToAllvPull,        // as above with per-peer counts/displacements via the meta pad
  kBarrierOnly,
  kAllReduceNvlsOneShot, // multimem.ld_reduce everything -> local output
  kAllReduceNvlsTwoShot, // multimem.ld_reduce own slice -> multimem.st to all
  kReduceScatterNvls,    // multimem.ld_reduce own block -> local output
  kAllGatherNvls,        // multimem.st own block to all
  kAllReduceTwoShotCast, // reduce own slice into local 16-bit scratch, then pull all slices and widen to fp32
  kLlAllReduce,          // small messages: data+flag stores into per-sender slots, no barrier
  kLlAllGather,
  kLlReduceScatter,      // block p of the input goes to rank p, which reduces what it receives
  kLlAllToAll,           // block p of the input goes to rank p's output block `rank`
  kAllGatherRing,        // n-1 steps: forward the block received in the previous step to the next rank
  kReduceScatterRing,    // n-1 steps: add the own block to the partial sum received and pass it on
  kAllReduceRing,        // ring reduce-scatter into the output, then ring all-gather of it
  kNumCollKinds
};

enum CollFlags : uint32_t {
  kFlagBeginBarrier = 1u << 0,
  kFlagEndBarrier = 1u << 1,
};

enum OutMode : int { kOutSame = 0, kOutFloat = 1, kOutBf16 = 2 };

// Which of a rank's buffers the kernel learns from its peers at run time
// (CollArgs::xchg).  A rank whose buffer is not inside a symmetric window cannot know
// on the host where its peers' buffers are; instead every rank tells each peer,
// before the kernel's first barrier, where ITS buffer is in that peer's address space.
enum XchgBits : uint32_t { kXchgIn = 1u << 0, kXchgOut = 1u << 1 };
// Pointer pad of a rank (inside its internal window): [parity][cta slot][source rank][in,out].
#define FLAGCX_PTRPAD_WORDS (2 * FLAGCX_COLL_BARRIER_SLOTS * FLAGCX_MAX_RANKS * 2)

// Reduction operator as the kernels see it (flagcxAvg arrives as sum plus a scale).
enum : int { kOpSum = 0, kOpProd = 1, kOpMax = 2, kOpMin = 3, kOpRuntime = -1 };

// Elements per rank-slice when `count` elements are cut for nRanks, rounded up to
// whole 16-byte packs so slice boundaries stay vector-aligned.
#ifdef __CUDACC__
__host__ __device__
#endif
inline size_t sliceElems(size_t count, int nRanks, size_t elemSize) {
  size_t perPack = 16 / elemSize;
  size_t s = (count + nRanks - 1) / nRanks;
  return (s + perPack - 1) / perPack * perPack;
}

struct CollArgs {
  const char *in[FLAGCX_MAX_RANKS]; // in[p]: rank p's input as mapped here
  char *out[FLAGCX_MAX_RANKS];      // out[p]: rank p's output as mapped here
  const char *mcIn;                 // multicast alias of the inputs (NVLS kinds)
  char *mcOut;                      // multicast alias of the outputs (NVLS kinds)
  const char *userIn;               // if set: copied into in[rank] before the first barrier
  char *userOut;                    // if set: out[rank] is copied here after the last barrier
  const char *residual;             // optional: added to the result before the store
  unsigned long long *meta[FLAGCX_MAX_RANKS]; // per-rank pad of 2*FLAGCX_MAX_RANKS u64 (alltoallv)
  // run-time pointer exchange (xchg != 0): pubIn[p] / pubOut[p] is this rank's input /
  // output as rank p addresses it; ptrPad[p] is rank p's pointer pad as mapped here
  const char *pubIn[FLAGCX_MAX_RANKS];
  char *pubOut[FLAGCX_MAX_RANKS];
  unsigned long long *ptrPad[FLAGCX_MAX_RANKS];
  // aux[p]: a region of rank p's internal window as mapped here.  kAllReduceTwoShotCast:
  // the 16-bit scratch that holds rank p's reduced slice.  LL kinds: rank p's slot area,
  // laid out [parity][sender][llSlotBytes].
  char *aux[FLAGCX_MAX_RANKS];
  // ring kinds: step flags, one u64 per CTA slot, monotonic over the communicator's life.
  // A rank raises ringNext[b] at its successor and waits on ringMine[b]; step s of this
  // launch uses the value ringBase + s + 1.  aux[] holds each rank's partial-sum scratch
  // (n-1 slots of ringSlotElems elements, one per step, so no slot is reused in a launch).
  unsigned long long *ringNext, *ringMine;
  unsigned long long ringBase;
  size_t ringSlotElems;
  size_t llSlotBytes;
  uint32_t llEpoch;    // value of the flags of this operation (never 0)
  uint32_t llPad;
  uint32_t xchg;       // XchgBits
  uint32_t xchgParity; // alternates between consecutive exchanging launches of a communicator
  // Bytes every rank's input / output region spans from in[p] / out[p] (0: not known).
  // Only the bounds-checking build (FLAGCX_BOUNDS_CHECK) reads them: before its main
  // phase a kernel verifies that everything it is about to touch lies inside.
  size_t inBytes, outBytes;
  size_t count;        // elements: total (allreduce, reduce, broadcast) or per rank-block
  // Rank-blocks inside the in/out buffers start at multiples of these byte strides
  // (reduce-scatter, gather, scatter, allgather, alltoall).
  size_t inStride, outStride;
  // copy-in: nInBlocks blocks of inBlockBytes, block j read at userIn + j*userInStride
  // and stored at in[rank] + j*inStride (j*inBlockBytes when inStride is 0)
  size_t userInStride, inBlockBytes;
  int nInBlocks;
  // copy-out: same scheme from out[rank] to userOut
  int nOutBlocks;
  size_t userOutStride, outBlockBytes;
  // when blocks are laid back to back, the last one may be short: total bytes of
  // all blocks (0: every block is full)
  size_t inTotalBytes, outTotalBytes;
  float scale;  // result multiplier (1 = none), floating types
  int divisor;  // integer average: divide by this (0 = none)
  int kind, dtype, elemSize, redOp, outMode, root;
  uint32_t flags;
  int bulkDepth; // stages of that ring: 8 or 12
  int bulkStage; // push kinds: bytes per shared-memory stage of the bulk-copy path (0: per-thread loads/stores)
  // alltoallv (element units), this rank's view
  size_t sendCounts[FLAGCX_MAX_RANKS], sendDispls[FLAGCX_MAX_RANKS];
  size_t recvCounts[FLAGCX_MAX_RANKS], recvDispls[FLAGCX_MAX_RANKS];
};

// ---- grouped point-to-point -----------------------------------------------------
// One launch moves, for every peer, at most one message out and one message in.
// Transfers are chunked through a slot in the SENDER's staging: the sender waits
// until the receiver consumed the previous chunk, copies, and raises `ready` at the
// receiver; the receiver waits for `ready`, copies out of the sender's slot, and
// raises `done` at the sender.  Flags are per (pair, CTA) and count chunks since the
// communicator was created, so only the two ranks of a pair ever wait on each other.
#define FLAGCX_P2P_CTAS 8

struct P2pArgs {
  const char *sendSrc[FLAGCX_MAX_RANKS]; // local user pointers (NULL: nothing to send)
  char *recvDst[FLAGCX_MAX_RANKS];       // local user pointers (NULL: nothing to receive)
  size_t sendBytes[FLAGCX_MAX_RANKS];
  size_t recvBytes[FLAGCX_MAX_RANKS];
  char *stage[FLAGCX_MAX_RANKS];              // stage[p]: rank p's p2p staging; slot (s->r) at stage[s] + r*slotBytes
  unsigned long long *ready[FLAGCX_MAX_RANKS]; // ready[p]: rank p's pad, entry [src*FLAGCX_P2P_CTAS + cta]
  unsigned long long *done[FLAGCX_MAX_RANKS];  // done[p]:  rank p's pad, entry [dst*FLAGCX_P2P_CTAS + cta]
  unsigned long long sendSeq[FLAGCX_MAX_RANKS]; // chunks sent to / received from each peer before this launch
  unsigned long long recvSeq[FLAGCX_MAX_RANKS];
  size_t slotBytes;
};

} // namespace fcx
