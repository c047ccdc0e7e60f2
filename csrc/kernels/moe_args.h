// moe_args.h -- argument block of the MoE dispatch / combine kernels.
#pragma once
#include <cuda_bf16.h>
#include <stddef.h>

#include "flagcx_device.cuh"

#define FLAGCX_MOE_MAX_TOPK 8
#define FLAGCX_MOE_MAX_EXPERTS 1024

namespace fcx {

struct MoeArgs {
  const __nv_bfloat16 *x;  // [T, H] local activations (dispatch input)
  const int *topkIdx;      // [T, K] global expert ids
  const float *topkW;      // [T, K] gate weights (combine)
  __nv_bfloat16 *out;      // [T, H] combine output
  int *countsAll[FLAGCX_MAX_RANKS]; // countsAll[p]: rank p's table [nRanks][E]; row r = counts of rank r
  int *pos;                // [T*K] index of the pair within its (source rank, expert) group
  int *route;              // [T*K][2] destination rank and row of each pair
  char *recv[FLAGCX_MAX_RANKS];      // recv[p]: rank p's receive buffer [capacity, H] bf16
  char *expertOut[FLAGCX_MAX_RANKS]; // expertOut[p]: rank p's expert outputs, same row order
  int *expertOffsets;      // local [EPR + 1]: row range of each local expert
  // A token that goes to several experts of one rank crosses NVLink once: the first copy
  // lands in its final row, and a (source row, destination row) record asks the receiver
  // to make the other copies locally.  dupList[p] / dupCount[p]: rank p's record area
  // [sender][CTA][dupCapPerCta] and count table [sender][CTA], as mapped here.
  int2 *dupList[FLAGCX_MAX_RANKS];
  int *dupCount[FLAGCX_MAX_RANKS];
  int dupRecordsPerSender; // records reserved per sender in a rank's area
  int maxT;                // largest token count any rank may pass (fixes the per-CTA share of that area)
  int dedup;               // 0: every (token, expert) pair crosses NVLink on its own
  int T, H, K, E, EPR;
  size_t capacity;         // rows in recv / expertOut
};

} // namespace fcx
