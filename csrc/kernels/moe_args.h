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
  // A token that goes to several experts of one rank crosses NVLink once.  For every
  // (token, destination rank) the sender leaves the destination a GROUP record: the rows
  // that token occupies there, leader first (rows[0] got the data over NVLink; the
  // receiver copies it to the others).  The combine uses the same records the other way:
  // the expert rank adds up a group's weighted outputs locally and the token's owner pulls
  // one row per group.  grpList[p] / grpCount[p]: rank p's record area
  // [sender][CTA][records per CTA] and count table [sender][CTA], as mapped here.
  int *grpList[FLAGCX_MAX_RANKS];   // records of FLAGCX_MOE_MAX_TOPK ints, -1 = unused
  int *grpCount[FLAGCX_MAX_RANKS];
  int grpRecordsPerSender; // records reserved per sender in a rank's area
  int maxT;                // largest token count any rank may pass (fixes the per-CTA share of that area)
  int dedup;               // 0: every (token, expert) pair crosses NVLink on its own (groups of one)
  int preReduce;           // combine: 1 = expert ranks pre-reduce each group, 0 = owners pull every pair
  int *lead;               // local [T*K]: per token, the pair indices of its group leaders packed to the front, then -1
  float *wRow[FLAGCX_MAX_RANKS];     // wRow[p]: rank p's gate weight per received row (pushed by the combine)
  char *partial[FLAGCX_MAX_RANKS];   // partial[p]: rank p's pre-reduced rows, indexed by the group's leader row
  int T, H, K, E, EPR;
  size_t capacity;         // rows in recv / expertOut
};

} // namespace fcx
