// tp_gemm_args.h -- argument block of the tcgen05 GEMM / fused tensor-parallel kernels.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <stddef.h>

#include "flagcx_device.cuh"

namespace fcx {

enum TpGemmMode : int { kPlain = 0, kAllGatherGemm = 1, kGemmReduceScatter = 2 };

// GEMM -> reduce-scatter: tensor maps of every rank's partial buffer [nRanks * rowsPerRank, N]
// (box 64 columns x 32 rows, 128-byte swizzle) for the epilogue's TMA stores.
struct TpStoreMaps {
  CUtensorMap m[FLAGCX_MAX_RANKS];
};

struct TpGemmArgs {
  __nv_bfloat16 *D; // [M, N] output (plain, all-gather modes)
  int M, N, K, mode;
  int rowsPerRank;  // M / nRanks
  int piecesPerChunk; // all-gather mode: a 128-row chunk travels in this many 4 KiB pieces per peer
  int groupRows;      // tile order: this many row blocks are walked together, column by column
  unsigned long long epoch; // call counter of this handle, starts at 1
  // all-gather -> GEMM
  __nv_bfloat16 *gathered[FLAGCX_MAX_RANKS];      // rank p's gather buffer [M, K] as mapped here
  // counters are spaced 128 bytes apart (16 u64): polls of one never delay atomics on another
  unsigned long long *chunkFlags[FLAGCX_MAX_RANKS]; // rank p's counters [nRanks][rowsPerRank/128]
  // GEMM -> reduce-scatter
  __nv_bfloat16 *partial[FLAGCX_MAX_RANKS];       // rank p's partial buffer [nRanks][rowsPerRank, N]
  unsigned long long *rowFlags[FLAGCX_MAX_RANKS];   // rank p's counters [rowsPerRank/128]
  __nv_bfloat16 *out;                              // [rowsPerRank, N] reduced rows of this rank
};

} // namespace fcx
