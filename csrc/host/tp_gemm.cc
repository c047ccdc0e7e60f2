// tp_gemm.cc -- host side of the tcgen05 GEMM and of the fused tensor-parallel kernels
// (all-gather -> GEMM, GEMM -> reduce-scatter): symmetric buffers and flags, TMA tensor
// maps, launches.
#include <algorithm>
#include <map>

#include "../kernels/launch.h"
#include "../kernels/tp_gemm_args.h"
#include "comm.h"
#include "flagcx_ext.h"

namespace fcx {
size_t tpGemmSmemBytes(bool pair);
cudaError_t launchTpGemm(cudaStream_t stream, const CUtensorMap &tmA, const CUtensorMap &tmB, const TpStoreMaps *maps,
                         const flagcxDevComm &c, const TpGemmArgs &a, int nCtas, bool pair);
} // namespace fcx

using namespace fcx;

struct flagcxTpGemm {
  flagcxComm *comm;
  int mode, M, N, K, rowsPerRank;
  void *buf = nullptr, *flags = nullptr;
  Window *wBuf = nullptr, *wFlags = nullptr;
  bool vmmBuf = false, vmmFlags = false;
  unsigned long long epoch = 0;
  CUtensorMap tmGather;
  TpStoreMaps storeMaps;
  std::map<const void *, CUtensorMap> mapsA, mapsB;
};

namespace {

// CTA pairs (256-row tiles, cta_group::2) whenever the row blocks allow it.
bool usePair(int rowsPerOwner) { return readParam("GEMM_PAIR", 1) != 0 && rowsPerOwner % 256 == 0; }

// Row blocks walked together by the tile order: the grid (74 pairs or 148 CTAs) then
// covers a near-square patch of the output at any moment.
int groupRows(bool pair) { return std::max(1, (int)readParam("GEMM_GROUP", pair ? 8 : 16)); }

int smCount() {
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms > 0 ? sms : 1;
}

flagcxResult_t checkShape(int M, int N, int K) {
  FCX_ARGCHECK(M > 0 && N > 0 && K > 0 && M % 128 == 0 && N % 256 == 0 && K % 64 == 0,
               "tcgen05 GEMM needs M %% 128 == 0, N %% 256 == 0, K %% 64 == 0 (got %d x %d x %d)", M, N, K);
  return flagcxSuccess;
}

flagcxResult_t symAlloc(flagcxComm *c, size_t bytes, void **ptr, Window **win, bool *isVmm) {
  cu::VmmBlock b;
  if (cu::vmmSupported(c->cudaDev) && readParam("VMM_ENABLE", 1) != 0) {
    FCXCHECK(cu::vmmAlloc(bytes, c->cudaDev, &b));
    *ptr = b.ptr;
    *isVmm = true;
  } else {
    FCX_CUDACHECK(cudaMalloc(ptr, bytes));
    *isVmm = false;
  }
  return windowRegister(c, *ptr, bytes, FLAGCX_WIN_COLL_SYMMETRIC, win);
}

void symFree(flagcxComm *c, void *ptr, Window *win, bool isVmm) {
  if (!ptr) return;
  if (win) windowDeregister(c, win);
  if (isVmm) {
    if (const cu::VmmBlock *b = cu::vmmLookup(ptr)) { cu::VmmBlock copy = *b; cu::vmmFree(&copy); }
  } else {
    cudaFree(ptr);
  }
}

flagcxResult_t cachedMap(std::map<const void *, CUtensorMap> &cache, const void *base, uint64_t rows, uint64_t cols,
                         uint32_t boxRows, const CUtensorMap **out) {
  auto it = cache.find(base);
  if (it == cache.end()) {
    CUtensorMap m;
    FCXCHECK(cu::tensorMap2dBf16(&m, base, rows, cols, boxRows, 64));
    if (cache.size() > 256) cache.clear();
    it = cache.emplace(base, m).first;
  }
  *out = &it->second;
  return flagcxSuccess;
}

} // namespace

extern "C" {

flagcxResult_t flagcxGemmBf16(const void *A, const void *B, void *D, int M, int N, int K, flagcxStream_t stream) {
  if (!A || !B || !D) return flagcxInvalidArgument;
  if (!cu::available()) return flagcxNotSupported;
  FCXCHECK(checkShape(M, N, K));
  CUtensorMap ta, tb;
  FCXCHECK(cu::tensorMap2dBf16(&ta, A, M, K, 128, 64));
  const bool pair = usePair(M);
  FCXCHECK(cu::tensorMap2dBf16(&tb, B, N, K, pair ? 128 : 256, 64));
  flagcxDevComm c;
  memset(&c, 0, sizeof c);
  c.nRanks = 1;
  c.timeoutNs = 4000000000ull;
  TpGemmArgs a;
  memset(&a, 0, sizeof a);
  a.D = (__nv_bfloat16 *)D;
  a.M = M; a.N = N; a.K = K;
  a.mode = kPlain;
  a.rowsPerRank = M;
  a.groupRows = groupRows(pair);
  int tiles = (M / 128) * (N / 256);
  if (pair) tiles = 2 * ((M / 256) * (N / 256));
  cudaError_t e = launchTpGemm(stream ? stream->base : nullptr, ta, tb, nullptr, c, a, std::min(tiles, smCount()), pair);
  if (e != cudaSuccess) { FCX_WARN("GEMM launch failed: %s", cudaGetErrorString(e)); return flagcxUnhandledDeviceError; }
  return flagcxSuccess;
}

flagcxResult_t flagcxTpGemmCreate(flagcxComm_t comm, int mode, int M, int N, int K, flagcxTpGemm_t *out) {
  if (!commValid(comm) || !out) return flagcxInvalidArgument;
  if (!comm->devicePath || comm->emu) return flagcxNotSupported;
  FCXCHECK(checkShape(M, N, K));
  const int n = comm->nranks;
  FCX_ARGCHECK((mode == kAllGatherGemm || mode == kGemmReduceScatter) && M % (128 * n) == 0,
               "flagcxTpGemmCreate: mode must be 1 (all-gather->GEMM) or 2 (GEMM->reduce-scatter) and M a multiple of 128 x ranks");
  auto *h = new flagcxTpGemm();
  h->comm = comm;
  h->mode = mode;
  h->M = M; h->N = N; h->K = K;
  h->rowsPerRank = M / n;
  const int chunks = h->rowsPerRank / 128;
  size_t bufBytes = mode == kAllGatherGemm ? (size_t)M * K * 2 : (size_t)M * N * 2;
  size_t flagBytes = alignUp(128 * (size_t)n * chunks, 4096); // one counter per 128-byte line
  flagcxResult_t r = symAlloc(comm, bufBytes, &h->buf, &h->wBuf, &h->vmmBuf);
  if (r == flagcxSuccess) r = symAlloc(comm, flagBytes, &h->flags, &h->wFlags, &h->vmmFlags);
  if (r != flagcxSuccess) { delete h; return r; }
  FCX_CUDACHECK(cudaMemset(h->flags, 0, flagBytes));
  FCX_CUDACHECK(cudaDeviceSynchronize());
  if (mode == kAllGatherGemm) FCXCHECK(cu::tensorMap2dBf16(&h->tmGather, h->buf, M, K, 128, 64));
  memset(&h->storeMaps, 0, sizeof h->storeMaps);
  if (mode == kGemmReduceScatter)
    for (int p = 0; p < n; ++p) FCXCHECK(cu::tensorMap2dBf16(&h->storeMaps.m[p], h->wBuf->peer[p], M, N, 32, 64));
  FCXCHECK(comm->bootstrap->barrier()); // flags are zero everywhere before anyone raises one
  *out = h;
  return flagcxSuccess;
}

flagcxResult_t flagcxTpGemmDestroy(flagcxTpGemm_t h) {
  if (!h) return flagcxSuccess;
  flagcxComm *c = h->comm;
  cudaDeviceSynchronize();
  if (c->bootstrap) c->bootstrap->barrier();
  symFree(c, h->buf, h->wBuf, h->vmmBuf);
  symFree(c, h->flags, h->wFlags, h->vmmFlags);
  delete h;
  return flagcxSuccess;
}

flagcxResult_t flagcxTpGemmGetShard(flagcxTpGemm_t h, void **localShard) {
  if (!h || !localShard || h->mode != kAllGatherGemm) return flagcxInvalidArgument;
  *localShard = (char *)h->buf + (size_t)h->comm->rank * h->rowsPerRank * h->K * 2;
  return flagcxSuccess;
}

flagcxResult_t flagcxTpAllGatherGemm(flagcxTpGemm_t h, const void *B, void *D, flagcxStream_t stream) {
  if (!h || !B || !D || h->mode != kAllGatherGemm) return flagcxInvalidArgument;
  flagcxComm *c = h->comm;
  if (c->asyncError.load() != flagcxSuccess) return (flagcxResult_t)c->asyncError.load();
  const CUtensorMap *tb;
  const bool pair = usePair(h->rowsPerRank);
  FCXCHECK(cachedMap(h->mapsB, B, h->N, h->K, pair ? 128 : 256, &tb));
  TpGemmArgs a;
  memset(&a, 0, sizeof a);
  a.D = (__nv_bfloat16 *)D;
  a.M = h->M; a.N = h->N; a.K = h->K;
  a.mode = kAllGatherGemm;
  a.rowsPerRank = h->rowsPerRank;
  a.groupRows = groupRows(pair);
  a.epoch = ++h->epoch;
  for (int p = 0; p < c->nranks; ++p) {
    a.gathered[p] = (__nv_bfloat16 *)h->wBuf->peer[p];
    a.chunkFlags[p] = (unsigned long long *)h->wFlags->peer[p];
  }
  const int sms = smCount();
  a.piecesPerChunk = h->K / 16; // a chunk is 128 rows of K bf16 = K/16 pieces of 4 KiB
  cudaError_t e = launchTpGemm(stream ? stream->base : nullptr, h->tmGather, *tb, nullptr, c->dev, a, sms, pair);
  if (e != cudaSuccess) { FCX_WARN("all-gather GEMM launch failed: %s", cudaGetErrorString(e)); return flagcxUnhandledDeviceError; }
  return flagcxSuccess;
}

flagcxResult_t flagcxTpGemmReduceScatter(flagcxTpGemm_t h, const void *A, const void *B, void *out,
                                         flagcxStream_t stream) {
  if (!h || !A || !B || !out || h->mode != kGemmReduceScatter) return flagcxInvalidArgument;
  flagcxComm *c = h->comm;
  if (c->asyncError.load() != flagcxSuccess) return (flagcxResult_t)c->asyncError.load();
  const CUtensorMap *ta, *tb;
  const bool pair = usePair(h->rowsPerRank);
  FCXCHECK(cachedMap(h->mapsA, A, h->M, h->K, 128, &ta));
  FCXCHECK(cachedMap(h->mapsB, B, h->N, h->K, pair ? 128 : 256, &tb));
  TpGemmArgs a;
  memset(&a, 0, sizeof a);
  a.M = h->M; a.N = h->N; a.K = h->K;
  a.mode = kGemmReduceScatter;
  a.rowsPerRank = h->rowsPerRank;
  a.groupRows = groupRows(pair);
  a.epoch = ++h->epoch;
  a.out = (__nv_bfloat16 *)out;
  for (int p = 0; p < c->nranks; ++p) {
    a.partial[p] = (__nv_bfloat16 *)h->wBuf->peer[p];
    a.rowFlags[p] = (unsigned long long *)h->wFlags->peer[p];
  }
  cudaError_t e = launchTpGemm(stream ? stream->base : nullptr, *ta, *tb, &h->storeMaps, c->dev, a, smCount(), pair);
  if (e != cudaSuccess) { FCX_WARN("GEMM reduce-scatter launch failed: %s", cudaGetErrorString(e)); return flagcxUnhandledDeviceError; }
  return flagcxSuccess;
}

} // extern "C"
