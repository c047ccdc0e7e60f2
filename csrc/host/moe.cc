// moe.cc -- host side of the expert-parallel dispatch/combine kernels: owns the
// peer-mapped receive, expert-output and partial-sum buffers, the count tables and the
// group records, and launches dispatch and combine.
#include <algorithm>

#include "../kernels/launch.h"
#include "../kernels/moe_args.h"
#include "comm.h"
#include "flagcx_ext.h"

using namespace fcx;

struct flagcxMoe {
  flagcxComm *comm;
  int maxTokens, hidden, topk, nExperts, epr;
  size_t capacity;
  // symmetric
  void *recv = nullptr, *expertOut = nullptr, *table = nullptr, *grp = nullptr, *partial = nullptr;
  Window *wRecv = nullptr, *wOut = nullptr, *wTable = nullptr, *wGrp = nullptr, *wPartial = nullptr;
  bool vmm[5] = {false, false, false, false, false};
  int grpRecordsPerSender = 0;
  size_t grpCountOff = 0, wRowOff = 0; // byte offsets of the count table and the per-row weights inside `grp`
  // local
  int *pos = nullptr, *route = nullptr, *expertOffsets = nullptr, *lead = nullptr;
  int lastTokens = 0;
  const int *lastIdx = nullptr;
};

namespace {

flagcxResult_t symAlloc(flagcxComm *c, size_t bytes, void **ptr, Window **win, bool *isVmm) {
  if (c->emu) {
    FCX_CUDACHECK(cudaMalloc(ptr, bytes));
    *isVmm = false;
    return emuWindowRegister(c, *ptr, bytes, FLAGCX_WIN_COLL_SYMMETRIC, win);
  }
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

void fillArgs(flagcxMoe *m, MoeArgs &a, int nTokens) {
  flagcxComm *c = m->comm;
  memset(&a, 0, sizeof a);
  for (int p = 0; p < c->nranks; ++p) {
    a.countsAll[p] = (int *)m->wTable->peer[p];
    a.recv[p] = (char *)m->wRecv->peer[p];
    a.expertOut[p] = (char *)m->wOut->peer[p];
    a.grpList[p] = (int *)m->wGrp->peer[p];
    a.grpCount[p] = (int *)((char *)m->wGrp->peer[p] + m->grpCountOff);
    a.wRow[p] = (float *)((char *)m->wGrp->peer[p] + m->wRowOff);
    a.partial[p] = (char *)m->wPartial->peer[p];
  }
  a.grpRecordsPerSender = m->grpRecordsPerSender;
  a.maxT = m->maxTokens;
  a.dedup = readParam("MOE_DEDUP", 1) != 0 ? 1 : 0;
  // Pre-reducing on the expert rank pays when a token has, on average, at least two experts
  // per rank it goes to (one row crosses NVLink instead of two or more; 523 -> 370 us on two
  // B200s with 64 experts, top-8); with eight ranks, 256 experts and top-8 a token reaches
  // 5.25 ranks, the saving is a third, and the extra local pass and barrier cost more (885
  // against 692 us).  Expected ranks per token for uniform routing: n (1 - (1 - 1/n)^k).
  {
    const double n = c->nranks, k = m->topk;
    double miss = 1.0;
    for (int i = 0; i < m->topk; ++i) miss *= 1.0 - 1.0 / n;
    const double ranksPerToken = n * (1.0 - miss);
    const int64_t dflt = k / ranksPerToken >= 2.0 ? 1 : 0;
    a.preReduce = readParam("MOE_COMBINE_REDUCE", dflt) != 0 ? 1 : 0;
  }
  a.lead = m->lead;
  a.pos = m->pos;
  a.route = m->route;
  a.expertOffsets = m->expertOffsets;
  a.T = nTokens;
  a.H = m->hidden;
  a.K = m->topk;
  a.E = m->nExperts;
  a.EPR = m->epr;
  a.capacity = m->capacity;
}

cudaError_t emuDispatch(const LaunchCtx &lc, const void *d) {
  LaunchCtx l2 = lc;
  l2.emuBlob = d;
  MoeArgs dummy{};
  dummy.E = 0;
  return launchMoeDispatch(l2, dummy);
}
cudaError_t emuCombine(const LaunchCtx &lc, const void *d) {
  LaunchCtx l2 = lc;
  l2.emuBlob = d;
  MoeArgs dummy{};
  return launchMoeCombine(l2, dummy, false);
}
cudaError_t emuCombinePull(const LaunchCtx &lc, const void *d) {
  LaunchCtx l2 = lc;
  l2.emuBlob = d;
  MoeArgs dummy{};
  return launchMoeCombine(l2, dummy, true);
}

int moeCtas(flagcxComm *c) {
  int64_t v = readParam("MOE_CTAS", 128); // CTAs of 256 threads
  return (int)std::max<int64_t>(1, std::min<int64_t>(v, FLAGCX_COLL_BARRIER_SLOTS));
}

} // namespace

extern "C" {

flagcxResult_t flagcxMoeCreate(flagcxComm_t comm, int maxTokens, int hidden, int topk, int nExperts,
                               size_t capacityRows, flagcxMoe_t *out) {
  if (!commValid(comm) || !out) return flagcxInvalidArgument;
  if (!comm->devicePath) return flagcxNotSupported;
  FCX_ARGCHECK(maxTokens > 0 && hidden > 0 && hidden % 8 == 0 && topk >= 1 && topk <= FLAGCX_MOE_MAX_TOPK &&
                   nExperts % comm->nranks == 0 && nExperts <= FLAGCX_MOE_MAX_EXPERTS && capacityRows > 0,
               "flagcxMoeCreate: hidden must be a multiple of 8, top-k at most %d, experts divisible by ranks",
               FLAGCX_MOE_MAX_TOPK);
  auto *m = new flagcxMoe();
  m->comm = comm;
  m->maxTokens = maxTokens;
  m->hidden = hidden;
  m->topk = topk;
  m->nExperts = nExperts;
  m->epr = nExperts / comm->nranks;
  m->capacity = capacityRows;
  size_t rows = capacityRows * (size_t)hidden * 2;
  flagcxResult_t r = symAlloc(comm, rows, &m->recv, &m->wRecv, &m->vmm[0]);
  if (r == flagcxSuccess) r = symAlloc(comm, rows, &m->expertOut, &m->wOut, &m->vmm[1]);
  if (r == flagcxSuccess)
    r = symAlloc(comm, alignUp(sizeof(int) * (size_t)comm->nranks * nExperts, 4096), &m->table, &m->wTable, &m->vmm[2]);
  // group records: per sender (maxTokens + one token per possible CTA) x topk records of
  // FLAGCX_MOE_MAX_TOPK ints, then the [sender][CTA] count table, then one gate weight per
  // received row
  m->grpRecordsPerSender = (maxTokens + FLAGCX_COLL_BARRIER_SLOTS) * topk;
  m->grpCountOff = alignUp((size_t)comm->nranks * m->grpRecordsPerSender * FLAGCX_MOE_MAX_TOPK * sizeof(int), 4096);
  m->wRowOff = m->grpCountOff + alignUp(sizeof(int) * (size_t)comm->nranks * FLAGCX_COLL_BARRIER_SLOTS, 4096);
  if (r == flagcxSuccess)
    r = symAlloc(comm, m->wRowOff + alignUp(sizeof(float) * capacityRows, 4096), &m->grp, &m->wGrp, &m->vmm[3]);
  if (r == flagcxSuccess) r = symAlloc(comm, rows, &m->partial, &m->wPartial, &m->vmm[4]);
  if (r != flagcxSuccess) { delete m; return r; }
  size_t items = (size_t)maxTokens * topk;
  FCX_CUDACHECK(cudaMalloc((void **)&m->pos, sizeof(int) * items));
  FCX_CUDACHECK(cudaMalloc((void **)&m->route, sizeof(int) * items * 2));
  FCX_CUDACHECK(cudaMalloc((void **)&m->expertOffsets, sizeof(int) * (m->epr + 1)));
  FCX_CUDACHECK(cudaMalloc((void **)&m->lead, sizeof(int) * items));
  FCX_CUDACHECK(cudaMemset(m->table, 0, sizeof(int) * (size_t)comm->nranks * nExperts));
  FCX_CUDACHECK(cudaDeviceSynchronize());
  *out = m;
  return flagcxSuccess;
}

flagcxResult_t flagcxMoeDestroy(flagcxMoe_t m) {
  if (!m) return flagcxSuccess;
  flagcxComm *c = m->comm;
  cudaDeviceSynchronize();
  if (!c->emu && c->bootstrap) c->bootstrap->barrier();
  symFree(c, m->recv, m->wRecv, m->vmm[0]);
  symFree(c, m->expertOut, m->wOut, m->vmm[1]);
  symFree(c, m->table, m->wTable, m->vmm[2]);
  symFree(c, m->grp, m->wGrp, m->vmm[3]);
  symFree(c, m->partial, m->wPartial, m->vmm[4]);
  cudaFree(m->pos);
  cudaFree(m->route);
  cudaFree(m->expertOffsets);
  cudaFree(m->lead);
  delete m;
  return flagcxSuccess;
}

flagcxResult_t flagcxMoeGetBuffers(flagcxMoe_t m, void **recvRows, void **expertOutRows, int **expertOffsets) {
  if (!m) return flagcxInvalidArgument;
  if (recvRows) *recvRows = m->recv;
  if (expertOutRows) *expertOutRows = m->expertOut;
  if (expertOffsets) *expertOffsets = m->expertOffsets;
  return flagcxSuccess;
}

flagcxResult_t flagcxMoeDispatch(flagcxMoe_t m, const void *x, const int *topkIdx, int nTokens, flagcxStream_t stream) {
  if (!m || !x || !topkIdx || nTokens < 0 || nTokens > m->maxTokens) return flagcxInvalidArgument;
  flagcxComm *c = m->comm;
  if (c->asyncError.load() != flagcxSuccess) return (flagcxResult_t)c->asyncError.load();
  cudaStream_t s = stream ? stream->base : nullptr;
  MoeArgs a;
  fillArgs(m, a, nTokens);
  a.x = (const __nv_bfloat16 *)x;
  a.topkIdx = topkIdx;
  cudaError_t e;
  m->lastTokens = nTokens;
  m->lastIdx = topkIdx;
  c->stats[flagcxCommOpAlltoAllv].calls++;
  c->stats[flagcxCommOpAlltoAllv].bytes += (size_t)nTokens * m->topk * m->hidden * 2;
  if (c->emu) return emuSubmitBlob(c, 100, &a, sizeof a, moeCtas(c), s, emuDispatch);
  LaunchCtx lc;
  lc.comm = &c->dev;
  lc.stream = s;
  lc.nCtas = moeCtas(c);
  e = launchMoeDispatch(lc, a);
  if (e != cudaSuccess) { FCX_WARN("moe dispatch launch failed: %s", cudaGetErrorString(e)); return flagcxUnhandledDeviceError; }
  return flagcxSuccess;
}

flagcxResult_t flagcxMoeCombine(flagcxMoe_t m, const float *topkWeights, void *out, int nTokens, flagcxStream_t stream) {
  if (!m || !topkWeights || !out || nTokens != m->lastTokens) {
    FCX_WARN("flagcxMoeCombine must follow a flagcxMoeDispatch of the same tokens");
    return flagcxInvalidArgument;
  }
  flagcxComm *c = m->comm;
  if (c->asyncError.load() != flagcxSuccess) return (flagcxResult_t)c->asyncError.load();
  cudaStream_t s = stream ? stream->base : nullptr;
  MoeArgs a;
  fillArgs(m, a, nTokens);
  a.topkIdx = m->lastIdx;
  a.topkW = topkWeights;
  a.out = (__nv_bfloat16 *)out;
  const bool pull = a.preReduce == 0;
  if (c->emu) return emuSubmitBlob(c, pull ? 102 : 101, &a, sizeof a, moeCtas(c), s, pull ? emuCombinePull : emuCombine);
  LaunchCtx lc;
  lc.comm = &c->dev;
  lc.stream = s;
  lc.nCtas = moeCtas(c);
  cudaError_t e = launchMoeCombine(lc, a, pull);
  if (e != cudaSuccess) { FCX_WARN("moe combine launch failed: %s", cudaGetErrorString(e)); return flagcxUnhandledDeviceError; }
  return flagcxSuccess;
}

} // extern "C"
