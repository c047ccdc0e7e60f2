// emu.cc -- the emulated world: several ranks inside one process on one GPU.
//
// Kernels that wait on one another must not run as separate launches on one GPU
// (nothing guarantees they are co-resident).  So an emulated rank's collective call
// is only recorded; when the last rank of the world has made its call the world
// launches ONE cooperative kernel with gridDim.y = nranks, in which blockIdx.y
// selects the rank's communicator and argument block.  The kernels, barriers and
// peer accesses are exactly those of the multi-GPU path; "peer memory" is simply
// another rank's buffer on the same device.
#include <algorithm>

#include "../kernels/launch.h"
#include "comm.h"
#include "tuner.h"

namespace fcx {

constexpr int kArgRing = 16;

struct EmuWorld {
  int n = 0, dev = 0;
  std::vector<flagcxComm *> comms;
  std::vector<void *> internalBase;
  // pending submissions of the current collective
  int posted = 0;
  int family = -1, nCtas = 0;
  std::vector<char> has;
  std::vector<CollArgs> coll;
  std::vector<P2pArgs> p2p;
  // device copies
  flagcxDevComm *dComms = nullptr;
  CollArgs *dColl = nullptr; // kArgRing * n
  P2pArgs *dP2p = nullptr;   // kArgRing * n
  // generic kernels (MoE, fused GEMMs): opaque per-rank argument blocks
  std::vector<std::vector<char>> blob;
  char *dBlob = nullptr;     // kArgRing * n * kMaxBlobBytes
  int blobKernel = -1;
  int ring = 0;
  int maxGrid = 0;
};

flagcxResult_t emuWorldCreate(int nranks, int dev, flagcxComm **out) {
  if (nranks < 1 || nranks > FLAGCX_MAX_RANKS) return flagcxInvalidArgument;
  if (!cu::available()) { FCX_WARN("an emulated world needs a GPU"); return flagcxNotSupported; }
  logInit();
  FCX_CUDACHECK(cudaSetDevice(dev));
  int coop = 0;
  cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev);
  if (!coop) { FCX_WARN("device %d cannot do cooperative launches", dev); return flagcxNotSupported; }
  auto *w = new EmuWorld();
  w->n = nranks;
  w->dev = dev;
  w->has.assign(nranks, 0);
  w->coll.resize(nranks);
  w->p2p.resize(nranks);
  SyncLayout layout{};
  for (int r = 0; r < nranks; ++r) {
    auto *c = new flagcxComm();
    c->magic = kCommMagic;
    c->rank = r;
    c->nranks = nranks;
    c->localRank = r;
    c->localRanks = nranks;
    c->cudaDev = dev;
    c->devicePath = true;
    c->emu = w;
    w->comms.push_back(c);
  }
  // internal windows: cudaMalloc, peers are the other ranks' allocations
  layout = makeSyncLayout();
  for (int r = 0; r < nranks; ++r) {
    void *base = nullptr;
    FCX_CUDACHECK(cudaMalloc(&base, layout.total));
    FCX_CUDACHECK(cudaMemset(base, 0, layout.zeroedBytes));
    w->internalBase.push_back(base);
  }
  for (int r = 0; r < nranks; ++r) {
    flagcxComm *c = w->comms[r];
    c->layout = layout;
    FCXCHECK(allocLocalDeviceState(c));
    auto *win = new Window();
    win->local = w->internalBase[r];
    win->size = layout.total;
    win->internal = true;
    for (int p = 0; p < nranks; ++p) win->peer[p] = w->internalBase[p];
    c->internalWin = win;
    fillDevComm(c);
    c->tuner.reset(new Tuner());
    FCXCHECK(c->tuner->init(c));
  }
  FCX_CUDACHECK(cudaMalloc((void **)&w->dComms, sizeof(flagcxDevComm) * nranks));
  FCX_CUDACHECK(cudaMalloc((void **)&w->dColl, sizeof(CollArgs) * nranks * kArgRing));
  FCX_CUDACHECK(cudaMalloc((void **)&w->dP2p, sizeof(P2pArgs) * nranks * kArgRing));
  FCX_CUDACHECK(cudaMalloc((void **)&w->dBlob, (size_t)kMaxEmuBlobBytes * nranks * kArgRing));
  w->blob.resize(nranks);
  w->maxGrid = maxCoresidentCtas(FLAGCX_DEVICE_THREADS_PER_CTA);
  FCX_CUDACHECK(cudaDeviceSynchronize());
  for (int r = 0; r < nranks; ++r) out[r] = w->comms[r];
  FCX_INFO(SUB_INIT, "emulated world of %d ranks on device %d (up to %d co-resident CTAs)", nranks, dev, w->maxGrid);
  return flagcxSuccess;
}

// Window registration among emulated ranks: rank r's k-th registration pairs with
// every other rank's k-th; the peer tables are completed as ranks arrive.
flagcxResult_t emuWindowRegister(flagcxComm *c, void *buff, size_t size, int flags, Window **out) {
  EmuWorld *w = c->emu;
  auto *win = new Window();
  win->local = buff;
  win->size = size;
  win->flags = flags;
  win->peer[c->rank] = buff;
  for (int p = 0; p < c->nranks; ++p) win->selfAt[p] = buff; // one address space
  const int seq = c->winSeq++;
  for (flagcxComm *o : w->comms) {
    if (o == c) continue;
    for (Window *ow : o->windows.all()) {
      if (ow->internal || ow->flags < 0) continue;
      if (ow->emuSeq == seq) {
        ow->peer[c->rank] = buff;
        win->peer[o->rank] = ow->local;
      }
    }
  }
  win->emuSeq = seq;
  c->windows.add(win);
  *out = win;
  return flagcxSuccess;
}

flagcxResult_t emuWorldDestroy(flagcxComm *any) {
  EmuWorld *w = any->emu;
  if (!w) return flagcxInvalidArgument;
  cudaSetDevice(w->dev);
  cudaDeviceSynchronize();
  for (int r = 0; r < w->n; ++r) {
    flagcxComm *c = w->comms[r];
    for (Window *win : c->windows.all()) delete win;
    delete c->internalWin;
    if (c->localSync) cudaFree(c->localSync);
    if (c->status) cudaFreeHost(c->status);
    if (c->internalStream) cudaStreamDestroy(c->internalStream);
    cudaFree(w->internalBase[r]);
    c->magic = 0;
    delete c;
  }
  cudaFree(w->dComms);
  cudaFree(w->dColl);
  cudaFree(w->dP2p);
  cudaFree(w->dBlob);
  delete w;
  return flagcxSuccess;
}

flagcxResult_t emuSubmit(flagcxComm *c, int family, const CollArgs *coll, const P2pArgs *p2p, int nCtas,
                         cudaStream_t stream) {
  EmuWorld *w = c->emu;
  const int n = w->n, r = c->rank;
  if (w->has[r]) {
    FCX_WARN("emulated rank %d posted a second collective before the others posted their first", r);
    return flagcxInvalidUsage;
  }
  if (w->posted == 0) { w->family = family; w->nCtas = nCtas; }
  if (family != w->family) {
    FCX_WARN("emulated ranks posted different kinds of operations");
    return flagcxInvalidUsage;
  }
  w->nCtas = std::min(w->nCtas, nCtas);
  if (coll) w->coll[r] = *coll;
  if (p2p) w->p2p[r] = *p2p;
  w->has[r] = 1;
  if (++w->posted < n) return flagcxSuccess;

  // everybody is here: complete the peer tables and launch once
  w->posted = 0;
  std::fill(w->has.begin(), w->has.end(), 0);
  const int slot = w->ring++ % kArgRing;
  LaunchCtx lc;
  lc.stream = stream;
  lc.emuRanks = n;
  lc.nCtas = std::max(1, std::min(w->nCtas, std::max(1, w->maxGrid / n)));
  std::vector<flagcxDevComm> devs(n);
  for (int q = 0; q < n; ++q) devs[q] = w->comms[q]->dev;
  FCX_CUDACHECK(cudaMemcpyAsync(w->dComms, devs.data(), sizeof(flagcxDevComm) * n, cudaMemcpyHostToDevice, stream));
  lc.emuComms = w->dComms;
  cudaError_t e;
  if (family == 3) {
    lc.nCtas = FLAGCX_P2P_CTAS;
    if (FLAGCX_P2P_CTAS * n > w->maxGrid) { FCX_WARN("p2p grid does not fit the device"); return flagcxInternalError; }
    P2pArgs *d = w->dP2p + (size_t)slot * n;
    FCX_CUDACHECK(cudaMemcpyAsync(d, w->p2p.data(), sizeof(P2pArgs) * n, cudaMemcpyHostToDevice, stream));
    lc.emuP2p = d;
    e = launchP2pKernel(lc, w->p2p[0]);
  } else {
    for (int q = 0; q < n; ++q) {
      if (w->coll[q].kind != w->coll[0].kind) { FCX_WARN("emulated ranks chose different algorithms"); return flagcxInvalidUsage; }
      for (int p = 0; p < n; ++p) {
        // a rank that exchanges pointers inside the kernel must get them from there
        if (!w->coll[q].in[p] && !(w->coll[q].xchg & kXchgIn)) w->coll[q].in[p] = w->coll[p].in[p];
        if (!w->coll[q].out[p] && !(w->coll[q].xchg & kXchgOut)) w->coll[q].out[p] = w->coll[p].out[p];
      }
    }
    for (int q = 0; q < n; ++q) lc.emuBulk |= w->coll[q].bulkStage != 0;
    CollArgs *d = w->dColl + (size_t)slot * n;
    FCX_CUDACHECK(cudaMemcpyAsync(d, w->coll.data(), sizeof(CollArgs) * n, cudaMemcpyHostToDevice, stream));
    lc.emuArgs = d;
    e = family == 0   ? launchReduceKernel(lc, w->coll[0], n)
        : family == 1 ? launchCopyKernel(lc, w->coll[0])
        : family == 4 ? launchLlKernel(lc, w->coll[0])
                      : cudaErrorNotSupported;
  }
  if (e != cudaSuccess) {
    FCX_WARN("emulated-world launch failed: %s", cudaGetErrorString(e));
    return flagcxUnhandledDeviceError;
  }
  return flagcxSuccess;
}

// Generic variant for kernels with their own argument block (MoE, fused GEMMs): the
// blocks are parked per rank; the last arrival copies them to the device and calls
// `launch(ctx, deviceArray)`, which must do ONE cooperative launch with
// gridDim.y = ctx.emuRanks.
flagcxResult_t emuSubmitBlob(flagcxComm *c, int kernelId, const void *args, size_t argBytes, int nCtas,
                             cudaStream_t stream, EmuBlobLaunch launch) {
  EmuWorld *w = c->emu;
  const int n = w->n, r = c->rank;
  if (argBytes > (size_t)kMaxEmuBlobBytes) return flagcxInternalError;
  if (w->has[r]) {
    FCX_WARN("emulated rank %d posted a second operation before the others posted their first", r);
    return flagcxInvalidUsage;
  }
  if (w->posted == 0) { w->blobKernel = kernelId; w->nCtas = nCtas; }
  if (kernelId != w->blobKernel) {
    FCX_WARN("emulated ranks posted different kinds of operations");
    return flagcxInvalidUsage;
  }
  w->nCtas = std::min(w->nCtas, nCtas);
  w->blob[r].assign((const char *)args, (const char *)args + argBytes);
  w->has[r] = 1;
  if (++w->posted < n) return flagcxSuccess;
  w->posted = 0;
  std::fill(w->has.begin(), w->has.end(), 0);
  const int slot = w->ring++ % kArgRing;
  std::vector<flagcxDevComm> devs(n);
  for (int q = 0; q < n; ++q) devs[q] = w->comms[q]->dev;
  FCX_CUDACHECK(cudaMemcpyAsync(w->dComms, devs.data(), sizeof(flagcxDevComm) * n, cudaMemcpyHostToDevice, stream));
  char *d = w->dBlob + (size_t)slot * n * kMaxEmuBlobBytes;
  std::vector<char> packed((size_t)n * argBytes);
  for (int q = 0; q < n; ++q) memcpy(packed.data() + (size_t)q * argBytes, w->blob[q].data(), argBytes);
  FCX_CUDACHECK(cudaMemcpyAsync(d, packed.data(), packed.size(), cudaMemcpyHostToDevice, stream));
  LaunchCtx lc;
  lc.stream = stream;
  lc.emuRanks = n;
  lc.emuComms = w->dComms;
  lc.nCtas = std::max(1, std::min(w->nCtas, std::max(1, w->maxGrid / n)));
  cudaError_t e = launch(lc, d);
  if (e != cudaSuccess) {
    FCX_WARN("emulated-world launch failed: %s", cudaGetErrorString(e));
    return flagcxUnhandledDeviceError;
  }
  return flagcxSuccess;
}

} // namespace fcx
