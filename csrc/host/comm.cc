// comm.cc -- communicator construction/destruction, the device world (internal
// window with barrier inboxes, signal pads, alltoallv pads and staging), window
// registration over CUDA VMM file descriptors or legacy IPC handles, optional
// NVLink multicast binding, and the device-status watchdog.
//
// What FlagCX spreads over flagcx/flagcx.cc:1943-2358 (init), core/init.cc:90-262
// (peer info, same-host detection, duplicate-GPU check), core/sym_heap.cc:23-377
// (symmetric window: physical alloc, fd exchange, flat map, multicast bind) and
// adaptor/flagcx_device.cc:295-437 (IPC peer pointers) happens here once per
// communicator, without proxy threads.
#include "comm.h"

#include <unistd.h>

#include <algorithm>
#include <chrono>

#include "tuner.h"

namespace fcx {

// Collectives on unregistered buffers pass through this window in chunks of its size; on
// B200 pairs 256 MiB measured 389 GB/s against 298 with 64 MiB (all-reduce, 256 MiB bf16),
// and 0.14 % of the HBM is a small price.
FCX_PARAM(StagingBytes, "STAGING_BYTES", 256ll << 20)
FCX_PARAM(WaitTimeoutMs, "WAIT_TIMEOUT_MS", 10000)
FCX_PARAM(P2pDisable, "P2P_DISABLE", 0)
FCX_PARAM(VmmEnable, "VMM_ENABLE", 1)
FCX_PARAM(NvlsEnable, "NVLS_ENABLE", 0)
FCX_PARAM(WatchdogMs, "WATCHDOG_MS", 200)
FCX_PARAM(P2pSlotBytes, "P2P_SLOT_BYTES", 4ll << 20)
FCX_PARAM(UserBufferExport, "USER_BUFFER_EXPORT", 1)
// largest message (bytes of data) the LL slots can hold; every rank keeps
// 2 * FLAGCX_MAX_RANKS slots of twice this size
FCX_PARAM(LlSlotDataBytes, "LL_SLOT_BYTES", 64 << 10)

// ---------------------------------------------------------------------------
// window registry
// ---------------------------------------------------------------------------
void WindowRegistry::add(Window *w) {
  std::lock_guard<std::mutex> g(mu_);
  byBase_[(uintptr_t)w->local] = w;
}
void WindowRegistry::remove(Window *w) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = byBase_.find((uintptr_t)w->local);
  if (it != byBase_.end() && it->second == w) byBase_.erase(it);
}
Window *WindowRegistry::find(const void *p, size_t bytes) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = byBase_.upper_bound((uintptr_t)p);
  if (it == byBase_.begin()) return nullptr;
  --it;
  Window *w = it->second;
  uintptr_t b = it->first;
  if ((uintptr_t)p >= b && (uintptr_t)p + bytes <= b + w->size) return w;
  return nullptr;
}
std::vector<Window *> WindowRegistry::all() const {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<Window *> v;
  for (auto &kv : byBase_) v.push_back(kv.second);
  return v;
}

bool commValid(const flagcxComm *c) { return c && c->magic == kCommMagic; }

// ---------------------------------------------------------------------------
// peer discovery
// ---------------------------------------------------------------------------
namespace {

struct PeerInfo {
  uint64_t hostHash;
  uint64_t pidHash;
  int32_t cudaDev; // -1: no GPU
  int32_t vmm;     // VMM + fd export usable
  int32_t mc;      // multicast usable
  int32_t pad;
  char busId[32];
};

SyncLayout makeLayout() {
  SyncLayout l;
  size_t off = 0;
  l.inboxOff = off;
  off += (size_t)FLAGCX_BARRIER_SLOTS * FLAGCX_MAX_RANKS * sizeof(uint64_t);
  l.signalOff = off;
  off += (size_t)FLAGCX_MAX_SIGNALS * sizeof(uint64_t);
  l.metaOff = off;
  off += 4 * FLAGCX_MAX_RANKS * sizeof(uint64_t);
  l.p2pReadyOff = off;
  off += (size_t)FLAGCX_MAX_RANKS * FLAGCX_P2P_CTAS * sizeof(uint64_t);
  l.p2pDoneOff = off;
  off += (size_t)FLAGCX_MAX_RANKS * FLAGCX_P2P_CTAS * sizeof(uint64_t);
  l.ptrPadOff = off;
  off += (size_t)FLAGCX_PTRPAD_WORDS * sizeof(uint64_t);
  l.ringOff = off;
  off += (size_t)FLAGCX_COLL_BARRIER_SLOTS * sizeof(uint64_t);
  // LL slots are compared against flag values: they start zeroed like the pads above
  off = alignUp(off, 256);
  l.llOff = off;
  l.llSlotBytes = alignUp((size_t)std::max<int64_t>(paramLlSlotDataBytes(), 1024) * 2, 256);
  off += 2 * (size_t)FLAGCX_MAX_RANKS * l.llSlotBytes;
  off = alignUp(off, 1 << 16);
  l.zeroedBytes = off;
  l.stagingOff = off;
  l.stagingBytes = alignUp((size_t)std::max<int64_t>(paramStagingBytes(), 1 << 20), 1 << 16);
  off += l.stagingBytes;
  l.p2pStageOff = off;
  l.p2pSlotBytes = alignUp((size_t)std::max<int64_t>(paramP2pSlotBytes(), 1 << 16), 1 << 16);
  off += l.p2pSlotBytes * FLAGCX_MAX_RANKS;
  l.total = off;
  return l;
}

void watchdogMain(flagcxComm *c) {
  while (!c->watchdogStop.load()) {
    commCheckDevice(c);
    std::this_thread::sleep_for(std::chrono::milliseconds(paramWatchdogMs()));
  }
}

} // namespace

SyncLayout makeSyncLayout() { return makeLayout(); }

void fillDevComm(flagcxComm *c) {
  flagcxDevComm &d = c->dev;
  memset(&d, 0, sizeof d);
  d.rank = c->rank;
  d.nRanks = c->nranks;
  d.intraRank = c->localRank;
  d.intraSize = c->localRanks;
  for (int p = 0; p < c->nranks; ++p) {
    char *base = (char *)c->internalWin->peer[p];
    d.barrierInbox[p] = (unsigned long long *)(base + c->layout.inboxOff);
    d.signalPad[p] = (unsigned long long *)(base + c->layout.signalOff);
  }
  char *ls = (char *)c->localSync;
  d.barrierEpoch = (unsigned long long *)ls;
  d.signalShadow = d.barrierEpoch + FLAGCX_BARRIER_SLOTS;
  d.counters = d.signalShadow + FLAGCX_MAX_SIGNALS;
  d.mcSignalPad = c->internalWin->mc ? (unsigned long long *)((char *)c->internalWin->mc + c->layout.signalOff) : nullptr;
  d.status = c->statusDev;
  d.timeoutNs = (unsigned long long)std::max<int64_t>(readParam("WAIT_TIMEOUT_MS", paramWaitTimeoutMs()), 1) * 1000000ull;
  d.nSignals = FLAGCX_MAX_SIGNALS;
  d.nCounters = FLAGCX_MAX_COUNTERS;
  d.nvlsBarrier = d.mcSignalPad && readParam("NVLS_BARRIER", 0) != 0 ? 1 : 0;
}

flagcxResult_t allocLocalDeviceState(flagcxComm *c) {
  size_t syncWords = (size_t)FLAGCX_BARRIER_SLOTS + FLAGCX_MAX_SIGNALS + FLAGCX_MAX_COUNTERS;
  size_t localBytes = syncWords * sizeof(uint64_t) + 256;
  FCX_CUDACHECK(cudaMalloc(&c->localSync, localBytes));
  FCX_CUDACHECK(cudaMemset(c->localSync, 0, localBytes));
  c->putArrival = (unsigned int *)((char *)c->localSync + syncWords * sizeof(uint64_t));
  FCX_CUDACHECK(cudaHostAlloc((void **)&c->rmaCounter, sizeof(uint64_t), cudaHostAllocMapped));
  *c->rmaCounter = 0;
  FCX_CUDACHECK(cudaHostAlloc((void **)&c->status, sizeof(flagcxDevStatus), cudaHostAllocMapped));
  memset(c->status, 0, sizeof(flagcxDevStatus));
  FCX_CUDACHECK(cudaHostGetDevicePointer((void **)&c->statusDev, c->status, 0));
  FCX_CUDACHECK(cudaStreamCreateWithFlags(&c->internalStream, cudaStreamNonBlocking));
  c->signalSent.assign(c->nranks, 0);
  c->signalSeen.assign(c->nranks, 0);
  return flagcxSuccess;
}

// ---------------------------------------------------------------------------
// window registration
// ---------------------------------------------------------------------------
namespace {

struct WinExchange {
  uint64_t size;      // window size
  uint64_t offset;    // offset of the window inside its allocation
  uint64_t allocSize; // size of the allocation (what gets mapped)
  int32_t method;     // 0: VMM fd, 1: cudaIpc
  int32_t wantMc;
  cudaIpcMemHandle_t ipc;
};

} // namespace

flagcxResult_t windowRegister(flagcxComm *c, void *buff, size_t size, int flags, Window **out) {
  if (!c->devicePath) return flagcxNotSupported;
  const int n = c->nranks, me = c->rank;
  auto w = std::make_unique<Window>();
  w->local = buff;
  w->size = size;
  w->flags = flags;

  const cu::VmmBlock *blk = cu::vmmLookup(buff);
  std::vector<WinExchange> ex(n);
  WinExchange &mine = ex[me];
  memset(&mine, 0, sizeof mine);
  mine.size = size;
  if (blk) {
    mine.method = 0;
    mine.offset = (uintptr_t)buff - (uintptr_t)blk->ptr;
    mine.allocSize = blk->size;
    mine.wantMc = (c->nvls && mine.offset == 0) ? 1 : 0;
  } else {
    void *base = nullptr;
    size_t asz = 0;
    FCXCHECK(cu::addressRange(buff, &base, &asz));
    mine.method = 1;
    mine.offset = (uintptr_t)buff - (uintptr_t)base;
    mine.allocSize = asz;
    FCX_CUDACHECK(cudaIpcGetMemHandle(&mine.ipc, base));
  }
  FCXCHECK(c->bootstrap->allGather(ex.data(), sizeof(WinExchange)));
  bool sameMethod = true, sameSize = true, allMc = true;
  for (int p = 0; p < n; ++p) {
    sameMethod &= ex[p].method == mine.method;
    sameSize &= ex[p].size == mine.size;
    allMc &= ex[p].wantMc == 1 && ex[p].allocSize == mine.allocSize;
  }
  if (!sameMethod || !sameSize) {
    FCX_WARN("window registration: ranks disagree on size or allocator (all ranks must pass buffers of "
             "one size from the same kind of allocation)");
    return flagcxInvalidArgument;
  }
  w->peer[me] = buff;
  const int seq = ++c->winSeq; // same order of collective calls on every rank
  if (mine.method == 0) {
    FdChannel ch;
    uint64_t key = c->bootstrap->nonce() ^ ((uint64_t)seq << 48) ^ 0x57494eull;
    FCXCHECK(ch.open(key, me));
    FCXCHECK(c->bootstrap->barrier()); // every rank is bound before anyone sends
    int fd = -1;
    FCXCHECK(cu::vmmExportFd(*blk, &fd));
    for (int i = 1; i < n; ++i) FCXCHECK(ch.sendFd(key, (me + i) % n, fd, (uint64_t)me));
    for (int i = 1; i < n; ++i) {
      int pfd = -1;
      uint64_t from = 0;
      FCXCHECK(ch.recvFd(&pfd, &from, defaultSocketTimeoutMs()));
      if (from >= (uint64_t)n || w->peer[from]) { ::close(pfd); return flagcxInternalError; }
      cu::VmmBlock imp;
      flagcxResult_t r = cu::vmmImportFd(pfd, ex[from].allocSize, c->cudaDev, &imp);
      ::close(pfd);
      FCXCHECK(r);
      w->imports.push_back(imp);
      w->peer[from] = (char *)imp.ptr + ex[from].offset;
    }
    ::close(fd);
    // optional NVLink multicast over the whole allocation
    if (allMc && cu::mcSupported(c->cudaDev)) {
      uint64_t mkey = key ^ 0x4d43ull;
      FdChannel mch;
      FCXCHECK(mch.open(mkey, me));
      FCXCHECK(c->bootstrap->barrier());
      flagcxResult_t mr = flagcxSuccess;
      if (me == 0) {
        mr = cu::mcCreate(n, mine.allocSize, &w->mcObj);
        if (mr == flagcxSuccess) {
          int mfd = -1;
          mr = cu::mcExportFd(w->mcObj, &mfd);
          for (int p = 1; p < n && mr == flagcxSuccess; ++p) mr = mch.sendFd(mkey, p, mfd, 0);
          if (mfd >= 0) ::close(mfd);
        }
      } else {
        int mfd = -1;
        uint64_t tag;
        mr = mch.recvFd(&mfd, &tag, defaultSocketTimeoutMs());
        if (mr == flagcxSuccess) { mr = cu::mcImportFd(mfd, mine.allocSize, &w->mcObj); ::close(mfd); }
      }
      if (mr == flagcxSuccess) mr = cu::mcAddDevice(&w->mcObj, c->cudaDev);
      // agree before binding: a partial bind would leave peers waiting on the switch
      std::vector<int32_t> okv(n, 0);
      okv[me] = mr == flagcxSuccess;
      FCXCHECK(c->bootstrap->allGather(okv.data(), sizeof(int32_t)));
      bool allOk = true;
      for (int v : okv) allOk &= v != 0;
      if (allOk) {
        mr = cu::mcBindAndMap(&w->mcObj, *blk);
        okv.assign(n, 0);
        okv[me] = mr == flagcxSuccess;
        FCXCHECK(c->bootstrap->allGather(okv.data(), sizeof(int32_t)));
        allOk = true;
        for (int v : okv) allOk &= v != 0;
      }
      if (allOk) {
        w->mc = (char *)w->mcObj.ptr + mine.offset;
        FCX_INFO(SUB_NVLS, "window %p: multicast bound (%zu bytes)", buff, (size_t)mine.allocSize);
      } else {
        cu::mcRelease(&w->mcObj);
        FCX_INFO(SUB_NVLS, "window %p: multicast unavailable, using peer loads/stores only", buff);
      }
    }
  } else {
    for (int p = 0; p < n; ++p) {
      if (p == me) continue;
      void *opened = nullptr;
      FCX_CUDACHECK(cudaIpcOpenMemHandle(&opened, ex[p].ipc, cudaIpcMemLazyEnablePeerAccess));
      w->ipcOpened.push_back(opened);
      w->peer[p] = (char *)opened + ex[p].offset;
    }
  }
  {
    // where every rank mapped every other rank's copy: row p of the table is rank p's view
    std::vector<void *> table((size_t)n * FLAGCX_MAX_RANKS, nullptr);
    for (int p = 0; p < n; ++p) table[(size_t)me * FLAGCX_MAX_RANKS + p] = w->peer[p];
    FCXCHECK(c->bootstrap->allGather(table.data(), sizeof(void *) * FLAGCX_MAX_RANKS));
    for (int p = 0; p < n; ++p) w->selfAt[p] = table[(size_t)p * FLAGCX_MAX_RANKS + me];
  }
  c->windows.add(w.get());
  FCX_INFO(SUB_REG, "rank %d registered window %p (%zu bytes, %s%s)", me, buff, size,
           mine.method == 0 ? "vmm" : "ipc", w->mc ? ", multicast" : "");
  *out = w.release();
  return flagcxSuccess;
}

flagcxResult_t windowDeregister(flagcxComm *c, Window *w) {
  if (!w) return flagcxSuccess;
  c->windows.remove(w);
  if (c->emu) { delete w; return flagcxSuccess; }
  // Nobody may touch the peers' mappings any more: drain our own work first.
  if (c->devicePath) cudaDeviceSynchronize();
  cu::mcRelease(&w->mcObj);
  for (auto &b : w->imports) cu::vmmFree(&b);
  for (void *p : w->ipcOpened) cudaIpcCloseMemHandle(p);
  if (w->owned.ptr) cu::vmmFree(&w->owned);
  delete w;
  return flagcxSuccess;
}

// ---------------------------------------------------------------------------
// construction / destruction
// ---------------------------------------------------------------------------
static flagcxResult_t setupDeviceWorld(flagcxComm *c, const std::vector<PeerInfo> &peers) {
  const int n = c->nranks;
  c->layout = makeLayout();
  FCXCHECK(allocLocalDeviceState(c));
  bool allMc = true, allVmm = true;
  for (auto &p : peers) { allMc &= p.mc != 0; allVmm &= p.vmm != 0; }
  c->nvls = allMc && allVmm && n > 1 && readParam("NVLS_ENABLE", paramNvlsEnable()) != 0;

  void *base = nullptr;
  cu::VmmBlock blk;
  if (allVmm) {
    FCXCHECK(cu::vmmAlloc(c->layout.total, c->cudaDev, &blk));
    base = blk.ptr;
  } else {
    FCX_CUDACHECK(cudaMalloc(&base, c->layout.total));
  }
  FCX_CUDACHECK(cudaMemset(base, 0, c->layout.zeroedBytes));
  FCX_CUDACHECK(cudaDeviceSynchronize());
  Window *w = nullptr;
  c->devicePath = true;
  flagcxResult_t r = windowRegister(c, base, c->layout.total, FLAGCX_WIN_COLL_SYMMETRIC, &w);
  if (r != flagcxSuccess) { c->devicePath = false; return r; }
  w->internal = true;
  if (allVmm) w->owned = blk;
  c->internalWin = w;
  fillDevComm(c);
  c->tuner.reset(new Tuner());
  FCXCHECK(c->tuner->init(c));
  // registration service for user buffers: every rank must have one, or nobody uses it
  {
    std::vector<int32_t> up(n, 0);
    if (n > 1 && readParam("USER_BUFFER_EXPORT", paramUserBufferExport()) != 0) {
      c->reg.reset(new RegCache());
      up[c->rank] = c->reg->start(c->bootstrap->nonce(), c->rank, n, cudaRegBackend(c->cudaDev)) == flagcxSuccess;
    }
    FCXCHECK(c->bootstrap->allGather(up.data(), sizeof(int32_t)));
    bool all = true;
    for (int v : up) all &= v != 0;
    if (all) {
      // open one small allocation at every peer now, while no kernel is running: the first
      // inter-process mapping between two devices also sets up their peer access
      void *va[FLAGCX_MAX_RANKS];
      up.assign(n, 0);
      up[c->rank] = c->reg->lookup(c->localSync, 8, va) ? 1 : 0;
      FCXCHECK(c->bootstrap->allGather(up.data(), sizeof(int32_t)));
      for (int v : up) all &= v != 0;
    }
    c->exportUserBuffers = all;
    c->autoExport = all && readParam("USER_BUFFER_EXPORT", paramUserBufferExport()) >= 2;
    if (!all && c->reg) { c->reg->stop(); c->reg.reset(); }
  }
  FCX_INFO(SUB_INIT, "rank %d: device path over NVLink, %d ranks, staging %zu MiB, nvls %d, user-buffer export %d",
           c->rank, n, c->layout.stagingBytes >> 20, (int)c->nvls, (int)c->exportUserBuffers);
  return flagcxSuccess;
}

flagcxResult_t commCreate(flagcxComm **out, int nranks, const flagcxUniqueId &id, int rank) {
  logInit();
  // Settings of the FlagCX project that select machinery this library does not have:
  // say so once instead of ignoring them silently.
  static const bool warned = [] {
    static const char *const unsupported[] = {
        "FLAGCX_CLUSTER_SPLIT_LIST",    // heterogeneous cluster planner
        "FLAGCX_CCL_ADAPTOR_PLUGIN",    // vendor collective-library plugins
        "FLAGCX_DEVICE_ADAPTOR_PLUGIN", // vendor device-runtime plugins
        "FLAGCX_TOPO_FILE",             // PCI/NIC topology XML
        "FLAGCX_INTERSERVER_ROUTE_FILE"};
    for (const char *name : unsupported)
      if (getEnv(name)) FCX_WARN("%s is set but has no effect: single-vendor NVLink library (see docs/environment_variables.md)", name);
    return true;
  }();
  (void)warned;
  auto c = std::make_unique<flagcxComm>();
  c->magic = kCommMagic;
  c->rank = rank;
  c->nranks = nranks;
  c->bootstrap.reset(new Bootstrap());
  FCXCHECK(c->bootstrap->init(id, rank, nranks));

  std::vector<PeerInfo> peers(nranks);
  PeerInfo &me = peers[rank];
  memset(&me, 0, sizeof me);
  me.hostHash = hostHash();
  me.pidHash = pidHash();
  me.cudaDev = -1;
  if (cu::available() && !getEnv("FLAGCX_FORCE_HOST")) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) {
      me.cudaDev = dev;
      me.vmm = cu::vmmSupported(dev) && readParam("VMM_ENABLE", paramVmmEnable()) != 0;
      me.mc = cu::mcSupported(dev);
      cudaDeviceGetPCIBusId(me.busId, sizeof me.busId, dev);
    }
  }
  FCXCHECK(c->bootstrap->allGather(peers.data(), sizeof(PeerInfo)));

  // ranks on this machine
  c->localRanks = 0;
  for (int p = 0; p < nranks; ++p) {
    if (peers[p].hostHash == me.hostHash) {
      if (p == rank) c->localRank = c->localRanks;
      ++c->localRanks;
    }
  }
  c->cudaDev = me.cudaDev;

  bool canDevice = nranks <= FLAGCX_MAX_RANKS && readParam("P2P_DISABLE", paramP2pDisable()) == 0;
  for (int p = 0; p < nranks && canDevice; ++p) {
    canDevice &= peers[p].cudaDev >= 0 && peers[p].hostHash == me.hostHash;
    for (int q = 0; q < p && canDevice; ++q)
      if (!strcmp(peers[p].busId, peers[q].busId)) {
        if (rank == 0) FCX_WARN("ranks %d and %d use the same GPU %s; taking the host path", q, p, peers[p].busId);
        canDevice = false;
      }
  }
  if (canDevice) {
    for (int p = 0; p < nranks; ++p) {
      if (p == rank) continue;
      int ok = 0;
      if (cudaDeviceCanAccessPeer(&ok, me.cudaDev, peers[p].cudaDev) != cudaSuccess || !ok) canDevice = false;
    }
  }
  // all ranks must agree
  std::vector<int32_t> votes(nranks, 0);
  votes[rank] = canDevice;
  FCXCHECK(c->bootstrap->allGather(votes.data(), sizeof(int32_t)));
  for (int v : votes) canDevice &= v != 0;

  if (canDevice) {
    FCXCHECK(setupDeviceWorld(c.get(), peers));
    c->watchdog = std::thread(watchdogMain, c.get());
  } else {
    FCX_INFO(SUB_INIT, "rank %d: host path (sockets)%s", rank, me.cudaDev >= 0 ? " with staged device buffers" : "");
    // several NVLink domains: NVLink kernels inside each, the host network between them
    bool gpus = true;
    std::vector<uint64_t> hashes(nranks);
    std::vector<int> hasGpu(nranks);
    for (int p = 0; p < nranks; ++p) {
      hashes[p] = peers[p].hostHash;
      hasGpu[p] = peers[p].cudaDev >= 0;
      gpus &= hasGpu[p] != 0;
    }
    if (gpus && nranks > 1 && readParam("P2P_DISABLE", paramP2pDisable()) == 0 && !getEnv("FLAGCX_FORCE_HOST"))
      FCXCHECK(hierSetup(c.get(), hashes, hasGpu));
  }
  *out = c.release();
  return flagcxSuccess;
}

flagcxResult_t commCheckDevice(flagcxComm *c) {
  if (!c->status) return flagcxSuccess;
  unsigned code = *(volatile unsigned *)&c->status->code;
  if (code != FLAGCX_DEV_OK && c->asyncError.load() == flagcxSuccess) {
    static const char *what[] = {"", "barrier", "signal", "counter", "kernel"};
    unsigned where = c->status->where < 5 ? c->status->where : 0;
    char buf[256];
    snprintf(buf, sizeof buf, "rank %d: device-side %s at %s (peer %d, detail %llu)", c->rank,
             code == FLAGCX_DEV_TIMEOUT ? "wait timed out" : code == FLAGCX_DEV_ABORTED ? "wait aborted" : "bounds check failed",
             what[where], (int)c->status->peer, (unsigned long long)c->status->detail);
    c->lastError = buf;
    FCX_WARN("%s", buf);
    c->asyncError.store(code == FLAGCX_DEV_BOUNDS ? flagcxInvalidArgument : flagcxRemoteError);
  }
  return (flagcxResult_t)c->asyncError.load();
}

flagcxResult_t commDestroy(flagcxComm *c) {
  if (!commValid(c)) return flagcxInvalidArgument;
  if (c->emu) return emuWorldDestroy(c);
  c->watchdogStop.store(true);
  if (c->watchdog.joinable()) c->watchdog.join();
  hierTeardown(c);
  if (c->devicePath) {
    cudaSetDevice(c->cudaDev);
    cudaDeviceSynchronize();
    // Peers may still be inside a kernel that touches our memory: leave together.
    if (!c->aborted && c->asyncError.load() == flagcxSuccess) c->bootstrap->barrier();
    if (c->reg) {
      // unmap what this rank opened for its peers, then meet again: nobody frees an
      // allocation that a peer still has mapped
      c->reg->stop();
      c->reg.reset();
      if (!c->aborted && c->asyncError.load() == flagcxSuccess) c->bootstrap->barrier();
    }
    for (void *&b : c->bounce)
      if (b) { cudaFree(b); b = nullptr; }
    for (Window *w : c->windows.all())
      if (!w->internal) windowDeregister(c, w);
    void *internalBase = c->internalWin ? c->internalWin->local : nullptr;
    bool ownedVmm = c->internalWin && c->internalWin->owned.ptr;
    if (c->internalWin) windowDeregister(c, c->internalWin);
    if (internalBase && !ownedVmm) cudaFree(internalBase);
    if (c->localSync) cudaFree(c->localSync);
    if (c->status) cudaFreeHost(c->status);
    if (c->internalStream) cudaStreamDestroy(c->internalStream);
    if (!c->aborted && c->asyncError.load() == flagcxSuccess) c->bootstrap->barrier();
  }
  if (c->hostStage) {
    if (cu::available()) cudaFreeHost(c->hostStage); else free(c->hostStage);
  }
  c->tuner.reset();
  if (c->hostNet) c->hostNet->close();
  c->bootstrap->close();
  c->magic = 0;
  delete c;
  return flagcxSuccess;
}

} // namespace fcx
