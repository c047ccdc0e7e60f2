// device_coll.cc -- host side of the device path: turns one collective call into
// one (or, for unregistered buffers larger than the staging area, a few) kernel
// launches: finds out whether the buffers are peer-visible, asks the tuner for an
// algorithm and CTA count, fills the argument block and launches.
//
// Buffers inside a registered window are used in place by every rank (offsets are
// symmetric, as with NCCL window registration).  Anything else is staged through
// the communicator's internal window inside the same kernel.
#include <algorithm>

#include "../kernels/launch.h"
#include "comm.h"
#include "tuner.h"

namespace fcx {

namespace {

enum Family { kFamReduce = 0, kFamCopy = 1, kFamNvls = 2, kFamP2p = 3, kFamLl = 4 };

struct BufView {
  Window *win = nullptr;
  size_t off = 0;
  bool visible() const { return win != nullptr; }
};

BufView viewOf(flagcxComm *c, const void *p, size_t bytes) {
  BufView v;
  if (c->emu || !p) return v;
  v.win = c->windows.find(p, bytes ? bytes : 1);
  if (v.win) v.off = (uintptr_t)p - (uintptr_t)v.win->local;
  return v;
}

// In an emulated world every buffer is visible to every rank; the launcher fills
// the other ranks' entries when all of them have posted.
bool emuVisible(flagcxComm *c) { return c->emu && !getEnv("FLAGCX_EMU_FORCE_STAGING"); }

void setIn(flagcxComm *c, CollArgs &a, const BufView &v, const void *local, size_t extraOff = 0) {
  for (int p = 0; p < c->nranks; ++p) a.in[p] = nullptr;
  if (v.win) {
    for (int p = 0; p < c->nranks; ++p) a.in[p] = (const char *)v.win->peer[p] + v.off + extraOff;
    if (v.win->mc) a.mcIn = (const char *)v.win->mc + v.off + extraOff;
  } else {
    a.in[c->rank] = (const char *)local + extraOff;
  }
}
void setOut(flagcxComm *c, CollArgs &a, const BufView &v, void *local, size_t extraOff = 0) {
  for (int p = 0; p < c->nranks; ++p) a.out[p] = nullptr;
  if (v.win) {
    for (int p = 0; p < c->nranks; ++p) a.out[p] = (char *)v.win->peer[p] + v.off + extraOff;
    if (v.win->mc) a.mcOut = (char *)v.win->mc + v.off + extraOff;
  } else {
    a.out[c->rank] = (char *)local + extraOff;
  }
}
// ---- user buffers outside windows ------------------------------------------------------
// How the peers' kernels reach a buffer of this rank.
enum Reach {
  kReachNone = 0, // they cannot: the legacy path stages it through the internal window
  kReachWindow,   // inside a symmetric window: every address is known on the host
  kReachEmu,      // emulated world: the launcher fills in the other ranks' addresses
  kReachExport    // exported on demand (reg_cache.h); peers learn the address inside the kernel
};

struct UserBuf {
  Reach reach = kReachNone;
  BufView view;
  void *user = nullptr;  // what the caller passed
  void *local = nullptr; // what the local kernel uses: the same, or an exportable stand-in
  size_t bytes = 0;
  void *peerVa[FLAGCX_MAX_RANKS] = {};
  bool visible() const { return reach != kReachNone; }
  bool bounced() const { return local != user; }
};

// A device allocation of at least `bytes` that can be exported (cudaMalloc memory),
// kept per communicator and direction.
flagcxResult_t bounceBuffer(flagcxComm *c, int which, size_t bytes, void **out) {
  if (c->bounceBytes[which] < bytes) {
    if (c->bounce[which]) {
      FCX_CUDACHECK(cudaDeviceSynchronize()); // earlier collectives may still use it, peers included
      c->reg->forget(c->bounce[which]);
      FCX_CUDACHECK(cudaFree(c->bounce[which]));
      c->bounce[which] = nullptr;
      c->bounceBytes[which] = 0;
    }
    size_t want = alignUp(bytes, (size_t)2 << 20);
    FCX_CUDACHECK(cudaMalloc(&c->bounce[which], want));
    c->bounceBytes[which] = want;
    FCX_INFO(SUB_REG, "rank %d: %zu MiB stand-in for %s buffers that cannot be exported", c->rank, want >> 20,
             which ? "output" : "input");
  }
  *out = c->bounce[which];
  return flagcxSuccess;
}

// Finds out how `p` is reachable.  With on-demand export enabled this never answers
// kReachNone for a non-null buffer: a buffer that cannot be exported (memory that is
// not a cudaMalloc block) is replaced by an exportable stand-in, filled from it
// (inputs) on `stream` here or copied back (outputs) by finishOut().
flagcxResult_t resolve(flagcxComm *c, const void *p, size_t bytes, int which, cudaStream_t stream, UserBuf *u) {
  *u = UserBuf();
  u->user = u->local = const_cast<void *>(p);
  u->bytes = bytes;
  if (!p) return flagcxSuccess;
  if (c->emu) {
    if (getEnv("FLAGCX_EMU_FORCE_STAGING")) return flagcxSuccess;
    if (getEnv("FLAGCX_EMU_EXCHANGE")) { // one address space: every rank sees the buffer where it is
      u->reach = kReachExport;
      for (int r = 0; r < c->nranks; ++r) u->peerVa[r] = u->local;
    } else {
      u->reach = kReachEmu;
    }
    return flagcxSuccess;
  }
  u->view = viewOf(c, p, bytes);
  if (u->view.visible()) { u->reach = kReachWindow; return flagcxSuccess; }
  if (!c->exportUserBuffers || c->nranks == 1) return flagcxSuccess;
  if (!c->autoExport) {
    // only what the caller registered (flagcxCommRegister, on every rank) is exported;
    // anything else goes through the staging window
    if (c->reg->lookupKnown(p, bytes ? bytes : 1, u->peerVa)) u->reach = kReachExport;
    return flagcxSuccess;
  }
  if (c->reg->lookup(p, bytes ? bytes : 1, u->peerVa)) { u->reach = kReachExport; return flagcxSuccess; }
  void *b = nullptr;
  FCXCHECK(bounceBuffer(c, which, bytes, &b));
  if (!c->reg->lookup(b, bytes ? bytes : 1, u->peerVa)) {
    FCX_WARN("rank %d: neither the user buffer %p nor a stand-in could be exported to the peers", c->rank, p);
    return flagcxUnhandledDeviceError;
  }
  u->local = b;
  u->reach = kReachExport;
  if (which == 0 && bytes) FCX_CUDACHECK(cudaMemcpyAsync(b, p, bytes, cudaMemcpyDeviceToDevice, stream));
  return flagcxSuccess;
}

flagcxResult_t finishOut(const UserBuf &u, cudaStream_t stream) {
  if (u.bounced() && u.bytes) FCX_CUDACHECK(cudaMemcpyAsync(u.user, u.local, u.bytes, cudaMemcpyDeviceToDevice, stream));
  return flagcxSuccess;
}

void applyIn(flagcxComm *c, CollArgs &a, const UserBuf &u, size_t extraOff = 0) {
  if (u.reach == kReachWindow) { setIn(c, a, u.view, u.user, extraOff); return; }
  setIn(c, a, BufView(), u.local, extraOff);
  if (u.reach == kReachExport) {
    a.xchg |= kXchgIn;
    for (int p = 0; p < c->nranks; ++p) a.pubIn[p] = (const char *)u.peerVa[p] + extraOff;
  }
}
void applyOut(flagcxComm *c, CollArgs &a, const UserBuf &u, size_t extraOff = 0) {
  if (u.reach == kReachWindow) { setOut(c, a, u.view, u.user, extraOff); return; }
  setOut(c, a, BufView(), u.local, extraOff);
  if (u.reach == kReachExport) {
    a.xchg |= kXchgOut;
    for (int p = 0; p < c->nranks; ++p) a.pubOut[p] = (char *)u.peerVa[p] + extraOff;
  }
}
// The output is only written by the local kernel: no peer needs its address.
void applyOutLocal(flagcxComm *c, CollArgs &a, const UserBuf &u, size_t extraOff = 0) {
  setOut(c, a, BufView(), u.local, extraOff);
}

// Staging region [off, off+...) of every rank.
void setInStage(flagcxComm *c, CollArgs &a, size_t off) {
  BufView v{c->internalWin, c->layout.stagingOff + off};
  setIn(c, a, v, nullptr);
}
void setOutStage(flagcxComm *c, CollArgs &a, size_t off) {
  BufView v{c->internalWin, c->layout.stagingOff + off};
  setOut(c, a, v, nullptr);
}

void initArgs(flagcxComm *c, CollArgs &a, int kind, flagcxDataType_t dt) {
  memset(&a, 0, sizeof a);
  a.kind = kind;
  a.dtype = dt;
  a.elemSize = (int)getFlagcxDataTypeSize(dt);
  a.scale = 1.0f;
  a.flags = kFlagBeginBarrier | kFlagEndBarrier;
  for (int p = 0; p < c->nranks; ++p) {
    a.meta[p] = (unsigned long long *)((char *)c->internalWin->peer[p] + c->layout.metaOff);
    a.ptrPad[p] = (unsigned long long *)((char *)c->internalWin->peer[p] + c->layout.ptrPadOff);
  }
}

// Push kinds whose blocks are large and 16-byte aligned move through the bulk-copy
// engine (one thread per CTA drives a ring of shared-memory stages) instead of
// per-thread loads and stores.  Returns the stage size in bytes, 0 for the thread path.
int bulkStageFor(flagcxComm *c, const CollArgs &a) {
  if (a.kind != kAllGatherPush && a.kind != kAllToAllPush && a.kind != kBroadcastPush) return 0;
  // measured on B200 pairs: the engine wins (about 670 against 590 GB/s per direction)
  // once a rank sends some tens of MB; below that its start-up costs more than it saves
  const int64_t enable = readParam("BULK_COPY", 1), minBytes = readParam("BULK_COPY_MIN_BYTES", 64 << 20);
  const size_t blk = a.count * (size_t)a.elemSize;
  if (!enable || blk * (size_t)std::max(1, c->nranks - 1) < (size_t)minBytes || blk % 16) return 0;
  uintptr_t bits = (uintptr_t)a.in[c->rank] | a.inStride | a.outStride;
  for (int p = 0; p < c->nranks; ++p) bits |= (uintptr_t)a.out[p];
  return (bits & 15) ? 0 : 16384;
}

// The sum reductions at 2, 4 and 8 ranks have a variant whose inputs arrive through
// the bulk-copy engine (Reducer::sliceBulk).  1 selects it.
int bulkReduceFor(flagcxComm *c, const CollArgs &a) {
  if (a.kind != kAllReduceTwoShot && a.kind != kAllReduceTwoShotCast && a.kind != kReduceScatter) return 0;
  const int n = c->nranks;
  if (a.redOp != kOpSum || (n != 2 && n != 4 && n != 8)) return 0;
  if (a.dtype != flagcxFloat32 && a.dtype != flagcxBfloat16 && a.dtype != flagcxFloat16) return 0;
  // measured on 8 B200s: reduce-scatter gains from 64 MB of peer input on (667 against 606 GB/s
  // at 4 GiB), the two-shot all-reduce only from about 400 MB on
  // Off by default: with the default cap of 32 CTAs the per-thread loads reach 555 GB/s on a
  // B200 pair (436 MB reduce-scatter) where this path reaches 263; it only catches up near
  // 96 CTAs, which a collective that runs beside GEMMs should not take.
  const int64_t enable = readParam("BULK_REDUCE", 0), minBytes = readParam("BULK_COPY_MIN_BYTES", 64 << 20),
                minAllReduce = readParam("BULK_ALLREDUCE_MIN_BYTES", 400 << 20);
  const size_t es = (size_t)a.elemSize, bytes = a.count * es;
  if (!enable || bytes % 16) return 0;
  const size_t slice = a.kind == kReduceScatter ? a.count : sliceElems(a.count, n, es);
  if (slice * es * (size_t)(n - 1) < (size_t)(a.kind != kReduceScatter ? std::max(minBytes, minAllReduce) : minBytes)) return 0;
  if (a.outMode == kOutBf16 && slice % 8) return 0; // output slices must start on 16 bytes too
  uintptr_t bits = (uintptr_t)a.residual | (a.kind == kReduceScatter ? a.inStride : 0);
  for (int p = 0; p < n; ++p) bits |= (uintptr_t)a.in[p] | (uintptr_t)a.out[p];
  return (bits & 15) ? 0 : 1;
}

// Extents of the regions behind in[] / out[] for the bounds-checking kernel build.  The
// regions of a launch are what the operation's definition says they are; a test can make
// the host understate them (FLAGCX_BOUNDS_TEST_SHRINK bytes) to see a violation reported.
void setExtents(CollArgs &a, size_t inBytes, size_t outBytes) {
  static const int64_t shrink = readParam("BOUNDS_TEST_SHRINK", 0);
  a.inBytes = inBytes > (size_t)shrink ? inBytes - (size_t)shrink : inBytes;
  a.outBytes = outBytes > (size_t)shrink ? outBytes - (size_t)shrink : outBytes;
}

flagcxResult_t launch(flagcxComm *c, int family, const CollArgs &a0, int nCtas, cudaStream_t stream) {
  nCtas = std::max(1, std::min(nCtas, FLAGCX_COLL_BARRIER_SLOTS));
  CollArgs a = a0;
  // every rank issues the same sequence of collective launches, so the parity agrees
  // whether or not a given rank exchanges pointers in a given launch
  a.xchgParity = (uint32_t)(c->xchgSeq++ & 1);
  if (a.xchg) a.flags |= kFlagBeginBarrier | kFlagEndBarrier;
  if (family == kFamCopy) {
    a.bulkStage = bulkStageFor(c, a);
    a.bulkDepth = readParam("BULK_STAGES", 8) >= 12 ? 12 : 8;
  } else if (family == kFamReduce) {
    a.bulkStage = bulkReduceFor(c, a);
  }
  if (c->emu) return emuSubmit(c, family, &a, nullptr, nCtas, stream);
  LaunchCtx lc;
  lc.comm = &c->dev;
  lc.stream = stream;
  lc.nCtas = nCtas;
  cudaError_t e;
  if (family == kFamCopy) e = launchCopyKernel(lc, a);
  else if (family == kFamReduce) e = launchReduceKernel(lc, a, c->nranks);
  else if (family == kFamLl) e = launchLlKernel(lc, a);
  else e = launchNvlsKernel(lc, a);
  if (e != cudaSuccess) {
    FCX_WARN("kernel launch failed: %s", cudaGetErrorString(e));
    return flagcxUnhandledDeviceError;
  }
  return flagcxSuccess;
}

bool isFloatType(flagcxDataType_t t) {
  return t == flagcxFloat16 || t == flagcxFloat32 || t == flagcxFloat64 || t == flagcxBfloat16;
}

// Reduction operator and epilogue fields common to the reduce family.
flagcxResult_t setReduceEpilogue(flagcxComm *c, CollArgs &a, const DeviceCollRequest &rq) {
  a.redOp = rq.redOp == flagcxAvg ? kOpSum : (int)rq.redOp;
  a.scale = rq.scale;
  a.divisor = 0;
  if (rq.redOp == flagcxAvg) {
    if (isFloatType(rq.dtype) && rq.dtype != flagcxFloat64) a.scale *= 1.0f / (float)c->nranks;
    else a.divisor = c->nranks;
  }
  a.outMode = kOutSame;
  if (rq.outDtype != flagcxNumTypes && rq.outDtype != rq.dtype) {
    if (rq.outDtype == flagcxFloat32 && (rq.dtype == flagcxBfloat16 || rq.dtype == flagcxFloat16)) a.outMode = kOutFloat;
    else if (rq.outDtype == flagcxBfloat16 && rq.dtype == flagcxFloat32) a.outMode = kOutBf16;
    else {
      FCX_WARN("fused cast %s -> %s is not supported", dtypeName(rq.dtype), dtypeName(rq.outDtype));
      return flagcxInvalidArgument;
    }
  }
  a.residual = (const char *)rq.residual;
  return flagcxSuccess;
}

size_t outElemSize(const CollArgs &a) {
  return a.outMode == kOutFloat ? 4 : a.outMode == kOutBf16 ? 2 : (size_t)a.elemSize;
}

bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

bool nvlsEligible(flagcxComm *c, const DeviceCollRequest &rq, size_t count) {
  if (!c->nvls || c->emu) return false;
  if (rq.dtype != flagcxFloat32 && rq.dtype != flagcxBfloat16 && rq.dtype != flagcxFloat16) return false;
  bool addLike = rq.redOp == flagcxSum || rq.redOp == flagcxAvg;
  bool minmax = (rq.redOp == flagcxMin || rq.redOp == flagcxMax) && rq.dtype != flagcxFloat32;
  if (!addLike && !minmax) return false;
  if (rq.residual || (rq.outDtype != flagcxNumTypes && rq.outDtype != rq.dtype)) return false;
  size_t es = getFlagcxDataTypeSize(rq.dtype);
  return (count * es) % 16 == 0 && aligned16(rq.send) && aligned16(rq.recv);
}

void note(flagcxComm *c, flagcxCommOp_t op, size_t bytes, int algo, int nCtas) {
  OpStats &s = c->stats[op];
  s.calls++;
  s.bytes += bytes;
  s.lastAlgo = algo;
  s.lastCtas = nCtas;
}

int pickCtas(flagcxComm *c, const DeviceCollRequest &rq, const TuneChoice &ch) {
  int n = rq.nCtas > 0 ? rq.nCtas : ch.nCtas;
  return std::max(1, std::min(n, FLAGCX_COLL_BARRIER_SLOTS));
}

// ---- ring kinds ---------------------------------------------------------------------------
// Step flags and, for the reducing kinds, the partial-sum scratch (the staging window cut
// into n-1 slots).  Returns the largest slot in elements of `es` bytes.
size_t setRing(flagcxComm *c, CollArgs &a, size_t es, int steps) {
  const int n = c->nranks, next = (c->rank + 1) % n;
  a.ringNext = (unsigned long long *)((char *)c->internalWin->peer[next] + c->layout.ringOff);
  a.ringMine = (unsigned long long *)((char *)c->internalWin->peer[c->rank] + c->layout.ringOff);
  a.ringBase = c->ringSeq;
  c->ringSeq += (uint64_t)steps;
  for (int p = 0; p < n; ++p) a.aux[p] = (char *)c->internalWin->peer[p] + c->layout.stagingOff;
  const size_t slot = c->layout.stagingBytes / (size_t)std::max(1, n - 1) / es / 16 * 16;
  a.ringSlotElems = slot;
  return slot;
}

// ---- LL: small messages ---------------------------------------------------------------
flagcxResult_t launchLl(flagcxComm *c, CollArgs &a, size_t bytes, cudaStream_t stream) {
  for (int p = 0; p < c->nranks; ++p) a.aux[p] = (char *)c->internalWin->peer[p] + c->layout.llOff;
  a.llSlotBytes = c->layout.llSlotBytes;
  const uint64_t seq = ++c->llSeq; // parity alternates with every operation; the flag is never 0
  a.llEpoch = (uint32_t)(seq & 0x7fffffffu) | 0x80000000u;
  if ((a.llEpoch & 1u) != (uint32_t)(seq & 1u)) return flagcxInternalError;
  a.flags = 0;
  const size_t units = (bytes + 7) / 8;
  const int nCtas = (int)std::max<size_t>(1, std::min<size_t>((units + FLAGCX_DEVICE_THREADS_PER_CTA - 1) / FLAGCX_DEVICE_THREADS_PER_CTA, 16));
  if (c->emu) return emuSubmit(c, kFamLl, &a, nullptr, nCtas, stream);
  LaunchCtx lc;
  lc.comm = &c->dev;
  lc.stream = stream;
  lc.nCtas = nCtas;
  cudaError_t e = launchLlKernel(lc, a);
  if (e != cudaSuccess) {
    FCX_WARN("LL kernel launch failed: %s", cudaGetErrorString(e));
    return flagcxUnhandledDeviceError;
  }
  return flagcxSuccess;
}

// ---------------------------------------------------------------------------
flagcxResult_t allReduce(flagcxComm *c, const DeviceCollRequest &rq, cudaStream_t stream) {
  const int n = c->nranks;
  CollArgs a;
  initArgs(c, a, kAllReduceOneShot, rq.dtype);
  FCXCHECK(setReduceEpilogue(c, a, rq));
  const size_t es = a.elemSize, oes = outElemSize(a);
  const size_t count = rq.count;
  // Small messages: no barrier, no registration, any buffer.  The choice depends only on
  // what every rank knows (size, type, settings, tuner table), so all ranks agree on it.
  {
    TuneChoice pre = c->tuner->choose(flagcxCommOpAllReduce, count * es, n, true, false, (int)es);
    const int want = rq.algo >= 0 ? rq.algo : pre.algo;
    if (want == FLAGCX_ALGO_LL && n > 1 && count > 0 && a.outMode == kOutSame && !a.residual &&
        count * es <= c->layout.llSlotBytes / 2) {
      a.kind = kLlAllReduce;
      a.count = count;
      setIn(c, a, BufView(), rq.send);
      setOut(c, a, BufView(), rq.recv);
      note(c, flagcxCommOpAllReduce, count * es, FLAGCX_ALGO_LL, 0);
      setExtents(a, count * es, count * es);
      return launchLl(c, a, count * es, stream);
    }
  }
  UserBuf uin, uout;
  FCXCHECK(resolve(c, rq.send, count * es, 0, stream, &uin));
  if (rq.send == rq.recv) uout = uin; // in place stays in place, stand-in included
  else FCXCHECK(resolve(c, rq.recv, count * oes, 1, stream, &uout));
  const bool inVis = uin.visible(), outVis = uout.visible();
  const bool nvlsOk = nvlsEligible(c, rq, count);
  TuneChoice ch = c->tuner->choose(flagcxCommOpAllReduce, count * es, n, inVis && outVis, nvlsOk, (int)es);
  int algo = rq.algo >= 0 ? rq.algo : ch.algo;
  if ((algo == FLAGCX_ALGO_NVLS_ONESHOT || algo == FLAGCX_ALGO_NVLS_TWOSHOT) && !nvlsOk) algo = FLAGCX_ALGO_TWOSHOT;
  if (algo == FLAGCX_ALGO_LL) algo = FLAGCX_ALGO_ONESHOT; // not eligible above
  if (algo != FLAGCX_ALGO_ONESHOT && algo != FLAGCX_ALGO_TWOSHOT && algo != FLAGCX_ALGO_NVLS_ONESHOT &&
      algo != FLAGCX_ALGO_NVLS_TWOSHOT && algo != FLAGCX_ALGO_RING)
    algo = FLAGCX_ALGO_TWOSHOT;
  // one-shot writes its output while peers may still read the same addresses
  if (algo == FLAGCX_ALGO_ONESHOT && uin.local == uout.local && inVis) algo = FLAGCX_ALGO_TWOSHOT;
  if (n == 1) algo = FLAGCX_ALGO_ONESHOT;
  const int nCtas = pickCtas(c, rq, ch);
  note(c, flagcxCommOpAllReduce, count * es, algo, nCtas);
  const size_t S = c->layout.stagingBytes, half = S / 2;
  const bool nvlsAlgo = algo == FLAGCX_ALGO_NVLS_ONESHOT || algo == FLAGCX_ALGO_NVLS_TWOSHOT;
  // multimem needs multicast aliases: windows bound at registration, else the staging
  const bool inMc = uin.view.win && uin.view.win->mc, outMc = uout.view.win && uout.view.win->mc;

  if (algo == FLAGCX_ALGO_ONESHOT || algo == FLAGCX_ALGO_NVLS_ONESHOT) {
    a.kind = nvlsAlgo ? kAllReduceNvlsOneShot : kAllReduceOneShot;
    const bool direct = nvlsAlgo ? inMc : inVis;
    if (direct) {
      a.count = count;
      setExtents(a, count * es, count * oes);
      applyIn(c, a, uin);
      applyOutLocal(c, a, uout);
      FCXCHECK(launch(c, nvlsAlgo ? kFamNvls : kFamReduce, a, nCtas, stream));
      return finishOut(uout, stream);
    }
    // Staged input.  The closing barrier stays: the next collective, whatever its kind,
    // overwrites the staging from offset 0 on, and must not start before every peer has
    // finished reading this one's.
    size_t chunk = S / es / 16 * 16;
    for (size_t off = 0; off < count || off == 0; off += chunk) {
      size_t cnt = std::min(chunk, count - off);
      a.count = cnt;
      setInStage(c, a, 0);
      a.userIn = (const char *)uin.local + off * es;
      a.nInBlocks = 1;
      a.inBlockBytes = cnt * es;
      applyOutLocal(c, a, uout, off * oes);
      a.residual = rq.residual ? (const char *)rq.residual + off * oes : nullptr;
      FCXCHECK(launch(c, nvlsAlgo ? kFamNvls : kFamReduce, a, nCtas, stream));
      if (count == 0) break;
    }
    return finishOut(uout, stream);
  }

  // ring: reduce-scatter round the ring into the output, then all-gather round the ring
  if (algo == FLAGCX_ALGO_RING && n > 1 && a.outMode == kOutSame && !a.residual && outVis) {
    a.kind = kAllReduceRing;
    CollArgs probe = a;
    const size_t slot = setRing(c, probe, es, 0);
    const size_t perLaunch = slot * (size_t)n;
    for (size_t off = 0; off < count || off == 0; off += perLaunch) {
      const size_t cnt = std::min(perLaunch, count - off);
      a.count = cnt;
      a.xchg = 0;
      setRing(c, a, es, 2 * (n - 1));
      setExtents(a, cnt * es, cnt * oes);
      setIn(c, a, BufView(), uin.local, off * es); // only this rank reads its input
      applyOut(c, a, uout, off * oes);
      FCXCHECK(launch(c, kFamReduce, a, nCtas, stream));
      if (count == 0) break;
    }
    return finishOut(uout, stream);
  }
  if (algo == FLAGCX_ALGO_RING) algo = FLAGCX_ALGO_TWOSHOT;

  // two-shot with a widening result: 16-bit values cross NVLink in both phases
  if (!nvlsAlgo && a.outMode == kOutFloat && inVis && n > 1) {
    a.kind = kAllReduceTwoShotCast;
    for (int p = 0; p < n; ++p) a.aux[p] = (char *)c->internalWin->peer[p] + c->layout.stagingOff;
    // one launch reduces n slices of at most the scratch size
    const size_t perLaunch = S / es / 16 * 16 * (size_t)n;
    for (size_t off = 0; off < count || off == 0; off += perLaunch) {
      const size_t cnt = std::min(perLaunch, count - off);
      a.count = cnt;
      a.xchg = 0;
      setExtents(a, cnt * es, cnt * oes);
      applyIn(c, a, uin, off * es);
      applyOutLocal(c, a, uout, off * oes);
      a.residual = rq.residual ? (const char *)rq.residual + off * oes : nullptr;
      FCXCHECK(launch(c, kFamReduce, a, nCtas, stream));
      if (count == 0) break;
    }
    return finishOut(uout, stream);
  }

  // two-shot
  a.kind = nvlsAlgo ? kAllReduceNvlsTwoShot : kAllReduceTwoShot;
  const bool inDirect = nvlsAlgo ? inMc : inVis, outDirect = nvlsAlgo ? outMc : outVis;
  if (inDirect && outDirect) {
    a.count = count;
    setExtents(a, count * es, count * oes);
    applyIn(c, a, uin);
    applyOut(c, a, uout);
    FCXCHECK(launch(c, nvlsAlgo ? kFamNvls : kFamReduce, a, nCtas, stream));
    return finishOut(uout, stream);
  }
  size_t chunk = half / std::max(es, oes) / (16 * (size_t)n) * (16 * (size_t)n);
  for (size_t off = 0; off < count || off == 0; off += chunk) {
    size_t cnt = std::min(chunk, count - off);
    a.count = cnt;
    a.xchg = 0;
    size_t slice = sliceElems(cnt, n, es);
    if (inDirect) {
      applyIn(c, a, uin, off * es);
      a.userIn = nullptr;
    } else {
      setInStage(c, a, 0);
      a.userIn = (const char *)uin.local + off * es;
      a.nInBlocks = n;
      a.inBlockBytes = slice * es;
      a.userInStride = slice * es;
      a.inTotalBytes = cnt * es;
    }
    if (outDirect) {
      applyOut(c, a, uout, off * oes);
      a.userOut = nullptr;
    } else {
      setOutStage(c, a, half);
      a.userOut = (char *)uout.local + off * oes;
      a.nOutBlocks = n;
      a.outBlockBytes = slice * oes;
      a.userOutStride = slice * oes;
      a.outTotalBytes = cnt * oes;
    }
    a.residual = rq.residual ? (const char *)rq.residual + off * oes : nullptr;
    FCXCHECK(launch(c, nvlsAlgo ? kFamNvls : kFamReduce, a, nCtas, stream));
    if (count == 0) break;
  }
  return finishOut(uout, stream);
}

flagcxResult_t reduceScatter(flagcxComm *c, const DeviceCollRequest &rq, cudaStream_t stream) {
  const int n = c->nranks;
  CollArgs a;
  initArgs(c, a, kReduceScatter, rq.dtype);
  FCXCHECK(setReduceEpilogue(c, a, rq));
  const size_t es = a.elemSize, oes = outElemSize(a), count = rq.count;
  if (n > 1 && count > 0 && a.outMode == kOutSame && !a.residual && count * es <= c->layout.llSlotBytes / 2) {
    TuneChoice pre = c->tuner->choose(flagcxCommOpReduceScatter, count * es * n, n, true, false, (int)es);
    if ((rq.algo >= 0 ? rq.algo : pre.algo) == FLAGCX_ALGO_LL) {
      a.kind = kLlReduceScatter;
      a.count = count;
      a.inStride = count * es;
      setIn(c, a, BufView(), rq.send);
      setOut(c, a, BufView(), rq.recv);
      setExtents(a, count * es * n, count * es);
      note(c, flagcxCommOpReduceScatter, count * es * n, FLAGCX_ALGO_LL, 0);
      return launchLl(c, a, count * es, stream);
    }
  }
  UserBuf uin;
  FCXCHECK(resolve(c, rq.send, count * es * n, 0, stream, &uin));
  const bool inVis = uin.visible();
  const bool nvlsOk = nvlsEligible(c, rq, count) && uin.view.win && uin.view.win->mc;
  TuneChoice ch = c->tuner->choose(flagcxCommOpReduceScatter, count * es * n, n, inVis, nvlsOk, (int)es);
  int algo = rq.algo >= 0 ? rq.algo : ch.algo;
  if (algo == FLAGCX_ALGO_NVLS && !nvlsOk) algo = FLAGCX_ALGO_PULL;
  if (algo == FLAGCX_ALGO_LL) algo = FLAGCX_ALGO_PULL; // not eligible above
  const int nCtas = pickCtas(c, rq, ch);
  note(c, flagcxCommOpReduceScatter, count * es * n, algo, nCtas);
  if (algo == FLAGCX_ALGO_COPY_ENGINE) {
    if (n > 1 && !c->emu && count > 0) {
      // The transport runs on the copy engines: every rank copies block p of its input into
      // slot `rank` of peer p's staging area (n-1 peer copies between two one-CTA barrier
      // kernels), then a kernel without any barrier reduces the n blocks that are now all
      // in local memory.  No SM moves a byte over NVLink, and no buffer has to be visible
      // to the peers.
      const size_t S = c->layout.stagingBytes;
      const size_t chunk = S / n / es / 16 * 16; // elements per slot
      char *stage[FLAGCX_MAX_RANKS];
      for (int p = 0; p < n; ++p) stage[p] = (char *)c->internalWin->peer[p] + c->layout.stagingOff;
      const int me = c->rank;
      for (size_t off = 0; off < count; off += chunk) {
        const size_t cnt = std::min(chunk, count - off);
        FCXCHECK(deviceBarrier(c, stream)); // the slots are free: every rank has finished the reduce before
        for (int i = 1; i < n; ++i) {
          const int p = (me + i) % n;
          FCX_CUDACHECK(cudaMemcpyAsync(stage[p] + (size_t)me * chunk * es, (const char *)rq.send + ((size_t)p * count + off) * es,
                                        cnt * es, cudaMemcpyDeviceToDevice, stream));
        }
        FCXCHECK(deviceBarrier(c, stream)); // every rank's copies have completed
        CollArgs r = a;
        r.kind = kReduceScatter;
        r.count = cnt;
        r.inStride = 0; // in[q] points at the block itself
        r.flags = 0;
        for (int q = 0; q < n; ++q)
          r.in[q] = q == me ? (const char *)rq.send + ((size_t)me * count + off) * es : stage[me] + (size_t)q * chunk * es;
        setOut(c, r, BufView(), rq.recv, off * oes);
        r.residual = rq.residual ? (const char *)rq.residual + off * oes : nullptr;
        setExtents(r, cnt * es, cnt * oes);
        FCXCHECK(launch(c, kFamReduce, r, nCtas, stream));
      }
      return flagcxSuccess;
    }
    algo = FLAGCX_ALGO_PULL;
  }
  if (algo == FLAGCX_ALGO_RING && n > 1 && a.outMode == kOutSame && !a.residual) {
    // neighbours only ever write into each other's scratch: no buffer needs to be visible
    a.kind = kReduceScatterRing;
    CollArgs probe = a;
    const size_t slot = setRing(c, probe, es, 0);
    if (count <= slot) {
      a.count = count;
      setExtents(a, count * es * n, count * oes);
      setRing(c, a, es, n - 1);
      setIn(c, a, BufView(), uin.local);
      setOut(c, a, BufView(), rq.recv);
      return launch(c, kFamReduce, a, nCtas, stream);
    }
    algo = FLAGCX_ALGO_PULL; // blocks larger than a scratch slot take the direct path
  }
  if (inVis) {
    a.kind = algo == FLAGCX_ALGO_NVLS ? kReduceScatterNvls : kReduceScatter;
    a.count = count;
    a.inStride = count * es;
    setExtents(a, count * es * n, count * oes);
    applyIn(c, a, uin);
    setOut(c, a, BufView(), rq.recv);
    return launch(c, algo == FLAGCX_ALGO_NVLS ? kFamNvls : kFamReduce, a, nCtas, stream);
  }
  const size_t S = c->layout.stagingBytes;
  size_t chunk = S / n / es / 16 * 16;
  for (size_t off = 0; off < count || off == 0; off += chunk) {
    size_t cnt = std::min(chunk, count - off);
    a.count = cnt;
    a.inStride = cnt * es;
    setInStage(c, a, 0);
    a.userIn = (const char *)rq.send + off * es;
    a.nInBlocks = n;
    a.inBlockBytes = cnt * es;
    a.userInStride = count * es;
    setOut(c, a, BufView(), rq.recv, off * oes);
    a.residual = rq.residual ? (const char *)rq.residual + off * oes : nullptr;
    FCXCHECK(launch(c, kFamReduce, a, nCtas, stream));
    if (count == 0) break;
  }
  return flagcxSuccess;
}

flagcxResult_t reduceToRoot(flagcxComm *c, const DeviceCollRequest &rq, cudaStream_t stream) {
  const int n = c->nranks;
  CollArgs a;
  initArgs(c, a, kReduceToRoot, rq.dtype);
  FCXCHECK(setReduceEpilogue(c, a, rq));
  a.root = rq.root;
  const size_t es = a.elemSize, oes = outElemSize(a), count = rq.count;
  UserBuf uin;
  FCXCHECK(resolve(c, rq.send, count * es, 0, stream, &uin));
  const bool inVis = uin.visible();
  TuneChoice ch = c->tuner->choose(flagcxCommOpReduce, count * es, n, inVis, false, (int)es);
  const int nCtas = pickCtas(c, rq, ch);
  note(c, flagcxCommOpReduce, count * es, FLAGCX_ALGO_PULL, nCtas);
  if (inVis) {
    a.count = count;
    setExtents(a, count * es, count * oes);
    applyIn(c, a, uin);
    setOut(c, a, BufView(), rq.recv);
    return launch(c, kFamReduce, a, nCtas, stream);
  }
  const size_t S = c->layout.stagingBytes;
  size_t chunk = S / es / 16 * 16;
  for (size_t off = 0; off < count || off == 0; off += chunk) {
    size_t cnt = std::min(chunk, count - off);
    a.count = cnt;
    setInStage(c, a, 0);
    a.userIn = (const char *)rq.send + off * es;
    a.nInBlocks = 1;
    a.inBlockBytes = cnt * es;
    setOut(c, a, BufView(), rq.recv, off * oes);
    FCXCHECK(launch(c, kFamReduce, a, nCtas, stream));
    if (count == 0) break;
  }
  return flagcxSuccess;
}

// ---- copy family: everything in bytes -----------------------------------------------
flagcxResult_t copyCollective(flagcxComm *c, const DeviceCollRequest &rq, cudaStream_t stream) {
  const int n = c->nranks, me = c->rank;
  const size_t es = getFlagcxDataTypeSize(rq.dtype);
  const size_t blk = rq.count * es; // bytes per rank-block (or the whole message)
  CollArgs a;
  initArgs(c, a, kBarrierOnly, flagcxUint8);
  a.elemSize = 1;
  a.root = rq.root;

  size_t sendBytes = blk, recvBytes = blk;
  int pushKind = -1, pullKind = -1;
  bool nBlocksIn = false; // the input holds one block per rank
  switch (rq.op) {
    case flagcxCommOpAllGather: recvBytes = blk * n; pushKind = kAllGatherPush; pullKind = kAllGatherPull; break;
    case flagcxCommOpBroadcast: pushKind = kBroadcastPush; pullKind = kBroadcastPull; break;
    case flagcxCommOpGather: recvBytes = blk * n; pullKind = kGatherPull; break;
    case flagcxCommOpScatter: sendBytes = blk * n; pullKind = kScatterPull; nBlocksIn = true; break;
    case flagcxCommOpAlltoAll:
      sendBytes = recvBytes = blk * n; pushKind = kAllToAllPush; pullKind = kAllToAllPull; nBlocksIn = true;
      break;
    default: return flagcxInternalError;
  }
  // Rooted operations: only the root's send (scatter, broadcast) or recv (gather)
  // argument is meaningful, so visibility is judged on the argument every rank has.
  const bool sendEverywhere = rq.op != flagcxCommOpBroadcast && rq.op != flagcxCommOpScatter;
  const bool recvEverywhere = rq.op != flagcxCommOpGather;
  const bool iAmRoot = me == rq.root;
  if ((rq.op == flagcxCommOpAllGather || rq.op == flagcxCommOpAlltoAll) && n > 1 && blk > 0 &&
      blk <= c->layout.llSlotBytes / 2) {
    TuneChoice pre = c->tuner->choose(rq.op, recvBytes, n, true, false);
    if ((rq.algo >= 0 ? rq.algo : pre.algo) == FLAGCX_ALGO_LL) {
      a.kind = rq.op == flagcxCommOpAllGather ? kLlAllGather : kLlAllToAll;
      a.count = blk;
      a.inStride = blk;
      a.outStride = blk;
      setIn(c, a, BufView(), rq.send);
      setOut(c, a, BufView(), rq.recv);
      note(c, rq.op, recvBytes, FLAGCX_ALGO_LL, 0);
      setExtents(a, sendBytes, recvBytes);
      return launchLl(c, a, blk, stream);
    }
  }
  UserBuf uin, uout;
  if (sendEverywhere) FCXCHECK(resolve(c, rq.send, sendBytes, 0, stream, &uin));
  if (recvEverywhere) FCXCHECK(resolve(c, rq.recv, recvBytes, 1, stream, &uout));
  bool inVis = uin.visible(), outVis = uout.visible();
  // Scatter has no argument that every rank owns: with run-time pointer exchange the
  // root alone publishes its input and the others learn it.
  const bool exchanging = c->emu ? getEnv("FLAGCX_EMU_EXCHANGE") != nullptr : c->autoExport;
  bool scatterExchange = false;
  if (rq.op == flagcxCommOpScatter && exchanging && n > 1) {
    if (iAmRoot) {
      FCXCHECK(resolve(c, rq.send, sendBytes, 0, stream, &uin));
      if (uin.reach == kReachWindow) { // peers passed no pointer they could look up: tell them
        Window *w = uin.view.win;
        bool known = true;
        for (int p = 0; p < n; ++p) known &= w->selfAt[p] != nullptr;
        if (known) {
          for (int p = 0; p < n; ++p) uin.peerVa[p] = (char *)w->selfAt[p] + uin.view.off;
          uin.reach = kReachExport;
        }
      }
      scatterExchange = uin.reach == kReachExport;
      if (!scatterExchange) { FCX_WARN("scatter: the root's buffer cannot be published to the peers"); return flagcxInternalError; }
    } else {
      scatterExchange = true;
    }
    inVis = true;
  }
  const bool nvlsOk = rq.op == flagcxCommOpAllGather && c->nvls && !c->emu && uout.view.win && uout.view.win->mc &&
                      blk % 16 == 0 && aligned16(rq.send);
  TuneChoice ch = c->tuner->choose(rq.op, std::max(sendBytes, recvBytes), n, inVis || outVis, nvlsOk);
  int algo = rq.algo >= 0 ? rq.algo : ch.algo;
  if (algo == FLAGCX_ALGO_NVLS && !nvlsOk) algo = FLAGCX_ALGO_PUSH;
  if (algo == FLAGCX_ALGO_LL) algo = FLAGCX_ALGO_PUSH; // not eligible above
  // Copy-engine all-gather: needs every rank's output inside a window (the host must know
  // the peers' addresses) and real peers.
  const bool ceWanted = algo == FLAGCX_ALGO_COPY_ENGINE && rq.op == flagcxCommOpAllGather && n > 1 && !c->emu &&
                        uout.reach == kReachWindow && blk > 0;
  if (algo == FLAGCX_ALGO_COPY_ENGINE && !ceWanted) algo = FLAGCX_ALGO_PUSH;
  const bool ringWanted = algo == FLAGCX_ALGO_RING && rq.op == flagcxCommOpAllGather && n > 1;
  if (algo == FLAGCX_ALGO_RING) algo = FLAGCX_ALGO_PUSH;
  if (algo == FLAGCX_ALGO_PUSH && !(outVis && pushKind >= 0)) algo = FLAGCX_ALGO_PULL;
  if (algo == FLAGCX_ALGO_PULL && !inVis && outVis && pushKind >= 0) algo = FLAGCX_ALGO_PUSH; // avoids staging
  if (algo != FLAGCX_ALGO_PUSH && algo != FLAGCX_ALGO_NVLS && !ceWanted) algo = FLAGCX_ALGO_PULL;
  const int nCtas = pickCtas(c, rq, ch);
  note(c, rq.op, std::max(sendBytes, recvBytes), algo, nCtas);

  if (ceWanted) {
    // 1. a one-CTA barrier kernel: every rank has reached this call in its stream, so
    //    nobody still reads the previous contents of its output;
    // 2. n-1 peer copies and the local one, on the copy engines, nearest neighbour first
    //    so that no rank is the target of all the others at once;
    // 3. the barrier again: it starts after this rank's copies have completed (stream
    //    order) and ends when every rank's have.
    FCXCHECK(deviceBarrier(c, stream));
    Window *w = uout.view.win;
    for (int i = 0; i < n; ++i) {
      const int p = (me + i) % n;
      char *dst = (char *)w->peer[p] + uout.view.off + (size_t)me * blk;
      if (p == me && dst == (const char *)rq.send) continue; // in place
      FCX_CUDACHECK(cudaMemcpyAsync(dst, rq.send, blk, cudaMemcpyDeviceToDevice, stream));
    }
    return deviceBarrier(c, stream);
  }
  if (algo == FLAGCX_ALGO_NVLS) {
    a.kind = kAllGatherNvls;
    a.dtype = flagcxFloat32; // multimem.st moves raw 16-byte packs
    a.elemSize = 4;
    a.count = blk / 4;
    a.outStride = blk;
    setIn(c, a, BufView(), rq.send);
    setOut(c, a, uout.view, rq.recv);
    return launch(c, kFamNvls, a, nCtas, stream);
  }
  if (ringWanted && outVis) {
    a.kind = kAllGatherRing;
    setExtents(a, sendBytes, recvBytes);
    a.count = blk;
    a.inStride = blk;
    a.outStride = blk;
    setRing(c, a, 1, n - 1);
    setIn(c, a, BufView(), rq.send);
    applyOut(c, a, uout);
    FCXCHECK(launch(c, kFamCopy, a, nCtas, stream));
    return finishOut(uout, stream);
  }
  if (algo == FLAGCX_ALGO_PUSH) {
    a.kind = pushKind;
    setExtents(a, sendBytes, recvBytes);
    a.count = blk;
    a.inStride = blk;
    a.outStride = blk;
    // the input is only read locally: a stand-in is not needed for it
    setIn(c, a, BufView(), rq.send);
    applyOut(c, a, uout);
    FCXCHECK(launch(c, kFamCopy, a, nCtas, stream));
    return finishOut(uout, stream);
  }
  a.kind = pullKind;
  if (inVis) {
    setExtents(a, sendBytes, recvBytes);
    a.count = blk;
    a.inStride = blk;
    a.outStride = blk;
    if (scatterExchange) {
      setIn(c, a, BufView(), iAmRoot ? uin.local : nullptr);
      a.xchg |= kXchgIn;
      for (int p = 0; p < n; ++p) a.pubIn[p] = iAmRoot ? (const char *)uin.peerVa[p] : nullptr;
    } else {
      applyIn(c, a, uin);
    }
    setOut(c, a, BufView(), rq.recv);
    return launch(c, kFamCopy, a, nCtas, stream);
  }
  // staged input
  const size_t S = c->layout.stagingBytes;
  size_t chunk = (nBlocksIn ? S / n : S) / 16 * 16;
  const bool iStage = !(rq.op == flagcxCommOpBroadcast || rq.op == flagcxCommOpScatter) || iAmRoot;
  for (size_t off = 0; off < blk || off == 0; off += chunk) {
    size_t len = std::min(chunk, blk - off);
    a.count = len;
    a.inStride = len;   // staged blocks are packed
    a.outStride = blk;  // the user's output keeps its own block stride
    setInStage(c, a, 0);
    a.userIn = iStage ? (const char *)rq.send + off : nullptr;
    a.nInBlocks = nBlocksIn ? n : 1;
    a.inBlockBytes = len;
    a.userInStride = blk;
    setOut(c, a, BufView(), rq.recv, off);
    FCXCHECK(launch(c, kFamCopy, a, nCtas, stream));
    if (blk == 0) break;
  }
  return flagcxSuccess;
}

flagcxResult_t allToAllv(flagcxComm *c, const DeviceCollRequest &rq, cudaStream_t stream) {
  const int n = c->nranks;
  const size_t es = getFlagcxDataTypeSize(rq.dtype);
  size_t sendSpan = 0, recvSpan = 0, total = 0;
  for (int p = 0; p < n; ++p) {
    sendSpan = std::max(sendSpan, (rq.sendDispls[p] + rq.sendCounts[p]) * es);
    recvSpan = std::max(recvSpan, (rq.recvDispls[p] + rq.recvCounts[p]) * es);
    total += rq.sendCounts[p] * es;
  }
  // Spans differ between ranks, so "is it inside a window / exportable" is decided on a
  // property every rank shares: the communicator's mode.  A rank whose buffer cannot be
  // exported gets a stand-in inside resolve().
  UserBuf uin;
  FCXCHECK(resolve(c, rq.send, sendSpan, 0, stream, &uin));
  if (!rq.send && c->autoExport) uin.reach = kReachExport; // nothing to send: publish a null pointer
  if (uin.visible()) {
    CollArgs a;
    initArgs(c, a, kAllToAllvPull, rq.dtype);
    for (int p = 0; p < n; ++p) {
      a.sendCounts[p] = rq.sendCounts[p];
      a.sendDispls[p] = rq.sendDispls[p];
      a.recvCounts[p] = rq.recvCounts[p];
      a.recvDispls[p] = rq.recvDispls[p];
    }
    applyIn(c, a, uin);
    setOut(c, a, BufView(), rq.recv);
    setExtents(a, sendSpan, recvSpan);
    // Every rank must launch the same grid (CTA b meets CTA b of its peers), but the byte
    // counts differ from rank to rank: the count cannot follow the size here.
    TuneChoice ch;
    ch.nCtas = (int)readParam("ALLTOALLV_CTAS", 16);
    const int nCtas = pickCtas(c, rq, ch);
    note(c, flagcxCommOpAlltoAllv, total, FLAGCX_ALGO_PULL, nCtas);
    return launch(c, kFamCopy, a, nCtas, stream);
  }
  // unregistered: n sends and n receives through the point-to-point slots
  note(c, flagcxCommOpAlltoAllv, total, FLAGCX_ALGO_PULL, FLAGCX_P2P_CTAS);
  for (int p = 0; p < n; ++p) {
    c->groupOps.push_back({true, p, (char *)const_cast<void *>(rq.send) + rq.sendDispls[p] * es,
                           rq.sendCounts[p] * es, stream});
    c->groupOps.push_back({false, p, (char *)rq.recv + rq.recvDispls[p] * es, rq.recvCounts[p] * es, stream});
  }
  return deviceGroupLaunch(c);
}

} // namespace

flagcxResult_t deviceBarrier(flagcxComm *c, cudaStream_t stream) {
  CollArgs a;
  initArgs(c, a, kBarrierOnly, flagcxUint8);
  a.flags = kFlagBeginBarrier;
  return launch(c, kFamCopy, a, 1, stream);
}

flagcxResult_t deviceCollective(flagcxComm *c, const DeviceCollRequest &rq, cudaStream_t stream) {
  if (c->asyncError.load() != flagcxSuccess) {
    FCX_WARN("communicator is in an error state; destroy it and create a new one");
    return (flagcxResult_t)c->asyncError.load();
  }
  if (getFlagcxDataTypeSize(rq.dtype) == 0) return flagcxInvalidArgument;
  switch (rq.op) {
    case flagcxCommOpAllReduce: return allReduce(c, rq, stream);
    case flagcxCommOpReduceScatter: return reduceScatter(c, rq, stream);
    case flagcxCommOpReduce: return reduceToRoot(c, rq, stream);
    case flagcxCommOpAllGather:
    case flagcxCommOpBroadcast:
    case flagcxCommOpGather:
    case flagcxCommOpScatter:
    case flagcxCommOpAlltoAll: return copyCollective(c, rq, stream);
    case flagcxCommOpAlltoAllv: return allToAllv(c, rq, stream);
    default: return flagcxInvalidArgument;
  }
}

// Launches everything queued by flagcxSend/flagcxRecv since flagcxGroupStart.  Each
// launch carries at most one message per peer and direction; later messages to the
// same peer go into the next launch, in call order on both sides.
flagcxResult_t deviceGroupLaunch(flagcxComm *c) {
  std::vector<GroupOp> ops;
  ops.swap(c->groupOps);
  const int n = c->nranks;
  size_t next = 0;
  std::vector<char> used(ops.size(), 0);
  size_t remaining = ops.size();
  bool first = true;
  while (remaining > 0 || (first && c->emu)) {
    first = false;
    P2pArgs a;
    memset(&a, 0, sizeof a);
    cudaStream_t stream = ops.empty() ? nullptr : ops[0].stream;
    for (size_t i = next; i < ops.size(); ++i) {
      if (used[i]) continue;
      GroupOp &op = ops[i];
      if (op.peer < 0 || op.peer >= n) return flagcxInvalidArgument;
      if (op.isSend) {
        if (a.sendSrc[op.peer]) continue; // slot of this peer is taken in this launch
        a.sendSrc[op.peer] = (const char *)op.buf;
        a.sendBytes[op.peer] = op.bytes;
        if (!op.buf) a.sendSrc[op.peer] = (const char *)c->internalWin->local; // zero-byte message
      } else {
        if (a.recvDst[op.peer]) continue;
        a.recvDst[op.peer] = (char *)op.buf;
        a.recvBytes[op.peer] = op.bytes;
        if (!op.buf) a.recvDst[op.peer] = (char *)c->internalWin->local;
      }
      used[i] = 1;
      --remaining;
    }
    if (a.sendSrc[c->rank] && a.recvDst[c->rank] && a.sendBytes[c->rank] != a.recvBytes[c->rank]) {
      FCX_WARN("send to self of %zu bytes meets a receive of %zu bytes", a.sendBytes[c->rank], a.recvBytes[c->rank]);
      return flagcxInvalidArgument;
    }
    a.slotBytes = c->layout.p2pSlotBytes;
    for (int p = 0; p < n; ++p) {
      char *base = (char *)c->internalWin->peer[p];
      a.stage[p] = base ? base + c->layout.p2pStageOff : nullptr;
      a.ready[p] = base ? (unsigned long long *)(base + c->layout.p2pReadyOff) : nullptr;
      a.done[p] = base ? (unsigned long long *)(base + c->layout.p2pDoneOff) : nullptr;
      a.sendSeq[p] = c->p2pSendSeq[p];
      a.recvSeq[p] = c->p2pRecvSeq[p];
      if (p != c->rank) {
        if (a.sendSrc[p]) c->p2pSendSeq[p] += (a.sendBytes[p] + a.slotBytes - 1) / a.slotBytes;
        if (a.recvDst[p]) c->p2pRecvSeq[p] += (a.recvBytes[p] + a.slotBytes - 1) / a.slotBytes;
      }
    }
    c->stats[flagcxCommOpSend].calls++;
    if (c->emu) {
      FCXCHECK(emuSubmit(c, 3, nullptr, &a, FLAGCX_P2P_CTAS, stream));
    } else {
      LaunchCtx lc;
      lc.comm = &c->dev;
      lc.stream = stream;
      lc.nCtas = FLAGCX_P2P_CTAS;
      cudaError_t e = launchP2pKernel(lc, a);
      if (e != cudaSuccess) {
        FCX_WARN("p2p kernel launch failed: %s", cudaGetErrorString(e));
        return flagcxUnhandledDeviceError;
      }
    }
  }
  return flagcxSuccess;
}

} // namespace fcx
