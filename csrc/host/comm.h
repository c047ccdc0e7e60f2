// comm.h -- the communicator and what hangs off it: the device world (peer-mapped
// windows, sync pads, staging), the window registry, the group queue, statistics
// and the tuner.
//
// One struct replaces the FlagCX pair flagcxComm / flagcxHeteroComm
// (flagcx/core/include/global_comm.h:73-139, flagcx/core/include/comm.h:170-386
// in the FlagCX project).  There is no runner table: a collective either runs on
// the device path (one kernel over NVLink) or on the host path (sockets).
#pragma once
#include <atomic>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "trace.h"
#include "bootstrap.h"
#include "cpu_coll.h"
#include "cuda_rt.h"
#include "flagcx.h"
#include "flagcx_device.cuh"
#include "reg_cache.h"
#include "../kernels/coll_args.h"

struct flagcxStream {
  cudaStream_t base;
};
struct flagcxEvent {
  cudaEvent_t base;
};

namespace fcx {

struct Tuner;

// A buffer that every rank of the NVLink domain has mapped.  peer[r] is rank r's
// copy as addressed from this process; offsets are symmetric.
struct Window {
  void *local = nullptr;
  size_t size = 0;
  void *peer[FLAGCX_MAX_RANKS] = {};
  void *selfAt[FLAGCX_MAX_RANKS] = {}; // this rank's copy as addressed by rank r (for published pointers)
  void *mc = nullptr;   // multicast alias (NVLS) or null
  int flags = 0;
  bool internal = false;
  int emuSeq = -1;      // emulated world: which registration round this window belongs to
  // resources to release
  std::vector<cu::VmmBlock> imports;    // VMM mappings of the peers' blocks
  std::vector<void *> ipcOpened;        // cudaIpcOpenMemHandle results
  cu::McObject mcObj;
  cu::VmmBlock owned;                   // set when the library allocated the local block
};

// Sorted interval map from local address to window.
class WindowRegistry {
 public:
  void add(Window *w);
  void remove(Window *w);
  // The window that fully contains [p, p+bytes), or nullptr.
  Window *find(const void *p, size_t bytes) const;
  std::vector<Window *> all() const;

 private:
  mutable std::mutex mu_;
  std::map<uintptr_t, Window *> byBase_;
};

struct OpStats {
  uint64_t calls = 0, bytes = 0;
  int lastAlgo = -1;
  int lastCtas = 0;
  float lastMs = 0.f;
};

// A queued operation of an open group.
struct GroupOp {
  bool isSend;
  int peer;
  void *buf;
  size_t bytes;
  cudaStream_t stream;
};

// Layout of the internal window of every rank (offsets are identical everywhere).
struct SyncLayout {
  size_t inboxOff, signalOff, metaOff, p2pReadyOff, p2pDoneOff, ptrPadOff, zeroedBytes;
  size_t stagingOff, stagingBytes;   // collectives on unregistered buffers
  size_t p2pStageOff, p2pSlotBytes;  // send/recv: FLAGCX_MAX_RANKS slots
  size_t llOff, llSlotBytes;         // LL slots: [parity 2][sender FLAGCX_MAX_RANKS][llSlotBytes]
  size_t ringOff;                    // ring step flags: one u64 per CTA slot
  size_t total;
};

struct EmuWorld; // several ranks in one process on one GPU (tests, 1-GPU boxes)

} // namespace fcx

struct flagcxComm {
  int rank = -1, nranks = 0;
  int localRank = 0, localRanks = 1;
  int cudaDev = -1;
  uint64_t magic = 0;

  // ---- host side (always present) ----
  std::unique_ptr<fcx::Bootstrap> bootstrap;
  std::unique_ptr<fcx::HostNet> hostNet;
  fcx::CpuColl cpu{nullptr};

  // ---- device side (present when every rank is a GPU on this host with P2P) ----
  bool devicePath = false;
  bool nvls = false;               // internal window is multicast-bound
  fcx::Window *internalWin = nullptr;
  fcx::SyncLayout layout{};
  flagcxDevComm dev{};             // host copy of what kernels receive
  flagcxDevStatus *status = nullptr; // pinned host page
  flagcxDevStatus *statusDev = nullptr; // device alias of the same page
  void *localSync = nullptr;       // epochs, shadows, counters (cudaMalloc)
  // User buffers outside symmetric windows: exported to the peers on first use
  // (reg_cache.h) and found by the peers' kernels through the run-time pointer
  // exchange.  Off (legacy in-kernel staging) when any rank could not start the service.
  std::unique_ptr<fcx::RegCache> reg;
  bool exportUserBuffers = false;
  // Export any buffer a collective meets, not only those the caller registered with
  // flagcxCommRegister.  Only safe when the library hears about frees (an exported
  // allocation must be unmapped at the peers before it is freed): set by allocator
  // integrations (the torch backend) or by FLAGCX_USER_BUFFER_EXPORT=2.
  bool autoExport = false;
  uint64_t xchgSeq = 0;            // collective launches so far (same on every rank)
  uint64_t llSeq = 0;              // LL operations so far (same on every rank)
  uint64_t ringSeq = 0;            // ring steps so far (same on every rank)
  void *bounce[2] = {nullptr, nullptr}; // exportable stand-ins for buffers that are not (input, output)
  size_t bounceBytes[2] = {0, 0};
  int winSeq = 0;                  // window registrations so far (same on every rank)
  unsigned int *putArrival = nullptr; // device word used by put kernels
  volatile uint64_t *rmaCounter = nullptr; // pinned: one-sided operations completed
  uint64_t rmaIssued = 0;
  fcx::Window *oneSideSignalWin = nullptr;
  uint64_t p2pSendSeq[FLAGCX_MAX_RANKS] = {}; // chunks sent to / received from each peer so far
  uint64_t p2pRecvSeq[FLAGCX_MAX_RANKS] = {};
  std::vector<uint64_t> signalSent; // per-peer count of flagcxSignal/PutSignal issued
  std::vector<uint64_t> signalSeen; // per-peer count consumed by flagcxWaitSignal
  fcx::WindowRegistry windows;
  std::vector<fcx::Window *> oneSideData; // memory regions in registration order
  std::vector<char> oneSideOwned;         // 1: the window was created by flagcxOneSideRegister
  cudaStream_t internalStream = nullptr;
  std::unique_ptr<fcx::Tuner> tuner;

  // ---- emulated world ----
  fcx::EmuWorld *emu = nullptr;

  // ---- group ----
  int groupDepth = 0;
  std::vector<fcx::GroupOp> groupOps;

  // ---- errors / observability ----
  std::atomic<int> asyncError{flagcxSuccess};
  std::string lastError;
  fcx::OpStats stats[flagcxNumCommOps];
  fcx::Trace trace;
  std::thread watchdog;
  std::atomic<bool> watchdogStop{false};
  bool finalized = false;
  bool aborted = false;

  // staged fallback when ranks cannot reach each other over NVLink
  void *hostStage = nullptr;
  size_t hostStageBytes = 0;
  // two-level route (hier.cc): child communicator of this node's ranks, node geometry,
  // pinned and device scratch of the inter-node step
  flagcxComm *intra = nullptr;
  int nNodes = 1, nodeRanks = 0;
  void *hierPinned = nullptr, *hierDev = nullptr;
  size_t hierPinnedBytes = 0, hierDevBytes = 0;
};

namespace fcx {

constexpr uint64_t kCommMagic = 0x464c4147434f4d4dull; // "FLAGCOMM"

// comm.cc
SyncLayout makeSyncLayout();
void fillDevComm(flagcxComm *c);
flagcxResult_t allocLocalDeviceState(flagcxComm *c);
flagcxResult_t commCreate(flagcxComm **out, int nranks, const flagcxUniqueId &id, int rank);
flagcxResult_t commDestroy(flagcxComm *c);
bool commValid(const flagcxComm *c);
flagcxResult_t windowRegister(flagcxComm *c, void *buff, size_t size, int flags, Window **out);
flagcxResult_t windowDeregister(flagcxComm *c, Window *w);
// Poll the device status block; turns a device-side error into the async error.
flagcxResult_t commCheckDevice(flagcxComm *c);

// device_coll.cc -- device path of every collective
struct DeviceCollRequest {
  flagcxCommOp_t op;
  const void *send;
  void *recv;
  size_t count; // per-rank-slice count for AG/RS/A2A, total otherwise
  flagcxDataType_t dtype;
  flagcxRedOp_t redOp;
  int root;
  // fused epilogue (reduce family)
  float scale = 1.0f;
  flagcxDataType_t outDtype = flagcxNumTypes; // flagcxNumTypes: same as dtype
  const void *residual = nullptr;
  // alltoallv
  const size_t *sendCounts = nullptr, *sendDispls = nullptr, *recvCounts = nullptr, *recvDispls = nullptr;
  // overrides (-1: let the tuner decide)
  int algo = -1;
  int nCtas = -1;
};
flagcxResult_t deviceCollective(flagcxComm *c, const DeviceCollRequest &rq, cudaStream_t stream);
flagcxResult_t deviceGroupLaunch(flagcxComm *c);
flagcxResult_t deviceBarrier(flagcxComm *c, cudaStream_t stream);

// hier.cc -- two-level route for communicators that span several NVLink domains
flagcxResult_t hierSetup(flagcxComm *c, const std::vector<uint64_t> &hostHashes, const std::vector<int> &hasGpu);
void hierTeardown(flagcxComm *c);
flagcxResult_t hierAllReduce(flagcxComm *c, const void *send, void *recv, size_t count, flagcxDataType_t dt,
                             flagcxRedOp_t op, cudaStream_t stream);
flagcxResult_t hierAllGather(flagcxComm *c, const void *send, void *recv, size_t count, flagcxDataType_t dt,
                             cudaStream_t stream);

// emu.cc
flagcxResult_t emuWorldCreate(int nranks, int dev, flagcxComm **comms);
flagcxResult_t emuWorldDestroy(flagcxComm *any);
// Called by deviceCollective for an emulated rank: parks the request until all
// ranks of the world have posted theirs, then launches once.
flagcxResult_t emuSubmit(flagcxComm *c, int family, const CollArgs *coll, const P2pArgs *p2p, int nCtas,
                         cudaStream_t stream);
flagcxResult_t emuWindowRegister(flagcxComm *c, void *buff, size_t size, int flags, Window **out);
// Generic form for kernels with their own argument block.
constexpr int kMaxEmuBlobBytes = 2048;
struct LaunchCtx;
typedef cudaError_t (*EmuBlobLaunch)(const LaunchCtx &lc, const void *deviceArgsArray);
flagcxResult_t emuSubmitBlob(flagcxComm *c, int kernelId, const void *args, size_t argBytes, int nCtas,
                             cudaStream_t stream, EmuBlobLaunch launch);

} // namespace fcx
