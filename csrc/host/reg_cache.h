// reg_cache.h -- user-buffer registration on demand: makes an ordinary device
// allocation (a cudaMalloc block, which is what a PyTorch caching-allocator segment
// is) readable and writable by the other ranks of the NVLink domain without any
// collective call.
//
// Takes the place of the registration pool and flagcxCommRegister of the FlagCX
// project (flagcx/core/reg_pool.cc, flagcx/flagcx.cc:1267-1390), which hand user
// buffers to NCCL for registration.  Here the mechanism is:
//
//   * every communicator runs a small service thread that listens on an abstract
//     Unix stream socket;
//   * the first time a rank passes a buffer from an allocation it has not exported
//     yet, it takes the allocation's cudaIpc handle and asks every peer's service
//     thread to open it; each peer answers with the address at which the allocation
//     is now mapped IN THE PEER'S address space;
//   * the collective kernel of the owning rank then publishes "my input/output is at
//     address X in your address space" to each peer before the kernel's first
//     barrier (publishPointers / learnPointers in kernels/coll_common.cuh), so no rank ever needs
//     to know on the host where a peer's buffer lives.
//
// Because the peers' main threads take no part, ranks need not meet a new allocation
// at the same call, or at all: registration is one-sided.  Entries are validated on
// every use against the driver's allocation id, so an address that was freed and
// handed out again is re-exported instead of being read through a stale mapping.
#pragma once
#include <atomic>
#include <functional>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "base.h"
#include "flagcx_device.cuh"

namespace fcx {

constexpr int kIpcHandleBytes = 64;

// What the cache needs from the CUDA layer; unit tests substitute plain memory.
struct RegBackend {
  // Base address, size and a never-reused id of the allocation holding p.
  std::function<bool(const void *p, void **base, size_t *size, uint64_t *id)> identify;
  // Fills the 64-byte inter-process handle of the allocation starting at base.
  std::function<bool(void *base, void *handle)> exportHandle;
  // Maps / unmaps an allocation of another process in this one (service thread).
  std::function<void *(const void *handle)> open;
  std::function<void(void *va)> close;
  // Called once at the start of the service thread (binds the thread to the device).
  std::function<void()> threadInit;
};
RegBackend cudaRegBackend(int dev);

class RegCache {
 public:
  RegCache() = default;
  ~RegCache() { stop(); }
  RegCache(const RegCache &) = delete;

  // key: shared by the ranks of one communicator and different between
  // communicators (the bootstrap nonce).  Starts the service thread.
  flagcxResult_t start(uint64_t key, int rank, int nranks, RegBackend backend);
  // Stops the service thread and unmaps whatever it opened for peers.  Callers
  // make sure no kernel of any rank still uses those mappings (the communicator
  // leaves through a barrier first).
  void stop();
  bool running() const { return running_.load(); }

  // Addresses of [p, p+bytes) as seen by each peer (peerVa[rank] = p).  Returns
  // false when the allocation cannot be exported (not a cudaMalloc block, a peer
  // failed to open it); the verdict is cached per allocation.
  bool lookup(const void *p, size_t bytes, void *peerVa[FLAGCX_MAX_RANKS]) { return find(p, bytes, peerVa, true); }
  // The same, but an allocation that has not been exported yet stays that way.
  bool lookupKnown(const void *p, size_t bytes, void *peerVa[FLAGCX_MAX_RANKS]) { return find(p, bytes, peerVa, false); }
  // Forgets the allocation that contains p (and has every peer unmap it).
  void forget(const void *p);

  struct Counters { uint64_t hits = 0, exports = 0, refused = 0, stale = 0, opened = 0, closed = 0; };
  Counters counters() const;

 private:
  struct Entry {
    void *base = nullptr;
    size_t size = 0;
    uint64_t id = 0;
    bool exportable = false;
    void *peerBase[FLAGCX_MAX_RANKS] = {};
  };
  struct Request { uint32_t op, srcRank; uint64_t va; unsigned char handle[kIpcHandleBytes]; };
  struct Reply { uint64_t va; };

  bool find(const void *p, size_t bytes, void *peerVa[FLAGCX_MAX_RANKS], bool exportNew);
  void serve();
  bool handle(int fd);
  int peerFd(int peer);
  bool call(int peer, const Request &rq, Reply *rp);
  bool exportEntry(Entry &e);
  void closeAtPeers(const Entry &e);

  uint64_t key_ = 0;
  int rank_ = -1, nranks_ = 0;
  RegBackend be_;
  std::atomic<bool> running_{false}, stopFlag_{false};
  int listenFd_ = -1, wakeFd_[2] = {-1, -1};
  std::thread thread_;
  // client side (caller threads)
  mutable std::mutex mu_;
  std::map<uintptr_t, Entry> entries_;
  std::vector<int> peerFds_;
  Counters cnt_;
  // service side: what this rank opened on behalf of its peers
  std::mutex openMu_;
  std::vector<void *> opened_;
  std::atomic<uint64_t> nOpened_{0}, nClosed_{0};
};

} // namespace fcx
