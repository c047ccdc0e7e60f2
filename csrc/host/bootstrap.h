// bootstrap.h -- out-of-band rendezvous and small-message exchange over TCP.
//
// Plays the role of flagcx/service/bootstrap.cc in the FlagCX project: a root
// listener (thread of the process that created the unique id) collects every
// rank's listening address and hands the complete table back; afterwards ranks
// talk pairwise over lazily opened connections with tagged messages, and the
// usual helpers (allgather, barrier, broadcast) are built on those.
#pragma once
#include <deque>
#include <memory>
#include <mutex>
#include <vector>

#include "socket.h"

namespace fcx {

// Layout of the opaque 256-byte flagcxUniqueId.
struct BootstrapId {
  uint64_t magic;
  uint64_t nonce;
  SockAddr root;
  uint32_t externalRoot; // 1: address came from FLAGCX_COMM_ID, rank 0 must serve it
  uint32_t pad;
};
static_assert(sizeof(BootstrapId) <= FLAGCX_UNIQUE_ID_BYTES, "id too large");

constexpr uint64_t kBootstrapMagic = 0x46434231424f4f54ull; // "FCB1BOOT"

// Creates an id; unless FLAGCX_COMM_ID names the address, also starts the root
// listener thread that serves exactly one communicator and then exits.
flagcxResult_t bootstrapCreateId(flagcxUniqueId *out);

class Bootstrap {
 public:
  Bootstrap() = default;
  ~Bootstrap() { close(); }
  Bootstrap(const Bootstrap &) = delete;

  flagcxResult_t init(const flagcxUniqueId &id, int rank, int nranks);
  void close();

  int rank() const { return rank_; }
  int nranks() const { return nranks_; }
  uint64_t nonce() const { return nonce_; }
  const SockAddr &peerAddr(int r) const { return addrs_[r]; }

  // Tagged, ordered per (peer, tag).  recv blocks until a message with that tag
  // from that peer arrives; messages with other tags are parked meanwhile.
  flagcxResult_t send(int peer, int tag, const void *data, size_t bytes);
  flagcxResult_t recv(int peer, int tag, void *data, size_t bytes);

  // data holds nranks slots of `bytes`; slot[rank] is the contribution.
  flagcxResult_t allGather(void *data, size_t bytes);
  flagcxResult_t barrier();
  flagcxResult_t broadcast(void *data, size_t bytes, int root);

  void setTimeoutMs(int ms) { timeoutMs_ = ms; }
  int timeoutMs() const { return timeoutMs_; }

 private:
  struct Parked { int tag; std::vector<char> data; };
  flagcxResult_t sendSock(int peer, Socket **s);
  flagcxResult_t recvSock(int peer, Socket **s);

  int rank_ = -1, nranks_ = 0;
  uint64_t magic_ = 0, nonce_ = 0;
  int timeoutMs_ = 120000;
  Socket listen_;
  std::vector<SockAddr> addrs_;
  std::vector<Socket> out_, in_;
  std::vector<std::deque<Parked>> parked_;
  std::mutex mu_;
};

} // namespace fcx
