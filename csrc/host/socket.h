// socket.h -- TCP sockets with deadlines, interface discovery, and Unix-domain
// sockets that pass file descriptors (used to hand CUDA VMM allocations to the
// other local ranks).
//
// Covers the role of flagcx/core/socket.cc and flagcx/core/ipcsocket.cc in the
// FlagCX project.  Every blocking operation takes a deadline and returns
// flagcxRemoteError when the peer closed or flagcxSystemError on timeout, so a
// dead rank surfaces as an error code instead of a hang.
#pragma once
#include <netinet/in.h>
#include <sys/socket.h>
#include <sys/un.h>

#include <string>
#include <vector>

#include "base.h"

namespace fcx {

union SockAddr {
  sockaddr sa;
  sockaddr_in in4;
  sockaddr_in6 in6;
  sockaddr_storage ss;
};
static_assert(sizeof(SockAddr) == 128, "address must fit the unique id");

struct NetIf {
  std::string name;
  SockAddr addr;
};

std::string addrToString(const SockAddr &a);
// Parses "ip:port", "[v6]:port" or "host:port".
flagcxResult_t addrFromString(const char *s, SockAddr *out);
int addrLen(const SockAddr &a);

// Interfaces usable for bootstrap/data traffic.  Honours
// FLAGCX_SOCKET_IFNAME ("eth0,eth1", "^docker", "=eth0" exact) and
// FLAGCX_SOCKET_FAMILY (AF_INET / AF_INET6).  Loopback is returned only when
// nothing else is up.
std::vector<NetIf> findInterfaces(int maxIfs = 16);
// Pure matcher behind FLAGCX_SOCKET_IFNAME, exposed for unit tests.
bool ifNameMatches(const char *spec, const char *ifname);

class Socket {
 public:
  Socket() = default;
  explicit Socket(int fd) : fd_(fd) {}
  Socket(Socket &&o) noexcept : fd_(o.fd_) { o.fd_ = -1; }
  Socket &operator=(Socket &&o) noexcept;
  Socket(const Socket &) = delete;
  Socket &operator=(const Socket &) = delete;
  ~Socket() { close(); }

  int fd() const { return fd_; }
  bool valid() const { return fd_ >= 0; }
  void close();
  int release() { int f = fd_; fd_ = -1; return f; }

  // Bind to `addr` (port 0 = ephemeral) and listen; `addr` receives the port.
  flagcxResult_t listen(SockAddr *addr);
  // Accept one connection, waiting at most timeoutMs (<0: forever).
  flagcxResult_t accept(Socket *out, int timeoutMs) const;
  // Connect with retries while the peer is not listening yet.
  flagcxResult_t connect(const SockAddr &addr, int timeoutMs);

  flagcxResult_t sendAll(const void *buf, size_t n, int timeoutMs) const;
  flagcxResult_t recvAll(void *buf, size_t n, int timeoutMs) const;
  // Non-blocking progress: moves up to n bytes, adds what moved to *done.
  flagcxResult_t sendSome(const void *buf, size_t n, size_t *done) const;
  flagcxResult_t recvSome(void *buf, size_t n, size_t *done) const;
  flagcxResult_t setNonBlocking(bool on) const;

 private:
  int fd_ = -1;
};

// Default deadline for bootstrap traffic (FLAGCX_SOCKET_TIMEOUT_MS, 120 s).
int defaultSocketTimeoutMs();

// ---- Unix-domain datagram socket for SCM_RIGHTS fd passing --------------------
class FdChannel {
 public:
  ~FdChannel() { close(); }
  // Binds an abstract-namespace address derived from (key, rank).
  flagcxResult_t open(uint64_t key, int rank);
  void close();
  flagcxResult_t sendFd(uint64_t key, int dstRank, int fd, uint64_t tag) const;
  flagcxResult_t recvFd(int *fd, uint64_t *tag, int timeoutMs) const;

 private:
  int fd_ = -1;
};

} // namespace fcx
