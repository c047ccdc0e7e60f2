// socket.cc -- see socket.h.
#include "socket.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netdb.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <unistd.h>

namespace fcx {

FCX_PARAM(SocketTimeoutMs, "SOCKET_TIMEOUT_MS", 120000)
int defaultSocketTimeoutMs() { return (int)paramSocketTimeoutMs(); }

int addrLen(const SockAddr &a) {
  return a.sa.sa_family == AF_INET6 ? sizeof(sockaddr_in6) : sizeof(sockaddr_in);
}

std::string addrToString(const SockAddr &a) {
  char host[NI_MAXHOST] = "?", serv[NI_MAXSERV] = "?";
  getnameinfo(&a.sa, addrLen(a), host, sizeof host, serv, sizeof serv,
              NI_NUMERICHOST | NI_NUMERICSERV);
  return a.sa.sa_family == AF_INET6 ? "[" + std::string(host) + "]:" + serv
                                    : std::string(host) + ":" + serv;
}

flagcxResult_t addrFromString(const char *s, SockAddr *out) {
  memset(out, 0, sizeof *out);
  std::string str(s), host, port;
  if (!str.empty() && str[0] == '[') {
    size_t rb = str.find(']');
    if (rb == std::string::npos || rb + 1 >= str.size() || str[rb + 1] != ':')
      return flagcxInvalidArgument;
    host = str.substr(1, rb - 1);
    port = str.substr(rb + 2);
  } else {
    size_t c = str.rfind(':');
    if (c == std::string::npos) return flagcxInvalidArgument;
    host = str.substr(0, c);
    port = str.substr(c + 1);
  }
  addrinfo hints = {}, *res = nullptr;
  hints.ai_family = AF_UNSPEC;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(host.c_str(), port.c_str(), &hints, &res) != 0 || !res) {
    FCX_WARN("cannot resolve '%s'", s);
    return flagcxInvalidArgument;
  }
  memcpy(out, res->ai_addr, res->ai_addrlen);
  freeaddrinfo(res);
  return flagcxSuccess;
}

bool ifNameMatches(const char *spec, const char *ifname) {
  // spec grammar: [^][=]name[,name...]; plain names match as prefixes.
  if (!spec || !*spec) return true;
  bool invert = false, exact = false;
  if (*spec == '^') { invert = true; ++spec; }
  if (*spec == '=') { exact = true; ++spec; }
  std::string list(spec);
  bool hit = false;
  size_t pos = 0;
  while (pos <= list.size()) {
    size_t c = list.find(',', pos);
    if (c == std::string::npos) c = list.size();
    std::string n = list.substr(pos, c - pos);
    if (!n.empty()) {
      if (exact ? (n == ifname) : (strncmp(n.c_str(), ifname, n.size()) == 0))
        hit = true;
    }
    pos = c + 1;
  }
  return invert ? !hit : hit;
}

std::vector<NetIf> findInterfaces(int maxIfs) {
  std::vector<NetIf> out, loop;
  const char *spec = getEnv("FLAGCX_SOCKET_IFNAME");
  int family = -1;
  if (const char *f = getEnv("FLAGCX_SOCKET_FAMILY")) {
    if (!strcmp(f, "AF_INET")) family = AF_INET;
    else if (!strcmp(f, "AF_INET6")) family = AF_INET6;
  }
  ifaddrs *ifs = nullptr;
  if (getifaddrs(&ifs) != 0) return out;
  for (ifaddrs *i = ifs; i; i = i->ifa_next) {
    if (!i->ifa_addr) continue;
    int fam = i->ifa_addr->sa_family;
    if (fam != AF_INET && fam != AF_INET6) continue;
    if (family != -1 && fam != family) continue;
    if (!(i->ifa_flags & IFF_UP)) continue;
    if (fam == AF_INET6) {
      auto *a6 = (sockaddr_in6 *)i->ifa_addr;
      if (IN6_IS_ADDR_LINKLOCAL(&a6->sin6_addr)) continue;
    }
    bool isLoop = i->ifa_flags & IFF_LOOPBACK;
    if (spec) {
      if (!ifNameMatches(spec, i->ifa_name)) continue;
    } else if (!isLoop && (!strncmp(i->ifa_name, "docker", 6) ||
                           !strncmp(i->ifa_name, "virbr", 5))) {
      continue;
    }
    NetIf n;
    n.name = i->ifa_name;
    memset(&n.addr, 0, sizeof n.addr);
    memcpy(&n.addr, i->ifa_addr,
           fam == AF_INET ? sizeof(sockaddr_in) : sizeof(sockaddr_in6));
    bool dup = false;
    for (auto &e : out) dup |= (e.name == n.name);
    for (auto &e : loop) dup |= (e.name == n.name);
    if (dup) continue;
    ((isLoop && !spec) ? loop : out).push_back(n);
  }
  freeifaddrs(ifs);
  if (out.empty()) out = loop;
  if ((int)out.size() > maxIfs) out.resize(maxIfs);
  return out;
}

// ---------------------------------------------------------------------------
Socket &Socket::operator=(Socket &&o) noexcept {
  if (this != &o) { close(); fd_ = o.fd_; o.fd_ = -1; }
  return *this;
}

void Socket::close() {
  if (fd_ >= 0) { ::close(fd_); fd_ = -1; }
}

static void tuneTcp(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
  int buf = 4 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof buf);
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof buf);
}

flagcxResult_t Socket::listen(SockAddr *addr) {
  close();
  fd_ = ::socket(addr->sa.sa_family, SOCK_STREAM | SOCK_CLOEXEC, 0);
  FCX_SYSCHECK(fd_, "socket");
  int one = 1;
  setsockopt(fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  FCX_SYSCHECK(::bind(fd_, &addr->sa, addrLen(*addr)), "bind");
  socklen_t l = sizeof(*addr);
  FCX_SYSCHECK(getsockname(fd_, &addr->sa, &l), "getsockname");
  FCX_SYSCHECK(::listen(fd_, 16384), "listen");
  return flagcxSuccess;
}

static int pollOne(int fd, short ev, int timeoutMs) {
  pollfd p = {fd, ev, 0};
  for (;;) {
    int r = ::poll(&p, 1, timeoutMs);
    if (r < 0 && errno == EINTR) continue;
    return r;
  }
}

flagcxResult_t Socket::accept(Socket *out, int timeoutMs) const {
  int r = pollOne(fd_, POLLIN, timeoutMs);
  if (r == 0) {
    FCX_WARN("accept timed out after %d ms", timeoutMs);
    return flagcxSystemError;
  }
  FCX_SYSCHECK(r, "poll");
  int c = ::accept4(fd_, nullptr, nullptr, SOCK_CLOEXEC);
  FCX_SYSCHECK(c, "accept");
  tuneTcp(c);
  *out = Socket(c);
  return flagcxSuccess;
}

flagcxResult_t Socket::connect(const SockAddr &addr, int timeoutMs) {
  uint64_t deadline = nowNs() + (uint64_t)(timeoutMs < 0 ? 3600000 : timeoutMs) * 1000000ull;
  int backoffUs = 1000;
  for (;;) {
    close();
    fd_ = ::socket(addr.sa.sa_family, SOCK_STREAM | SOCK_CLOEXEC, 0);
    FCX_SYSCHECK(fd_, "socket");
    tuneTcp(fd_);
    if (::connect(fd_, &addr.sa, addrLen(addr)) == 0) return flagcxSuccess;
    int e = errno;
    bool retry = (e == ECONNREFUSED || e == ETIMEDOUT || e == EINTR ||
                  e == EAGAIN || e == ENETUNREACH || e == EHOSTUNREACH);
    if (!retry || nowNs() > deadline) {
      FCX_WARN("connect to %s failed: %s", addrToString(addr).c_str(), strerror(e));
      close();
      return e == ECONNREFUSED ? flagcxRemoteError : flagcxSystemError;
    }
    usleep(backoffUs);
    if (backoffUs < 100000) backoffUs *= 2;
  }
}

flagcxResult_t Socket::setNonBlocking(bool on) const {
  int fl = fcntl(fd_, F_GETFL, 0);
  FCX_SYSCHECK(fl, "fcntl");
  fl = on ? (fl | O_NONBLOCK) : (fl & ~O_NONBLOCK);
  FCX_SYSCHECK(fcntl(fd_, F_SETFL, fl), "fcntl");
  return flagcxSuccess;
}

flagcxResult_t Socket::sendSome(const void *buf, size_t n, size_t *done) const {
  if (n == 0) return flagcxSuccess;
  ssize_t r = ::send(fd_, buf, n, MSG_NOSIGNAL | MSG_DONTWAIT);
  if (r < 0) {
    if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return flagcxSuccess;
    FCX_WARN("send failed: %s", strerror(errno));
    return (errno == EPIPE || errno == ECONNRESET) ? flagcxRemoteError : flagcxSystemError;
  }
  *done += (size_t)r;
  return flagcxSuccess;
}

flagcxResult_t Socket::recvSome(void *buf, size_t n, size_t *done) const {
  if (n == 0) return flagcxSuccess;
  ssize_t r = ::recv(fd_, buf, n, MSG_DONTWAIT);
  if (r == 0) {
    FCX_WARN("peer closed the connection");
    return flagcxRemoteError;
  }
  if (r < 0) {
    if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return flagcxSuccess;
    FCX_WARN("recv failed: %s", strerror(errno));
    return errno == ECONNRESET ? flagcxRemoteError : flagcxSystemError;
  }
  *done += (size_t)r;
  return flagcxSuccess;
}

flagcxResult_t Socket::sendAll(const void *buf, size_t n, int timeoutMs) const {
  size_t done = 0;
  const char *p = (const char *)buf;
  while (done < n) {
    size_t before = done;
    FCXCHECK(sendSome(p + done, n - done, &done));
    if (done == before) {
      int r = pollOne(fd_, POLLOUT, timeoutMs);
      if (r == 0) { FCX_WARN("send timed out after %d ms", timeoutMs); return flagcxSystemError; }
      FCX_SYSCHECK(r, "poll");
    }
  }
  return flagcxSuccess;
}

flagcxResult_t Socket::recvAll(void *buf, size_t n, int timeoutMs) const {
  size_t done = 0;
  char *p = (char *)buf;
  while (done < n) {
    size_t before = done;
    FCXCHECK(recvSome(p + done, n - done, &done));
    if (done == before) {
      int r = pollOne(fd_, POLLIN, timeoutMs);
      if (r == 0) { FCX_WARN("recv timed out after %d ms", timeoutMs); return flagcxSystemError; }
      FCX_SYSCHECK(r, "poll");
    }
  }
  return flagcxSuccess;
}

// ---------------------------------------------------------------------------
// fd passing
// ---------------------------------------------------------------------------
static socklen_t fdAddr(sockaddr_un *a, uint64_t key, int rank) {
  memset(a, 0, sizeof *a);
  a->sun_family = AF_UNIX;
  // Abstract namespace (leading NUL): nothing to unlink, dies with the process.
  int n = snprintf(a->sun_path + 1, sizeof a->sun_path - 1, "flagcx-%016llx-%d",
                   (unsigned long long)key, rank);
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

flagcxResult_t FdChannel::open(uint64_t key, int rank) {
  close();
  fd_ = ::socket(AF_UNIX, SOCK_DGRAM | SOCK_CLOEXEC, 0);
  FCX_SYSCHECK(fd_, "socket(AF_UNIX)");
  sockaddr_un a;
  socklen_t l = fdAddr(&a, key, rank);
  FCX_SYSCHECK(::bind(fd_, (sockaddr *)&a, l), "bind(AF_UNIX)");
  return flagcxSuccess;
}

void FdChannel::close() {
  if (fd_ >= 0) { ::close(fd_); fd_ = -1; }
}

flagcxResult_t FdChannel::sendFd(uint64_t key, int dstRank, int fd, uint64_t tag) const {
  sockaddr_un a;
  socklen_t l = fdAddr(&a, key, dstRank);
  msghdr msg = {};
  iovec iov = {&tag, sizeof tag};
  char ctrl[CMSG_SPACE(sizeof(int))] = {0};
  msg.msg_name = &a;
  msg.msg_namelen = l;
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof ctrl;
  cmsghdr *c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  // The receiver may not have bound yet: retry for a bounded time.
  uint64_t deadline = nowNs() + (uint64_t)defaultSocketTimeoutMs() * 1000000ull;
  for (;;) {
    if (::sendmsg(fd_, &msg, 0) >= 0) return flagcxSuccess;
    if ((errno == ECONNREFUSED || errno == ENOENT || errno == EAGAIN) && nowNs() < deadline) {
      usleep(1000);
      continue;
    }
    FCX_WARN("sendmsg(SCM_RIGHTS) to rank %d failed: %s", dstRank, strerror(errno));
    return flagcxSystemError;
  }
}

flagcxResult_t FdChannel::recvFd(int *fd, uint64_t *tag, int timeoutMs) const {
  int r = pollOne(fd_, POLLIN, timeoutMs);
  if (r == 0) { FCX_WARN("fd receive timed out"); return flagcxSystemError; }
  FCX_SYSCHECK(r, "poll");
  msghdr msg = {};
  uint64_t t = 0;
  iovec iov = {&t, sizeof t};
  char ctrl[CMSG_SPACE(sizeof(int))] = {0};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof ctrl;
  ssize_t n = ::recvmsg(fd_, &msg, MSG_CMSG_CLOEXEC);
  FCX_SYSCHECK(n, "recvmsg");
  cmsghdr *c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_type != SCM_RIGHTS) {
    FCX_WARN("datagram without a file descriptor");
    return flagcxInternalError;
  }
  memcpy(fd, CMSG_DATA(c), sizeof(int));
  *tag = t;
  return flagcxSuccess;
}

} // namespace fcx
