// reg_cache.cc -- see reg_cache.h.
#include "reg_cache.h"

#include <errno.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <array>

#include "cuda_rt.h"

namespace fcx {

namespace {

enum : uint32_t { kOpOpen = 1, kOpClose = 2 };

// Abstract-namespace address "\0flagcx-reg-<key>-<rank>".
socklen_t serviceAddr(uint64_t key, int rank, sockaddr_un *sa) {
  memset(sa, 0, sizeof *sa);
  sa->sun_family = AF_UNIX;
  int n = snprintf(sa->sun_path + 1, sizeof(sa->sun_path) - 1, "flagcx-reg-%016llx-%d", (unsigned long long)key, rank);
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

bool sendAll(int fd, const void *buf, size_t n) {
  const char *p = (const char *)buf;
  while (n) {
    ssize_t k = ::send(fd, p, n, MSG_NOSIGNAL);
    if (k < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    p += k;
    n -= (size_t)k;
  }
  return true;
}

// Reads exactly n bytes, waiting at most timeoutMs for each piece.
bool recvAll(int fd, void *buf, size_t n, int timeoutMs) {
  char *p = (char *)buf;
  while (n) {
    pollfd pf{fd, POLLIN, 0};
    int r = ::poll(&pf, 1, timeoutMs);
    if (r < 0 && errno == EINTR) continue;
    if (r <= 0) return false;
    ssize_t k = ::recv(fd, p, n, 0);
    if (k < 0 && errno == EINTR) continue;
    if (k <= 0) return false;
    p += k;
    n -= (size_t)k;
  }
  return true;
}

// One process may hold several communicators whose peers export the same
// allocation; a handle is opened once per process and counted.
struct OpenedHandle { void *va; int refs; };
std::mutex gOpenMu;
std::map<std::array<unsigned char, kIpcHandleBytes>, OpenedHandle> gOpenByHandle;

} // namespace

RegBackend cudaRegBackend(int dev) {
  RegBackend b;
  b.identify = [](const void *p, void **base, size_t *size, uint64_t *id) {
    return cu::allocationInfo(p, base, size, id) == flagcxSuccess;
  };
  b.exportHandle = [](void *base, void *handle) {
    static_assert(sizeof(cudaIpcMemHandle_t) == kIpcHandleBytes, "handle size");
    if (cu::vmmLookup(base)) return false; // VMM blocks travel as file descriptors (window registration)
    cudaError_t e = cudaIpcGetMemHandle((cudaIpcMemHandle_t *)handle, base);
    if (e != cudaSuccess) {
      cudaGetLastError(); // not an error of the caller's: the buffer simply is not exportable
      return false;
    }
    return true;
  };
  b.open = [](const void *handle) -> void * {
    std::array<unsigned char, kIpcHandleBytes> k;
    memcpy(k.data(), handle, kIpcHandleBytes);
    std::lock_guard<std::mutex> g(gOpenMu);
    auto it = gOpenByHandle.find(k);
    if (it != gOpenByHandle.end()) {
      it->second.refs++;
      return it->second.va;
    }
    void *va = nullptr;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof h);
    cudaError_t e = cudaIpcOpenMemHandle(&va, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
      cudaGetLastError();
      FCX_INFO(SUB_REG, "cudaIpcOpenMemHandle failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    gOpenByHandle[k] = OpenedHandle{va, 1};
    return va;
  };
  b.close = [](void *va) {
    std::lock_guard<std::mutex> g(gOpenMu);
    for (auto it = gOpenByHandle.begin(); it != gOpenByHandle.end(); ++it) {
      if (it->second.va != va) continue;
      if (--it->second.refs == 0) {
        cudaIpcCloseMemHandle(va);
        gOpenByHandle.erase(it);
      }
      return;
    }
  };
  b.threadInit = [dev]() { cudaSetDevice(dev); };
  return b;
}

flagcxResult_t RegCache::start(uint64_t key, int rank, int nranks, RegBackend backend) {
  if (running_.load()) return flagcxInvalidUsage;
  key_ = key;
  rank_ = rank;
  nranks_ = nranks;
  be_ = std::move(backend);
  peerFds_.assign(nranks, -1);
  listenFd_ = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  FCX_SYSCHECK(listenFd_, "socket(AF_UNIX)");
  sockaddr_un sa;
  socklen_t len = serviceAddr(key, rank, &sa);
  if (::bind(listenFd_, (sockaddr *)&sa, len) != 0 || ::listen(listenFd_, 64) != 0) {
    FCX_WARN("registration service: bind/listen failed: %s", strerror(errno));
    ::close(listenFd_);
    listenFd_ = -1;
    return flagcxSystemError;
  }
  if (::pipe(wakeFd_) != 0) {
    ::close(listenFd_);
    listenFd_ = -1;
    return flagcxSystemError;
  }
  stopFlag_.store(false);
  running_.store(true);
  thread_ = std::thread([this] { serve(); });
  return flagcxSuccess;
}

void RegCache::stop() {
  if (!running_.exchange(false)) return;
  stopFlag_.store(true);
  char one = 1;
  if (wakeFd_[1] >= 0 && ::write(wakeFd_[1], &one, 1) < 0) { /* the thread also polls the flag */ }
  if (thread_.joinable()) thread_.join();
  {
    std::lock_guard<std::mutex> g(mu_);
    for (int &fd : peerFds_)
      if (fd >= 0) { ::close(fd); fd = -1; }
    entries_.clear();
  }
  {
    std::lock_guard<std::mutex> g(openMu_);
    for (void *va : opened_)
      if (be_.close) be_.close(va);
    opened_.clear();
  }
  if (listenFd_ >= 0) ::close(listenFd_);
  if (wakeFd_[0] >= 0) ::close(wakeFd_[0]);
  if (wakeFd_[1] >= 0) ::close(wakeFd_[1]);
  listenFd_ = wakeFd_[0] = wakeFd_[1] = -1;
}

// ---- service side -----------------------------------------------------------------
bool RegCache::handle(int fd) {
  Request rq;
  if (!recvAll(fd, &rq, sizeof rq, 2000)) return false;
  Reply rp{0};
  if (rq.op == kOpOpen) {
    void *va = be_.open ? be_.open(rq.handle) : nullptr;
    if (va) {
      std::lock_guard<std::mutex> g(openMu_);
      opened_.push_back(va);
      nOpened_++;
    }
    rp.va = (uint64_t)(uintptr_t)va;
  } else if (rq.op == kOpClose) {
    void *va = (void *)(uintptr_t)rq.va;
    std::lock_guard<std::mutex> g(openMu_);
    for (size_t i = 0; i < opened_.size(); ++i)
      if (opened_[i] == va) {
        if (be_.close) be_.close(va);
        opened_.erase(opened_.begin() + (long)i);
        nClosed_++;
        rp.va = 1;
        break;
      }
  } else {
    return false;
  }
  return sendAll(fd, &rp, sizeof rp);
}

void RegCache::serve() {
  if (be_.threadInit) be_.threadInit();
  std::vector<int> conns;
  while (!stopFlag_.load()) {
    std::vector<pollfd> pfs;
    pfs.push_back({listenFd_, POLLIN, 0});
    pfs.push_back({wakeFd_[0], POLLIN, 0});
    for (int fd : conns) pfs.push_back({fd, POLLIN, 0});
    int r = ::poll(pfs.data(), (nfds_t)pfs.size(), 500);
    if (r < 0 && errno != EINTR) break;
    if (r <= 0) continue;
    if (pfs[1].revents) break;
    if (pfs[0].revents & POLLIN) {
      int fd = ::accept4(listenFd_, nullptr, nullptr, SOCK_CLOEXEC);
      if (fd >= 0) conns.push_back(fd);
    }
    for (size_t i = 2; i < pfs.size(); ++i) {
      if (!pfs[i].revents) continue;
      int fd = pfs[i].fd;
      if (!(pfs[i].revents & POLLIN) || !handle(fd)) {
        ::close(fd);
        for (size_t k = 0; k < conns.size(); ++k)
          if (conns[k] == fd) { conns.erase(conns.begin() + (long)k); break; }
      }
    }
  }
  for (int fd : conns) ::close(fd);
}

// ---- client side --------------------------------------------------------------------
int RegCache::peerFd(int peer) {
  if (peerFds_[peer] >= 0) return peerFds_[peer];
  int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return -1;
  sockaddr_un sa;
  socklen_t len = serviceAddr(key_, peer, &sa);
  // the peer's service starts during its communicator creation: allow it a moment
  const uint64_t deadline = nowNs() + 20ull * 1000000000ull;
  while (::connect(fd, (sockaddr *)&sa, len) != 0) {
    if ((errno != ECONNREFUSED && errno != ENOENT && errno != EAGAIN && errno != EINTR) || nowNs() > deadline) {
      FCX_INFO(SUB_REG, "registration service of rank %d unreachable: %s", peer, strerror(errno));
      ::close(fd);
      return -1;
    }
    ::usleep(2000);
  }
  peerFds_[peer] = fd;
  return fd;
}

bool RegCache::call(int peer, const Request &rq, Reply *rp) {
  int fd = peerFd(peer);
  if (fd < 0) return false;
  if (!sendAll(fd, &rq, sizeof rq) || !recvAll(fd, rp, sizeof *rp, 30000)) {
    ::close(fd);
    peerFds_[peer] = -1;
    return false;
  }
  return true;
}

bool RegCache::exportEntry(Entry &e) {
  Request rq;
  memset(&rq, 0, sizeof rq);
  rq.op = kOpOpen;
  rq.srcRank = (uint32_t)rank_;
  if (!be_.exportHandle || !be_.exportHandle(e.base, rq.handle)) return false;
  bool ok = true;
  for (int p = 0; p < nranks_; ++p) {
    if (p == rank_) { e.peerBase[p] = e.base; continue; }
    Reply rp{0};
    if (!call(p, rq, &rp) || !rp.va) { ok = false; break; }
    e.peerBase[p] = (void *)(uintptr_t)rp.va;
  }
  if (!ok) closeAtPeers(e); // leave no half-registered allocation behind
  return ok;
}

void RegCache::closeAtPeers(const Entry &e) {
  for (int p = 0; p < nranks_; ++p) {
    if (p == rank_ || !e.peerBase[p]) continue;
    Request rq;
    memset(&rq, 0, sizeof rq);
    rq.op = kOpClose;
    rq.srcRank = (uint32_t)rank_;
    rq.va = (uint64_t)(uintptr_t)e.peerBase[p];
    Reply rp;
    call(p, rq, &rp);
  }
}

bool RegCache::find(const void *p, size_t bytes, void *peerVa[FLAGCX_MAX_RANKS], bool exportNew) {
  if (!running_.load() || !p) return false;
  void *base = nullptr;
  size_t size = 0;
  uint64_t id = 0;
  if (!be_.identify || !be_.identify(p, &base, &size, &id)) return false;
  if ((uintptr_t)p + bytes > (uintptr_t)base + size) return false;
  std::lock_guard<std::mutex> g(mu_);
  auto it = entries_.find((uintptr_t)base);
  if (it != entries_.end() && (it->second.id != id || it->second.size != size)) {
    // the address was freed and allocated again: the peers' mappings show the old memory
    cnt_.stale++;
    if (it->second.exportable) closeAtPeers(it->second);
    entries_.erase(it);
    it = entries_.end();
  }
  if (it == entries_.end()) {
    if (!exportNew) return false;
    Entry e;
    e.base = base;
    e.size = size;
    e.id = id;
    e.exportable = exportEntry(e);
    if (e.exportable) {
      cnt_.exports++;
      FCX_INFO(SUB_REG, "rank %d exported allocation %p (%zu bytes) to %d peers", rank_, base, size, nranks_ - 1);
    } else {
      cnt_.refused++;
      for (auto &v : e.peerBase) v = nullptr;
      FCX_INFO(SUB_REG, "rank %d: allocation %p (%zu bytes) cannot be exported", rank_, base, size);
    }
    it = entries_.emplace((uintptr_t)base, e).first;
  } else {
    cnt_.hits++;
  }
  const Entry &e = it->second;
  if (!e.exportable) return false;
  const size_t off = (uintptr_t)p - (uintptr_t)base;
  for (int r = 0; r < nranks_; ++r) peerVa[r] = (char *)e.peerBase[r] + off;
  return true;
}

void RegCache::forget(const void *p) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = entries_.upper_bound((uintptr_t)p);
  if (it == entries_.begin()) return;
  --it;
  if ((uintptr_t)p >= it->first + it->second.size) return;
  if (it->second.exportable) closeAtPeers(it->second);
  entries_.erase(it);
}

RegCache::Counters RegCache::counters() const {
  std::lock_guard<std::mutex> g(mu_);
  Counters c = cnt_;
  c.opened = nOpened_.load();
  c.closed = nClosed_.load();
  return c;
}

} // namespace fcx
