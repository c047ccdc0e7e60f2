// net_socket.cc -- the built-in "socket" network adaptor and the plugin loader.
//
// One logical connection is FLAGCX_NSOCKS_PERTHREAD x max(1, FLAGCX_SOCKET_NTHREADS)
// TCP connections.  A message is a 16-byte header on connection 0 followed by
// the payload cut into equal contiguous stripes, one per connection, so large
// transfers use several kernel socket buffers (and cores) at once.  Requests on
// one connection complete in posting order.  With FLAGCX_SOCKET_NTHREADS > 0 a
// helper thread per connection drives the I/O; otherwise test() does.
//
// Same job as flagcx/adaptor/net/socket_adaptor.cc in the FlagCX project.
#include <poll.h>
#include <unistd.h>
#include <dlfcn.h>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "base.h"
#include "flagcx_net.h"
#include "socket.h"

namespace fcx {
namespace {

FCX_PARAM(NSocksPerThread, "NSOCKS_PERTHREAD", 2)
FCX_PARAM(SocketNThreads, "SOCKET_NTHREADS", 0)
FCX_PARAM(SocketStripeMin, "SOCKET_STRIPE_MIN", 65536)

constexpr uint64_t kNetMagic = 0x46434e4554303031ull; // "FCNET001"
constexpr int kMaxSocks = 16;

// Wire form of a listening address; IPv4/IPv6 socket addresses need 28 bytes.
struct ListenHandle {
  uint64_t magic;
  char addr[64];
};
static_assert(sizeof(ListenHandle) <= FLAGCX_NET_HANDLE_BYTES, "handle size");
static_assert(sizeof(sockaddr_in6) <= 64, "address does not fit the handle");

struct ConnHello {
  uint64_t magic;
  uint64_t connId;
  int32_t index;
  int32_t nsocks;
};

struct WireHeader {
  uint64_t bytes;
  int32_t tag;
  int32_t pad;
};

struct Conn;

struct Request {
  Conn *conn = nullptr;
  bool isSend = false;
  char *data = nullptr;
  size_t capacity = 0;   // posted size (recv: maximum)
  size_t bytes = 0;      // actual size (known after the header for recv)
  int tag = 0;
  WireHeader hdr{};
  size_t hdrDone = 0;
  bool layoutKnown = false;
  size_t off[kMaxSocks]{}, len[kMaxSocks]{}, done[kMaxSocks]{};
  int partsLeft = 0;
  std::atomic<int> finished{0};
  flagcxResult_t status = flagcxSuccess;
};

struct Conn {
  bool isSend = false;
  int nsocks = 0;
  Socket socks[kMaxSocks];
  std::deque<Request *> queue; // posting order; front completes first
  std::mutex mu;
  // helper thread (optional)
  std::thread worker;
  std::condition_variable cv;
  bool stop = false;
  flagcxResult_t broken = flagcxSuccess;
};

struct ListenComm {
  Socket sock;
  // partially assembled inbound connections keyed by connId
  std::map<uint64_t, Conn *> pending;
};

void layout(Request *r, int nsocks) {
  int use = (r->bytes >= (size_t)paramSocketStripeMin()) ? nsocks : 1;
  size_t per = divUp(r->bytes, (size_t)use);
  per = alignUp(per ? per : 1, 64);
  size_t o = 0;
  r->partsLeft = 0;
  for (int s = 0; s < nsocks; ++s) {
    size_t l = (s < use && o < r->bytes) ? std::min(per, r->bytes - o) : 0;
    r->off[s] = o;
    r->len[s] = l;
    r->done[s] = 0;
    o += l;
    if (l) ++r->partsLeft;
  }
  r->layoutKnown = true;
}

// Moves as many bytes as the sockets take without blocking.  Caller holds mu.
// Returns true if anything moved.
bool progress(Conn *c) {
  if (c->broken != flagcxSuccess) {
    for (Request *r : c->queue) { r->status = c->broken; r->finished.store(1); }
    c->queue.clear();
    return false;
  }
  bool moved = false;
  for (int s = 0; s < c->nsocks; ++s) {
    for (Request *r : c->queue) {
      flagcxResult_t res = flagcxSuccess;
      if (s == 0 && r->hdrDone < sizeof(WireHeader)) {
        size_t before = r->hdrDone;
        char *h = (char *)&r->hdr;
        res = c->isSend ? c->socks[0].sendSome(h + before, sizeof(WireHeader) - before, &r->hdrDone)
                        : c->socks[0].recvSome(h + before, sizeof(WireHeader) - before, &r->hdrDone);
        if (res != flagcxSuccess) { c->broken = res; return progress(c); }
        moved |= r->hdrDone != before;
        if (r->hdrDone < sizeof(WireHeader)) break; // socket 0 is busy with this header
        if (!c->isSend) {
          if (r->hdr.bytes > r->capacity) {
            FCX_WARN("socket net: message of %llu bytes does not fit the posted %zu",
                     (unsigned long long)r->hdr.bytes, r->capacity);
            c->broken = flagcxInternalError;
            return progress(c);
          }
          r->bytes = r->hdr.bytes;
          r->tag = r->hdr.tag;
          layout(r, c->nsocks);
        }
      }
      if (!r->layoutKnown) break; // stripes of later requests must wait for this header
      if (r->done[s] < r->len[s]) {
        size_t before = r->done[s];
        char *p = r->data + r->off[s] + before;
        res = c->isSend ? c->socks[s].sendSome(p, r->len[s] - before, &r->done[s])
                        : c->socks[s].recvSome(p, r->len[s] - before, &r->done[s]);
        if (res != flagcxSuccess) { c->broken = res; return progress(c); }
        moved |= r->done[s] != before;
        if (r->done[s] < r->len[s]) break; // this socket is busy with this request
        --r->partsLeft;
      }
    }
  }
  while (!c->queue.empty()) {
    Request *r = c->queue.front();
    if (r->hdrDone == sizeof(WireHeader) && r->layoutKnown && r->partsLeft == 0) {
      c->queue.pop_front();
      r->finished.store(1, std::memory_order_release);
    } else break;
  }
  return moved;
}

void workerMain(Conn *c) {
  std::unique_lock<std::mutex> lk(c->mu);
  while (!c->stop) {
    if (c->queue.empty()) { c->cv.wait(lk); continue; }
    bool moved = progress(c);
    if (!moved) {
      lk.unlock();
      std::vector<pollfd> fds;
      for (int s = 0; s < c->nsocks; ++s)
        fds.push_back({c->socks[s].fd(), (short)(c->isSend ? POLLOUT : POLLIN), 0});
      ::poll(fds.data(), fds.size(), 1);
      lk.lock();
    }
  }
}

void startWorker(Conn *c) {
  if (paramSocketNThreads() > 0) c->worker = std::thread(workerMain, c);
}

void destroyConn(Conn *c) {
  if (!c) return;
  {
    std::lock_guard<std::mutex> g(c->mu);
    c->stop = true;
    c->cv.notify_all();
  }
  if (c->worker.joinable()) c->worker.join();
  for (Request *r : c->queue) { r->status = flagcxRemoteError; r->finished.store(1); }
  delete c;
}

int socksPerConn() {
  int64_t n = paramNSocksPerThread() * std::max<int64_t>(1, paramSocketNThreads());
  return (int)std::min<int64_t>(std::max<int64_t>(n, 1), kMaxSocks);
}

// ---- adaptor entry points -----------------------------------------------------
flagcxResult_t sockInit() { return flagcxSuccess; }

std::vector<NetIf> &ifaces() {
  static std::vector<NetIf> v = findInterfaces();
  return v;
}

flagcxResult_t sockDevices(int *ndev) {
  *ndev = (int)ifaces().size();
  return flagcxSuccess;
}

flagcxResult_t sockGetProperties(int dev, void *props) {
  if (dev < 0 || dev >= (int)ifaces().size()) return flagcxInvalidArgument;
  flagcxNetProperties_t *p = (flagcxNetProperties_t *)props;
  memset(p, 0, sizeof *p);
  snprintf(p->name, sizeof p->name, "%s", ifaces()[dev].name.c_str());
  p->speedMbps = 10000;
  char path[256];
  snprintf(path, sizeof path, "/sys/class/net/%s/speed", p->name);
  if (FILE *f = fopen(path, "r")) {
    int sp = 0;
    if (fscanf(f, "%d", &sp) == 1 && sp > 0) p->speedMbps = sp;
    fclose(f);
  }
  p->maxComms = 65536;
  p->supportsDeviceMemory = 0;
  return flagcxSuccess;
}

flagcxResult_t sockListen(int dev, void *handle, void **listenComm) {
  if (dev < 0 || dev >= (int)ifaces().size()) return flagcxInvalidArgument;
  auto *lc = new ListenComm();
  ListenHandle h;
  memset(&h, 0, sizeof h);
  h.magic = kNetMagic;
  SockAddr a = ifaces()[dev].addr;
  if (a.sa.sa_family == AF_INET) a.in4.sin_port = 0;
  else a.in6.sin6_port = 0;
  flagcxResult_t r = lc->sock.listen(&a);
  if (r != flagcxSuccess) { delete lc; return r; }
  memcpy(h.addr, &a, sizeof h.addr);
  memset(handle, 0, FLAGCX_NET_HANDLE_BYTES);
  memcpy(handle, &h, sizeof h);
  *listenComm = lc;
  return flagcxSuccess;
}

flagcxResult_t sockConnect(int, void *handle, void **sendComm) {
  ListenHandle h;
  memcpy(&h, handle, sizeof h);
  if (h.magic != kNetMagic) { FCX_WARN("socket net: bad listen handle"); return flagcxInvalidArgument; }
  SockAddr peer;
  memset(&peer, 0, sizeof peer);
  memcpy(&peer, h.addr, sizeof h.addr);
  auto *c = new Conn();
  c->isSend = true;
  c->nsocks = socksPerConn();
  uint64_t connId = nowNs() ^ (pidHash() * 0x9e3779b97f4a7c15ull) ^ (uint64_t)(uintptr_t)c;
  for (int s = 0; s < c->nsocks; ++s) {
    flagcxResult_t r = c->socks[s].connect(peer, defaultSocketTimeoutMs());
    ConnHello hello = {kNetMagic, connId, s, c->nsocks};
    if (r == flagcxSuccess) r = c->socks[s].sendAll(&hello, sizeof hello, defaultSocketTimeoutMs());
    if (r != flagcxSuccess) { delete c; return r; }
  }
  startWorker(c);
  *sendComm = c;
  return flagcxSuccess;
}

flagcxResult_t sockAccept(void *listenComm, void **recvComm) {
  auto *lc = (ListenComm *)listenComm;
  for (;;) {
    // a connection completed by an earlier accept round?
    for (auto it = lc->pending.begin(); it != lc->pending.end(); ++it) {
      Conn *c = it->second;
      bool full = true;
      for (int s = 0; s < c->nsocks; ++s) full &= c->socks[s].valid();
      if (full) {
        lc->pending.erase(it);
        startWorker(c);
        *recvComm = c;
        return flagcxSuccess;
      }
    }
    Socket s;
    FCXCHECK(lc->sock.accept(&s, defaultSocketTimeoutMs()));
    ConnHello hello;
    if (s.recvAll(&hello, sizeof hello, defaultSocketTimeoutMs()) != flagcxSuccess) continue;
    if (hello.magic != kNetMagic || hello.nsocks < 1 || hello.nsocks > kMaxSocks ||
        hello.index < 0 || hello.index >= hello.nsocks) {
      FCX_WARN("socket net: dropped a connection with a foreign magic");
      continue;
    }
    Conn *&c = lc->pending[hello.connId];
    if (!c) { c = new Conn(); c->isSend = false; c->nsocks = hello.nsocks; }
    c->socks[hello.index] = std::move(s);
  }
}

flagcxResult_t sockCloseConn(void *c) { destroyConn((Conn *)c); return flagcxSuccess; }
flagcxResult_t sockCloseListen(void *l) {
  auto *lc = (ListenComm *)l;
  if (lc) { for (auto &p : lc->pending) destroyConn(p.second); delete lc; }
  return flagcxSuccess;
}

flagcxResult_t sockRegMr(void *, void *, size_t, int type, int, void **mhandle) {
  if (type != flagcxMemHost) return flagcxNotSupported; // host pointers only
  *mhandle = nullptr;
  return flagcxSuccess;
}
flagcxResult_t sockRegMrDmaBuf(void *, void *, size_t, int, uint64_t, int, int, void **) {
  return flagcxNotSupported;
}
flagcxResult_t sockDeregMr(void *, void *) { return flagcxSuccess; }

flagcxResult_t post(Conn *c, Request *r) {
  std::lock_guard<std::mutex> g(c->mu);
  if (c->broken != flagcxSuccess) { delete r; return c->broken; }
  c->queue.push_back(r);
  if (c->worker.joinable()) c->cv.notify_one();
  else progress(c);
  return flagcxSuccess;
}

flagcxResult_t sockIsend(void *sendComm, void *data, size_t size, int tag, void *, void *,
                         void **request) {
  Conn *c = (Conn *)sendComm;
  auto *r = new Request();
  r->conn = c;
  r->isSend = true;
  r->data = (char *)data;
  r->capacity = r->bytes = size;
  r->tag = tag;
  r->hdr = {size, tag, 0};
  layout(r, c->nsocks);
  *request = r;
  flagcxResult_t res = post(c, r);
  if (res != flagcxSuccess) *request = nullptr;
  return res;
}

flagcxResult_t sockIrecv(void *recvComm, int n, void **data, size_t *sizes, int *tags, void **,
                         void **, void **request) {
  if (n != 1) return flagcxNotSupported;
  Conn *c = (Conn *)recvComm;
  auto *r = new Request();
  r->conn = c;
  r->isSend = false;
  r->data = (char *)data[0];
  r->capacity = sizes[0];
  r->tag = tags ? tags[0] : 0;
  *request = r;
  flagcxResult_t res = post(c, r);
  if (res != flagcxSuccess) *request = nullptr;
  return res;
}

flagcxResult_t sockIflush(void *, int, void **, int *, void **, void **request) {
  *request = nullptr; // host memory needs no flush
  return flagcxSuccess;
}

flagcxResult_t sockTest(void *request, int *done, int *sizes) {
  auto *r = (Request *)request;
  if (!r) { *done = 1; return flagcxSuccess; }
  if (!r->finished.load(std::memory_order_acquire)) {
    Conn *c = r->conn;
    if (!c->worker.joinable()) {
      std::lock_guard<std::mutex> g(c->mu);
      progress(c);
    }
  }
  if (r->finished.load(std::memory_order_acquire)) {
    *done = 1;
    if (sizes) sizes[0] = (int)r->bytes;
    flagcxResult_t st = r->status;
    delete r;
    return st;
  }
  *done = 0;
  return flagcxSuccess;
}

flagcxResult_t sockGetDevFromName(char *name, int *dev) {
  for (size_t i = 0; i < ifaces().size(); ++i)
    if (ifaces()[i].name == name) { *dev = (int)i; return flagcxSuccess; }
  return flagcxInvalidArgument;
}

const flagcxNetAdaptor_v1 kSocketAdaptor = {
    "socket",        sockInit,      sockDevices,   sockGetProperties, sockListen,
    sockConnect,     sockAccept,    sockCloseConn, sockCloseConn,     sockCloseListen,
    sockRegMr,       sockRegMrDmaBuf, sockDeregMr, sockIsend,         sockIrecv,
    sockIflush,      sockTest,      nullptr,       nullptr,           nullptr,
    sockGetDevFromName};

const flagcxNetAdaptor_v1 *loadPlugin() {
  const char *path = getEnv("FLAGCX_NET_ADAPTOR_PLUGIN");
  if (!path || !*path || !strcasecmp(path, "none")) return nullptr;
  void *h = dlopen(path, RTLD_NOW | RTLD_LOCAL);
  if (!h) {
    FCX_WARN("net plugin %s: %s; using the socket adaptor", path, dlerror());
    return nullptr;
  }
  auto *a = (const flagcxNetAdaptor_v1 *)dlsym(h, "flagcxNetAdaptorPlugin_v1");
  if (!a || !a->name || !a->init || !a->listen || !a->connect || !a->accept || !a->isend ||
      !a->irecv || !a->test) {
    FCX_WARN("net plugin %s lacks a complete flagcxNetAdaptorPlugin_v1; using the socket adaptor", path);
    return nullptr;
  }
  if (a->init() != flagcxSuccess) {
    FCX_WARN("net plugin %s failed to initialise; using the socket adaptor", path);
    return nullptr;
  }
  FCX_INFO(SUB_NET, "using net plugin '%s' from %s", a->name, path);
  return a;
}

} // namespace
} // namespace fcx

extern "C" const struct flagcxNetAdaptor_v1 *flagcxGetNetAdaptor(void) {
  static const flagcxNetAdaptor_v1 *chosen = [] {
    const flagcxNetAdaptor_v1 *p = fcx::loadPlugin();
    return p ? p : &fcx::kSocketAdaptor;
  }();
  return chosen;
}
