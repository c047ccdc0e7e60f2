// p2p_engine.cc -- the transfer engine of flagcx_p2p.h.
//
// A connection is two TCP sockets: on `out` this side sends requests and reads the
// answers (one request at a time, under a mutex); on `in` a service thread answers the
// peer's requests.  Device memory of a peer on the same machine never touches the
// sockets: its descriptor carries the CUDA IPC handle of the allocation, the first use
// maps it, and a transfer is a cudaMemcpyAsync between the caller's pointer and the
// mapping.  Everything else (host regions, peers on other machines) is copied by the
// owner's service thread from / to the bytes that travel with the request.
//
// Plays the role of flagcx/core/p2p_engine*.cc of the FlagCX project (RDMA verbs there).
#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <deque>
#include <iterator>
#include <map>
#include <memory>
#include <mutex>
#include <poll.h>
#include <string>
#include <thread>
#include <unistd.h>
#include <vector>

#include "comm.h"
#include "cuda_rt.h"
#include "flagcx_p2p.h"
#include "socket.h"

using namespace fcx;

namespace {

constexpr uint32_t kMagic = 0x50325046; // "FP2P"
constexpr size_t kStageBytes = 4u << 20;

enum Kind : uint32_t { kKindHost = 0, kKindCudaIpc = 1 };
enum Op : uint32_t { kOpWrite = 1, kOpRead = 2, kOpNotif = 3, kOpLookup = 4, kOpBye = 5 };

struct DescBody {
  uint32_t magic, kind;
  uint64_t pid, hostId;
  uint64_t base, allocSize; // the allocation (cudaIpc) or the region (host), in the owner's address space
  uint64_t addr, len;       // the described range, owner's address space
  int32_t dev;
  uint32_t pad;
  unsigned char ipc[64];
};
static_assert(sizeof(DescBody) == FLAGCX_P2P_DESC_BYTES, "descriptor layout");

struct Hello {
  uint32_t magic, role; // role 0: requests flow initiator -> acceptor on this socket; 1: the other way
  uint64_t connId, pid, hostId;
  int32_t dev;
  uint32_t pad;
};

struct Request {
  uint32_t magic, op;
  uint64_t addr, len;
};
struct Reply {
  uint32_t magic;
  int32_t status;
  uint64_t len;
};

struct Region {
  uintptr_t addr = 0;
  size_t size = 0;
  Kind kind = kKindHost;
  uintptr_t base = 0; // allocation base (cudaIpc)
  size_t allocSize = 0;
  unsigned char ipc[64] = {};
};

} // namespace

struct flagcxP2pConn;

struct flagcxP2pEngine {
  int dev = -1;
  uint64_t hostId = 0;
  Socket listener;
  SockAddr addr{};
  std::mutex mu;
  std::condition_variable cv;
  std::map<uint64_t, Region> regions;
  uint64_t nextMr = 1;
  std::thread acceptThread;
  std::atomic<bool> stop{false};
  std::map<uint64_t, Socket> halfOpen;       // first socket of a connection, waiting for the second
  std::map<uint64_t, Hello> halfHello;
  std::deque<flagcxP2pConn *> accepted;       // complete, not yet handed to flagcxP2pEngineAccept
  std::vector<flagcxP2pConn *> conns;         // everything alive, for teardown
  std::map<std::string, flagcxP2pConn *> sessions; // flagcxP2pEngineGetConn's cache, by "ip:port"

  bool findRegion(uintptr_t a, size_t len, Region *out) {
    std::lock_guard<std::mutex> lk(mu);
    for (auto &kv : regions) {
      const Region &r = kv.second;
      if (a >= r.addr && a + len <= r.addr + r.size && a + len >= a) { *out = r; return true; }
    }
    return false;
  }
};

struct flagcxP2pConn {
  flagcxP2pEngine *engine = nullptr;
  Socket out, in;
  std::mutex outMu;
  std::thread server;
  std::atomic<bool> stop{false};
  uint64_t peerPid = 0, peerHost = 0;
  int peerDev = -1;
  std::mutex mu;
  std::condition_variable cv;
  std::deque<std::string> notifs;
  std::map<std::pair<uint64_t, uint64_t>, void *> mapped; // (owner pid, allocation base) -> local mapping
  void *stage = nullptr;                                  // pinned (or plain) bounce buffer of the requester
  void *serverStage = nullptr;                            // the same for the service thread
  cudaStream_t stream = nullptr;
  bool local() const { return peerHost == engine->hostId; }
};

namespace {

int timeoutMs() { return defaultSocketTimeoutMs(); }

bool cudaUsable(const flagcxP2pEngine *e) { return e->dev >= 0 && cu::available(); }

flagcxResult_t stageBuffer(flagcxP2pEngine *e, void **slot) {
  if (*slot) return flagcxSuccess;
  if (cudaUsable(e)) {
    FCX_CUDACHECK(cudaSetDevice(e->dev));
    FCX_CUDACHECK(cudaHostAlloc(slot, kStageBytes, cudaHostAllocDefault));
  } else {
    *slot = malloc(kStageBytes);
    if (!*slot) return flagcxSystemError;
  }
  return flagcxSuccess;
}
void freeStage(flagcxP2pEngine *e, void *p) {
  if (!p) return;
  if (cudaUsable(e)) cudaFreeHost(p);
  else free(p);
}

bool isDevicePtr(const flagcxP2pEngine *e, const void *p) {
  if (!cudaUsable(e)) return false;
  int d = -1;
  return cu::classify(p, &d) != cu::kPtrHost;
}

// Copies between this process's memory (host or device) and a host buffer.
flagcxResult_t copyOut(flagcxP2pEngine *e, void *hostDst, const void *src, size_t n) {
  if (isDevicePtr(e, src)) FCX_CUDACHECK(cudaMemcpy(hostDst, src, n, cudaMemcpyDeviceToHost));
  else memcpy(hostDst, src, n);
  return flagcxSuccess;
}
flagcxResult_t copyIn(flagcxP2pEngine *e, void *dst, const void *hostSrc, size_t n) {
  if (isDevicePtr(e, dst)) FCX_CUDACHECK(cudaMemcpy(dst, hostSrc, n, cudaMemcpyHostToDevice));
  else memcpy(dst, hostSrc, n);
  return flagcxSuccess;
}

void fillDesc(const flagcxP2pEngine *e, const Region &r, uintptr_t addr, size_t len, flagcxP2pDesc_t *out) {
  DescBody d{};
  d.magic = kMagic;
  d.kind = r.kind;
  d.pid = (uint64_t)getpid();
  d.hostId = e->hostId;
  d.base = r.kind == kKindCudaIpc ? r.base : r.addr;
  d.allocSize = r.kind == kKindCudaIpc ? r.allocSize : r.size;
  d.addr = addr;
  d.len = len;
  d.dev = e->dev;
  memcpy(d.ipc, r.ipc, sizeof d.ipc);
  memcpy(out->bytes, &d, sizeof d);
}

// ---- the owner's side of a connection ---------------------------------------------
void serve(flagcxP2pConn *c) {
  flagcxP2pEngine *e = c->engine;
  if (cudaUsable(e)) cudaSetDevice(e->dev);
  while (!c->stop.load()) {
    Request rq;
    if (c->in.recvAll(&rq, sizeof rq, -1) != flagcxSuccess || rq.magic != kMagic) break;
    Reply rp{kMagic, flagcxSuccess, 0};
    if (rq.op == kOpBye) break;
    if (rq.op == kOpNotif) {
      std::string msg(rq.len <= FLAGCX_P2P_MAX_NOTIF_BYTES ? rq.len : 0, '\0');
      if (rq.len > FLAGCX_P2P_MAX_NOTIF_BYTES) break; // a frame we cannot skip safely
      if (rq.len && c->in.recvAll(&msg[0], rq.len, timeoutMs()) != flagcxSuccess) break;
      {
        std::lock_guard<std::mutex> lk(c->mu);
        c->notifs.push_back(std::move(msg));
      }
      c->cv.notify_all();
      if (c->in.sendAll(&rp, sizeof rp, timeoutMs()) != flagcxSuccess) break;
      continue;
    }
    Region r;
    const bool known = e->findRegion((uintptr_t)rq.addr, rq.len, &r);
    if (rq.op == kOpLookup) {
      flagcxP2pDesc_t d{};
      if (known) fillDesc(e, r, (uintptr_t)rq.addr, rq.len, &d);
      else rp.status = flagcxInvalidArgument;
      rp.len = known ? sizeof d : 0;
      if (c->in.sendAll(&rp, sizeof rp, timeoutMs()) != flagcxSuccess) break;
      if (known && c->in.sendAll(&d, sizeof d, timeoutMs()) != flagcxSuccess) break;
      continue;
    }
    if (stageBuffer(e, &c->serverStage) != flagcxSuccess) break;
    bool broken = false;
    if (rq.op == kOpWrite) {
      // the payload follows in pieces of at most kStageBytes; it must be drained even when
      // the range is refused, or the stream would lose its framing
      for (size_t off = 0; off < rq.len && !broken; off += kStageBytes) {
        const size_t n = std::min(kStageBytes, (size_t)rq.len - off);
        if (c->in.recvAll(c->serverStage, n, timeoutMs()) != flagcxSuccess) { broken = true; break; }
        if (known && copyIn(e, (char *)(uintptr_t)rq.addr + off, c->serverStage, n) != flagcxSuccess) rp.status = flagcxUnhandledDeviceError;
      }
      if (!known) rp.status = flagcxInvalidArgument;
      if (broken || c->in.sendAll(&rp, sizeof rp, timeoutMs()) != flagcxSuccess) break;
    } else if (rq.op == kOpRead) {
      if (!known) rp.status = flagcxInvalidArgument;
      rp.len = known ? rq.len : 0;
      if (c->in.sendAll(&rp, sizeof rp, timeoutMs()) != flagcxSuccess) break;
      for (size_t off = 0; known && off < rq.len && !broken; off += kStageBytes) {
        const size_t n = std::min(kStageBytes, (size_t)rq.len - off);
        if (copyOut(e, c->serverStage, (const char *)(uintptr_t)rq.addr + off, n) != flagcxSuccess) memset(c->serverStage, 0, n);
        if (c->in.sendAll(c->serverStage, n, timeoutMs()) != flagcxSuccess) broken = true;
      }
      if (broken) break;
    } else {
      break;
    }
  }
  c->stop.store(true);
  c->cv.notify_all();
}

flagcxP2pConn *makeConn(flagcxP2pEngine *e, Socket &&out, Socket &&in, const Hello &peer) {
  auto *c = new flagcxP2pConn();
  c->engine = e;
  c->out = std::move(out);
  c->in = std::move(in);
  c->peerPid = peer.pid;
  c->peerHost = peer.hostId;
  c->peerDev = peer.dev;
  c->server = std::thread(serve, c);
  {
    std::lock_guard<std::mutex> lk(e->mu);
    e->conns.push_back(c);
  }
  return c;
}

Hello myHello(const flagcxP2pEngine *e, uint32_t role, uint64_t connId) {
  Hello h{};
  h.magic = kMagic;
  h.role = role;
  h.connId = connId;
  h.pid = (uint64_t)getpid();
  h.hostId = e->hostId;
  h.dev = e->dev;
  return h;
}

void acceptLoop(flagcxP2pEngine *e) {
  while (!e->stop.load()) {
    // wait for a connection in slices so that the stop flag is seen
    pollfd pfd{e->listener.fd(), POLLIN, 0};
    if (::poll(&pfd, 1, 200) <= 0 || !(pfd.revents & POLLIN)) continue;
    Socket s;
    if (e->listener.accept(&s, 1000) != flagcxSuccess) continue;
    Hello h;
    if (s.recvAll(&h, sizeof h, 5000) != flagcxSuccess || h.magic != kMagic) continue;
    Hello mine = myHello(e, h.role, h.connId);
    if (s.sendAll(&mine, sizeof mine, 5000) != flagcxSuccess) continue;
    std::unique_lock<std::mutex> lk(e->mu);
    auto it = e->halfOpen.find(h.connId);
    if (it == e->halfOpen.end()) {
      e->halfOpen.emplace(h.connId, std::move(s));
      e->halfHello[h.connId] = h;
      continue;
    }
    // second socket of the pair: role 0 carries the initiator's requests (we serve it),
    // role 1 carries ours
    Socket other = std::move(it->second);
    Hello first = e->halfHello[h.connId];
    e->halfOpen.erase(it);
    e->halfHello.erase(h.connId);
    lk.unlock();
    Socket in = h.role == 0 ? std::move(s) : std::move(other);
    Socket out = h.role == 0 ? std::move(other) : std::move(s);
    (void)first;
    flagcxP2pConn *c = makeConn(e, std::move(out), std::move(in), h);
    lk.lock();
    e->accepted.push_back(c);
    lk.unlock();
    e->cv.notify_all();
  }
}

// One request / reply exchange on the requester's socket; payloads are handled by the caller
// between the two halves, under the same lock.
struct Exchange {
  flagcxP2pConn *c;
  std::unique_lock<std::mutex> lk;
  explicit Exchange(flagcxP2pConn *conn) : c(conn), lk(conn->outMu) {}
  flagcxResult_t request(uint32_t op, uint64_t addr, uint64_t len) {
    if (c->stop.load()) return flagcxRemoteError;
    Request rq{kMagic, op, addr, len};
    return c->out.sendAll(&rq, sizeof rq, timeoutMs());
  }
  flagcxResult_t reply(Reply *rp) {
    FCXCHECK(c->out.recvAll(rp, sizeof *rp, timeoutMs()));
    return rp->magic == kMagic ? flagcxSuccess : flagcxRemoteError;
  }
};

bool parseDesc(const flagcxP2pDesc_t *d, DescBody *out) {
  memcpy(out, d->bytes, sizeof *out);
  return out->magic == kMagic;
}

// The peer's allocation as mapped in this process (opened on first use).
flagcxResult_t mapRemote(flagcxP2pConn *c, const DescBody &d, void **mapping) {
  std::lock_guard<std::mutex> lk(c->mu);
  auto key = std::make_pair(d.pid, d.base);
  auto it = c->mapped.find(key);
  if (it != c->mapped.end()) { *mapping = it->second; return flagcxSuccess; }
  if (d.pid == (uint64_t)getpid()) { // an engine of this very process: the address is valid as it is
    c->mapped[key] = (void *)(uintptr_t)d.base;
    *mapping = (void *)(uintptr_t)d.base;
    return flagcxSuccess;
  }
  cudaIpcMemHandle_t h;
  static_assert(sizeof h == 64, "CUDA IPC handle size");
  memcpy(&h, d.ipc, sizeof h);
  void *p = nullptr;
  FCX_CUDACHECK(cudaSetDevice(c->engine->dev));
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    FCX_WARN("p2p engine: cannot map the peer's allocation (%s)", cudaGetErrorString(e));
    return flagcxUnhandledDeviceError;
  }
  c->mapped[key] = p;
  *mapping = p;
  return flagcxSuccess;
}

flagcxResult_t transfer(flagcxP2pConn *c, bool isWrite, void *local, const flagcxP2pDesc_t *remote, size_t bytes,
                        flagcxStream_t stream) {
  if (!c || !remote || (!local && bytes)) return flagcxInvalidArgument;
  DescBody d;
  if (!parseDesc(remote, &d) || bytes > d.len) {
    FCX_WARN("p2p engine: bad descriptor, or %zu bytes asked of a %llu-byte range", bytes, (unsigned long long)d.len);
    return flagcxInvalidArgument;
  }
  if (bytes == 0) return flagcxSuccess;
  flagcxP2pEngine *e = c->engine;
  // fast path: the peer's device memory on this machine, reached by the copy engines
  if (d.kind == kKindCudaIpc && d.hostId == e->hostId && cudaUsable(e)) {
    void *mapping = nullptr;
    FCXCHECK(mapRemote(c, d, &mapping));
    char *rem = (char *)mapping + (d.addr - d.base);
    cudaStream_t s = stream ? stream->base : c->stream;
    FCX_CUDACHECK(cudaSetDevice(e->dev));
    if (!stream && !c->stream) {
      FCX_CUDACHECK(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
      s = c->stream;
    }
    FCX_CUDACHECK(cudaMemcpyAsync(isWrite ? (void *)rem : local, isWrite ? (const void *)local : (const void *)rem, bytes,
                                  cudaMemcpyDefault, s));
    if (!stream) FCX_CUDACHECK(cudaStreamSynchronize(s));
    return flagcxSuccess;
  }
  // through the owner
  if (stream) FCX_CUDACHECK(cudaStreamSynchronize(stream->base)); // what the caller queued before is part of the data
  FCXCHECK(stageBuffer(e, &c->stage));
  Exchange x(c);
  FCXCHECK(x.request(isWrite ? kOpWrite : kOpRead, d.addr, bytes));
  Reply rp;
  if (isWrite) {
    for (size_t off = 0; off < bytes; off += kStageBytes) {
      const size_t n = std::min(kStageBytes, bytes - off);
      FCXCHECK(copyOut(e, c->stage, (const char *)local + off, n));
      FCXCHECK(c->out.sendAll(c->stage, n, timeoutMs()));
    }
    FCXCHECK(x.reply(&rp));
    return (flagcxResult_t)rp.status;
  }
  FCXCHECK(x.reply(&rp));
  if (rp.status != flagcxSuccess) return (flagcxResult_t)rp.status;
  for (size_t off = 0; off < bytes; off += kStageBytes) {
    const size_t n = std::min(kStageBytes, bytes - off);
    FCXCHECK(c->out.recvAll(c->stage, n, timeoutMs()));
    FCXCHECK(copyIn(e, (char *)local + off, c->stage, n));
  }
  return flagcxSuccess;
}

} // namespace

extern "C" {

flagcxResult_t flagcxP2pEngineCreate(int cudaDevice, flagcxP2pEngine_t *engine) {
  if (!engine) return flagcxInvalidArgument;
  auto e = std::make_unique<flagcxP2pEngine>();
  e->dev = cudaDevice;
  e->hostId = hostHash();
  if (cudaDevice >= 0) {
    if (!cu::available()) { FCX_WARN("p2p engine: device %d requested but no CUDA driver is present", cudaDevice); return flagcxInvalidArgument; }
    FCX_CUDACHECK(cudaSetDevice(cudaDevice));
  }
  std::vector<NetIf> ifs = findInterfaces(1);
  if (ifs.empty()) return flagcxSystemError;
  e->addr = ifs[0].addr;
  e->addr.in4.sin_port = 0; // same offset for both families
  FCXCHECK(e->listener.listen(&e->addr));
  e->acceptThread = std::thread(acceptLoop, e.get());
  *engine = e.release();
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pEngineDestroy(flagcxP2pEngine_t e) {
  if (!e) return flagcxSuccess;
  e->stop.store(true);
  if (e->acceptThread.joinable()) e->acceptThread.join();
  std::vector<flagcxP2pConn *> conns;
  {
    std::lock_guard<std::mutex> lk(e->mu);
    conns.swap(e->conns);
    e->accepted.clear();
  }
  for (flagcxP2pConn *c : conns) {
    c->engine = e; // flagcxP2pConnDestroy must not look the connection up again
    flagcxP2pConnDestroy(c);
  }
  delete e;
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pEngineGetPort(flagcxP2pEngine_t e, int *port) {
  if (!e || !port) return flagcxInvalidArgument;
  *port = ntohs(e->addr.in4.sin_port);
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pEngineGetMetadata(flagcxP2pEngine_t e, char *buf, size_t len) {
  if (!e || !buf || !len) return flagcxInvalidArgument;
  std::string s = addrToString(e->addr);
  if (s.size() + 1 > len) return flagcxInvalidArgument;
  memcpy(buf, s.c_str(), s.size() + 1);
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pEngineConnect(flagcxP2pEngine_t e, const char *ipPort, flagcxP2pConn_t *conn) {
  if (!e || !ipPort || !conn) return flagcxInvalidArgument;
  SockAddr a;
  FCXCHECK(addrFromString(ipPort, &a));
  uint64_t id = ((uint64_t)getpid() << 32) ^ nowNs() ^ (uint64_t)(uintptr_t)e;
  Socket s[2];
  Hello peer{};
  for (uint32_t role = 0; role < 2; ++role) {
    FCXCHECK(s[role].connect(a, timeoutMs()));
    Hello h = myHello(e, role, id);
    FCXCHECK(s[role].sendAll(&h, sizeof h, timeoutMs()));
    FCXCHECK(s[role].recvAll(&peer, sizeof peer, timeoutMs()));
    if (peer.magic != kMagic) return flagcxRemoteError;
  }
  // role 0: my requests; role 1: the peer's
  *conn = makeConn(e, std::move(s[0]), std::move(s[1]), peer);
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pEngineGetConn(flagcxP2pEngine_t e, const char *ipPort, flagcxP2pConn_t *conn) {
  if (!e || !ipPort || !conn) return flagcxInvalidArgument;
  {
    std::lock_guard<std::mutex> lk(e->mu);
    auto it = e->sessions.find(ipPort);
    if (it != e->sessions.end() && !it->second->stop.load()) { *conn = it->second; return flagcxSuccess; }
  }
  flagcxP2pConn_t fresh = nullptr;
  FCXCHECK(flagcxP2pEngineConnect(e, ipPort, &fresh));
  std::lock_guard<std::mutex> lk(e->mu);
  e->sessions[ipPort] = fresh; // a broken predecessor stays in `conns` and is torn down with the engine
  *conn = fresh;
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pEngineAccept(flagcxP2pEngine_t e, flagcxP2pConn_t *conn, int waitMs) {
  if (!e || !conn) return flagcxInvalidArgument;
  std::unique_lock<std::mutex> lk(e->mu);
  auto ready = [&] { return !e->accepted.empty() || e->stop.load(); };
  if (waitMs < 0) e->cv.wait(lk, ready);
  else if (!e->cv.wait_for(lk, std::chrono::milliseconds(waitMs), ready)) return flagcxInProgress;
  if (e->accepted.empty()) return flagcxInProgress;
  *conn = e->accepted.front();
  e->accepted.pop_front();
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pConnDestroy(flagcxP2pConn_t c) {
  if (!c) return flagcxSuccess;
  flagcxP2pEngine *e = c->engine;
  {
    std::lock_guard<std::mutex> lk(e->mu);
    e->conns.erase(std::remove(e->conns.begin(), e->conns.end(), c), e->conns.end());
    e->accepted.erase(std::remove(e->accepted.begin(), e->accepted.end(), c), e->accepted.end());
    for (auto it = e->sessions.begin(); it != e->sessions.end();)
      it = it->second == c ? e->sessions.erase(it) : std::next(it);
  }
  if (!c->stop.load()) {
    std::lock_guard<std::mutex> lk(c->outMu);
    Request bye{kMagic, kOpBye, 0, 0};
    c->out.sendAll(&bye, sizeof bye, 1000); // lets the peer's service thread leave its read
  }
  c->stop.store(true);
  ::shutdown(c->in.fd(), SHUT_RDWR); // wakes this side's service thread
  if (c->server.joinable()) c->server.join();
  if (cudaUsable(e)) {
    cudaSetDevice(e->dev);
    for (auto &kv : c->mapped)
      if (kv.first.first != (uint64_t)getpid()) cudaIpcCloseMemHandle(kv.second);
    if (c->stream) cudaStreamDestroy(c->stream);
  }
  freeStage(e, c->stage);
  freeStage(e, c->serverStage);
  delete c;
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pConnIsLocal(flagcxP2pConn_t c, int *isLocal) {
  if (!c || !isLocal) return flagcxInvalidArgument;
  *isLocal = c->local() ? 1 : 0;
  return flagcxSuccess;
}
flagcxResult_t flagcxP2pConnPeerDevice(flagcxP2pConn_t c, int *device) {
  if (!c || !device) return flagcxInvalidArgument;
  *device = c->peerDev;
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pEngineReg(flagcxP2pEngine_t e, void *data, size_t size, flagcxP2pMr_t *mr) {
  if (!e || !data || !size || !mr) return flagcxInvalidArgument;
  Region r;
  r.addr = (uintptr_t)data;
  r.size = size;
  if (isDevicePtr(e, data)) {
    void *base = nullptr;
    size_t allocSize = 0;
    uint64_t id = 0;
    FCX_CUDACHECK(cudaSetDevice(e->dev));
    FCXCHECK(cu::allocationInfo(data, &base, &allocSize, &id));
    if ((uintptr_t)data + size > (uintptr_t)base + allocSize) {
      FCX_WARN("p2p engine: the region spans more than one device allocation");
      return flagcxInvalidArgument;
    }
    cudaIpcMemHandle_t h;
    cudaError_t ce = cudaIpcGetMemHandle(&h, base);
    if (ce != cudaSuccess) {
      cudaGetLastError();
      FCX_WARN("p2p engine: this device memory cannot be shared between processes (%s); allocate it with cudaMalloc",
               cudaGetErrorString(ce));
      return flagcxInvalidArgument;
    }
    r.kind = kKindCudaIpc;
    r.base = (uintptr_t)base;
    r.allocSize = allocSize;
    memcpy(r.ipc, &h, sizeof h);
  }
  std::lock_guard<std::mutex> lk(e->mu);
  *mr = e->nextMr++;
  e->regions[*mr] = r;
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pEngineDereg(flagcxP2pEngine_t e, flagcxP2pMr_t mr) {
  if (!e) return flagcxInvalidArgument;
  std::lock_guard<std::mutex> lk(e->mu);
  return e->regions.erase(mr) ? flagcxSuccess : flagcxInvalidArgument;
}

flagcxResult_t flagcxP2pEngineMakeDesc(flagcxP2pEngine_t e, flagcxP2pMr_t mr, const void *addr, size_t len,
                                       flagcxP2pDesc_t *desc) {
  if (!e || !desc) return flagcxInvalidArgument;
  Region r;
  {
    std::lock_guard<std::mutex> lk(e->mu);
    auto it = e->regions.find(mr);
    if (it == e->regions.end()) return flagcxInvalidArgument;
    r = it->second;
  }
  const uintptr_t a = addr ? (uintptr_t)addr : r.addr;
  if (a < r.addr || a + len > r.addr + r.size) {
    FCX_WARN("p2p engine: the range lies outside the region");
    return flagcxInvalidArgument;
  }
  fillDesc(e, r, a, len, desc);
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pConnLookup(flagcxP2pConn_t c, uint64_t remoteAddr, size_t len, flagcxP2pDesc_t *desc) {
  if (!c || !desc) return flagcxInvalidArgument;
  Exchange x(c);
  FCXCHECK(x.request(kOpLookup, remoteAddr, len));
  Reply rp;
  FCXCHECK(x.reply(&rp));
  if (rp.status != flagcxSuccess) return (flagcxResult_t)rp.status;
  return c->out.recvAll(desc, sizeof *desc, timeoutMs());
}

flagcxResult_t flagcxP2pWrite(flagcxP2pConn_t c, const void *local, const flagcxP2pDesc_t *remote, size_t bytes,
                              flagcxStream_t stream) {
  return transfer(c, true, const_cast<void *>(local), remote, bytes, stream);
}
flagcxResult_t flagcxP2pRead(flagcxP2pConn_t c, void *local, const flagcxP2pDesc_t *remote, size_t bytes,
                             flagcxStream_t stream) {
  return transfer(c, false, local, remote, bytes, stream);
}
flagcxResult_t flagcxP2pWriteVector(flagcxP2pConn_t c, int n, const void *const *locals, const flagcxP2pDesc_t *remotes,
                                    const size_t *bytes, flagcxStream_t stream) {
  if (n < 0 || (n && (!locals || !remotes || !bytes))) return flagcxInvalidArgument;
  for (int i = 0; i < n; ++i) FCXCHECK(transfer(c, true, const_cast<void *>(locals[i]), &remotes[i], bytes[i], stream));
  return flagcxSuccess;
}
flagcxResult_t flagcxP2pReadVector(flagcxP2pConn_t c, int n, void *const *locals, const flagcxP2pDesc_t *remotes,
                                   const size_t *bytes, flagcxStream_t stream) {
  if (n < 0 || (n && (!locals || !remotes || !bytes))) return flagcxInvalidArgument;
  for (int i = 0; i < n; ++i) FCXCHECK(transfer(c, false, locals[i], &remotes[i], bytes[i], stream));
  return flagcxSuccess;
}

flagcxResult_t flagcxP2pSendNotif(flagcxP2pConn_t c, const void *msg, size_t len) {
  if (!c || (!msg && len) || len > FLAGCX_P2P_MAX_NOTIF_BYTES) return flagcxInvalidArgument;
  Exchange x(c);
  FCXCHECK(x.request(kOpNotif, 0, len));
  if (len) FCXCHECK(c->out.sendAll(msg, len, timeoutMs()));
  Reply rp;
  FCXCHECK(x.reply(&rp));
  return (flagcxResult_t)rp.status;
}

flagcxResult_t flagcxP2pRecvNotif(flagcxP2pConn_t c, void *buf, size_t capacity, size_t *len, int waitMs) {
  if (!c || !buf || !len) return flagcxInvalidArgument;
  std::unique_lock<std::mutex> lk(c->mu);
  auto ready = [&] { return !c->notifs.empty() || c->stop.load(); };
  if (waitMs < 0) c->cv.wait(lk, ready);
  else if (!c->cv.wait_for(lk, std::chrono::milliseconds(waitMs), ready)) return flagcxInProgress;
  if (c->notifs.empty()) return c->stop.load() ? flagcxRemoteError : flagcxInProgress;
  std::string m = std::move(c->notifs.front());
  c->notifs.pop_front();
  if (m.size() > capacity) { c->notifs.push_front(std::move(m)); return flagcxInvalidArgument; }
  memcpy(buf, m.data(), m.size());
  *len = m.size();
  return flagcxSuccess;
}

} // extern "C"
