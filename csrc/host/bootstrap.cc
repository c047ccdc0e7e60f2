// bootstrap.cc -- see bootstrap.h.
#include "bootstrap.h"

#include <poll.h>
#include <unistd.h>

#include <random>
#include <thread>

namespace fcx {

FCX_PARAM(RootTimeoutMs, "BOOTSTRAP_ROOT_TIMEOUT_MS", 1800000)

namespace {

struct CheckIn {
  uint64_t magic;
  uint64_t nonce;
  int32_t rank;
  int32_t nranks;
  SockAddr listenAddr;
};

struct Hello {
  uint64_t magic;
  uint64_t nonce;
  int32_t rank;
  int32_t pad;
};

struct MsgHeader {
  int32_t tag;
  int32_t pad;
  uint64_t bytes;
};

uint64_t freshNonce() {
  std::random_device rd;
  uint64_t a = ((uint64_t)rd() << 32) ^ rd();
  return a ^ nowNs() ^ (pidHash() << 1);
}

// Serves one communicator: waits for every rank, then returns the address
// table to each of them.  A connection that opens with a wrong magic/nonce is
// dropped and does not count.
void rootMain(Socket listener, uint64_t nonce) {
  std::vector<Socket> socks;
  std::vector<SockAddr> addrs;
  int nranks = -1, got = 0;
  uint64_t deadline = nowNs() + (uint64_t)paramRootTimeoutMs() * 1000000ull;
  while (nranks < 0 || got < nranks) {
    int64_t leftMs = ((int64_t)deadline - (int64_t)nowNs()) / 1000000;
    if (leftMs <= 0) {
      FCX_WARN("bootstrap root: only %d of %d ranks checked in before the deadline", got, nranks);
      return;
    }
    Socket c;
    if (listener.accept(&c, (int)std::min<int64_t>(leftMs, 1000)) != flagcxSuccess) continue;
    CheckIn ci;
    if (c.recvAll(&ci, sizeof ci, 10000) != flagcxSuccess) continue;
    if (ci.magic != kBootstrapMagic || ci.nonce != nonce) {
      FCX_WARN("bootstrap root: dropped a connection with a foreign magic");
      continue;
    }
    if (nranks < 0) {
      nranks = ci.nranks;
      socks.resize(nranks);
      addrs.resize(nranks);
    }
    if (ci.nranks != nranks || ci.rank < 0 || ci.rank >= nranks || socks[ci.rank].valid()) {
      FCX_WARN("bootstrap root: inconsistent check-in (rank %d of %d, expected %d ranks)",
               ci.rank, ci.nranks, nranks);
      continue;
    }
    addrs[ci.rank] = ci.listenAddr;
    socks[ci.rank] = std::move(c);
    ++got;
  }
  for (int r = 0; r < nranks; ++r)
    socks[r].sendAll(addrs.data(), sizeof(SockAddr) * nranks, 30000);
  FCX_INFO(SUB_BOOTSTRAP, "bootstrap root: %d ranks connected", nranks);
}

flagcxResult_t startRoot(SockAddr *addr, uint64_t nonce) {
  Socket l;
  FCXCHECK(l.listen(addr));
  std::thread(rootMain, std::move(l), nonce).detach();
  return flagcxSuccess;
}

} // namespace

flagcxResult_t bootstrapCreateId(flagcxUniqueId *out) {
  memset(out, 0, sizeof *out);
  BootstrapId *id = (BootstrapId *)out->internal;
  id->magic = kBootstrapMagic;
  if (const char *fixed = getEnv("FLAGCX_COMM_ID")) {
    FCXCHECK(addrFromString(fixed, &id->root));
    id->nonce = hashBytes(fixed, strlen(fixed));
    id->externalRoot = 1;
    return flagcxSuccess;
  }
  auto ifs = findInterfaces(1);
  if (ifs.empty()) {
    FCX_WARN("no usable network interface for bootstrap");
    return flagcxSystemError;
  }
  id->root = ifs[0].addr;
  if (id->root.sa.sa_family == AF_INET) id->root.in4.sin_port = 0;
  else id->root.in6.sin6_port = 0;
  id->nonce = freshNonce();
  FCXCHECK(startRoot(&id->root, id->nonce));
  FCX_INFO(SUB_BOOTSTRAP, "bootstrap root listening on %s (%s)",
           addrToString(id->root).c_str(), ifs[0].name.c_str());
  return flagcxSuccess;
}

flagcxResult_t Bootstrap::init(const flagcxUniqueId &uid, int rank, int nranks) {
  const BootstrapId *id = (const BootstrapId *)uid.internal;
  if (id->magic != kBootstrapMagic) {
    FCX_WARN("unique id does not come from flagcxGetUniqueId");
    return flagcxInvalidArgument;
  }
  FCX_ARGCHECK(nranks > 0 && rank >= 0 && rank < nranks, "rank %d of %d is out of range", rank, nranks);
  rank_ = rank;
  nranks_ = nranks;
  magic_ = id->magic;
  nonce_ = id->nonce;
  timeoutMs_ = defaultSocketTimeoutMs();
  if (id->externalRoot && rank == 0) {
    SockAddr a = id->root;
    FCXCHECK(startRoot(&a, nonce_));
  }

  Socket toRoot;
  FCXCHECK(toRoot.connect(id->root, timeoutMs_));
  // Listen on the local address that routes to the root unless the user pinned
  // an interface.
  SockAddr mine;
  memset(&mine, 0, sizeof mine);
  if (getEnv("FLAGCX_SOCKET_IFNAME")) {
    auto ifs = findInterfaces(1);
    if (ifs.empty()) { FCX_WARN("FLAGCX_SOCKET_IFNAME matches no interface"); return flagcxSystemError; }
    mine = ifs[0].addr;
  } else {
    socklen_t l = sizeof mine;
    FCX_SYSCHECK(getsockname(toRoot.fd(), &mine.sa, &l), "getsockname");
  }
  if (mine.sa.sa_family == AF_INET) mine.in4.sin_port = 0;
  else mine.in6.sin6_port = 0;
  FCXCHECK(listen_.listen(&mine));

  CheckIn ci;
  memset(&ci, 0, sizeof ci);
  ci.magic = magic_;
  ci.nonce = nonce_;
  ci.rank = rank;
  ci.nranks = nranks;
  ci.listenAddr = mine;
  FCXCHECK(toRoot.sendAll(&ci, sizeof ci, timeoutMs_));
  addrs_.resize(nranks);
  FCXCHECK(toRoot.recvAll(addrs_.data(), sizeof(SockAddr) * nranks, timeoutMs_));
  out_.resize(nranks);
  in_.resize(nranks);
  parked_.resize(nranks);
  FCX_INFO(SUB_BOOTSTRAP, "rank %d/%d bootstrap ready, listening on %s", rank, nranks,
           addrToString(mine).c_str());
  return flagcxSuccess;
}

void Bootstrap::close() {
  for (auto &s : out_) s.close();
  for (auto &s : in_) s.close();
  listen_.close();
  out_.clear();
  in_.clear();
}

flagcxResult_t Bootstrap::sendSock(int peer, Socket **s) {
  if (!out_[peer].valid()) {
    FCXCHECK(out_[peer].connect(addrs_[peer], timeoutMs_));
    Hello h = {magic_, nonce_, rank_, 0};
    FCXCHECK(out_[peer].sendAll(&h, sizeof h, timeoutMs_));
  }
  *s = &out_[peer];
  return flagcxSuccess;
}

flagcxResult_t Bootstrap::recvSock(int peer, Socket **s) {
  uint64_t deadline = nowNs() + (uint64_t)timeoutMs_ * 1000000ull;
  while (!in_[peer].valid()) {
    int64_t leftMs = ((int64_t)deadline - (int64_t)nowNs()) / 1000000;
    if (leftMs <= 0) {
      FCX_WARN("rank %d: no connection from rank %d within %d ms", rank_, peer, timeoutMs_);
      return flagcxRemoteError;
    }
    Socket c;
    FCXCHECK(listen_.accept(&c, (int)leftMs));
    Hello h;
    if (c.recvAll(&h, sizeof h, timeoutMs_) != flagcxSuccess) continue;
    if (h.magic != magic_ || h.nonce != nonce_ || h.rank < 0 || h.rank >= nranks_) {
      FCX_WARN("rank %d: dropped a connection with a foreign magic", rank_);
      continue;
    }
    in_[h.rank] = std::move(c);
  }
  *s = &in_[peer];
  return flagcxSuccess;
}

flagcxResult_t Bootstrap::send(int peer, int tag, const void *data, size_t bytes) {
  FCX_ARGCHECK(peer >= 0 && peer < nranks_, "bootstrap send: bad peer %d", peer);
  std::lock_guard<std::mutex> g(mu_);
  if (peer == rank_) {
    Parked p{tag, std::vector<char>((const char *)data, (const char *)data + bytes)};
    parked_[peer].push_back(std::move(p));
    return flagcxSuccess;
  }
  Socket *s;
  FCXCHECK(sendSock(peer, &s));
  MsgHeader h = {tag, 0, bytes};
  FCXCHECK(s->sendAll(&h, sizeof h, timeoutMs_));
  FCXCHECK(s->sendAll(data, bytes, timeoutMs_));
  return flagcxSuccess;
}

flagcxResult_t Bootstrap::recv(int peer, int tag, void *data, size_t bytes) {
  FCX_ARGCHECK(peer >= 0 && peer < nranks_, "bootstrap recv: bad peer %d", peer);
  std::lock_guard<std::mutex> g(mu_);
  auto &q = parked_[peer];
  for (auto it = q.begin(); it != q.end(); ++it) {
    if (it->tag == tag) {
      if (it->data.size() != bytes) {
        FCX_WARN("bootstrap recv: rank %d sent %zu bytes for tag %d, expected %zu", peer,
                 it->data.size(), tag, bytes);
        return flagcxInternalError;
      }
      memcpy(data, it->data.data(), bytes);
      q.erase(it);
      return flagcxSuccess;
    }
  }
  if (peer == rank_) {
    FCX_WARN("bootstrap recv from self without a matching send (tag %d)", tag);
    return flagcxInvalidUsage;
  }
  Socket *s;
  FCXCHECK(recvSock(peer, &s));
  for (;;) {
    MsgHeader h;
    FCXCHECK(s->recvAll(&h, sizeof h, timeoutMs_));
    if (h.tag == tag) {
      if (h.bytes != bytes) {
        FCX_WARN("bootstrap recv: rank %d sent %llu bytes for tag %d, expected %zu", peer,
                 (unsigned long long)h.bytes, tag, bytes);
        return flagcxInternalError;
      }
      return s->recvAll(data, bytes, timeoutMs_);
    }
    Parked p{h.tag, std::vector<char>(h.bytes)};
    FCXCHECK(s->recvAll(p.data.data(), h.bytes, timeoutMs_));
    q.push_back(std::move(p));
  }
}

// Bootstrap payloads are small (addresses, handles, counts), far below the
// socket buffers, so "send to the next rank, then receive from the previous"
// cannot block on a full pipe.
flagcxResult_t Bootstrap::allGather(void *data, size_t bytes) {
  if (nranks_ == 1) return flagcxSuccess;
  char *d = (char *)data;
  constexpr int kTag = -101;
  if (bytes * nranks_ <= (1u << 20)) {
    // direct exchange: one round trip instead of nranks-1 ring steps
    for (int i = 1; i < nranks_; ++i)
      FCXCHECK(send((rank_ + i) % nranks_, kTag, d + (size_t)rank_ * bytes, bytes));
    for (int i = 1; i < nranks_; ++i) {
      int src = (rank_ - i + nranks_) % nranks_;
      FCXCHECK(recv(src, kTag, d + (size_t)src * bytes, bytes));
    }
    return flagcxSuccess;
  }
  int next = (rank_ + 1) % nranks_, prev = (rank_ - 1 + nranks_) % nranks_;
  for (int step = 0; step < nranks_ - 1; ++step) {
    int sendSlot = (rank_ - step + nranks_) % nranks_;
    int recvSlot = (rank_ - step - 1 + nranks_) % nranks_;
    // split big slots so a ring of blocking sends cannot fill every pipe
    const size_t piece = 256 << 10;
    for (size_t off = 0; off < bytes; off += piece) {
      size_t n = std::min(piece, bytes - off);
      FCXCHECK(send(next, kTag, d + sendSlot * bytes + off, n));
      FCXCHECK(recv(prev, kTag, d + recvSlot * bytes + off, n));
    }
  }
  return flagcxSuccess;
}

flagcxResult_t Bootstrap::barrier() {
  // dissemination barrier: ceil(log2 n) rounds
  constexpr int kTag = -1000;
  for (int dist = 1; dist < nranks_; dist <<= 1) {
    char tok = 1, got = 0;
    FCXCHECK(send((rank_ + dist) % nranks_, kTag - dist, &tok, 1));
    FCXCHECK(recv((rank_ - dist + nranks_) % nranks_, kTag - dist, &got, 1));
  }
  return flagcxSuccess;
}

flagcxResult_t Bootstrap::broadcast(void *data, size_t bytes, int root) {
  constexpr int kTag = -103;
  if (nranks_ == 1) return flagcxSuccess;
  // binomial tree rooted at `root`
  int vr = (rank_ - root + nranks_) % nranks_;
  int mask = 1;
  while (mask < nranks_) {
    if (vr & mask) {
      int src = (vr - mask + root) % nranks_;
      FCXCHECK(recv(src, kTag, data, bytes));
      break;
    }
    mask <<= 1;
  }
  mask >>= 1;
  while (mask > 0) {
    if (vr + mask < nranks_) {
      int dst = (vr + mask + root) % nranks_;
      FCXCHECK(send(dst, kTag, data, bytes));
    }
    mask >>= 1;
  }
  return flagcxSuccess;
}

} // namespace fcx
