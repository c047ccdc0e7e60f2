// cpu_coll.cc -- see cpu_coll.h.
#include "cpu_coll.h"

#include <sched.h>
#include <string.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>

namespace fcx {

// ---------------------------------------------------------------------------
// 16-bit float conversions
// ---------------------------------------------------------------------------
float bf16ToFloat(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t floatToBf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40); // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1);
  return (uint16_t)(u >> 16);
}

float halfToFloat(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000) << 16;
  uint32_t exp = (h >> 10) & 0x1f, man = h & 0x3ff, u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400));
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t floatToHalf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint32_t sign = (u >> 16) & 0x8000;
  int32_t exp = (int32_t)((u >> 23) & 0xff) - 127 + 15;
  uint32_t man = u & 0x7fffff;
  if (((u >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00 | (man ? 0x200 : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000;
    int shift = 14 - exp;
    uint32_t half = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((uint32_t)exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1fff;
  if (rem > 0x1000 || (rem == 0x1000 && (half & 1))) ++half; // may carry into the exponent: correct
  return (uint16_t)(sign | half);
}

// ---------------------------------------------------------------------------
// element-wise reduction
// ---------------------------------------------------------------------------
namespace {

template <typename T>
inline T applyOp(T a, T b, flagcxRedOp_t op) {
  switch (op) {
    case flagcxProd: return (T)(a * b);
    case flagcxMax: return a > b ? a : b;
    case flagcxMin: return a < b ? a : b;
    default: return (T)(a + b); // sum, avg (divided afterwards)
  }
}

template <typename T>
void reduceTyped(T *dst, const T *src, size_t n, flagcxRedOp_t op) {
  switch (op) { // hoist the switch so the loops vectorise
    case flagcxProd: for (size_t i = 0; i < n; ++i) dst[i] = (T)(dst[i] * src[i]); break;
    case flagcxMax: for (size_t i = 0; i < n; ++i) dst[i] = dst[i] > src[i] ? dst[i] : src[i]; break;
    case flagcxMin: for (size_t i = 0; i < n; ++i) dst[i] = dst[i] < src[i] ? dst[i] : src[i]; break;
    default: for (size_t i = 0; i < n; ++i) dst[i] = (T)(dst[i] + src[i]); break;
  }
}

template <float (*toF)(uint16_t), uint16_t (*fromF)(float)>
void reduce16(uint16_t *dst, const uint16_t *src, size_t n, flagcxRedOp_t op) {
  for (size_t i = 0; i < n; ++i) dst[i] = fromF(applyOp<float>(toF(dst[i]), toF(src[i]), op));
}

} // namespace

flagcxResult_t hostReduce(void *dst, const void *src, size_t n, flagcxDataType_t dt,
                          flagcxRedOp_t op) {
  if ((int)op < 0 || op >= flagcxNumRedOps) return flagcxInvalidArgument;
  switch (dt) {
    case flagcxInt8: reduceTyped((int8_t *)dst, (const int8_t *)src, n, op); break;
    case flagcxUint8: reduceTyped((uint8_t *)dst, (const uint8_t *)src, n, op); break;
    case flagcxInt32: reduceTyped((int32_t *)dst, (const int32_t *)src, n, op); break;
    case flagcxUint32: reduceTyped((uint32_t *)dst, (const uint32_t *)src, n, op); break;
    case flagcxInt64: reduceTyped((int64_t *)dst, (const int64_t *)src, n, op); break;
    case flagcxUint64: reduceTyped((uint64_t *)dst, (const uint64_t *)src, n, op); break;
    case flagcxFloat32: reduceTyped((float *)dst, (const float *)src, n, op); break;
    case flagcxFloat64: reduceTyped((double *)dst, (const double *)src, n, op); break;
    case flagcxFloat16:
      reduce16<halfToFloat, floatToHalf>((uint16_t *)dst, (const uint16_t *)src, n, op);
      break;
    case flagcxBfloat16:
      reduce16<bf16ToFloat, floatToBf16>((uint16_t *)dst, (const uint16_t *)src, n, op);
      break;
    default: return flagcxInvalidArgument;
  }
  return flagcxSuccess;
}

flagcxResult_t hostDivide(void *dst, size_t n, flagcxDataType_t dt, int d) {
  switch (dt) {
    case flagcxInt8: for (size_t i = 0; i < n; ++i) ((int8_t *)dst)[i] /= d; break;
    case flagcxUint8: for (size_t i = 0; i < n; ++i) ((uint8_t *)dst)[i] /= d; break;
    case flagcxInt32: for (size_t i = 0; i < n; ++i) ((int32_t *)dst)[i] /= d; break;
    case flagcxUint32: for (size_t i = 0; i < n; ++i) ((uint32_t *)dst)[i] /= d; break;
    case flagcxInt64: for (size_t i = 0; i < n; ++i) ((int64_t *)dst)[i] /= d; break;
    case flagcxUint64: for (size_t i = 0; i < n; ++i) ((uint64_t *)dst)[i] /= d; break;
    case flagcxFloat32: for (size_t i = 0; i < n; ++i) ((float *)dst)[i] /= d; break;
    case flagcxFloat64: for (size_t i = 0; i < n; ++i) ((double *)dst)[i] /= d; break;
    case flagcxFloat16:
      for (size_t i = 0; i < n; ++i) ((uint16_t *)dst)[i] = floatToHalf(halfToFloat(((uint16_t *)dst)[i]) / d);
      break;
    case flagcxBfloat16:
      for (size_t i = 0; i < n; ++i) ((uint16_t *)dst)[i] = floatToBf16(bf16ToFloat(((uint16_t *)dst)[i]) / d);
      break;
    default: return flagcxInvalidArgument;
  }
  return flagcxSuccess;
}

// ---------------------------------------------------------------------------
// HostNet
// ---------------------------------------------------------------------------
constexpr int kTagNetHandle = -201;

flagcxResult_t HostNet::init(Bootstrap *bs) {
  bs_ = bs;
  net_ = flagcxGetNetAdaptor();
  int ndev = 0;
  FCXCHECK(net_->init());
  FCXCHECK(net_->devices(&ndev));
  if (ndev < 1) { FCX_WARN("net adaptor %s reports no device", net_->name); return flagcxSystemError; }
  int n = bs->nranks();
  handles_.assign((size_t)n * FLAGCX_NET_HANDLE_BYTES, 0);
  FCXCHECK(net_->listen(0, handles_.data() + (size_t)bs->rank() * FLAGCX_NET_HANDLE_BYTES, &listen_));
  FCXCHECK(bs->allGather(handles_.data(), FLAGCX_NET_HANDLE_BYTES));
  send_.assign(n, nullptr);
  recv_.assign(n, nullptr);
  return initShm();
}

// Every rank creates one ring towards each rank of its own machine; shared memory is
// used only if ALL ranks got ALL their rings (otherwise everybody closes them again and
// the adaptor carries everything), so the two ends of a pair never disagree.
flagcxResult_t HostNet::initShm() {
  const int n = bs_->nranks(), me = bs_->rank();
  shmSend_.clear();
  shmRecv_.clear();
  shmSend_.resize(n);
  shmRecv_.resize(n);
  struct Info {
    uint64_t host;
    int32_t pid;
    int32_t ok;
  };
  std::vector<Info> infos(n);
  infos[me] = {hostHash(), (int32_t)getpid(), 0};
  const bool want = n > 1 && readParam("HOST_SHM", 1) != 0 && !strcmp(net_->name, "socket");
  FCXCHECK(bs_->allGather(infos.data(), sizeof(Info)));
  size_t cap = (size_t)std::max<int64_t>(4096, readParam("SHM_RING_BYTES", 512 << 10));
  while (cap & (cap - 1)) cap &= cap - 1; // round down to a power of two
  auto nameOf = [&](int src, int dst) {
    char b[96];
    snprintf(b, sizeof b, "/flagcx-%016llx-%d-%d", (unsigned long long)bs_->nonce(), src, dst);
    return std::string(b);
  };
  bool ok = want;
  if (want) {
    for (int p = 0; p < n && ok; ++p) {
      if (p == me || infos[p].host != infos[me].host) continue;
      shmSend_[p].reset(new ShmRing());
      ok = shmSend_[p]->create(nameOf(me, p), cap) == flagcxSuccess;
    }
  }
  infos[me].ok = ok ? 1 : 0;
  FCXCHECK(bs_->allGather(infos.data(), sizeof(Info))); // also: every ring exists from here on
  bool all = true;
  for (int p = 0; p < n; ++p) all = all && infos[p].ok;
  pids_.assign(n, 0);
  for (int p = 0; p < n; ++p) pids_[p] = infos[p].pid;
  if (all) {
    for (int p = 0; p < n && all; ++p) {
      if (p == me || infos[p].host != infos[me].host) continue;
      shmRecv_[p].reset(new ShmRing());
      all = shmRecv_[p]->open(nameOf(p, me)) == flagcxSuccess;
    }
    if (!all) { FCX_WARN("host shm: a ring that its creator announced could not be opened"); return flagcxSystemError; }
  }
  if (!all) {
    for (auto &r : shmSend_) r.reset();
    for (auto &r : shmRecv_) r.reset();
  }
  shm_ = all;
  FCXCHECK(bs_->barrier()); // nobody writes before every receiver is attached and the names are gone
  if (want) FCX_INFO(SUB_SHM, "rank %d: host shared-memory rings %s (%zu KiB each)", me, shm_ ? "on" : "off", cap >> 10);
  return flagcxSuccess;
}

void HostNet::close() {
  shmSend_.clear();
  shmRecv_.clear();
  shm_ = false;
  if (!net_) return;
  for (void *&c : send_) if (c) { net_->closeSend(c); c = nullptr; }
  for (void *&c : recv_) if (c) { net_->closeRecv(c); c = nullptr; }
  if (listen_) { net_->closeListen(listen_); listen_ = nullptr; }
}

static flagcxResult_t waitReq(const flagcxNetAdaptor_v1 *net, void *req) {
  int done = 0, sz = 0;
  uint64_t deadline = nowNs() + (uint64_t)defaultSocketTimeoutMs() * 1000000ull;
  while (!done) {
    FCXCHECK(net->test(req, &done, &sz));
    if (!done) {
      if (nowNs() > deadline) { FCX_WARN("host net: request timed out"); return flagcxSystemError; }
      sched_yield();
    }
  }
  return flagcxSuccess;
}

flagcxResult_t HostNet::sendComm(int peer, void **c) {
  if (!send_[peer]) {
    FCXCHECK(net_->connect(0, handles_.data() + (size_t)peer * FLAGCX_NET_HANDLE_BYTES, &send_[peer]));
    // first message names the sender so the acceptor can file the connection
    int32_t me = bs_->rank();
    void *req = nullptr;
    FCXCHECK(net_->isend(send_[peer], &me, sizeof me, 0, nullptr, nullptr, &req));
    FCXCHECK(waitReq(net_, req));
  }
  *c = send_[peer];
  return flagcxSuccess;
}

flagcxResult_t HostNet::recvComm(int peer, void **c) {
  while (!recv_[peer]) {
    void *rc = nullptr;
    FCXCHECK(net_->accept(listen_, &rc));
    int32_t who = -1;
    void *data = &who;
    size_t sz = sizeof who;
    int tag = 0;
    void *req = nullptr;
    FCXCHECK(net_->irecv(rc, 1, &data, &sz, &tag, nullptr, nullptr, &req));
    FCXCHECK(waitReq(net_, req));
    if (who < 0 || who >= bs_->nranks() || recv_[who]) {
      FCX_WARN("host net: unexpected connection from rank %d", who);
      net_->closeRecv(rc);
      return flagcxInternalError;
    }
    recv_[who] = rc;
  }
  *c = recv_[peer];
  return flagcxSuccess;
}

flagcxResult_t HostNet::run(const std::vector<Op> &ops) {
  std::vector<void *> reqs(ops.size(), nullptr);
  std::vector<char> pending(ops.size(), 0);
  // Open outgoing connections first: connect never waits for the peer's accept,
  // so no ordering between ranks can deadlock here.
  auto viaShm = [&](const Op &op) { return shm_ && (op.isSend ? shmSend_[op.peer] : shmRecv_[op.peer]) != nullptr; };
  for (auto &op : ops)
    if (op.isSend && op.peer != bs_->rank() && !viaShm(op)) { void *c; FCXCHECK(sendComm(op.peer, &c)); }
  // shared-memory messages: an 8-byte length, then the bytes; state per op
  struct ShmState {
    uint64_t header = 0;
    size_t hdrDone = 0, done = 0;
  };
  std::vector<ShmState> shmState(ops.size());
  size_t left = 0;
  for (size_t i = 0; i < ops.size(); ++i) {
    const Op &op = ops[i];
    if (op.peer == bs_->rank()) continue; // self transfers are handled by the callers
    if (viaShm(op)) {
      shmState[i].header = op.bytes;
      pending[i] = 2;
      ++left;
      continue;
    }
    void *c;
    if (op.isSend) {
      FCXCHECK(sendComm(op.peer, &c));
      FCXCHECK(net_->isend(c, op.data, op.bytes, 0, nullptr, nullptr, &reqs[i]));
    } else {
      FCXCHECK(recvComm(op.peer, &c));
      void *d = op.data;
      size_t sz = op.bytes;
      int tag = 0;
      FCXCHECK(net_->irecv(c, 1, &d, &sz, &tag, nullptr, nullptr, &reqs[i]));
    }
    pending[i] = 1;
    ++left;
  }
  uint64_t deadline = nowNs() + (uint64_t)defaultSocketTimeoutMs() * 1000000ull;
  flagcxResult_t firstErr = flagcxSuccess;
  const int nr = bs_->nranks();
  std::vector<char> busy(2 * (size_t)nr);
  uint64_t lastAlive = nowNs();
  while (left) {
    size_t before = left;
    bool moved = false;
    std::fill(busy.begin(), busy.end(), 0);
    for (size_t i = 0; i < ops.size(); ++i) {
      if (pending[i] != 2) continue;
      const Op &op = ops[i];
      char &b = busy[(op.isSend ? 0 : nr) + op.peer];
      if (b) continue; // an earlier message of this ring is still under way
      ShmState &st = shmState[i];
      ShmRing &ring = op.isSend ? *shmSend_[op.peer] : *shmRecv_[op.peer];
      if (st.hdrDone < 8) {
        uint64_t h = st.header;
        size_t k = op.isSend ? ring.write((char *)&h + st.hdrDone, 8 - st.hdrDone)
                             : ring.read((char *)&st.header + st.hdrDone, 8 - st.hdrDone);
        st.hdrDone += k;
        moved = moved || k;
        if (st.hdrDone == 8 && !op.isSend && st.header != op.bytes) {
          FCX_WARN("host shm: rank %d sent %llu bytes where %zu were expected", op.peer,
                   (unsigned long long)st.header, op.bytes);
          return flagcxInternalError;
        }
      }
      if (st.hdrDone == 8 && st.done < op.bytes) {
        size_t k = op.isSend ? ring.write((char *)op.data + st.done, op.bytes - st.done)
                             : ring.read((char *)op.data + st.done, op.bytes - st.done);
        st.done += k;
        moved = moved || k;
      }
      if (st.hdrDone == 8 && st.done == op.bytes) { pending[i] = 0; --left; }
      else b = 1;
    }
    if (moved) deadline = nowNs() + (uint64_t)defaultSocketTimeoutMs() * 1000000ull;
    else if (nowNs() - lastAlive > 100000000ull) { // nothing moved for a while: is the other side still there?
      lastAlive = nowNs();
      for (size_t i = 0; i < ops.size(); ++i)
        if (pending[i] == 2 && processIsDead(pids_[ops[i].peer])) {
          FCX_WARN("host shm: rank %d (pid %d) is gone", ops[i].peer, pids_[ops[i].peer]);
          return flagcxRemoteError;
        }
    }
    for (size_t i = 0; i < ops.size(); ++i) {
      if (pending[i] != 1) continue;
      int done = 0, sz = 0;
      flagcxResult_t r = net_->test(reqs[i], &done, &sz);
      if (r != flagcxSuccess) { if (firstErr == flagcxSuccess) firstErr = r; done = 1; }
      if (done) { pending[i] = 0; --left; }
    }
    if (left == before) {
      if (!moved) {
        if (nowNs() > deadline) { FCX_WARN("host net: no progress before the deadline"); return flagcxSystemError; }
        sched_yield();
      }
    } else {
      deadline = nowNs() + (uint64_t)defaultSocketTimeoutMs() * 1000000ull;
    }
  }
  return firstErr;
}

flagcxResult_t HostNet::sendRecv(int sendPeer, const void *sbuf, size_t sbytes, int recvPeer,
                                 void *rbuf, size_t rbytes) {
  std::vector<Op> ops;
  ops.push_back({false, recvPeer, rbuf, rbytes});
  ops.push_back({true, sendPeer, const_cast<void *>(sbuf), sbytes});
  return run(ops);
}

// ---------------------------------------------------------------------------
// collectives
// ---------------------------------------------------------------------------
namespace {
// element range of chunk c when `count` elements are split over n chunks
inline size_t chunkBegin(size_t count, int n, int c) { return count * (size_t)c / (size_t)n; }
} // namespace

flagcxResult_t CpuColl::allReduce(const void *send, void *recv, size_t count, flagcxDataType_t dt,
                                  flagcxRedOp_t op) {
  const int n = net->nranks(), r = net->rank();
  const size_t es = getFlagcxDataTypeSize(dt);
  if (es == 0) return flagcxInvalidArgument;
  if (send != recv) memmove(recv, send, count * es);
  if (n > 1) {
    char *buf = (char *)recv;
    const int next = (r + 1) % n, prev = (r - 1 + n) % n;
    size_t maxChunk = 0;
    for (int c = 0; c < n; ++c) maxChunk = std::max(maxChunk, chunkBegin(count, n, c + 1) - chunkBegin(count, n, c));
    std::vector<char> tmp(maxChunk * es);
    // reduce-scatter: after n-1 steps rank r owns the finished chunk (r+1)%n
    for (int s = 0; s < n - 1; ++s) {
      int sc = (r - s + n) % n, rc = (r - s - 1 + n) % n;
      size_t sb = chunkBegin(count, n, sc), se = chunkBegin(count, n, sc + 1);
      size_t rb = chunkBegin(count, n, rc), re = chunkBegin(count, n, rc + 1);
      FCXCHECK(net->sendRecv(next, buf + sb * es, (se - sb) * es, prev, tmp.data(), (re - rb) * es));
      FCXCHECK(hostReduce(buf + rb * es, tmp.data(), re - rb, dt, op));
    }
    // all-gather of the finished chunks
    for (int s = 0; s < n - 1; ++s) {
      int sc = (r + 1 - s + n) % n, rc = (r - s + n) % n;
      size_t sb = chunkBegin(count, n, sc), se = chunkBegin(count, n, sc + 1);
      size_t rb = chunkBegin(count, n, rc), re = chunkBegin(count, n, rc + 1);
      FCXCHECK(net->sendRecv(next, buf + sb * es, (se - sb) * es, prev, buf + rb * es, (re - rb) * es));
    }
  }
  if (op == flagcxAvg) FCXCHECK(hostDivide(recv, count, dt, n));
  return flagcxSuccess;
}

flagcxResult_t CpuColl::reduceScatter(const void *send, void *recv, size_t recvCount,
                                      flagcxDataType_t dt, flagcxRedOp_t op) {
  const int n = net->nranks(), r = net->rank();
  const size_t es = getFlagcxDataTypeSize(dt);
  if (es == 0) return flagcxInvalidArgument;
  const size_t cb = recvCount * es;
  const char *in = (const char *)send;
  if (n == 1) {
    if (send != recv) memmove(recv, send, cb);
  } else {
    const int next = (r + 1) % n, prev = (r - 1 + n) % n;
    // acc travels round the ring; chunk c ends at rank c after n-1 hops, so the
    // chunk first sent by rank r is (r-1)%n.
    std::vector<char> acc(cb), in2(cb);
    memcpy(acc.data(), in + (size_t)((r - 1 + n) % n) * cb, cb);
    for (int s = 0; s < n - 1; ++s) {
      int rc = (r - 2 - s + 2 * n) % n; // chunk arriving at this step
      FCXCHECK(net->sendRecv(next, acc.data(), cb, prev, in2.data(), cb));
      memcpy(acc.data(), in + (size_t)rc * cb, cb);
      FCXCHECK(hostReduce(acc.data(), in2.data(), recvCount, dt, op));
    }
    memcpy(recv, acc.data(), cb);
  }
  if (op == flagcxAvg) FCXCHECK(hostDivide(recv, recvCount, dt, n));
  return flagcxSuccess;
}

flagcxResult_t CpuColl::allGather(const void *send, void *recv, size_t sendCount,
                                  flagcxDataType_t dt) {
  const int n = net->nranks(), r = net->rank();
  const size_t cb = sendCount * getFlagcxDataTypeSize(dt);
  char *out = (char *)recv;
  if ((const char *)send != out + (size_t)r * cb) memmove(out + (size_t)r * cb, send, cb);
  const int next = (r + 1) % n, prev = (r - 1 + n) % n;
  for (int s = 0; s < n - 1; ++s) {
    int sc = (r - s + n) % n, rc = (r - s - 1 + n) % n;
    FCXCHECK(net->sendRecv(next, out + (size_t)sc * cb, cb, prev, out + (size_t)rc * cb, cb));
  }
  return flagcxSuccess;
}

flagcxResult_t CpuColl::broadcast(const void *send, void *recv, size_t count, flagcxDataType_t dt,
                                  int root) {
  const int n = net->nranks(), r = net->rank();
  const size_t bytes = count * getFlagcxDataTypeSize(dt);
  if (r == root && send != recv) memmove(recv, send, bytes);
  int vr = (r - root + n) % n, mask = 1;
  while (mask < n) {
    if (vr & mask) {
      FCXCHECK(net->run({{false, (vr - mask + root) % n, recv, bytes}}));
      break;
    }
    mask <<= 1;
  }
  for (mask >>= 1; mask > 0; mask >>= 1)
    if (vr + mask < n) FCXCHECK(net->run({{true, (vr + mask + root) % n, recv, bytes}}));
  return flagcxSuccess;
}

flagcxResult_t CpuColl::reduce(const void *send, void *recv, size_t count, flagcxDataType_t dt,
                               flagcxRedOp_t op, int root) {
  const int n = net->nranks(), r = net->rank();
  const size_t bytes = count * getFlagcxDataTypeSize(dt);
  // binomial tree towards the root; non-roots accumulate in a scratch buffer
  std::vector<char> scratch, in(n > 1 ? bytes : 0);
  char *acc;
  if (r == root) {
    acc = (char *)recv;
    if (send != recv) memmove(recv, send, bytes);
  } else {
    scratch.assign((const char *)send, (const char *)send + bytes);
    acc = scratch.data();
  }
  int vr = (r - root + n) % n;
  for (int mask = 1; mask < n; mask <<= 1) {
    if (vr & mask) {
      FCXCHECK(net->run({{true, (vr - mask + root) % n, acc, bytes}}));
      break;
    }
    if (vr + mask < n) {
      FCXCHECK(net->run({{false, (vr + mask + root) % n, in.data(), bytes}}));
      FCXCHECK(hostReduce(acc, in.data(), count, dt, op));
    }
  }
  if (r == root && op == flagcxAvg) FCXCHECK(hostDivide(recv, count, dt, n));
  return flagcxSuccess;
}

flagcxResult_t CpuColl::gather(const void *send, void *recv, size_t count, flagcxDataType_t dt,
                               int root) {
  const int n = net->nranks(), r = net->rank();
  const size_t cb = count * getFlagcxDataTypeSize(dt);
  if (r != root) return net->run({{true, root, const_cast<void *>(send), cb}});
  std::vector<HostNet::Op> ops;
  for (int p = 0; p < n; ++p) {
    if (p == r) memmove((char *)recv + (size_t)p * cb, send, cb);
    else ops.push_back({false, p, (char *)recv + (size_t)p * cb, cb});
  }
  return net->run(ops);
}

flagcxResult_t CpuColl::scatter(const void *send, void *recv, size_t count, flagcxDataType_t dt,
                                int root) {
  const int n = net->nranks(), r = net->rank();
  const size_t cb = count * getFlagcxDataTypeSize(dt);
  if (r != root) return net->run({{false, root, recv, cb}});
  std::vector<HostNet::Op> ops;
  for (int p = 0; p < n; ++p) {
    const char *src = (const char *)send + (size_t)p * cb;
    if (p == r) memmove(recv, src, cb);
    else ops.push_back({true, p, const_cast<char *>(src), cb});
  }
  return net->run(ops);
}

flagcxResult_t CpuColl::allToAll(const void *send, void *recv, size_t count, flagcxDataType_t dt) {
  const int n = net->nranks();
  std::vector<size_t> counts(n, count), displs(n);
  for (int p = 0; p < n; ++p) displs[p] = (size_t)p * count;
  return allToAllv(send, counts.data(), displs.data(), recv, counts.data(), displs.data(), dt);
}

flagcxResult_t CpuColl::allToAllv(const void *send, const size_t *scounts, const size_t *sdispls,
                                  void *recv, const size_t *rcounts, const size_t *rdispls,
                                  flagcxDataType_t dt) {
  const int n = net->nranks(), r = net->rank();
  const size_t es = getFlagcxDataTypeSize(dt);
  if (es == 0) return flagcxInvalidArgument;
  if (send == recv) { FCX_WARN("alltoall(v) does not support in-place buffers"); return flagcxInvalidArgument; }
  memmove((char *)recv + rdispls[r] * es, (const char *)send + sdispls[r] * es, scounts[r] * es);
  std::vector<HostNet::Op> ops;
  for (int i = 1; i < n; ++i) {
    int to = (r + i) % n, from = (r - i + n) % n;
    ops.push_back({false, from, (char *)recv + rdispls[from] * es, rcounts[from] * es});
    ops.push_back({true, to, (char *)const_cast<void *>(send) + sdispls[to] * es, scounts[to] * es});
  }
  return net->run(ops);
}

} // namespace fcx
