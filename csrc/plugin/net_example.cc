// net_example.cc -- example network-adaptor plugin: one TCP connection per peer pair,
// length-prefixed messages, non-blocking progress inside test().
//
//   make -C csrc plugin-example
//   FLAGCX_NET_ADAPTOR_PLUGIN=<dir>/libflagcx_net_example.so  <program using libflagcx>
//
// The library loads the symbol flagcxNetAdaptorPlugin_v1 (flagcx_net.h) and routes the
// host-path collectives through it instead of the built-in socket adaptor.  Same role
// as the example under adaptor_plugin/net/ in the FlagCX project.  The counters at the
// end let a test see that the plugin really carried the traffic.
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdint.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <deque>
#include <mutex>
#include <new>

#include "flagcx_net.h"

namespace {

std::atomic<uint64_t> gBytesSent{0}, gBytesReceived{0}, gMessages{0};

struct Handle { // fits FLAGCX_NET_HANDLE_BYTES
  uint32_t magic;
  uint16_t port;
  uint32_t addr; // network byte order
};
constexpr uint32_t kMagic = 0x45584e54; // "EXNT"

struct Request;
struct Conn {
  int fd = -1;
  std::mutex mu;
  std::deque<Request *> queue; // requests complete in posting order
};
struct Listen {
  int fd = -1;
};
struct Request {
  Conn *conn;
  bool isSend;
  char *data;
  uint64_t size;     // payload bytes (send) / capacity (recv)
  uint64_t header;   // payload length on the wire
  uint64_t hdrDone = 0, done = 0;
  bool finished = false, failed = false;
};

void setNonBlocking(int fd, bool on) {
  int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, on ? (fl | O_NONBLOCK) : (fl & ~O_NONBLOCK));
}

// Moves as many bytes as the socket takes right now; returns false on a dead connection.
bool progressOne(Request *r) {
  int fd = r->conn->fd;
  for (;;) {
    char *p;
    uint64_t want;
    if (r->hdrDone < sizeof r->header) {
      p = (char *)&r->header + r->hdrDone;
      want = sizeof r->header - r->hdrDone;
    } else {
      uint64_t total = r->header;
      if (!r->isSend && total > r->size) return false; // message larger than the posted buffer
      if (r->done == total) { r->finished = true; return true; }
      p = r->data + r->done;
      want = total - r->done;
    }
    ssize_t n = r->isSend ? ::send(fd, p, want, MSG_NOSIGNAL) : ::recv(fd, p, want, 0);
    if (n == 0 && !r->isSend) return false;
    if (n < 0) {
      if (errno == EAGAIN || errno == EWOULDBLOCK || errno == EINTR) return true;
      return false;
    }
    if (r->hdrDone < sizeof r->header) r->hdrDone += (uint64_t)n;
    else {
      r->done += (uint64_t)n;
      (r->isSend ? gBytesSent : gBytesReceived) += (uint64_t)n;
    }
  }
}

flagcxResult_t exInit() { return flagcxSuccess; }
flagcxResult_t exDevices(int *ndev) { *ndev = 1; return flagcxSuccess; }
flagcxResult_t exGetProperties(int, void *props) {
  auto *p = (flagcxNetProperties_t *)props;
  memset(p, 0, sizeof *p);
  strncpy(p->name, "example-tcp", sizeof p->name - 1);
  p->speedMbps = 10000;
  p->maxComms = 65536;
  return flagcxSuccess;
}

flagcxResult_t exListen(int, void *handle, void **listenComm) {
  int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return flagcxSystemError;
  sockaddr_in sa{};
  sa.sin_family = AF_INET;
  sa.sin_addr.s_addr = htonl(INADDR_LOOPBACK); // an example: one host only
  sa.sin_port = 0;
  socklen_t len = sizeof sa;
  if (bind(fd, (sockaddr *)&sa, sizeof sa) || listen(fd, 1024) || getsockname(fd, (sockaddr *)&sa, &len)) {
    close(fd);
    return flagcxSystemError;
  }
  Handle h{kMagic, ntohs(sa.sin_port), sa.sin_addr.s_addr};
  memset(handle, 0, FLAGCX_NET_HANDLE_BYTES);
  memcpy(handle, &h, sizeof h);
  auto *l = new (std::nothrow) Listen();
  if (!l) { close(fd); return flagcxSystemError; }
  l->fd = fd;
  *listenComm = l;
  return flagcxSuccess;
}

flagcxResult_t finishConn(int fd, void **out) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
  setNonBlocking(fd, true);
  auto *c = new (std::nothrow) Conn();
  if (!c) { close(fd); return flagcxSystemError; }
  c->fd = fd;
  *out = c;
  return flagcxSuccess;
}

flagcxResult_t exConnect(int, void *handle, void **sendComm) {
  Handle h;
  memcpy(&h, handle, sizeof h);
  if (h.magic != kMagic) return flagcxInvalidArgument;
  int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return flagcxSystemError;
  sockaddr_in sa{};
  sa.sin_family = AF_INET;
  sa.sin_addr.s_addr = h.addr;
  sa.sin_port = htons(h.port);
  if (connect(fd, (sockaddr *)&sa, sizeof sa)) { close(fd); return flagcxSystemError; }
  return finishConn(fd, sendComm);
}

flagcxResult_t exAccept(void *listenComm, void **recvComm) {
  auto *l = (Listen *)listenComm;
  pollfd pfd{l->fd, POLLIN, 0};
  if (poll(&pfd, 1, 120000) <= 0) return flagcxSystemError; // nobody came within two minutes
  int fd = accept(l->fd, nullptr, nullptr);
  if (fd < 0) return flagcxSystemError;
  return finishConn(fd, recvComm);
}

flagcxResult_t exCloseConn(void *comm) {
  auto *c = (Conn *)comm;
  if (!c) return flagcxSuccess;
  if (c->fd >= 0) close(c->fd);
  for (Request *r : c->queue) delete r;
  delete c;
  return flagcxSuccess;
}
flagcxResult_t exCloseListen(void *listenComm) {
  auto *l = (Listen *)listenComm;
  if (!l) return flagcxSuccess;
  if (l->fd >= 0) close(l->fd);
  delete l;
  return flagcxSuccess;
}

// Host memory needs no registration here.
flagcxResult_t exRegMr(void *, void *, size_t, int, int, void **mhandle) { *mhandle = nullptr; return flagcxSuccess; }
flagcxResult_t exRegMrDmaBuf(void *, void *, size_t, int, uint64_t, int, int, void **) { return flagcxNotSupported; }
flagcxResult_t exDeregMr(void *, void *) { return flagcxSuccess; }

flagcxResult_t post(Conn *c, bool isSend, void *data, size_t size, void **request) {
  auto *r = new (std::nothrow) Request();
  if (!r) return flagcxSystemError;
  r->conn = c;
  r->isSend = isSend;
  r->data = (char *)data;
  r->size = size;
  r->header = isSend ? size : 0;
  std::lock_guard<std::mutex> lk(c->mu);
  c->queue.push_back(r);
  *request = r;
  ++gMessages;
  return flagcxSuccess;
}

flagcxResult_t exIsend(void *sendComm, void *data, size_t size, int, void *, void *, void **request) {
  return post((Conn *)sendComm, true, data, size, request);
}
flagcxResult_t exIrecv(void *recvComm, int n, void **data, size_t *sizes, int *, void **, void **, void **request) {
  if (n != 1) return flagcxInvalidArgument;
  return post((Conn *)recvComm, false, data[0], sizes[0], request);
}
flagcxResult_t exIflush(void *, int, void **, int *, void **, void **request) { *request = nullptr; return flagcxSuccess; }

flagcxResult_t exTest(void *request, int *done, int *sizes) {
  *done = 0;
  if (!request) { *done = 1; return flagcxSuccess; }
  auto *r = (Request *)request;
  Conn *c = r->conn;
  std::lock_guard<std::mutex> lk(c->mu);
  // requests of one connection share one byte stream: drive them in posting order up
  // to this one; finished requests stay queued until their owner tests them
  for (Request *q : c->queue) {
    if (!q->finished && !q->failed && !progressOne(q)) q->failed = true;
    if (!q->finished && !q->failed) break; // the stream is busy with q
    if (q == r) break;
  }
  if (!r->finished && !r->failed) return flagcxSuccess;
  for (auto it = c->queue.begin(); it != c->queue.end(); ++it)
    if (*it == r) { c->queue.erase(it); break; }
  const bool failed = r->failed;
  if (sizes) sizes[0] = (int)r->done;
  delete r;
  *done = 1;
  return failed ? flagcxRemoteError : flagcxSuccess;
}

flagcxResult_t exGetDevFromName(char *, int *dev) { *dev = 0; return flagcxSuccess; }

} // namespace

extern "C" {

// (a const object has internal linkage in C++ unless it is declared extern first)
extern const struct flagcxNetAdaptor_v1 flagcxNetAdaptorPlugin_v1;
const struct flagcxNetAdaptor_v1 flagcxNetAdaptorPlugin_v1 = {
    "example-tcp", exInit,        exDevices,   exGetProperties, exListen,      exConnect, exAccept,
    exCloseConn,   exCloseConn,   exCloseListen, exRegMr,       exRegMrDmaBuf, exDeregMr, exIsend,
    exIrecv,       exIflush,      exTest,      nullptr,         nullptr,       nullptr,   exGetDevFromName};

// Traffic carried since the library was loaded (for tests and curiosity).
void flagcxNetExampleCounters(uint64_t *bytesSent, uint64_t *bytesReceived, uint64_t *messages) {
  if (bytesSent) *bytesSent = gBytesSent.load();
  if (bytesReceived) *bytesReceived = gBytesReceived.load();
  if (messages) *messages = gMessages.load();
}

} // extern "C"
