// p2p_transfer.cc -- the transfer engine of flagcx_p2p.h from plain C++: a forked "owner"
// process registers a buffer and publishes its metadata and a descriptor through a pipe; the
// parent connects, writes a pattern into the owner's buffer one-sidedly, tells the owner
// with a notification, reads the buffer back and checks it.  Host memory, so it runs on a
// machine without a GPU:
//
//     make -C csrc examples && csrc/build/examples/p2p_transfer [bytes]
//
// With device memory the calls are the same (flagcxP2pEngineCreate(device, ...), a
// cudaMalloc'ed buffer); the transfer is then one cudaMemcpyAsync over NVLink.
#include <sys/wait.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "flagcx_p2p.h"

#define CHECK(call)                                                                   \
  do {                                                                                \
    flagcxResult_t r_ = (call);                                                       \
    if (r_ != flagcxSuccess) {                                                        \
      fprintf(stderr, "%s:%d %s -> %s\n", __FILE__, __LINE__, #call, flagcxGetErrorString(r_)); \
      exit(1);                                                                        \
    }                                                                                 \
  } while (0)

struct Hello {
  char meta[128];
  flagcxP2pDesc_t desc;
};

static int owner(int wfd, size_t bytes) {
  flagcxP2pEngine_t eng;
  CHECK(flagcxP2pEngineCreate(-1, &eng));
  std::vector<unsigned char> buf(bytes, 0);
  flagcxP2pMr_t mr;
  CHECK(flagcxP2pEngineReg(eng, buf.data(), buf.size(), &mr));
  Hello h{};
  CHECK(flagcxP2pEngineGetMetadata(eng, h.meta, sizeof h.meta));
  CHECK(flagcxP2pEngineMakeDesc(eng, mr, buf.data(), buf.size(), &h.desc));
  if (write(wfd, &h, sizeof h) != (ssize_t)sizeof h) return 1;
  flagcxP2pConn_t conn;
  CHECK(flagcxP2pEngineAccept(eng, &conn, 30000));
  char msg[64];
  size_t len = 0;
  CHECK(flagcxP2pRecvNotif(conn, msg, sizeof msg, &len, 30000)); // "written"
  size_t bad = 0;
  for (size_t i = 0; i < bytes; ++i) bad += buf[i] != (unsigned char)(i * 31 + 7);
  printf("owner: %zu bytes arrived, %zu wrong\n", bytes, bad);
  fflush(stdout);
  for (size_t i = 0; i < bytes; ++i) buf[i] = (unsigned char)(i * 13 + 1);
  CHECK(flagcxP2pSendNotif(conn, "refilled", 8));
  CHECK(flagcxP2pRecvNotif(conn, msg, sizeof msg, &len, 30000)); // "bye"
  CHECK(flagcxP2pConnDestroy(conn));
  CHECK(flagcxP2pEngineDereg(eng, mr));
  CHECK(flagcxP2pEngineDestroy(eng));
  return bad ? 1 : 0;
}

int main(int argc, char **argv) {
  const size_t bytes = argc > 1 ? strtoull(argv[1], nullptr, 0) : (8u << 20);
  int fds[2];
  if (pipe(fds) != 0) return 1;
  pid_t pid = fork();
  if (pid == 0) {
    close(fds[0]);
    _exit(owner(fds[1], bytes));
  }
  close(fds[1]);
  Hello h;
  if (read(fds[0], &h, sizeof h) != (ssize_t)sizeof h) return 1;
  flagcxP2pEngine_t eng;
  CHECK(flagcxP2pEngineCreate(-1, &eng));
  flagcxP2pConn_t conn;
  CHECK(flagcxP2pEngineConnect(eng, h.meta, &conn));
  int local = 0;
  CHECK(flagcxP2pConnIsLocal(conn, &local));
  std::vector<unsigned char> src(bytes), back(bytes, 0);
  for (size_t i = 0; i < bytes; ++i) src[i] = (unsigned char)(i * 31 + 7);
  CHECK(flagcxP2pWrite(conn, src.data(), &h.desc, bytes, nullptr));
  CHECK(flagcxP2pSendNotif(conn, "written", 7));
  char msg[64];
  size_t len = 0;
  CHECK(flagcxP2pRecvNotif(conn, msg, sizeof msg, &len, 30000)); // "refilled"
  CHECK(flagcxP2pRead(conn, back.data(), &h.desc, bytes, nullptr));
  size_t bad = 0;
  for (size_t i = 0; i < bytes; ++i) bad += back[i] != (unsigned char)(i * 13 + 1);
  printf("initiator: peer %s, read %zu bytes back, %zu wrong\n", local ? "on this machine" : "remote", bytes, bad);
  CHECK(flagcxP2pSendNotif(conn, "bye", 3));
  CHECK(flagcxP2pConnDestroy(conn));
  CHECK(flagcxP2pEngineDestroy(eng));
  int status = 0;
  waitpid(pid, &status, 0);
  const bool ok = bad == 0 && WIFEXITED(status) && WEXITSTATUS(status) == 0;
  printf("%s\n", ok ? "ok" : "FAILED");
  return ok ? 0 : 1;
}
