// allreduce_perf.cc -- a program written against the public C API only: launches N ranks
// (one process each, one GPU each when GPUs are present, host buffers otherwise), runs
// one collective (-o allreduce|allgather|reducescatter|alltoall|broadcast, default
// allreduce) over a range of sizes, checks the result and prints time, algorithm
// bandwidth and bus bandwidth.  Same role as the test/perf/host_api/test_*.cpp programs of
// the FlagCX project, without mpirun: ranks are forked here and meet through
// FLAGCX_COMM_ID.
//
//   make -C csrc examples
//   csrc/build/examples/allreduce_perf -n 8 -b 1M -e 1G -f 2 -w 5 -i 20
//   csrc/build/examples/allreduce_perf -n 3 --host -b 1K -e 1M        (CPU ranks, host buffers)
//   csrc/build/examples/allreduce_perf -n 8 -o alltoall -b 1M -e 256M
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cmath>
#include <string>
#include <vector>

#include "flagcx.h"

#define CHECK(call)                                                                                  \
  do {                                                                                               \
    flagcxResult_t r_ = (call);                                                                      \
    if (r_ != flagcxSuccess) {                                                                       \
      fprintf(stderr, "rank %d: %s failed: %s (%s:%d)\n", gRank, #call, flagcxGetErrorString(r_), __FILE__, \
              __LINE__);                                                                             \
      exit(2);                                                                                       \
    }                                                                                                \
  } while (0)

static int gRank = -1;

static size_t parseSize(const char *s) {
  char *end = nullptr;
  double v = strtod(s, &end);
  switch (*end) {
    case 'K': case 'k': v *= 1 << 10; break;
    case 'M': case 'm': v *= 1 << 20; break;
    case 'G': case 'g': v *= 1 << 30; break;
    default: break;
  }
  return (size_t)v;
}

enum Op { kAllReduce, kAllGather, kReduceScatter, kAllToAll, kBroadcast };

// `bytes` is the size of the larger of the two buffers; count = elements of the call.
static flagcxResult_t runOp(Op op, const void *send, void *recv, size_t total, int n, flagcxComm_t comm,
                            flagcxStream_t stream) {
  switch (op) {
    case kAllReduce: return flagcxAllReduce(send, recv, total, flagcxFloat, flagcxSum, comm, stream);
    case kAllGather: return flagcxAllGather(send, recv, total / n, flagcxFloat, comm, stream);
    case kReduceScatter: return flagcxReduceScatter(send, recv, total / n, flagcxFloat, flagcxSum, comm, stream);
    case kAllToAll: return flagcxAlltoAll(send, recv, total / n, flagcxFloat, comm, stream);
    case kBroadcast: return flagcxBroadcast(send, recv, total, flagcxFloat, 0, comm, stream);
  }
  return flagcxInvalidArgument;
}

// What element i of the output must hold when rank r's input element j is (j % 13) + r.
static float expected(Op op, size_t i, size_t total, int n, int rank) {
  const size_t per = total / n;
  const float ranks = (float)(n * (n - 1) / 2);
  switch (op) {
    case kAllReduce: return (float)n * (float)(i % 13) + ranks;
    case kAllGather: return (float)((i % per) % 13) + (float)(i / per);
    case kReduceScatter: return (float)n * (float)((rank * per + i) % 13) + ranks;
    case kAllToAll: return (float)((rank * per + i % per) % 13) + (float)(i / per);
    case kBroadcast: return (float)(i % 13);
  }
  return 0.f;
}

static int runRank(Op op, int rank, int n, bool host, size_t minBytes, size_t maxBytes, int factor, int warmup, int iters) {
  gRank = rank;
  flagcxDeviceHandle_t dev;
  CHECK(flagcxDeviceHandleInit(&dev));
  int ndev = 0;
  if (!host) dev->getDeviceCount(&ndev);
  const bool onGpu = !host && ndev > 0;
  if (onGpu) CHECK(dev->setDevice(rank % ndev));
  if (host) setenv("FLAGCX_FORCE_HOST", "1", 1);

  flagcxUniqueId id; // every rank derives the same id from FLAGCX_COMM_ID; rank 0 serves it
  CHECK(flagcxGetUniqueId(&id));
  flagcxComm_t comm;
  CHECK(flagcxCommInitRank(&comm, n, &id, rank));

  flagcxStream_t stream;
  CHECK(dev->streamCreate(&stream));
  flagcxEvent_t e0, e1;
  CHECK(dev->eventCreate(&e0, flagcxEventDefault));
  CHECK(dev->eventCreate(&e1, flagcxEventDefault));
  const flagcxMemType_t where = onGpu ? flagcxMemDevice : flagcxMemHost;
  void *send = nullptr, *recv = nullptr;
  CHECK(dev->deviceMalloc(&send, maxBytes, where, stream));
  CHECK(dev->deviceMalloc(&recv, maxBytes, where, stream));
  std::vector<float> h(maxBytes / 4), back(maxBytes / 4);
  for (size_t i = 0; i < h.size(); ++i) h[i] = (float)((i % 13) + rank);
  CHECK(dev->deviceMemcpy(send, h.data(), maxBytes, flagcxMemcpyHostToDevice, stream));
  CHECK(dev->streamSynchronize(stream));

  static const char *names[] = {"allreduce", "allgather", "reducescatter", "alltoall", "broadcast"};
  if (rank == 0) printf("# %s, %d ranks, %s buffers\n# %12s %10s %10s %10s %8s\n", names[op], n, onGpu ? "device" : "host",
                        "bytes", "time(us)", "algbw GB/s", "busbw GB/s", "check");
  int bad = 0;
  for (size_t bytes = minBytes; bytes <= maxBytes; bytes *= factor) {
    const size_t count = bytes / 4 / n * n; // elements of the larger buffer, a multiple of the ranks
    if (count == 0) continue;
    const size_t outCount = op == kReduceScatter ? count / n : count;
    for (int i = 0; i < warmup; ++i) CHECK(runOp(op, send, recv, count, n, comm, stream));
    CHECK(dev->streamSynchronize(stream));
    CHECK(flagcxBarrier(comm, stream));
    CHECK(dev->streamSynchronize(stream));
    CHECK(dev->eventRecord(e0, stream));
    for (int i = 0; i < iters; ++i) CHECK(runOp(op, send, recv, count, n, comm, stream));
    CHECK(dev->eventRecord(e1, stream));
    CHECK(dev->eventSynchronize(e1));
    float ms = 0;
    CHECK(dev->eventElapsedTime(&ms, e0, e1));
    // slowest rank counts
    float mine = ms * 1000.f / iters, worst = 0;
    {
      std::vector<float> all(n, 0.f), out(n, 0.f);
      all[rank] = mine;
      void *a = nullptr, *o = nullptr;
      CHECK(dev->deviceMalloc(&a, n * 4, where, stream));
      CHECK(dev->deviceMalloc(&o, n * 4, where, stream));
      CHECK(dev->deviceMemcpy(a, all.data(), n * 4, flagcxMemcpyHostToDevice, stream));
      CHECK(flagcxAllReduce(a, o, n, flagcxFloat, flagcxMax, comm, stream));
      CHECK(dev->deviceMemcpy(out.data(), o, n * 4, flagcxMemcpyDeviceToHost, stream));
      CHECK(dev->streamSynchronize(stream));
      for (float v : out) worst = std::fmax(worst, v);
      dev->deviceFree(a, where, stream);
      dev->deviceFree(o, where, stream);
    }
    CHECK(dev->deviceMemcpy(back.data(), recv, outCount * 4, flagcxMemcpyDeviceToHost, stream));
    CHECK(dev->streamSynchronize(stream));
    bool ok = true;
    for (size_t i = 0; i < outCount && ok; i += (outCount / 257) + 1) {
      float want = expected(op, i, count, n, rank);
      ok = std::fabs(back[i] - want) <= 1e-5f * std::fabs(want) + 1e-6f;
    }
    bad += !ok;
    if (rank == 0) {
      double alg = (double)(count * 4) / worst / 1e3;
      double factorBus = op == kAllReduce ? 2.0 * (n - 1) / n : op == kBroadcast ? 1.0 : (double)(n - 1) / n;
      printf("  %12zu %10.1f %10.2f %10.2f %8s\n", count * 4, worst, alg, alg * factorBus, ok ? "ok" : "WRONG");
      fflush(stdout);
    }
    if (bytes == 0 || factor < 2) break;
  }
  dev->deviceFree(send, where, stream);
  dev->deviceFree(recv, where, stream);
  dev->eventDestroy(e0);
  dev->eventDestroy(e1);
  dev->streamDestroy(stream);
  CHECK(flagcxCommDestroy(comm));
  flagcxDeviceHandleFree(dev);
  return bad ? 1 : 0;
}

int main(int argc, char **argv) {
  int n = 2, factor = 2, warmup = 5, iters = 20, port = 0;
  size_t minBytes = 1 << 20, maxBytes = 64 << 20;
  bool host = false;
  Op op = kAllReduce;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() -> const char * { return i + 1 < argc ? argv[++i] : "0"; };
    if (a == "-n") n = atoi(next());
    else if (a == "-b") minBytes = parseSize(next());
    else if (a == "-e") maxBytes = parseSize(next());
    else if (a == "-f") factor = atoi(next());
    else if (a == "-w") warmup = atoi(next());
    else if (a == "-i") iters = atoi(next());
    else if (a == "-p") port = atoi(next());
    else if (a == "--host") host = true;
    else if (a == "-o") {
      std::string o = next();
      if (o == "allreduce") op = kAllReduce;
      else if (o == "allgather") op = kAllGather;
      else if (o == "reducescatter") op = kReduceScatter;
      else if (o == "alltoall") op = kAllToAll;
      else if (o == "broadcast") op = kBroadcast;
      else { fprintf(stderr, "unknown operation %s\n", o.c_str()); return 64; }
    }
    else { fprintf(stderr, "usage: %s [-n ranks] [-b min] [-e max] [-f factor] [-w warmup] [-i iters] [-p port] [-o op] [--host]\n", argv[0]); return 64; }
  }
  minBytes = (minBytes + 3) / 4 * 4;
  if (maxBytes < minBytes) maxBytes = minBytes;
  if (!getenv("FLAGCX_COMM_ID")) {
    char id[64];
    snprintf(id, sizeof id, "127.0.0.1:%d", port ? port : 20000 + (int)(getpid() % 20000));
    setenv("FLAGCX_COMM_ID", id, 1);
  }
  // fork before anything touches the library or CUDA: every rank starts clean
  std::vector<pid_t> kids;
  for (int r = 0; r < n; ++r) {
    pid_t p = fork();
    if (p == 0) return runRank(op, r, n, host, minBytes, maxBytes, factor, warmup, iters);
    if (p < 0) { perror("fork"); return 1; }
    kids.push_back(p);
  }
  int rc = 0;
  for (pid_t p : kids) {
    int st = 0;
    waitpid(p, &st, 0);
    if (!WIFEXITED(st) || WEXITSTATUS(st)) rc = 1;
  }
  return rc;
}
