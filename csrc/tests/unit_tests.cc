// unit_tests.cc -- host-only unit tests of the library's internals, linked against
// libflagcx.so and run without a GPU: parameters and config files, the interface-name
// matcher, address parsing, 16-bit float conversions, the window registry, the tuner's
// heuristic and JSON round trip, bootstrap primitives among threads, and the socket
// network adaptor.  Prints one line per check; the exit code is the number of failures.
#include <unistd.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <thread>
#include <vector>

#include "../host/bootstrap.h"
#include "../host/comm.h"
#include "../host/cpu_coll.h"
#include "../host/reg_cache.h"
#include "../host/shm.h"
#include "../host/tuner.h"
#include "flagcx_net.h"
#include "flagcx_p2p.h"

using namespace fcx;

static int failures = 0;
#define EXPECT(cond)                                                                  \
  do {                                                                                \
    if (!(cond)) { ++failures; printf("FAIL %s:%d  %s\n", __FILE__, __LINE__, #cond); } \
  } while (0)

static void testParams() {
  // the config files are read once, at the first lookup the environment cannot answer
  char path[] = "/tmp/flagcx_ut_confXXXXXX";
  int fd = mkstemp(path);
  const char *text = "# comment\nFLAGCX_UT_FROM_FILE = 99\nFLAGCX_UT_NUMBER=1\n";
  EXPECT(write(fd, text, strlen(text)) > 0);
  close(fd);
  setenv("FLAGCX_CONF_FILE", path, 1);
  setenv("FLAGCX_UT_NUMBER", "42", 1);
  setenv("FLAGCX_UT_SIZE", "3M", 1);
  setenv("FLAGCX_UT_BAD", "abc", 1);
  EXPECT(loadParam("FLAGCX_UT_NUMBER", 7) == 42);
  EXPECT(loadParam("FLAGCX_UT_SIZE", 7) == 3 << 20);
  EXPECT(loadParam("FLAGCX_UT_BAD", 7) == 7);
  EXPECT(loadParam("FLAGCX_UT_MISSING", -5) == -5);
  EXPECT(readParam("UT_NUMBER", 0) == 42);
  // values from a config file are used when the environment has none
  EXPECT(loadParam("FLAGCX_UT_FROM_FILE", 0) == 99);
  EXPECT(loadParam("FLAGCX_UT_NUMBER", 0) == 42); // environment wins
  unlink(path);
}

static void testIfMatcher() {
  EXPECT(ifNameMatches(nullptr, "eth0"));
  EXPECT(ifNameMatches("eth", "eth0") && ifNameMatches("eth", "eth1") && !ifNameMatches("eth", "ib0"));
  EXPECT(ifNameMatches("ib,eth1", "eth1") && !ifNameMatches("ib,eth1", "eth0"));
  EXPECT(ifNameMatches("=eth0", "eth0") && !ifNameMatches("=eth0", "eth00"));
  EXPECT(!ifNameMatches("^docker,lo", "docker0") && !ifNameMatches("^docker,lo", "lo") && ifNameMatches("^docker,lo", "eth0"));
  EXPECT(ifNameMatches("^=lo", "lo0") && !ifNameMatches("^=lo", "lo"));
}

static void testAddresses() {
  SockAddr a;
  EXPECT(addrFromString("127.0.0.1:2345", &a) == flagcxSuccess);
  EXPECT(a.sa.sa_family == AF_INET && ntohs(a.in4.sin_port) == 2345);
  EXPECT(addrToString(a) == "127.0.0.1:2345");
  EXPECT(addrFromString("[::1]:77", &a) == flagcxSuccess && a.sa.sa_family == AF_INET6);
  EXPECT(addrToString(a) == "[::1]:77");
  EXPECT(addrFromString("no-port", &a) == flagcxInvalidArgument);
  EXPECT(!findInterfaces().empty());
}

static void testHalfFloats() {
  for (float f : {0.f, 1.f, -2.5f, 65504.f, 1e-5f, 3.14159f, -0.33333f}) {
    EXPECT(std::fabs(halfToFloat(floatToHalf(f)) - f) <= std::fabs(f) * 1e-3f + 1e-7f);
    EXPECT(std::fabs(bf16ToFloat(floatToBf16(f)) - f) <= std::fabs(f) * 8e-3f + 1e-38f);
  }
  EXPECT(halfToFloat(floatToHalf(1e6f)) == INFINITY);
  EXPECT(std::isnan(halfToFloat(floatToHalf(NAN))) && std::isnan(bf16ToFloat(floatToBf16(NAN))));
  // round to nearest even: 1 + 2^-8 is exactly between two bf16 values, 1 + 2^-11 between two halves
  EXPECT(bf16ToFloat(floatToBf16(1.0f + 0.00390625f)) == 1.0f);
  EXPECT(halfToFloat(floatToHalf(1.0f + 0.00048828125f)) == 1.0f);
  EXPECT(halfToFloat(floatToHalf(6e-8f)) > 0.f); // subnormal survives
}

static void testRegistry() {
  WindowRegistry reg;
  Window a, b;
  a.local = (void *)0x10000; a.size = 0x1000;
  b.local = (void *)0x20000; b.size = 0x8000;
  reg.add(&a);
  reg.add(&b);
  EXPECT(reg.find((void *)0x10000, 16) == &a);
  EXPECT(reg.find((void *)0x10ff0, 16) == &a);
  EXPECT(reg.find((void *)0x10ff0, 17) == nullptr); // runs past the end
  EXPECT(reg.find((void *)0x27fff, 1) == &b);
  EXPECT(reg.find((void *)0x1ffff, 1) == nullptr);
  EXPECT(reg.find((void *)0x0fff0, 32) == nullptr);
  EXPECT(reg.all().size() == 2);
  reg.remove(&a);
  EXPECT(reg.find((void *)0x10000, 16) == nullptr && reg.all().size() == 1);
}

static void testTuner() {
  Tuner t;
  t.maxCtas = 48;
  TuneChoice small = t.heuristic(flagcxCommOpAllReduce, 8 << 10, 8, true, false);
  TuneChoice big = t.heuristic(flagcxCommOpAllReduce, 64 << 20, 8, true, false);
  EXPECT(small.algo == FLAGCX_ALGO_ONESHOT && big.algo == FLAGCX_ALGO_TWOSHOT);
  EXPECT(small.nCtas >= 1 && small.nCtas <= big.nCtas && big.nCtas <= 48);
  EXPECT(t.heuristic(flagcxCommOpAllReduce, 64 << 20, 8, true, true).algo == FLAGCX_ALGO_NVLS_TWOSHOT);
  EXPECT(t.heuristic(flagcxCommOpAllGather, 1 << 20, 4, true, false).algo == FLAGCX_ALGO_PUSH);
  EXPECT(t.heuristic(flagcxCommOpReduceScatter, 1 << 20, 4, true, false).algo == FLAGCX_ALGO_PULL);
  EXPECT(Tuner::bucketOf(1) == 0 && Tuner::bucketOf(1024) == 10 && Tuner::bucketOf(1025) == 11);
  // a measured entry overrides the heuristic for its bucket only, and survives JSON
  TuneChoice forced;
  forced.algo = FLAGCX_ALGO_TWOSHOT;
  forced.nCtas = 7;
  forced.usec = 12.5f;
  t.table[(int)flagcxCommOpAllReduce * 1000 + 13 * 2 + 1] = forced;
  EXPECT(t.choose(flagcxCommOpAllReduce, 8 << 10, 8, true, false).nCtas == 7);
  EXPECT(t.choose(flagcxCommOpAllReduce, 8 << 10, 8, false, false).algo == FLAGCX_ALGO_ONESHOT);
  Tuner u;
  u.maxCtas = 48;
  EXPECT(u.fromJson(t.toJson()) == flagcxSuccess);
  EXPECT(u.table.size() == 1 && u.choose(flagcxCommOpAllReduce, 8 << 10, 8, true, false).nCtas == 7);
  // an entry for 2-byte elements wins for bf16 calls of that bucket; 4-byte calls keep the
  // size-agnostic entry; a table without elem_size (older files) still loads
  TuneChoice two;
  two.algo = FLAGCX_ALGO_TWOSHOT;
  two.nCtas = 9;
  t.table[2 * 100000 + (int)flagcxCommOpAllReduce * 1000 + 13 * 2 + 1] = two;
  EXPECT(t.choose(flagcxCommOpAllReduce, 8 << 10, 8, true, false, 2).nCtas == 9);
  EXPECT(t.choose(flagcxCommOpAllReduce, 8 << 10, 8, true, false, 4).nCtas == 7);
  EXPECT(t.choose(flagcxCommOpAllGather, 8 << 10, 8, true, false, 2).algo != FLAGCX_ALGO_TWOSHOT);
  EXPECT(u.fromJson(t.toJson()) == flagcxSuccess && u.table.size() == 2);
  EXPECT(u.choose(flagcxCommOpAllReduce, 8 << 10, 8, true, false, 2).nCtas == 9);
  t.table.erase(2 * 100000 + (int)flagcxCommOpAllReduce * 1000 + 13 * 2 + 1);
  EXPECT(u.fromJson("{\"entries\": [{\"op\": 6, \"bucket\": 13, \"registered\": 1, \"algo\": 1, \"nctas\": 5}]}") == flagcxSuccess);
  EXPECT(u.choose(flagcxCommOpAllReduce, 8 << 10, 8, true, false, 2).nCtas == 5);
  EXPECT(u.fromJson("{\"entries\": [{\"op\": 99, \"bucket\": 3}]}") == flagcxInvalidArgument);
  EXPECT(u.fromJson("not json") == flagcxInvalidArgument);
  // an NVLS entry is ignored when multimem is not usable for the call
  TuneChoice nv;
  nv.algo = FLAGCX_ALGO_NVLS_ONESHOT;
  nv.nCtas = 4;
  t.table[(int)flagcxCommOpAllReduce * 1000 + 20 * 2 + 1] = nv;
  EXPECT(t.choose(flagcxCommOpAllReduce, 1 << 20, 8, true, false).algo != FLAGCX_ALGO_NVLS_ONESHOT);
  EXPECT(t.choose(flagcxCommOpAllReduce, 1 << 20, 8, true, true).algo == FLAGCX_ALGO_NVLS_ONESHOT);
}

static void testBootstrapThreads() {
  const int n = 5;
  flagcxUniqueId id;
  EXPECT(bootstrapCreateId(&id) == flagcxSuccess);
  std::atomic<int> bad{0};
  std::vector<std::thread> th;
  for (int r = 0; r < n; ++r)
    th.emplace_back([&, r] {
      Bootstrap b;
      if (b.init(id, r, n) != flagcxSuccess) { ++bad; return; }
      std::vector<int> all(n, -1);
      all[r] = r * r;
      if (b.allGather(all.data(), sizeof(int)) != flagcxSuccess) ++bad;
      for (int p = 0; p < n; ++p) if (all[p] != p * p) ++bad;
      int v = r == 2 ? 77 : 0;
      if (b.broadcast(&v, sizeof v, 2) != flagcxSuccess || v != 77) ++bad;
      if (b.barrier() != flagcxSuccess) ++bad;
      // out-of-order tags: send tag 9 then tag 8, receive 8 then 9
      int next = (r + 1) % n, prev = (r + n - 1) % n, x9 = 900 + r, x8 = 800 + r, g8 = 0, g9 = 0;
      if (b.send(next, 9, &x9, sizeof x9) != flagcxSuccess || b.send(next, 8, &x8, sizeof x8) != flagcxSuccess) ++bad;
      if (b.recv(prev, 8, &g8, sizeof g8) != flagcxSuccess || b.recv(prev, 9, &g9, sizeof g9) != flagcxSuccess) ++bad;
      if (g8 != 800 + prev || g9 != 900 + prev) ++bad;
      // big ring allgather (forces the chunked path)
      std::vector<char> bigbuf((size_t)n * (300 << 10));
      memset(bigbuf.data() + (size_t)r * (300 << 10), 'a' + r, 300 << 10);
      if (b.allGather(bigbuf.data(), 300 << 10) != flagcxSuccess) ++bad;
      for (int p = 0; p < n; ++p) if (bigbuf[(size_t)p * (300 << 10) + 12345] != 'a' + p) ++bad;
      b.barrier();
    });
  for (auto &t : th) t.join();
  EXPECT(bad.load() == 0);
}

// Whole communicators as threads of one process (host buffers): the public API from
// several threads at once, over shared-memory rings and over the socket adaptor.
static void testCommunicatorsInThreads() {
  const int n = 4;
  const size_t count = 50000;
  flagcxUniqueId id;
  EXPECT(flagcxGetUniqueId(&id) == flagcxSuccess);
  std::atomic<int> bad{0};
  std::vector<std::thread> th;
  for (int r = 0; r < n; ++r)
    th.emplace_back([&, r] {
      flagcxComm_t comm = nullptr;
      if (flagcxCommInitRank(&comm, n, &id, r) != flagcxSuccess) { ++bad; return; }
      std::vector<float> x(count), out(count);
      for (size_t i = 0; i < count; ++i) x[i] = (float)(i % 7) + r;
      if (flagcxAllReduce(x.data(), out.data(), count, flagcxFloat, flagcxSum, comm, nullptr) != flagcxSuccess) ++bad;
      for (size_t i = 0; i < count; i += 97)
        if (out[i] != (float)n * (float)(i % 7) + (float)(n * (n - 1) / 2)) { ++bad; break; }
      const size_t per = count / n;
      std::vector<float> a2a(per * n);
      if (flagcxAlltoAll(x.data(), a2a.data(), per, flagcxFloat, comm, nullptr) != flagcxSuccess) ++bad;
      for (int p = 0; p < n; ++p)
        if (a2a[p * per + 5] != (float)((r * per + 5) % 7) + p) ++bad;
      int next = (r + 1) % n, prev = (r + n - 1) % n;
      std::vector<float> got(count);
      if (flagcxGroupStart(comm) != flagcxSuccess) ++bad;
      if (flagcxSend(x.data(), count, flagcxFloat, next, comm, nullptr) != flagcxSuccess) ++bad;
      if (flagcxRecv(got.data(), count, flagcxFloat, prev, comm, nullptr) != flagcxSuccess) ++bad;
      if (flagcxGroupEnd(comm) != flagcxSuccess) ++bad;
      if (got[3] != 3.f + prev) ++bad;
      if (flagcxBarrier(comm, nullptr) != flagcxSuccess) ++bad;
      if (flagcxCommDestroy(comm) != flagcxSuccess) ++bad;
    });
  for (auto &t : th) t.join();
  EXPECT(bad.load() == 0);
}

static void testSocketAdaptor() {
  const flagcxNetAdaptor_v1 *net = flagcxGetNetAdaptor();
  EXPECT(net && std::string(net->name) == "socket");
  int ndev = 0;
  EXPECT(net->devices(&ndev) == flagcxSuccess && ndev >= 1);
  flagcxNetProperties_t props;
  EXPECT(net->getProperties(0, &props) == flagcxSuccess && props.speedMbps > 0);
  char handle[FLAGCX_NET_HANDLE_BYTES];
  void *lc = nullptr, *sc = nullptr, *rc = nullptr;
  EXPECT(net->listen(0, handle, &lc) == flagcxSuccess);
  std::thread connector([&] { EXPECT(net->connect(0, handle, &sc) == flagcxSuccess); });
  EXPECT(net->accept(lc, &rc) == flagcxSuccess);
  connector.join();
  const size_t big = (3 << 20) + 17;
  std::vector<char> src(big), dst(big, 0), small(100, 'x'), smallDst(100, 0);
  for (size_t i = 0; i < big; ++i) src[i] = (char)(i * 31 + 7);
  void *r1 = nullptr, *r2 = nullptr, *s1 = nullptr, *s2 = nullptr;
  void *d1 = dst.data(), *d2 = smallDst.data();
  size_t z1 = big, z2 = 100;
  int tag = 0;
  EXPECT(net->irecv(rc, 1, &d1, &z1, &tag, nullptr, nullptr, &r1) == flagcxSuccess);
  EXPECT(net->irecv(rc, 1, &d2, &z2, &tag, nullptr, nullptr, &r2) == flagcxSuccess);
  EXPECT(net->isend(sc, src.data(), big, 0, nullptr, nullptr, &s1) == flagcxSuccess);
  EXPECT(net->isend(sc, small.data(), 100, 0, nullptr, nullptr, &s2) == flagcxSuccess);
  void *reqs[4] = {r1, r2, s1, s2};
  int done[4] = {0, 0, 0, 0}, sizes[4] = {0, 0, 0, 0}, left = 4;
  for (int spin = 0; spin < 20000000 && left; ++spin)
    for (int i = 0; i < 4; ++i)
      if (!done[i]) { EXPECT(net->test(reqs[i], &done[i], &sizes[i]) == flagcxSuccess); if (done[i]) --left; }
  EXPECT(left == 0 && sizes[0] == (int)big && sizes[1] == 100);
  EXPECT(dst == src && smallDst == small);
  EXPECT(net->closeSend(sc) == flagcxSuccess && net->closeRecv(rc) == flagcxSuccess && net->closeListen(lc) == flagcxSuccess);
}

static void testHostReduce() {
  float a[5] = {1, 2, 3, 4, 5}, b[5] = {5, 4, 3, 2, 1};
  EXPECT(hostReduce(a, b, 5, flagcxFloat32, flagcxMax) == flagcxSuccess && a[0] == 5 && a[4] == 5 && a[2] == 3);
  int64_t x[3] = {6, -9, 10};
  EXPECT(hostDivide(x, 3, flagcxInt64, 3) == flagcxSuccess && x[0] == 2 && x[1] == -3 && x[2] == 3);
  EXPECT(hostReduce(a, b, 5, (flagcxDataType_t)42, flagcxSum) == flagcxInvalidArgument);
  EXPECT(getFlagcxDataTypeSize(flagcxBfloat16) == 2 && getFlagcxDataTypeSize((flagcxDataType_t)42) == 0);
}

// Shared-memory ring: creation rules, wrap-around, a producer and a consumer thread.
static void testShmRing() {
  char name[64];
  snprintf(name, sizeof name, "/flagcx-unit-%d", (int)getpid());
  ShmRing tx, rx;
  EXPECT(tx.create(name, 5000) == flagcxInvalidArgument); // not a power of two
  EXPECT(tx.create(name, 8192) == flagcxSuccess);
  ShmRing dup;
  EXPECT(dup.create(name, 8192) == flagcxSystemError); // the name is taken
  EXPECT(rx.open(name) == flagcxSuccess);
  ShmRing late;
  EXPECT(late.open(name) != flagcxSuccess); // the receiver removed the name
  char small[16] = "hello, ring", got[16] = {0};
  EXPECT(rx.read(got, sizeof got) == 0);
  EXPECT(tx.write(small, 12) == 12 && rx.read(got, sizeof got) == 12 && !strcmp(got, small));
  // far more than the capacity, odd piece sizes so that every wrap position is hit
  const size_t total = 1 << 20;
  std::vector<unsigned char> src(total), dst(total, 0);
  for (size_t i = 0; i < total; ++i) src[i] = (unsigned char)(i * 131 + (i >> 9));
  std::thread producer([&] {
    size_t off = 0, piece = 1;
    while (off < total) {
      size_t want = std::min(piece, total - off);
      off += tx.write(src.data() + off, want);
      piece = piece % 3001 + 7;
    }
  });
  size_t off = 0, piece = 5;
  while (off < total) {
    off += rx.read(dst.data() + off, std::min(piece, total - off));
    piece = piece % 4099 + 11;
  }
  producer.join();
  EXPECT(src == dst);
  EXPECT(processIsDead(getpid()) == false && processIsDead(0x3ffffff) == true);
}

// On-demand registration among three "ranks" (threads) with a backend that stands in
// for the CUDA layer: allocations are heap blocks, "opening" a handle returns the
// owner's address plus a per-opener offset so that each rank sees its own mapping.
static void testRegCache() {
  struct FakeAlloc { char *base; size_t size; uint64_t id; };
  static std::mutex mu;
  static std::vector<FakeAlloc> allocs;
  static std::atomic<uint64_t> nextId{100};
  static std::atomic<int> opens{0}, closes{0};
  auto backendFor = [](int rank) {
    RegBackend b;
    b.identify = [](const void *p, void **base, size_t *size, uint64_t *id) {
      std::lock_guard<std::mutex> g(mu);
      for (auto &a : allocs)
        if ((const char *)p >= a.base && (const char *)p < a.base + a.size) { *base = a.base; *size = a.size; *id = a.id; return true; }
      return false;
    };
    b.exportHandle = [](void *base, void *handle) {
      std::lock_guard<std::mutex> g(mu);
      for (auto &a : allocs)
        if (a.base == base) {
          if (a.size == 4096) return false; // this size plays the allocation that cannot be exported
          memset(handle, 0, kIpcHandleBytes);
          memcpy(handle, &a.base, sizeof a.base);
          memcpy((char *)handle + 8, &a.id, sizeof a.id);
          return true;
        }
      return false;
    };
    b.open = [rank](const void *handle) -> void * {
      char *base;
      memcpy(&base, handle, sizeof base);
      ++opens;
      return base + ((size_t)(rank + 1) << 40); // a different address in every "process"
    };
    b.close = [](void *) { ++closes; };
    return b;
  };
  auto alloc = [](size_t size) {
    char *p = (char *)malloc(size);
    std::lock_guard<std::mutex> g(mu);
    allocs.push_back({p, size, nextId++});
    return p;
  };
  const int n = 3;
  const uint64_t key = 0xabcdef12345ull ^ (uint64_t)getpid();
  RegCache rc[n];
  for (int r = 0; r < n; ++r) EXPECT(rc[r].start(key, r, n, backendFor(r)) == flagcxSuccess);
  char *x = alloc(1 << 16), *bad = alloc(4096);
  void *va[FLAGCX_MAX_RANKS] = {};
  // rank 1 exports x: ranks 0 and 2 open it, each at its own address; offsets carry over
  EXPECT(rc[1].lookup(x + 256, 1024, va));
  EXPECT(va[1] == x + 256 && va[0] == x + 256 + ((size_t)1 << 40) && va[2] == x + 256 + ((size_t)3 << 40));
  EXPECT(opens.load() == 2);
  EXPECT(rc[1].lookup(x, 1 << 16, va) && opens.load() == 2 && rc[1].counters().hits == 1);
  EXPECT(!rc[1].lookup(x + 100, 1 << 16, va)); // runs past the allocation
  // an allocation that cannot be exported: refused, and the verdict is remembered
  EXPECT(!rc[0].lookup(bad, 16, va) && !rc[0].lookup(bad, 16, va) && rc[0].counters().refused == 1);
  EXPECT(!rc[0].lookup(&key, 8, va)); // not a device allocation at all
  // the address is freed and handed out again under a new id: peers unmap and map anew
  {
    std::lock_guard<std::mutex> g(mu);
    for (auto &a : allocs) if (a.base == x) a.id = nextId++;
  }
  EXPECT(rc[1].lookup(x, 64, va) && rc[1].counters().stale == 1 && opens.load() == 4 && closes.load() == 2);
  // two ranks register at the same time, each serving the other
  std::thread t0([&] { void *v[FLAGCX_MAX_RANKS]; for (int i = 0; i < 50; ++i) { char *p = alloc(8192); EXPECT(rc[0].lookup(p, 8192, v)); } });
  std::thread t2([&] { void *v[FLAGCX_MAX_RANKS]; for (int i = 0; i < 50; ++i) { char *p = alloc(8192); EXPECT(rc[2].lookup(p, 8192, v)); } });
  t0.join();
  t2.join();
  EXPECT(rc[0].counters().exports == 50 && rc[2].counters().exports == 50);
  rc[1].forget(x + 5);
  EXPECT(closes.load() == 4);
  const int openedBefore = opens.load();
  for (int r = 0; r < n; ++r) rc[r].stop();
  EXPECT(closes.load() == openedBefore); // everything a rank opened for its peers is unmapped at stop
  EXPECT(!rc[1].lookup(x, 8, va));       // stopped: nothing is exportable any more
  std::lock_guard<std::mutex> g(mu);
  for (auto &a : allocs) free(a.base);
  allocs.clear();
}

// Two transfer engines in one process (host memory): an owner thread that accepts and
// waits for notifications, an initiator that writes, looks ranges up by address, reads
// back, and provokes the two range errors.  Under the sanitizers this is the check of the
// engine's threads (accept loop, per-connection service thread, requester).
static void testP2pEngine() {
  flagcxP2pEngine_t owner = nullptr, user = nullptr;
  EXPECT(flagcxP2pEngineCreate(-1, &owner) == flagcxSuccess);
  EXPECT(flagcxP2pEngineCreate(-1, &user) == flagcxSuccess);
  if (!owner || !user) return;
  std::vector<unsigned char> mem(1 << 18, 0), src(1 << 18), back(1 << 18, 0);
  for (size_t i = 0; i < src.size(); ++i) src[i] = (unsigned char)(i * 7 + 3);
  flagcxP2pMr_t mr = 0;
  EXPECT(flagcxP2pEngineReg(owner, mem.data(), mem.size(), &mr) == flagcxSuccess);
  flagcxP2pDesc_t whole;
  EXPECT(flagcxP2pEngineMakeDesc(owner, mr, mem.data(), mem.size(), &whole) == flagcxSuccess);
  EXPECT(flagcxP2pEngineMakeDesc(owner, mr, mem.data() + mem.size() - 8, 16, &whole) == flagcxInvalidArgument);
  EXPECT(flagcxP2pEngineMakeDesc(owner, mr, mem.data(), mem.size(), &whole) == flagcxSuccess);
  char meta[128];
  EXPECT(flagcxP2pEngineGetMetadata(owner, meta, sizeof meta) == flagcxSuccess);
  std::atomic<int> ownerOk{0};
  std::thread ownerThread([&] {
    flagcxP2pConn_t c = nullptr;
    if (flagcxP2pEngineAccept(owner, &c, 20000) != flagcxSuccess) return;
    char msg[64];
    size_t len = 0;
    if (flagcxP2pRecvNotif(c, msg, sizeof msg, &len, 20000) == flagcxSuccess && len == 4 && !memcmp(msg, "done", 4) &&
        !memcmp(mem.data(), src.data(), mem.size()))
      ownerOk.store(1);
    flagcxP2pSendNotif(c, "ok", 2);
    // the peer says goodbye by closing; wait for that so that its reads are served
    flagcxResult_t r = flagcxP2pRecvNotif(c, msg, sizeof msg, &len, 20000);
    if (r == flagcxRemoteError) ownerOk.fetch_add(1);
    flagcxP2pConnDestroy(c);
  });
  flagcxP2pConn_t c = nullptr, again = nullptr;
  EXPECT(flagcxP2pEngineGetConn(user, meta, &c) == flagcxSuccess);
  EXPECT(flagcxP2pEngineGetConn(user, meta, &again) == flagcxSuccess && again == c); // cached
  if (c) {
    int local = 0;
    EXPECT(flagcxP2pConnIsLocal(c, &local) == flagcxSuccess && local == 1);
    EXPECT(flagcxP2pWrite(c, src.data(), &whole, src.size(), nullptr) == flagcxSuccess);
    EXPECT(flagcxP2pSendNotif(c, "done", 4) == flagcxSuccess);
    char msg[8];
    size_t len = 0;
    EXPECT(flagcxP2pRecvNotif(c, msg, sizeof msg, &len, 20000) == flagcxSuccess && len == 2);
    flagcxP2pDesc_t part;
    EXPECT(flagcxP2pConnLookup(c, (uint64_t)(uintptr_t)mem.data() + 1000, 5000, &part) == flagcxSuccess);
    EXPECT(flagcxP2pRead(c, back.data(), &part, 5000, nullptr) == flagcxSuccess && !memcmp(back.data(), src.data() + 1000, 5000));
    EXPECT(flagcxP2pRead(c, back.data(), &part, 5001, nullptr) == flagcxInvalidArgument);
    EXPECT(flagcxP2pConnLookup(c, (uint64_t)(uintptr_t)mem.data() + mem.size() - 4, 64, &part) == flagcxInvalidArgument);
    EXPECT(flagcxP2pRecvNotif(c, msg, sizeof msg, &len, 10) == flagcxInProgress);
    EXPECT(flagcxP2pConnDestroy(c) == flagcxSuccess);
  }
  ownerThread.join();
  EXPECT(ownerOk.load() == 2);
  EXPECT(flagcxP2pEngineDereg(owner, mr) == flagcxSuccess);
  EXPECT(flagcxP2pEngineDestroy(user) == flagcxSuccess);
  EXPECT(flagcxP2pEngineDestroy(owner) == flagcxSuccess);
}

int main() {
  testRegCache();
  testShmRing();
  testParams();
  testIfMatcher();
  testAddresses();
  testHalfFloats();
  testRegistry();
  testTuner();
  testHostReduce();
  testSocketAdaptor();
  testBootstrapThreads();
  testCommunicatorsInThreads();
  testP2pEngine();
  printf("%s: %d failure(s)\n", failures ? "FAILED" : "ok", failures);
  return failures;
}
