// trace.cc -- see trace.h.
#include "trace.h"

#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <cstdio>

#include "base.h"
#include "comm.h"

namespace fcx {

Trace::~Trace() { enable(0); }

void Trace::enable(int capacity) {
  std::lock_guard<std::mutex> lk(mu_);
  for (auto &r : ring_) {
    if (r.e0) cudaEventDestroy(r.e0);
    if (r.e1) cudaEventDestroy(r.e1);
  }
  ring_.clear();
  capacity_ = capacity > 0 ? capacity : 0;
  ring_.resize((size_t)capacity_);
  next_ = 0;
}

int Trace::begin(flagcxComm *c, flagcxCommOp_t op, size_t bytes, int route, cudaStream_t stream) {
  if (capacity_ <= 0) return -1;
  std::lock_guard<std::mutex> lk(mu_);
  const int slot = (int)(next_ % (uint64_t)capacity_);
  TraceRecord &r = ring_[slot];
  r.seq = next_++;
  r.op = (int)op;
  r.bytes = bytes;
  r.route = route;
  r.algo = -1;
  r.nCtas = 0;
  r.deviceMs = 0.f;
  r.timed = false;
  r.hostEndNs = 0;
  // the emulated world launches when its last rank submits, outside this bracket
  if (route == 0 && c->devicePath && !c->emu) {
    if (!r.e0) cudaEventCreate(&r.e0);
    if (!r.e1) cudaEventCreate(&r.e1);
    if (r.e0 && r.e1 && cudaEventRecord(r.e0, stream) == cudaSuccess) r.timed = true;
  }
  r.hostStartNs = nowNs();
  return slot;
}

void Trace::end(flagcxComm *c, int slot, cudaStream_t stream) {
  if (slot < 0) return;
  std::lock_guard<std::mutex> lk(mu_);
  if (slot >= capacity_) return;
  TraceRecord &r = ring_[slot];
  r.hostEndNs = nowNs();
  if (r.timed && cudaEventRecord(r.e1, stream) != cudaSuccess) r.timed = false;
  const OpStats &s = c->stats[r.op];
  r.algo = s.lastAlgo;
  r.nCtas = s.lastCtas;
}

void Trace::resolve(flagcxComm *c) {
  std::lock_guard<std::mutex> lk(mu_);
  for (auto &r : ring_) {
    if (!r.timed || r.hostEndNs == 0) continue;
    if (cudaEventSynchronize(r.e1) != cudaSuccess) continue;
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.e0, r.e1) == cudaSuccess) {
      r.deviceMs = ms;
      // newest record of each op wins
      bool newest = true;
      for (auto &o : ring_)
        if (o.op == r.op && o.timed && o.hostEndNs && o.seq > r.seq) newest = false;
      if (newest) c->stats[r.op].lastMs = ms;
    }
  }
}

flagcxResult_t Trace::dump(flagcxComm *c, const char *path) {
  if (!path) return flagcxInvalidArgument;
  resolve(c);
  std::lock_guard<std::mutex> lk(mu_);
  FILE *f = fopen(path, "w");
  if (!f) { FCX_WARN("trace: cannot open %s", path); return flagcxSystemError; }
  static const char *routes[] = {"device", "host", "staged"};
  fprintf(f, "{\"rank\": %d, \"nranks\": %d, \"records\": [", c->rank, c->nranks);
  // oldest first
  std::vector<const TraceRecord *> order;
  for (auto &r : ring_)
    if (r.hostEndNs) order.push_back(&r);
  std::sort(order.begin(), order.end(), [](const TraceRecord *a, const TraceRecord *b) { return a->seq < b->seq; });
  bool first = true;
  for (const TraceRecord *r : order) {
    fprintf(f, "%s\n {\"seq\": %llu, \"op\": \"%s\", \"bytes\": %zu, \"route\": \"%s\", \"algo\": %d, \"ctas\": %d, "
               "\"host_us\": %.1f, \"device_ms\": %.4f}",
            first ? "" : ",", (unsigned long long)r->seq, commOpName((flagcxCommOp_t)r->op), r->bytes,
            routes[r->route < 0 || r->route > 2 ? 0 : r->route], r->algo, r->nCtas,
            (double)(r->hostEndNs - r->hostStartNs) / 1e3, r->timed ? r->deviceMs : 0.0);
    first = false;
  }
  fprintf(f, "\n]}\n");
  fclose(f);
  return flagcxSuccess;
}

static bool nvtxOn() {
  static const bool on = readParam("NVTX", 0) != 0;
  return on;
}
void nvtxPush(const char *name) {
  if (nvtxOn()) nvtxRangePushA(name);
}
void nvtxPop() {
  if (nvtxOn()) nvtxRangePop();
}

} // namespace fcx
