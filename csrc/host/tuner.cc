// tuner.cc -- see tuner.h.
#include "tuner.h"

#include <algorithm>
#include <cmath>
#include <fstream>
#include <sstream>
#include <vector>

#include "comm.h"

namespace fcx {

// Past about 32 CTAs (512 threads each) a B200 pair gains nothing: 590 GB/s at 32,
// 500-600 at 48 and 96 (all-gather and reduce-scatter of 436 MB), and every extra CTA is
// an SM that a GEMM running beside the collective does not get.
FCX_PARAM(MaxCtas, "MAX_CTAS", 32)
FCX_PARAM(OneShotMaxBytes, "ONESHOT_MAX_BYTES", 0)

int Tuner::bucketOf(size_t bytes) {
  int b = 0;
  while (b < 62 && ((size_t)1 << b) < bytes) ++b;
  return b;
}

static int keyOf(flagcxCommOp_t op, int bucket, bool registered, int elemSize = 0) {
  return elemSize * 100000 + (int)op * 1000 + bucket * 2 + (registered ? 1 : 0);
}
// Only reductions do arithmetic per element; everything else is keyed size-agnostic.
static int elemClass(flagcxCommOp_t op, int elemSize) {
  const bool reduces = op == flagcxCommOpAllReduce || op == flagcxCommOpReduceScatter || op == flagcxCommOpReduce;
  return reduces && elemSize > 0 && elemSize <= 8 ? elemSize : 0;
}

flagcxResult_t Tuner::init(flagcxComm *c) {
  maxCtas = (int)std::max<int64_t>(1, std::min<int64_t>(readParam("MAX_CTAS", paramMaxCtas()), FLAGCX_COLL_BARRIER_SLOTS));
  forcedCtas = (int)readParam("NCTAS", 0);
  forcedAlgo = FLAGCX_ALGO_AUTO;
  {
    const size_t cap = c->layout.llSlotBytes / 2;
    const int64_t ar = readParam("LL_MAX_BYTES", c->nranks <= 2 ? (64 << 10) : c->nranks <= 4 ? (32 << 10) : (16 << 10));
    const int64_t ag = readParam("LL_ALLGATHER_MAX_BYTES", 8 << 10); // per-rank block
    llMaxAllReduce = c->nranks > 1 ? (size_t)std::max<int64_t>(0, std::min<int64_t>(ar, (int64_t)cap)) : 0;
    llMaxAllGather = c->nranks > 1 ? (size_t)std::max<int64_t>(0, std::min<int64_t>(ag, (int64_t)cap)) : 0;
  }
  if (const char *s = getEnv("FLAGCX_ALGO")) {
    static const struct { const char *n; int v; } names[] = {
        {"oneshot", FLAGCX_ALGO_ONESHOT}, {"twoshot", FLAGCX_ALGO_TWOSHOT},
        {"nvls_oneshot", FLAGCX_ALGO_NVLS_ONESHOT}, {"nvls_twoshot", FLAGCX_ALGO_NVLS_TWOSHOT},
        {"push", FLAGCX_ALGO_PUSH}, {"pull", FLAGCX_ALGO_PULL}, {"nvls", FLAGCX_ALGO_NVLS}, {"ll", FLAGCX_ALGO_LL}, {"ring", FLAGCX_ALGO_RING},
        {"copy_engine", FLAGCX_ALGO_COPY_ENGINE}};
    for (auto &e : names)
      if (!strcasecmp(s, e.n)) forcedAlgo = e.v;
  }
  if (const char *f = getEnv("FLAGCX_TUNE_FILE")) {
    if (load(f) == flagcxSuccess) FCX_INFO(SUB_TUNING, "rank %d: loaded %zu tuned entries from %s", c->rank, table.size(), f);
  }
  return flagcxSuccess;
}

TuneChoice Tuner::heuristic(flagcxCommOp_t op, size_t bytes, int nranks, bool registered, bool nvlsOk) const {
  TuneChoice ch;
  size_t work = bytes; // bytes this rank produces or moves
  switch (op) {
    case flagcxCommOpAllReduce: {
      size_t oneShotMax = paramOneShotMaxBytes() > 0 ? (size_t)paramOneShotMaxBytes()
                          : nranks <= 2 ? (8u << 20) : nranks <= 4 ? (512u << 10) : (256u << 10);
      // with two ranks the switch saves no traffic over a plain peer read
      // every rank sends its whole input to every peer in the LL path, so its range shrinks
      // as the world grows
      if (bytes <= llMaxAllReduce) ch.algo = FLAGCX_ALGO_LL;
      else if (nvlsOk && nranks > 2) ch.algo = bytes < (1u << 20) ? FLAGCX_ALGO_NVLS_ONESHOT : FLAGCX_ALGO_NVLS_TWOSHOT;
      else ch.algo = bytes <= oneShotMax ? FLAGCX_ALGO_ONESHOT : FLAGCX_ALGO_TWOSHOT;
      if (ch.algo == FLAGCX_ALGO_TWOSHOT || ch.algo == FLAGCX_ALGO_NVLS_TWOSHOT) work = bytes / std::max(1, nranks);
      break;
    }
    case flagcxCommOpReduceScatter: {
      if (bytes / std::max(1, nranks) <= llMaxAllGather) { ch.algo = FLAGCX_ALGO_LL; break; }
      ch.algo = nvlsOk && nranks > 2 && bytes >= (1u << 20) ? FLAGCX_ALGO_NVLS : FLAGCX_ALGO_PULL;
      work = bytes / std::max(1, nranks);
      // Callers that overlap their collectives with compute (a training framework's
      // gradient reduce-scatter) do better with the copy engines carrying the bytes and a
      // few CTAs adding from local memory: FLAGCX_COPY_ENGINE_MIN_BYTES > 0 asks for that
      // from the given total size on (off by default).
      static const int64_t ceMin = readParam("COPY_ENGINE_MIN_BYTES", 0);
      if (ceMin > 0 && bytes >= (size_t)ceMin && nranks > 1) {
        ch.algo = FLAGCX_ALGO_COPY_ENGINE;
        ch.nCtas = std::min(16, maxCtas);
        return ch;
      }
      break;
    }
    case flagcxCommOpAllGather:
      if (bytes / std::max(1, nranks) <= llMaxAllGather) { ch.algo = FLAGCX_ALGO_LL; break; }
      ch.algo = FLAGCX_ALGO_PUSH;
      break;
    case flagcxCommOpAlltoAll:
      if (bytes / std::max(1, nranks) <= llMaxAllGather) { ch.algo = FLAGCX_ALGO_LL; break; }
      ch.algo = FLAGCX_ALGO_PUSH;
      break;
    case flagcxCommOpBroadcast:
      ch.algo = FLAGCX_ALGO_PUSH; // the launcher falls back to pull when the output is not registered
      break;
    default:
      ch.algo = FLAGCX_ALGO_PULL;
      break;
  }
  (void)registered;
  // work per CTA below which another CTA costs more (its barrier flags on every peer)
  // than it brings; the offline tuner on B200 pairs picked 8 CTAs for 1-2 MiB
  // (FLAGCX_BYTES_PER_CTA is that figure for a pair).  With more ranks a CTA's work splits
  // into n-1 streams and the tuner wants more CTAs for the same bytes: 16-64 CTAs for a
  // 1-8 MiB all-reduce or reduce-scatter on eight B200s, i.e. about 16 KiB each.
  static const size_t perCtaPair = (size_t)std::max<int64_t>(1024, readParam("BYTES_PER_CTA", 64 << 10));
  const size_t perCta = std::max<size_t>(8 << 10, perCtaPair * 2 / (size_t)std::max(2, nranks));
  // all-to-all moves n separate streams per CTA and keeps gaining up to about 96 CTAs
  // (365 GB/s at 32, 616 at 96 on a B200 pair, 1 GiB); everything else is flat beyond 32
  size_t cap = op == flagcxCommOpAlltoAll && work >= (16u << 20)
                   ? std::min<size_t>(3 * (size_t)maxCtas, FLAGCX_COLL_BARRIER_SLOTS)
                   : (size_t)maxCtas;
  ch.nCtas = (int)std::max<size_t>(1, std::min<size_t>((work + perCta - 1) / perCta, cap));
  return ch;
}

TuneChoice Tuner::choose(flagcxCommOp_t op, size_t bytes, int nranks, bool registered, bool nvlsOk, int elemSize) const {
  TuneChoice ch = heuristic(op, bytes, nranks, registered, nvlsOk);
  const int bucket = bucketOf(bytes);
  auto it = table.find(keyOf(op, bucket, registered, elemClass(op, elemSize)));
  if (it == table.end()) it = table.find(keyOf(op, bucket, registered, 0));
  for (int es = 1; it == table.end() && es <= 8; es *= 2) it = table.find(keyOf(op, bucket, registered, es));
  if (it != table.end()) {
    bool needsNvls = it->second.algo == FLAGCX_ALGO_NVLS_ONESHOT || it->second.algo == FLAGCX_ALGO_NVLS_TWOSHOT ||
                     it->second.algo == FLAGCX_ALGO_NVLS;
    if (!needsNvls || nvlsOk) ch = it->second;
  }
  if (forcedAlgo != FLAGCX_ALGO_AUTO) ch.algo = forcedAlgo;
  if (forcedCtas > 0) ch.nCtas = forcedCtas;
  return ch;
}

// ---------------------------------------------------------------------------
// persistence
// ---------------------------------------------------------------------------
std::string Tuner::toJson() const {
  std::ostringstream o;
  o << "{\n  \"version\": 1,\n  \"entries\": [\n";
  bool firstEntry = true;
  for (auto &kv : table) {
    int es = kv.first / 100000, op = kv.first % 100000 / 1000, rest = kv.first % 1000;
    if (!firstEntry) o << ",\n";
    firstEntry = false;
    o << "    {\"op\": " << op << ", \"elem_size\": " << es << ", \"bucket\": " << rest / 2 << ", \"registered\": " << rest % 2
      << ", \"algo\": " << kv.second.algo << ", \"nctas\": " << kv.second.nCtas << ", \"usec\": " << kv.second.usec
      << ", \"best_usec\": " << kv.second.bestUsec << "}";
  }
  o << "\n  ]\n}\n";
  return o.str();
}

flagcxResult_t Tuner::fromJson(const std::string &text) {
  size_t pos = text.find("\"entries\"");
  if (pos == std::string::npos) return flagcxInvalidArgument;
  std::map<int, TuneChoice> parsed;
  while ((pos = text.find('{', pos)) != std::string::npos) {
    size_t end = text.find('}', pos);
    if (end == std::string::npos) return flagcxInvalidArgument;
    std::string obj = text.substr(pos + 1, end - pos - 1);
    auto field = [&](const char *name, double dflt) {
      std::string k = std::string("\"") + name + "\"";
      size_t p = obj.find(k);
      if (p == std::string::npos) return dflt;
      p = obj.find(':', p);
      return p == std::string::npos ? dflt : atof(obj.c_str() + p + 1);
    };
    int op = (int)field("op", -1), bucket = (int)field("bucket", -1), reg = (int)field("registered", 0);
    int es = (int)field("elem_size", 0); // absent in tables written before the key had it
    TuneChoice ch;
    ch.algo = (int)field("algo", -1);
    ch.nCtas = (int)field("nctas", 0);
    ch.usec = (float)field("usec", 0);
    ch.bestUsec = (float)field("best_usec", 0);
    if (op < 0 || op >= flagcxNumCommOps || bucket < 0 || bucket > 62 || ch.algo < 0 || ch.algo >= FLAGCX_ALGO_COUNT ||
        ch.nCtas < 1 || ch.nCtas > FLAGCX_COLL_BARRIER_SLOTS || es < 0 || es > 8)
      return flagcxInvalidArgument;
    parsed[keyOf((flagcxCommOp_t)op, bucket, reg != 0, es)] = ch;
    pos = end + 1;
  }
  table = parsed;
  return flagcxSuccess;
}

flagcxResult_t Tuner::save(const char *path) const {
  std::ofstream f(path);
  if (!f) { FCX_WARN("cannot write %s", path); return flagcxSystemError; }
  f << toJson();
  return flagcxSuccess;
}

flagcxResult_t Tuner::load(const char *path) {
  std::ifstream f(path);
  if (!f) return flagcxSystemError;
  std::stringstream ss;
  ss << f.rdbuf();
  flagcxResult_t r = fromJson(ss.str());
  if (r != flagcxSuccess) FCX_WARN("tune file %s is malformed; ignoring it", path);
  return r;
}

// ---------------------------------------------------------------------------
// measurement
// ---------------------------------------------------------------------------
namespace {

struct Candidate { int algo, nCtas; };

std::vector<Candidate> candidatesFor(flagcxCommOp_t op, size_t bytes, int n, bool registered, bool nvls, int maxCtas,
                                     size_t llCap) {
  std::vector<int> algos;
  switch (op) {
    case flagcxCommOpAllReduce:
      if (bytes <= (16u << 20)) algos.push_back(FLAGCX_ALGO_ONESHOT);
      algos.push_back(FLAGCX_ALGO_TWOSHOT);
      if (nvls) {
        if (bytes <= (16u << 20)) algos.push_back(FLAGCX_ALGO_NVLS_ONESHOT);
        algos.push_back(FLAGCX_ALGO_NVLS_TWOSHOT);
      }
      if (bytes >= (1u << 20)) algos.push_back(FLAGCX_ALGO_RING);
      break;
    case flagcxCommOpReduceScatter:
      algos.push_back(FLAGCX_ALGO_PULL);
      if (bytes >= (1u << 20)) algos.push_back(FLAGCX_ALGO_RING);
      if (nvls && registered) algos.push_back(FLAGCX_ALGO_NVLS);
      break;
    case flagcxCommOpAllGather:
      if (registered) algos.push_back(FLAGCX_ALGO_PUSH);
      algos.push_back(FLAGCX_ALGO_PULL);
      if (registered && bytes >= (1u << 20)) algos.push_back(FLAGCX_ALGO_RING);
      if (nvls && registered) algos.push_back(FLAGCX_ALGO_NVLS);
      break;
    case flagcxCommOpAlltoAll:
      if (registered) algos.push_back(FLAGCX_ALGO_PUSH);
      algos.push_back(FLAGCX_ALGO_PULL);
      break;
    default: algos.push_back(FLAGCX_ALGO_PULL); break;
  }
  std::vector<Candidate> out;
  for (int a : algos)
    for (int ctas : {1, 2, 4, 8, 16, 32, 64, 96, 128}) {
      if (ctas > maxCtas && ctas != 1) continue;
      // more CTAs than 4 KiB pieces of work only adds barrier traffic
      if (ctas > 1 && (size_t)ctas * 4096 > bytes) continue;
      out.push_back({a, ctas});
    }
  // the copy engines move the data: no CTA count to choose
  if (n > 1 && op == flagcxCommOpAllGather && registered && bytes >= (1u << 20)) out.push_back({FLAGCX_ALGO_COPY_ENGINE, 1});
  // reduce-scatter: copy engines for the transport, then a local reduce with `ctas` CTAs
  if (n > 1 && op == flagcxCommOpReduceScatter && bytes >= (1u << 20))
    for (int ctas : {8, 16, 32})
      if (ctas <= maxCtas) out.push_back({FLAGCX_ALGO_COPY_ENGINE, ctas});
  // the barrier-free path picks its own CTA count
  if (n > 1 && ((op == flagcxCommOpAllReduce && bytes <= llCap) ||
                ((op == flagcxCommOpAllGather || op == flagcxCommOpReduceScatter || op == flagcxCommOpAlltoAll) &&
                 bytes / n <= llCap)))
    out.push_back({FLAGCX_ALGO_LL, 1});
  return out;
}

} // namespace

flagcxResult_t Tuner::tune(flagcxComm *c, flagcxCommOp_t op, flagcxDataType_t dtype, size_t minBytes,
                           size_t maxBytes, int iters) {
  if (!c->devicePath || c->emu) return flagcxNotSupported;
  if (op != flagcxCommOpAllReduce && op != flagcxCommOpAllGather && op != flagcxCommOpReduceScatter &&
      op != flagcxCommOpAlltoAll)
    return flagcxNotSupported;
  const int n = c->nranks;
  const size_t es = getFlagcxDataTypeSize(dtype);
  if (es == 0 || minBytes == 0 || maxBytes < minBytes) return flagcxInvalidArgument;
  iters = std::max(iters, 3);
  const int tuneMaxCtas = (int)std::min<int64_t>(readParam("TUNE_MAX_CTAS", 128), FLAGCX_COLL_BARRIER_SLOTS);

  // registered pair and unregistered pair of scratch buffers
  cu::VmmBlock sb, rb;
  FCXCHECK(cu::vmmAlloc(maxBytes, c->cudaDev, &sb));
  FCXCHECK(cu::vmmAlloc(maxBytes, c->cudaDev, &rb));
  Window *ws = nullptr, *wr = nullptr;
  FCXCHECK(windowRegister(c, sb.ptr, sb.size, FLAGCX_WIN_COLL_SYMMETRIC, &ws));
  FCXCHECK(windowRegister(c, rb.ptr, rb.size, FLAGCX_WIN_COLL_SYMMETRIC, &wr));
  void *us = nullptr, *ur = nullptr;
  FCX_CUDACHECK(cudaMalloc(&us, maxBytes));
  FCX_CUDACHECK(cudaMalloc(&ur, maxBytes));
  FCX_CUDACHECK(cudaMemset(sb.ptr, 0, maxBytes));
  FCX_CUDACHECK(cudaMemset(us, 0, maxBytes));
  cudaEvent_t e0, e1;
  FCX_CUDACHECK(cudaEventCreate(&e0));
  FCX_CUDACHECK(cudaEventCreate(&e1));
  cudaStream_t stream = c->internalStream;
  const int savedForcedAlgo = forcedAlgo, savedForcedCtas = forcedCtas;
  forcedAlgo = FLAGCX_ALGO_AUTO;
  forcedCtas = 0;
  flagcxResult_t res = flagcxSuccess;

  for (size_t bytes = minBytes; bytes <= maxBytes && res == flagcxSuccess; bytes *= 2) {
    for (int registered = 1; registered >= 0 && res == flagcxSuccess; --registered) {
      DeviceCollRequest rq{};
      rq.op = op;
      rq.dtype = dtype;
      rq.redOp = flagcxSum;
      rq.root = 0;
      rq.send = registered ? sb.ptr : us;
      rq.recv = registered ? rb.ptr : ur;
      size_t elems = bytes / es;
      rq.count = (op == flagcxCommOpAllReduce) ? elems : std::max<size_t>(1, elems / n);
      const bool nvlsOk = c->nvls && registered && ws->mc && wr->mc && (rq.count * es) % 16 == 0;
      TuneChoice base = heuristic(op, bytes, n, registered, nvlsOk);
      auto cands = candidatesFor(op, bytes, n, registered, nvlsOk, tuneMaxCtas, c->layout.llSlotBytes / 2);
      cands.push_back({base.algo, base.nCtas});
      float bestUs = 0, baseUs = 0;
      Candidate best{base.algo, base.nCtas};
      for (size_t ci = 0; ci < cands.size() && res == flagcxSuccess; ++ci) {
        rq.algo = cands[ci].algo;
        rq.nCtas = cands[ci].nCtas;
        for (int w = 0; w < 2 && res == flagcxSuccess; ++w) res = deviceCollective(c, rq, stream);
        if (res != flagcxSuccess) break;
        cudaEventRecord(e0, stream);
        for (int i = 0; i < iters && res == flagcxSuccess; ++i) res = deviceCollective(c, rq, stream);
        cudaEventRecord(e1, stream);
        if (cudaEventSynchronize(e1) != cudaSuccess) { res = flagcxUnhandledDeviceError; break; }
        float ms = 0;
        cudaEventElapsedTime(&ms, e0, e1);
        std::vector<float> all(n, 0.f);
        all[c->rank] = ms * 1000.f / iters;
        res = c->bootstrap->allGather(all.data(), sizeof(float));
        if (res != flagcxSuccess) break;
        float us = *std::max_element(all.begin(), all.end());
        if (ci + 1 == cands.size()) baseUs = us;
        if (bestUs == 0 || us < bestUs) { bestUs = us; best = cands[ci]; }
        if (commCheckDevice(c) != flagcxSuccess) res = flagcxRemoteError;
      }
      if (res != flagcxSuccess) break;
      TuneChoice ch;
      if (baseUs > 0 && bestUs >= 0.95f * baseUs) { ch = base; ch.usec = baseUs; } // hysteresis
      else { ch.algo = best.algo; ch.nCtas = best.nCtas; ch.usec = bestUs; }
      ch.bestUsec = bestUs;
      table[keyOf(op, bucketOf(bytes), registered != 0, elemClass(op, (int)getFlagcxDataTypeSize(dtype)))] = ch;
      if (c->rank == 0)
        FCX_INFO(SUB_TUNING, "%s %zu B %s: algo %d ctas %d %.1f us (heuristic %.1f us)", commOpName(op), bytes,
                 registered ? "registered" : "staged", ch.algo, ch.nCtas, ch.usec, baseUs);
    }
  }
  forcedAlgo = savedForcedAlgo;
  forcedCtas = savedForcedCtas;
  cudaStreamSynchronize(stream);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  c->bootstrap->barrier();
  windowDeregister(c, ws);
  windowDeregister(c, wr);
  cu::vmmFree(&sb);
  cu::vmmFree(&rb);
  cudaFree(us);
  cudaFree(ur);
  return res;
}

} // namespace fcx
