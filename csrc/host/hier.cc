// hier.cc -- two-level collectives for communicators whose ranks do not all share one
// NVLink domain: several machines, or one machine that FLAGCX_HOSTID splits into
// several "nodes".  Inside each node the ranks form a child communicator and run the
// NVLink kernels; between nodes, rank k of one node talks to rank k of every other node
// (a "rail") over the host network.
//
// Plays the role of the FlagCX hybrid runner and its cluster-to-cluster planner
// (flagcx/runner/hybrid_runner.cc:124-151, flagcx/runner/c2c_algo.cc:1474, :2268 in the
// FlagCX project) for the two operations that dominate training traffic:
//
//   all-reduce   intra-node all-reduce (device kernel); every rail sums its 1/L slice
//                across the nodes (pinned host memory + sockets); intra-node all-gather
//                of the finished slices (device kernel);
//   all-gather   every rank swaps its block with its rail peers over the host network;
//                one intra-node all-gather per node puts the blocks in place.
//
// Other operations on such communicators keep the flat route (device buffer -> pinned
// host memory -> socket collective -> device buffer).  Nodes must have equally many
// ranks, numbered contiguously (ranks [i*L, (i+1)*L) form node i).
#include <algorithm>
#include <map>

#include "comm.h"

namespace fcx {

flagcxResult_t ensureHostNet(flagcxComm *c); // api.cc

namespace {

constexpr int kTagHierId = 0x48494552; // "HIER"

flagcxResult_t growPinned(flagcxComm *c, size_t bytes) {
  if (c->hierPinnedBytes >= bytes) return flagcxSuccess;
  if (c->hierPinned) cudaFreeHost(c->hierPinned);
  c->hierPinned = nullptr;
  c->hierPinnedBytes = 0;
  const size_t want = alignUp(std::max(bytes, (size_t)1 << 20), 1 << 20);
  FCX_CUDACHECK(cudaHostAlloc(&c->hierPinned, want, cudaHostAllocDefault));
  c->hierPinnedBytes = want;
  return flagcxSuccess;
}

flagcxResult_t growDevice(flagcxComm *c, size_t bytes) {
  if (c->hierDevBytes >= bytes) return flagcxSuccess;
  if (c->hierDev) {
    FCX_CUDACHECK(cudaDeviceSynchronize());
    FCX_CUDACHECK(cudaFree(c->hierDev));
  }
  c->hierDev = nullptr;
  c->hierDevBytes = 0;
  const size_t want = alignUp(std::max(bytes, (size_t)1 << 20), 1 << 20);
  FCX_CUDACHECK(cudaMalloc(&c->hierDev, want));
  c->hierDevBytes = want;
  return flagcxSuccess;
}

flagcxResult_t intraCollective(flagcxComm *c, flagcxCommOp_t op, const void *send, void *recv, size_t count,
                               flagcxDataType_t dt, flagcxRedOp_t red, int root, cudaStream_t stream) {
  DeviceCollRequest rq{op, send, recv, count, dt, red, root};
  return deviceCollective(c->intra, rq, stream);
}

} // namespace

// Called by commCreate on every rank once it is known that the ranks cannot all reach
// each other over NVLink.  hostHashes[r] identifies rank r's node; hasGpu[r] says whether
// it has a device.  Leaves c->intra null when the shape does not fit.
flagcxResult_t hierSetup(flagcxComm *c, const std::vector<uint64_t> &hostHashes, const std::vector<int> &hasGpu) {
  const int n = c->nranks;
  if (readParam("HIERARCHICAL", 1) == 0 || getEnv("FLAGCX_COMM_ID")) return flagcxSuccess;
  std::map<uint64_t, int> nodeIdx;
  std::vector<int> nodeOf(n), sizeOf;
  bool fits = true;
  for (int r = 0; r < n; ++r) {
    auto it = nodeIdx.find(hostHashes[r]);
    if (it == nodeIdx.end()) {
      it = nodeIdx.emplace(hostHashes[r], (int)sizeOf.size()).first;
      sizeOf.push_back(0);
    }
    nodeOf[r] = it->second;
    sizeOf[it->second]++;
    fits &= hasGpu[r] != 0;
  }
  const int m = (int)sizeOf.size();
  const int L = sizeOf[0];
  for (int s : sizeOf) fits &= s == L;
  for (int r = 0; r < n && fits; ++r) fits &= nodeOf[r] == r / L; // contiguous numbering
  fits &= m > 1 && L <= FLAGCX_MAX_RANKS;
  if (!fits) return flagcxSuccess;

  const int node = c->rank / L, k = c->rank % L, leader = node * L;
  flagcxUniqueId id;
  memset(&id, 0, sizeof id);
  if (k == 0) {
    FCXCHECK(bootstrapCreateId(&id));
    for (int p = 1; p < L; ++p) FCXCHECK(c->bootstrap->send(leader + p, kTagHierId, &id, sizeof id));
  } else {
    FCXCHECK(c->bootstrap->recv(leader, kTagHierId, &id, sizeof id));
  }
  flagcxComm *child = nullptr;
  flagcxResult_t r = commCreate(&child, L, id, k);
  // every rank of the big communicator must agree, or the nodes would take different routes
  std::vector<int32_t> ok(n, 0);
  ok[c->rank] = r == flagcxSuccess && child && child->devicePath;
  FCXCHECK(c->bootstrap->allGather(ok.data(), sizeof(int32_t)));
  bool all = true;
  for (int v : ok) all &= v != 0;
  if (!all) {
    if (child) commDestroy(child);
    FCX_INFO(SUB_INIT, "rank %d: no two-level route (a node has no NVLink path among its ranks)", c->rank);
    return flagcxSuccess;
  }
  c->intra = child;
  c->nNodes = m;
  c->nodeRanks = L;
  FCX_INFO(SUB_INIT, "rank %d: two-level route, %d nodes x %d ranks (NVLink inside a node, host network between)",
           c->rank, m, L);
  return flagcxSuccess;
}

void hierTeardown(flagcxComm *c) {
  if (c->intra) { commDestroy(c->intra); c->intra = nullptr; }
  if (c->hierPinned) { cudaFreeHost(c->hierPinned); c->hierPinned = nullptr; }
  if (c->hierDev) { cudaFree(c->hierDev); c->hierDev = nullptr; }
}

flagcxResult_t hierAllReduce(flagcxComm *c, const void *send, void *recv, size_t count, flagcxDataType_t dt,
                             flagcxRedOp_t op, cudaStream_t stream) {
  const int L = c->nodeRanks, m = c->nNodes, node = c->rank / L, k = c->rank % L;
  const size_t es = getFlagcxDataTypeSize(dt);
  const flagcxRedOp_t inner = op == flagcxAvg ? flagcxSum : op;
  // 1. node-level result on every rank of the node
  FCXCHECK(intraCollective(c, flagcxCommOpAllReduce, send, recv, count, dt, inner, 0, stream));
  // 2. rail k owns slice k; rail 0 also owns what is left over after L equal slices
  const size_t base = count / (size_t)L / 8 * 8, tailBegin = base * (size_t)L, tail = count - tailBegin;
  struct Piece { size_t begin, elems; };
  std::vector<Piece> mine;
  if (base) mine.push_back({base * (size_t)k, base});
  if (k == 0 && tail) mine.push_back({tailBegin, tail});
  size_t myElems = 0;
  for (auto &p : mine) myElems += p.elems;
  if (myElems) {
    FCXCHECK(growPinned(c, myElems * es * (size_t)m));
    FCXCHECK(ensureHostNet(c));
    char *own = (char *)c->hierPinned, *theirs = own + myElems * es;
    size_t off = 0;
    for (auto &p : mine) {
      FCX_CUDACHECK(cudaMemcpyAsync(own + off, (char *)recv + p.begin * es, p.elems * es, cudaMemcpyDeviceToHost, stream));
      off += p.elems * es;
    }
    FCX_CUDACHECK(cudaStreamSynchronize(stream));
    std::vector<HostNet::Op> ops;
    int slot = 0;
    for (int j = 0; j < m; ++j) {
      if (j == node) continue;
      ops.push_back({true, j * L + k, own, myElems * es});
      ops.push_back({false, j * L + k, theirs + (size_t)slot++ * myElems * es, myElems * es});
    }
    FCXCHECK(c->hostNet->run(ops));
    // sum in node order so that every node computes bit-identical results
    std::vector<char> acc(myElems * es);
    slot = 0;
    bool first = true;
    for (int j = 0; j < m; ++j) {
      const char *src = j == node ? own : theirs + (size_t)slot++ * myElems * es;
      if (first) { memcpy(acc.data(), src, myElems * es); first = false; }
      else FCXCHECK(hostReduce(acc.data(), src, myElems, dt, inner));
    }
    if (op == flagcxAvg) FCXCHECK(hostDivide(acc.data(), myElems, dt, c->nranks));
    memcpy(own, acc.data(), myElems * es);
    off = 0;
    for (auto &p : mine) {
      FCX_CUDACHECK(cudaMemcpyAsync((char *)recv + p.begin * es, own + off, p.elems * es, cudaMemcpyHostToDevice, stream));
      off += p.elems * es;
    }
  }
  // 3. the finished slices back to every rank of the node
  if (base)
    FCXCHECK(intraCollective(c, flagcxCommOpAllGather, (char *)recv + base * (size_t)k * es, recv, base, dt, flagcxSum, 0, stream));
  if (tail)
    FCXCHECK(intraCollective(c, flagcxCommOpBroadcast, (char *)recv + tailBegin * es, (char *)recv + tailBegin * es, tail, dt,
                             flagcxSum, 0, stream));
  // the pinned buffer is reused by the next call
  FCX_CUDACHECK(cudaStreamSynchronize(stream));
  return flagcxSuccess;
}

flagcxResult_t hierAllGather(flagcxComm *c, const void *send, void *recv, size_t count, flagcxDataType_t dt,
                             cudaStream_t stream) {
  const int L = c->nodeRanks, m = c->nNodes, node = c->rank / L, k = c->rank % L;
  const size_t blk = count * getFlagcxDataTypeSize(dt);
  if (blk == 0) return flagcxSuccess;
  // A. my block to my rail peers, theirs into a device scratch (one slot per node)
  FCXCHECK(growPinned(c, blk * (size_t)m));
  FCXCHECK(growDevice(c, blk * (size_t)m));
  FCXCHECK(ensureHostNet(c));
  char *own = (char *)c->hierPinned;
  FCX_CUDACHECK(cudaMemcpyAsync(own + (size_t)node * blk, send, blk, cudaMemcpyDeviceToHost, stream));
  FCX_CUDACHECK(cudaStreamSynchronize(stream));
  std::vector<HostNet::Op> ops;
  for (int j = 0; j < m; ++j) {
    if (j == node) continue;
    ops.push_back({true, j * L + k, own + (size_t)node * blk, blk});
    ops.push_back({false, j * L + k, own + (size_t)j * blk, blk});
  }
  FCXCHECK(c->hostNet->run(ops));
  for (int j = 0; j < m; ++j)
    if (j != node)
      FCX_CUDACHECK(cudaMemcpyAsync((char *)c->hierDev + (size_t)j * blk, own + (size_t)j * blk, blk, cudaMemcpyHostToDevice, stream));
  // B. one node-level all-gather per node: blocks (j, 0..L-1) land at recv[(j*L + .) * blk]
  for (int j = 0; j < m; ++j) {
    const void *in = j == node ? send : (const void *)((char *)c->hierDev + (size_t)j * blk);
    FCXCHECK(intraCollective(c, flagcxCommOpAllGather, in, (char *)recv + (size_t)j * L * blk, count, dt, flagcxSum, 0, stream));
  }
  FCX_CUDACHECK(cudaStreamSynchronize(stream));
  return flagcxSuccess;
}

} // namespace fcx
