// process_group_flagcx.cpp -- torch.distributed backend "flagcx".
//
// A c10d::Backend whose every operation is a call into libflagcx: CUDA tensors run
// as NVLink kernels on a dedicated communication stream (ordered after the caller's
// current stream by an event, and the returned Work orders the caller's stream
// after the collective), CPU tensors run over sockets.  The unique id travels
// through the c10d Store.  Same operation list as the FlagCX torch plugin
// (plugin/torch/flagcx/src/backend_flagcx.cpp:656-1437 in the FlagCX project):
// allreduce(+coalesced), broadcast, reduce, allgather(+base, +coalesced),
// reduce_scatter(+base, +coalesced), alltoall(+base with splits), gather, scatter,
// send, recv, barrier, coalescing.
#include <ATen/cuda/CUDAContext.h>
#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>
#include <torch/extension.h>
#include <pybind11/chrono.h>

#include <atomic>
#include <cstdlib>
#include <memory>
#include <mutex>
#include <optional>
#include <set>

#include "flagcx.h"
#include "flagcx_ext.h"

struct flagcxStream {
  cudaStream_t base;
};

namespace {

#define FCX_TORCH_CHECK(call, comm)                                                     \
  do {                                                                                  \
    flagcxResult_t r__ = (call);                                                        \
    TORCH_CHECK(r__ == flagcxSuccess, "flagcx: ", #call, " failed: ",                   \
                flagcxGetErrorString(r__), " (", flagcxGetLastError(comm), ")");        \
  } while (0)

flagcxDataType_t toFlagcxType(at::ScalarType t) {
  switch (t) {
    case at::kChar: return flagcxInt8;
    case at::kByte: return flagcxUint8;
    case at::kBool: return flagcxUint8;
    case at::kInt: return flagcxInt32;
    case at::kLong: return flagcxInt64;
    case at::kHalf: return flagcxHalf;
    case at::kFloat: return flagcxFloat;
    case at::kDouble: return flagcxDouble;
    case at::kBFloat16: return flagcxBfloat16;
    case at::kFloat8_e4m3fn:
    case at::kFloat8_e5m2: return flagcxUint8; // moved as bytes; not reducible
    default: TORCH_CHECK(false, "flagcx: unsupported tensor dtype ", t);
  }
}

flagcxRedOp_t toFlagcxOp(const c10d::ReduceOp &op, at::ScalarType t) {
  if (t == at::kBool) {
    // bool travels as uint8: a sum would wrap at 256 ranks' worth of ones and, worse,
    // yield values other than 0/1.  Sum is a logical or (max), product a logical and (min).
    switch (op) {
      case c10d::ReduceOp::SUM:
      case c10d::ReduceOp::MAX: return flagcxMax;
      case c10d::ReduceOp::PRODUCT:
      case c10d::ReduceOp::MIN: return flagcxMin;
      default: TORCH_CHECK(false, "flagcx: this reduce op is not defined for bool tensors");
    }
  }
  switch (op) {
    case c10d::ReduceOp::SUM: return flagcxSum;
    case c10d::ReduceOp::PRODUCT: return flagcxProd;
    case c10d::ReduceOp::MAX: return flagcxMax;
    case c10d::ReduceOp::MIN: return flagcxMin;
    case c10d::ReduceOp::AVG: return flagcxAvg;
    default: TORCH_CHECK(false, "flagcx: unsupported reduce op for dtype ", t);
  }
}

class WorkFlagCX : public c10d::Work {
 public:
  WorkFlagCX(c10d::OpType op, std::optional<at::Device> dev) : c10d::Work(-1, op), device_(dev) {
    if (dev && dev->is_cuda()) event_ = std::make_unique<at::cuda::CUDAEvent>(cudaEventDisableTiming);
  }
  bool isCompleted() override { return !event_ || event_->query(); }
  bool isSuccess() const override { return true; }
  bool wait(std::chrono::milliseconds = kNoTimeout) override {
    // stream semantics, like the NCCL backend: the caller's stream waits, the host does not
    if (event_) event_->block(at::cuda::getCurrentCUDAStream(device_->index()));
    return true;
  }
  void synchronize() override { wait(); }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }
  std::vector<at::Tensor> result() override { return outputs_; }

  std::optional<at::Device> device_;
  std::unique_ptr<at::cuda::CUDAEvent> event_;
  std::vector<at::Tensor> outputs_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
};

// Communicators that must hear about segments the caching allocator hands back to the
// driver: an allocation that peers have mapped (on-demand export of user buffers) has to
// be unmapped there before it is freed.  The allocator calls its trace trackers right
// before cudaFree of a segment, under its own lock; the callback below only talks to the
// peers' registration threads over a socket and calls nothing of torch.
std::mutex gLiveMu;
std::set<std::pair<flagcxComm_t, int>> gLiveComms; // (communicator, CUDA device)

void followAllocator(flagcxComm_t comm, int device) {
  static std::once_flag once;
  std::call_once(once, [] {
    c10::cuda::CUDACachingAllocator::attachAllocatorTraceTracker([](const c10::cuda::CUDACachingAllocator::TraceEntry &te) {
      if (te.action_ != c10::cuda::CUDACachingAllocator::TraceEntry::SEGMENT_FREE) return;
      std::lock_guard<std::mutex> g(gLiveMu);
      for (auto &cd : gLiveComms)
        if (cd.second == (int)te.device_) flagcxCommForgetUserBuffer(cd.first, (const void *)te.addr_);
    });
  });
  {
    std::lock_guard<std::mutex> g(gLiveMu);
    gLiveComms.insert({comm, device});
  }
  // frees are now announced to the peers, so any tensor may be exported on first use
  flagcxCommSetAutoExport(comm, 1);
}
void unfollowAllocator(flagcxComm_t comm) {
  std::lock_guard<std::mutex> g(gLiveMu);
  for (auto it = gLiveComms.begin(); it != gLiveComms.end();)
    it = it->first == comm ? gLiveComms.erase(it) : std::next(it);
}

// Options of the backend, same two fields as the FlagCX torch plugin
// (plugin/torch/flagcx/include/backend_flagcx.hpp:104-114 in the FlagCX project).  With
// enableTuner every collective's (operation, bytes) is remembered as a "tune object";
// flagcx_b200.torch_backend.tune_recorded() later measures exactly those sizes.
struct FlagcxOptions {
  bool enableTuner = false;
  int tuneGroupIdx = 0;
};

class ProcessGroupFlagCX : public c10d::Backend {
 public:
  ProcessGroupFlagCX(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size, FlagcxOptions options = {})
      : c10d::Backend(rank, size), store_(store), options_(options) {
    const char *cur = std::getenv("FLAGCX_TORCH_USE_CURRENT_STREAM");
    useCurrentStream_ = cur && std::atoi(cur) != 0;
  }

  ~ProcessGroupFlagCX() override {
    if (comm_) { unfollowAllocator(comm_); flagcxCommDestroy(comm_); }
  }

  const std::string getBackendName() const override { return "flagcx"; }
  bool supportsCoalescing() const override { return true; }
  void setSequenceNumberForGroup() override {}
  uint64_t getSequenceNumberForGroup() override { return seq_; }
  void abort() override {
    if (comm_) { unfollowAllocator(comm_); flagcxCommAbort(comm_); comm_ = nullptr; }
  }
  void shutdown() override {
    if (comm_) { unfollowAllocator(comm_); flagcxCommDestroy(comm_); comm_ = nullptr; }
  }
  void eagerConnectSingleDevice(at::Device device) override { ensureComm(device); }

  flagcxComm_t comm(const at::Device &device) {
    ensureComm(device);
    return comm_;
  }
  const FlagcxOptions &options() const { return options_; }
  // (operation, bytes) of every distinct collective seen so far (enableTuner only)
  std::vector<std::pair<int, uint64_t>> tuneObjects() {
    std::lock_guard<std::mutex> g(mu_);
    return std::vector<std::pair<int, uint64_t>>(tuneObjects_.begin(), tuneObjects_.end());
  }

  // ---- coalescing --------------------------------------------------------------
  void startCoalescing() override {
    coalescing_ = true;
    coalescedDevice_.reset();
  }
  c10::intrusive_ptr<c10d::Work> endCoalescing() override {
    coalescing_ = false;
    if (groupOpen_) {
      FCX_TORCH_CHECK(flagcxGroupEnd(comm_), comm_);
      groupOpen_ = false;
    }
    auto work = c10::make_intrusive<WorkFlagCX>(c10d::OpType::COALESCED, coalescedDevice_);
    finish(work, {});
    return work;
  }

  // ---- collectives -----------------------------------------------------------------
  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor> &tensors,
                                           const c10d::AllreduceOptions &opts) override {
    auto &t = single(tensors);
    return run(c10d::OpType::ALLREDUCE, {t}, {t}, [&](flagcxStream_t s) {
      return flagcxAllReduce(t.data_ptr(), t.data_ptr(), t.numel(), toFlagcxType(t.scalar_type()),
                             toFlagcxOp(opts.reduceOp, t.scalar_type()), comm_, s);
    });
  }

  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor> &tensors,
                                                     const c10d::AllreduceCoalescedOptions &opts) override {
    for (auto &t : tensors) checkContiguous(t);
    return run(c10d::OpType::ALLREDUCE_COALESCED, tensors, tensors, [&](flagcxStream_t s) {
      for (auto &t : tensors) {
        flagcxResult_t r = flagcxAllReduce(t.data_ptr(), t.data_ptr(), t.numel(), toFlagcxType(t.scalar_type()),
                                           toFlagcxOp(opts.reduceOp, t.scalar_type()), comm_, s);
        if (r != flagcxSuccess) return r;
      }
      return flagcxSuccess;
    });
  }

  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor> &tensors,
                                           const c10d::BroadcastOptions &opts) override {
    auto &t = single(tensors);
    int root = (int)(opts.rootRank + opts.rootTensor);
    return run(c10d::OpType::BROADCAST, {t}, {t}, [&](flagcxStream_t s) {
      return flagcxBroadcast(t.data_ptr(), t.data_ptr(), t.numel(), toFlagcxType(t.scalar_type()), root, comm_, s);
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor> &tensors, const c10d::ReduceOptions &opts) override {
    auto &t = single(tensors);
    int root = (int)(opts.rootRank + opts.rootTensor);
    // non-roots must not see their input overwritten: reduce into a scratch there
    at::Tensor out = getRank() == root ? t : at::empty_like(t);
    return run(c10d::OpType::REDUCE, {t}, {t, out}, [&](flagcxStream_t s) {
      return flagcxReduce(t.data_ptr(), out.data_ptr(), t.numel(), toFlagcxType(t.scalar_type()),
                          toFlagcxOp(opts.reduceOp, t.scalar_type()), root, comm_, s);
    });
  }

  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor &output, at::Tensor &input,
                                                 const c10d::AllgatherOptions &) override {
    checkContiguous(output);
    checkContiguous(input);
    TORCH_CHECK(output.numel() == input.numel() * getSize(), "flagcx: allgather output must be world_size x input");
    return run(c10d::OpType::_ALLGATHER_BASE, {input}, {output}, [&](flagcxStream_t s) {
      return flagcxAllGather(input.data_ptr(), output.data_ptr(), input.numel(), toFlagcxType(input.scalar_type()),
                             comm_, s);
    });
  }

  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>> &outputs,
                                           std::vector<at::Tensor> &inputs,
                                           const c10d::AllgatherOptions &opts) override {
    auto &in = single(inputs);
    TORCH_CHECK(outputs.size() == 1 && (int)outputs[0].size() == getSize(), "flagcx: allgather needs world_size outputs");
    auto &outs = outputs[0];
    at::Tensor flat = flatAlias(outs);
    bool direct = flat.defined();
    if (!direct) flat = at::empty({(int64_t)getSize() * in.numel()}, in.options());
    auto work = run(c10d::OpType::ALLGATHER, {in}, {flat}, [&](flagcxStream_t s) {
      return flagcxAllGather(in.data_ptr(), flat.data_ptr(), in.numel(), toFlagcxType(in.scalar_type()), comm_, s);
    }, [&]() {
      if (!direct)
        for (int r = 0; r < getSize(); ++r) outs[r].copy_(flat.narrow(0, r * in.numel(), in.numel()).view_as(outs[r]), true);
    });
    (void)opts;
    return work;
  }

  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(std::vector<at::Tensor> &outputs,
                                                                 std::vector<at::Tensor> &inputs,
                                                                 const c10d::AllgatherOptions &) override {
    TORCH_CHECK(outputs.size() == inputs.size(), "flagcx: mismatched coalesced allgather lists");
    return run(c10d::OpType::COALESCED, inputs, outputs, [&](flagcxStream_t s) {
      for (size_t i = 0; i < inputs.size(); ++i) {
        flagcxResult_t r = flagcxAllGather(inputs[i].data_ptr(), outputs[i].data_ptr(), inputs[i].numel(),
                                           toFlagcxType(inputs[i].scalar_type()), comm_, s);
        if (r != flagcxSuccess) return r;
      }
      return flagcxSuccess;
    });
  }

  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor &output, at::Tensor &input,
                                                      const c10d::ReduceScatterOptions &opts) override {
    checkContiguous(output);
    checkContiguous(input);
    TORCH_CHECK(input.numel() == output.numel() * getSize(), "flagcx: reduce_scatter input must be world_size x output");
    return run(c10d::OpType::_REDUCE_SCATTER_BASE, {input}, {output}, [&](flagcxStream_t s) {
      return flagcxReduceScatter(input.data_ptr(), output.data_ptr(), output.numel(),
                                 toFlagcxType(input.scalar_type()), toFlagcxOp(opts.reduceOp, input.scalar_type()),
                                 comm_, s);
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor> &outputs,
                                                std::vector<std::vector<at::Tensor>> &inputs,
                                                const c10d::ReduceScatterOptions &opts) override {
    auto &out = single(outputs);
    TORCH_CHECK(inputs.size() == 1 && (int)inputs[0].size() == getSize(), "flagcx: reduce_scatter needs world_size inputs");
    at::Tensor flat = flatAlias(inputs[0]);
    if (!flat.defined()) {
      std::vector<at::Tensor> pieces;
      for (auto &t : inputs[0]) pieces.push_back(t.reshape({-1}));
      flat = at::cat(pieces);
    }
    return run(c10d::OpType::REDUCE_SCATTER, {flat}, {out}, [&](flagcxStream_t s) {
      return flagcxReduceScatter(flat.data_ptr(), out.data_ptr(), out.numel(), toFlagcxType(out.scalar_type()),
                                 toFlagcxOp(opts.reduceOp, out.scalar_type()), comm_, s);
    });
  }

  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor> &outputs,
                                                                 std::vector<at::Tensor> &inputs,
                                                                 const c10d::ReduceScatterOptions &opts) override {
    TORCH_CHECK(outputs.size() == inputs.size(), "flagcx: mismatched coalesced reduce_scatter lists");
    return run(c10d::OpType::COALESCED, inputs, outputs, [&](flagcxStream_t s) {
      for (size_t i = 0; i < inputs.size(); ++i) {
        flagcxResult_t r = flagcxReduceScatter(inputs[i].data_ptr(), outputs[i].data_ptr(), outputs[i].numel(),
                                               toFlagcxType(inputs[i].scalar_type()),
                                               toFlagcxOp(opts.reduceOp, inputs[i].scalar_type()), comm_, s);
        if (r != flagcxSuccess) return r;
      }
      return flagcxSuccess;
    });
  }

  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor &output, at::Tensor &input,
                                               std::vector<int64_t> &outSplits, std::vector<int64_t> &inSplits,
                                               const c10d::AllToAllOptions &) override {
    checkContiguous(output);
    checkContiguous(input);
    const int n = getSize();
    auto dt = toFlagcxType(input.scalar_type());
    if (outSplits.empty() && inSplits.empty()) {
      TORCH_CHECK(input.numel() % n == 0 && input.numel() == output.numel(), "flagcx: alltoall sizes must divide evenly");
      return run(c10d::OpType::ALLTOALL_BASE, {input}, {output}, [&](flagcxStream_t s) {
        return flagcxAlltoAll(input.data_ptr(), output.data_ptr(), input.numel() / n, dt, comm_, s);
      });
    }
    // rows of dimension 0 are split unevenly: counts in elements
    int64_t inRow = input.dim() > 0 && input.size(0) > 0 ? input.numel() / input.size(0) : 1;
    int64_t outRow = output.dim() > 0 && output.size(0) > 0 ? output.numel() / output.size(0) : 1;
    std::vector<size_t> sc(n), sd(n), rc(n), rd(n);
    size_t so = 0, ro = 0;
    for (int p = 0; p < n; ++p) {
      sc[p] = (size_t)((inSplits.empty() ? input.size(0) / n : inSplits[p]) * inRow);
      rc[p] = (size_t)((outSplits.empty() ? output.size(0) / n : outSplits[p]) * outRow);
      sd[p] = so; so += sc[p];
      rd[p] = ro; ro += rc[p];
    }
    return run(c10d::OpType::ALLTOALL_BASE, {input}, {output}, [&](flagcxStream_t s) {
      return flagcxAlltoAllv(input.data_ptr(), sc.data(), sd.data(), output.data_ptr(), rc.data(), rd.data(), dt,
                             comm_, s);
    });
  }

  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor> &outputs, std::vector<at::Tensor> &inputs,
                                          const c10d::AllToAllOptions &) override {
    const int n = getSize();
    TORCH_CHECK((int)outputs.size() == n && (int)inputs.size() == n, "flagcx: alltoall needs world_size tensors");
    std::vector<size_t> sc(n), sd(n), rc(n), rd(n);
    size_t so = 0, ro = 0;
    std::vector<at::Tensor> pieces;
    for (int p = 0; p < n; ++p) {
      sc[p] = inputs[p].numel(); sd[p] = so; so += sc[p];
      rc[p] = outputs[p].numel(); rd[p] = ro; ro += rc[p];
      pieces.push_back(inputs[p].reshape({-1}));
    }
    at::Tensor in = at::cat(pieces);
    at::Tensor out = at::empty({(int64_t)ro}, inputs[0].options());
    auto dt = toFlagcxType(in.scalar_type());
    return run(c10d::OpType::ALLTOALL, {in}, {out}, [&](flagcxStream_t s) {
      return flagcxAlltoAllv(in.data_ptr(), sc.data(), sd.data(), out.data_ptr(), rc.data(), rd.data(), dt, comm_, s);
    }, [&]() {
      for (int p = 0; p < n; ++p) outputs[p].copy_(out.narrow(0, rd[p], rc[p]).view_as(outputs[p]), true);
    });
  }

  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>> &outputs, std::vector<at::Tensor> &inputs,
                                        const c10d::GatherOptions &opts) override {
    auto &in = single(inputs);
    const int n = getSize(), root = (int)opts.rootRank;
    at::Tensor flat;
    if (getRank() == root) {
      TORCH_CHECK(outputs.size() == 1 && (int)outputs[0].size() == n, "flagcx: gather needs world_size outputs at the root");
      flat = at::empty({(int64_t)n * in.numel()}, in.options());
    }
    return run(c10d::OpType::GATHER, {in}, flat.defined() ? std::vector<at::Tensor>{flat} : std::vector<at::Tensor>{},
               [&](flagcxStream_t s) {
                 return flagcxGather(in.data_ptr(), flat.defined() ? flat.data_ptr() : nullptr, in.numel(),
                                     toFlagcxType(in.scalar_type()), root, comm_, s);
               },
               [&]() {
                 if (flat.defined())
                   for (int r = 0; r < n; ++r)
                     outputs[0][r].copy_(flat.narrow(0, r * in.numel(), in.numel()).view_as(outputs[0][r]), true);
               });
  }

  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor> &outputs, std::vector<std::vector<at::Tensor>> &inputs,
                                         const c10d::ScatterOptions &opts) override {
    auto &out = single(outputs);
    const int n = getSize(), root = (int)opts.rootRank;
    at::Tensor flat;
    if (getRank() == root) {
      TORCH_CHECK(inputs.size() == 1 && (int)inputs[0].size() == n, "flagcx: scatter needs world_size inputs at the root");
      std::vector<at::Tensor> pieces;
      for (auto &t : inputs[0]) pieces.push_back(t.reshape({-1}));
      flat = at::cat(pieces);
    }
    return run(c10d::OpType::SCATTER, flat.defined() ? std::vector<at::Tensor>{flat} : std::vector<at::Tensor>{}, {out},
               [&](flagcxStream_t s) {
                 return flagcxScatter(flat.defined() ? flat.data_ptr() : nullptr, out.data_ptr(), out.numel(),
                                      toFlagcxType(out.scalar_type()), root, comm_, s);
               });
  }

  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor> &tensors, int dst, int) override {
    auto &t = single(tensors);
    return run(c10d::OpType::SEND, {t}, {}, [&](flagcxStream_t s) {
      return flagcxSend(t.data_ptr(), t.numel(), toFlagcxType(t.scalar_type()), dst, comm_, s);
    }, {}, /*p2p=*/true);
  }

  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor> &tensors, int src, int) override {
    auto &t = single(tensors);
    return run(c10d::OpType::RECV, {}, {t}, [&](flagcxStream_t s) {
      return flagcxRecv(t.data_ptr(), t.numel(), toFlagcxType(t.scalar_type()), src, comm_, s);
    }, {}, /*p2p=*/true);
  }

  c10::intrusive_ptr<c10d::Work> recvAnysource(std::vector<at::Tensor> &, int) override {
    TORCH_CHECK(false, "flagcx: recvAnysource is not supported");
  }

  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions &opts) override {
    at::Device dev = at::Device(at::kCPU);
    if (opts.device.has_value()) dev = *opts.device;
    else if (lastDevice_) dev = *lastDevice_;
    else if (at::cuda::is_available()) dev = at::Device(at::kCUDA, c10::cuda::current_device());
    ensureComm(dev);
    auto work = c10::make_intrusive<WorkFlagCX>(c10d::OpType::BARRIER, dev);
    if (dev.is_cuda()) {
      c10::cuda::CUDAGuard g(dev);
      auto stream = commStream(dev);
      sync(dev, stream);
      flagcxStream fs{stream.stream()};
      FCX_TORCH_CHECK(flagcxBarrier(comm_, &fs), comm_);
      work->event_->record(stream);
    } else {
      FCX_TORCH_CHECK(flagcxBarrier(comm_, nullptr), comm_);
    }
    return work;
  }

 private:
  static void checkContiguous(const at::Tensor &t) {
    TORCH_CHECK(t.is_contiguous(), "flagcx: tensors must be contiguous");
  }
  static at::Tensor &single(std::vector<at::Tensor> &v) {
    TORCH_CHECK(v.size() == 1, "flagcx: expected exactly one tensor per rank");
    checkContiguous(v[0]);
    return v[0];
  }
  // If the list is a set of equal, back-to-back views of one buffer, returns that buffer.
  static at::Tensor flatAlias(const std::vector<at::Tensor> &ts) {
    if (ts.empty()) return {};
    const auto &t0 = ts[0];
    for (size_t i = 0; i < ts.size(); ++i) {
      const auto &t = ts[i];
      if (!t.is_contiguous() || t.numel() != t0.numel() || t.scalar_type() != t0.scalar_type() ||
          t.storage().data() != t0.storage().data() ||
          (char *)t.data_ptr() != (char *)t0.data_ptr() + i * t0.nbytes())
        return {};
    }
    return at::from_blob(t0.data_ptr(), {(int64_t)(ts.size() * t0.numel())}, t0.options());
  }

  at::cuda::CUDAStream commStream(const at::Device &dev) {
    if (useCurrentStream_) return at::cuda::getCurrentCUDAStream(dev.index());
    if (!stream_) stream_ = at::cuda::getStreamFromPool(/*isHighPriority=*/true, dev.index());
    return *stream_;
  }

  // The communication stream starts after everything already queued on the caller's stream.
  void sync(const at::Device &dev, at::cuda::CUDAStream &stream) {
    if (useCurrentStream_) return;
    if (coalescing_ && coalescedDevice_) return; // once per coalesced batch
    at::cuda::CUDAEvent ev(cudaEventDisableTiming);
    ev.record(at::cuda::getCurrentCUDAStream(dev.index()));
    ev.block(stream);
  }

  void ensureComm(const at::Device &dev) {
    std::lock_guard<std::mutex> g(mu_);
    if (dev.is_cuda()) lastDevice_ = dev;
    if (comm_) {
      // one communicator, bound to one GPU at creation: a tensor on another GPU of this
      // process cannot use it
      TORCH_CHECK(!dev.is_cuda() || commDevice_ < 0 || dev.index() == commDevice_,
                  "flagcx: this process group was initialised on cuda:", commDevice_, " but got a tensor on cuda:",
                  (int)dev.index(), "; call torch.cuda.set_device() before the first collective");
      return;
    }
    std::optional<c10::cuda::CUDAGuard> guard;
    if (dev.is_cuda()) guard.emplace(dev);
    // id exchange through the c10d store; one key per communicator instance
    static std::atomic<int> instance{0};
    std::string key = "flagcx/unique_id/" + std::to_string(groupCounter_) + "/" + getGroupUid();
    (void)instance;
    flagcxUniqueId id;
    if (getRank() == 0) {
      FCX_TORCH_CHECK(flagcxGetUniqueId(&id), nullptr);
      std::vector<uint8_t> bytes((uint8_t *)&id, (uint8_t *)&id + sizeof id);
      store_->set(key, bytes);
    } else {
      auto bytes = store_->get(key);
      TORCH_CHECK(bytes.size() == sizeof id, "flagcx: malformed unique id in the store");
      std::memcpy(&id, bytes.data(), sizeof id);
    }
    FCX_TORCH_CHECK(flagcxCommInitRank(&comm_, getSize(), &id, getRank()), nullptr);
    // the GPU the communicator bound itself to (the current device if the first tensor was
    // a CPU tensor); -1 on hosts without one
    int devNo = -1;
    if (flagcxCommGetDeviceNumber(comm_, &devNo) == flagcxSuccess) commDevice_ = devNo;
    if (commDevice_ >= 0) followAllocator(comm_, commDevice_);
  }

  static int commOpOf(c10d::OpType op) {
    switch (op) {
      case c10d::OpType::ALLREDUCE:
      case c10d::OpType::ALLREDUCE_COALESCED: return flagcxCommOpAllReduce;
      case c10d::OpType::BROADCAST: return flagcxCommOpBroadcast;
      case c10d::OpType::REDUCE: return flagcxCommOpReduce;
      case c10d::OpType::ALLGATHER:
      case c10d::OpType::_ALLGATHER_BASE: return flagcxCommOpAllGather;
      case c10d::OpType::REDUCE_SCATTER:
      case c10d::OpType::_REDUCE_SCATTER_BASE: return flagcxCommOpReduceScatter;
      case c10d::OpType::ALLTOALL_BASE:
      case c10d::OpType::ALLTOALL: return flagcxCommOpAlltoAll;
      case c10d::OpType::GATHER: return flagcxCommOpGather;
      case c10d::OpType::SCATTER: return flagcxCommOpScatter;
      default: return -1;
    }
  }

  template <typename Fn>
  c10::intrusive_ptr<c10d::Work> run(c10d::OpType op, const std::vector<at::Tensor> &inputs,
                                     const std::vector<at::Tensor> &outputs, Fn fn,
                                     std::function<void()> post = {}, bool p2p = false) {
    ++seq_;
    if (options_.enableTuner && commOpOf(op) >= 0) {
      // the size the library's tuner keys on: the larger side of the operation
      uint64_t in = 0, out = 0;
      for (auto &t : inputs) in += (uint64_t)t.nbytes();
      for (auto &t : outputs) out += (uint64_t)t.nbytes();
      std::lock_guard<std::mutex> g(mu_);
      tuneObjects_.insert({commOpOf(op), std::max(in, out)});
    }
    const at::Tensor &probe = !inputs.empty() ? inputs[0] : outputs[0];
    at::Device dev = probe.device();
    ensureComm(dev);
    auto work = c10::make_intrusive<WorkFlagCX>(op, dev);
    work->outputs_ = outputs;
    if (!dev.is_cuda()) {
      if (p2p && coalescing_ && !groupOpen_) { FCX_TORCH_CHECK(flagcxGroupStart(comm_), comm_); groupOpen_ = true; }
      FCX_TORCH_CHECK(fn(nullptr), comm_);
      if (post) post();
      finish(work, outputs);
      return work;
    }
    c10::cuda::CUDAGuard guard(dev);
    auto stream = commStream(dev);
    sync(dev, stream);
    if (coalescing_) coalescedDevice_ = dev;
    if (!useCurrentStream_) {
      for (auto &t : inputs) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), stream);
      for (auto &t : outputs) c10::cuda::CUDACachingAllocator::recordStream(t.storage().data_ptr(), stream);
    }
    {
      c10::cuda::CUDAStreamGuard sg(stream);
      if (p2p && coalescing_ && !groupOpen_) { FCX_TORCH_CHECK(flagcxGroupStart(comm_), comm_); groupOpen_ = true; }
      flagcxStream fs{stream.stream()};
      FCX_TORCH_CHECK(fn(&fs), comm_);
      if (post) post();
      if (!coalescing_) {
        work->event_->record(stream);
        work->future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()),
                                                                  std::vector<c10::Device>{dev});
        work->future_->markCompleted(c10::IValue(outputs));
      }
    }
    return work;
  }

  void finish(const c10::intrusive_ptr<WorkFlagCX> &work, const std::vector<at::Tensor> &outputs) {
    if (work->device_ && work->device_->is_cuda()) {
      c10::cuda::CUDAGuard guard(*work->device_);
      auto stream = commStream(*work->device_);
      c10::cuda::CUDAStreamGuard sg(stream);
      work->event_->record(stream);
      work->future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()),
                                                                std::vector<c10::Device>{*work->device_});
      work->future_->markCompleted(c10::IValue(outputs));
    } else {
      work->future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
      work->future_->markCompleted(c10::IValue(outputs));
    }
  }

  c10::intrusive_ptr<c10d::Store> store_;
  flagcxComm_t comm_ = nullptr;
  std::optional<at::cuda::CUDAStream> stream_;
  std::optional<at::Device> lastDevice_, coalescedDevice_;
  bool coalescing_ = false, groupOpen_ = false, useCurrentStream_ = false;
  uint64_t seq_ = 0;
  int groupCounter_ = 0;
  int commDevice_ = -1;
  FlagcxOptions options_;
  std::set<std::pair<int, uint64_t>> tuneObjects_;
  std::mutex mu_;
};

c10::intrusive_ptr<c10d::Backend> createBackend(const c10::intrusive_ptr<c10d::Store> &store, int rank, int size,
                                                const std::chrono::duration<float> &, bool enableTuner,
                                                int tuneGroupIdx) {
  return c10::make_intrusive<ProcessGroupFlagCX>(store, rank, size, FlagcxOptions{enableTuner, tuneGroupIdx});
}

std::vector<std::pair<int, uint64_t>> tuneObjects(const c10::intrusive_ptr<c10d::Backend> &backend) {
  auto *pg = dynamic_cast<ProcessGroupFlagCX *>(backend.get());
  TORCH_CHECK(pg, "not a flagcx backend");
  return pg->tuneObjects();
}
std::pair<bool, int> backendOptions(const c10::intrusive_ptr<c10d::Backend> &backend) {
  auto *pg = dynamic_cast<ProcessGroupFlagCX *>(backend.get());
  TORCH_CHECK(pg, "not a flagcx backend");
  return {pg->options().enableTuner, pg->options().tuneGroupIdx};
}

// Raw flagcxComm_t of a backend (as an integer) so Python can drive the C API --
// window registration, fused collectives, tuner -- on the same communicator.
uintptr_t commHandle(const c10::intrusive_ptr<c10d::Backend> &backend, const at::Device &device) {
  auto *pg = dynamic_cast<ProcessGroupFlagCX *>(backend.get());
  TORCH_CHECK(pg, "not a flagcx backend");
  return (uintptr_t)pg->comm(device);
}

} // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "torch.distributed backend 'flagcx' (B200-native collectives)";
  m.def("create_backend", &createBackend, py::arg("store"), py::arg("rank"), py::arg("size"), py::arg("timeout"),
        py::arg("enable_tuner") = false, py::arg("tune_group_idx") = 0);
  m.def("tune_objects", &tuneObjects, py::arg("backend"));
  m.def("follow_allocator", [](uintptr_t comm, int device) { followAllocator((flagcxComm_t)comm, device); },
        py::arg("comm_handle"), py::arg("device"),
        "Have a communicator created outside torch.distributed unmap, on its peers, every segment the caching "
        "allocator is about to free.");
  m.def("unfollow_allocator", [](uintptr_t comm) { unfollowAllocator((flagcxComm_t)comm); }, py::arg("comm_handle"));
  m.def("backend_options", &backendOptions, py::arg("backend"));
  m.def("comm_handle", &commHandle, py::arg("backend"), py::arg("device"));
}
