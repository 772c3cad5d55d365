#include "backend.h"

#include "core/numa.h"

#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/csrc/distributed/c10d/Types.hpp>
#include <torch/csrc/distributed/c10d/NCCLUtils.hpp>

#include <atomic>
#include <map>
#include <random>

#include "core/log.h"
#include "kernels/kernels_api.h"

// core errors become torch errors at the boundary
#define MOODIST_TRANSLATE(body)                 \
  try {                                         \
    body                                        \
  } catch (const moodist::Error& e) {           \
    TORCH_CHECK(false, e.what());               \
  }

namespace moodist {
namespace {

// Work for stream-ordered CUDA collectives: "complete" as soon as it is created; wait() makes the
// caller's current stream wait for the point in the launch stream where the collective ended.
class CudaWork final : public c10d::Work {
 public:
  CudaWork(int rank, c10d::OpType op, std::vector<at::Tensor> outputs, c10::cuda::CUDAStream stream)
      : c10d::Work(rank, op), outputs_(std::move(outputs)), device_(stream.device_index()) {
    event_.record(stream);
    future_ = c10::make_intrusive<at::ivalue::Future>(c10::ListType::create(c10::TensorType::get()),
                                                      std::vector<c10::Device>{stream.device()});
    future_->markCompleted(at::IValue(outputs_));
  }
  bool isCompleted() override { return true; }
  bool isSuccess() const override { return true; }
  bool wait(std::chrono::milliseconds) override {
    auto cur = c10::cuda::getCurrentCUDAStream(device_);
    event_.block(cur);
    return true;
  }
  void synchronize() override { wait(std::chrono::milliseconds(0)); }
  std::vector<at::Tensor> result() override { return outputs_; }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }

 private:
  std::vector<at::Tensor> outputs_;
  c10::DeviceIndex device_;
  at::cuda::CUDAEvent event_;
  c10::intrusive_ptr<at::ivalue::Future> future_;
};

// CPU collectives block inside the call, so their Work is simply done.
class DoneWork final : public c10d::Work {
 public:
  DoneWork(int rank, c10d::OpType op, std::vector<at::Tensor> outputs)
      : c10d::Work(rank, op), outputs_(std::move(outputs)) {
    future_ = c10::make_intrusive<at::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
    future_->markCompleted(at::IValue(outputs_));
  }
  bool isCompleted() override { return true; }
  bool isSuccess() const override { return true; }
  bool wait(std::chrono::milliseconds) override { return true; }
  void synchronize() override {}
  std::vector<at::Tensor> result() override { return outputs_; }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }

 private:
  std::vector<at::Tensor> outputs_;
  c10::intrusive_ptr<at::ivalue::Future> future_;
};

// A receive that has been posted and is completed by wait(): the message is matched in posting order whatever the
// order of the waits, so a rank may post its receives first and send afterwards (pipelines and rings do) without
// every rank sitting in a receive that nobody has sent to yet. `after` runs once, inside wait(), when the host
// part has arrived (the device part of a CUDA receive).
class RecvWork final : public c10d::Work {
 public:
  // `send` = true makes it the work of a posted send (completed when the receiver has taken the payload)
  RecvWork(int rank, std::vector<at::Tensor> outputs, c10::intrusive_ptr<MoodistBackend> owner,
           std::shared_ptr<void> posted, std::function<void()> after, bool send = false)
      : c10d::Work(rank, send ? c10d::OpType::SEND : c10d::OpType::RECV), outputs_(std::move(outputs)),
        owner_(std::move(owner)), posted_(std::move(posted)), after_(std::move(after)),
        has_after_(static_cast<bool>(after_)), send_(send) {
    future_ = c10::make_intrusive<at::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
  }
  bool isCompleted() override {
    // never blocks, also while another thread sits in wait(): a receive with a device part counts as complete
    // once wait() has run it
    if (done_.load()) return true;
    if (has_after_) return false;
    return send_ ? owner_->hostGroup().send_done(posted_) : owner_->hostGroup().recv_done(posted_);
  }
  bool isSuccess() const override { return true; }
  bool wait(std::chrono::milliseconds) override {
    std::lock_guard<std::mutex> lk(mu_);
    if (done_) return true;
    MOODIST_TRANSLATE(if (send_) owner_->hostGroup().send_wait(posted_); else owner_->hostGroup().recv_wait(posted_);)
    if (after_) {
      auto f = std::move(after_);
      after_ = nullptr;
      f();
    }
    done_ = true;
    future_->markCompleted(at::IValue(outputs_));
    return true;
  }
  void synchronize() override { wait(std::chrono::milliseconds(0)); }
  std::vector<at::Tensor> result() override { return outputs_; }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }
  // of a completed receive: the rank the message came from (what a receive from anybody wants to know)
  int sourceRank() const override { return send_ ? -1 : owner_->hostGroup().recv_source(posted_); }

 private:
  std::mutex mu_;
  std::atomic<bool> done_{false};
  std::vector<at::Tensor> outputs_;
  c10::intrusive_ptr<MoodistBackend> owner_;
  std::shared_ptr<void> posted_;
  std::function<void()> after_;
  const bool has_after_;
  const bool send_;
  c10::intrusive_ptr<at::ivalue::Future> future_;
};

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kByte: return MB_U8;
    case at::kBool: return MB_U8;
    case at::kChar: return MB_I8;
    case at::kShort: return MB_I16;
    case at::kInt: return MB_I32;
    case at::kLong: return MB_I64;
    case at::kHalf: return MB_F16;
    case at::kFloat: return MB_F32;
    case at::kDouble: return MB_F64;
    case at::kBFloat16: return MB_BF16;
    default: TORCH_CHECK(false, "moodist: unsupported dtype ", t);
  }
}

// torch ReduceOp -> (kernel op code, premul factor)
std::pair<int, double> reduce_code(const c10d::ReduceOp& op) {
  switch (op.op_) {
    case c10d::ReduceOp::SUM: return {MB_SUM, 1.0};
    case c10d::ReduceOp::AVG: return {MB_AVG, 1.0};
    case c10d::ReduceOp::MIN: return {MB_MIN, 1.0};
    case c10d::ReduceOp::MAX: return {MB_MAX, 1.0};
    case c10d::ReduceOp::PREMUL_SUM: {
      // the factor travels in the same supplement type NCCL's backend uses (reference:
      // wrapper/processgroup_wrapper.cc:41-53)
      auto* sup = reinterpret_cast<c10d::NCCLPreMulSumSupplement*>(op.supplement_.get());
      TORCH_CHECK(sup != nullptr, "moodist: PREMUL_SUM without a factor");
      if (sup->tensor_factor.defined()) return {MB_PREMUL_SUM, sup->tensor_factor.item<double>()};
      return {MB_PREMUL_SUM, sup->double_factor};
    }
    // host path only (the kernels implement the five above, as the reference's core does: core/group.h:26)
    case c10d::ReduceOp::PRODUCT: return {2, 1.0};
    case c10d::ReduceOp::BAND: return {5, 1.0};
    case c10d::ReduceOp::BOR: return {6, 1.0};
    case c10d::ReduceOp::BXOR: return {7, 1.0};
    default: TORCH_CHECK(false, "moodist: unsupported reduce op");
  }
}

// A bool tensor holds bytes 0 and 1, and must keep doing so: its "sum" is the logical or, its product the and.
int bool_op(at::ScalarType t, int op) {
  if (t != at::kBool) return op;
  if (op == MB_SUM || op == MB_AVG || op == MB_PREMUL_SUM || op == 6 /* BOR */) return MB_MAX;
  if (op == 2 /* PRODUCT */ || op == 5 /* BAND */) return MB_MIN;
  return op;
}

void check_cuda_op(int op) {
  TORCH_CHECK(op == MB_SUM || op == MB_AVG || op == MB_MIN || op == MB_MAX || op == MB_PREMUL_SUM,
              "moodist: CUDA tensors support SUM, AVG, MIN, MAX and PREMUL_SUM (PRODUCT and the bitwise reductions "
              "exist for CPU tensors only)");
}

void check_contig(const at::Tensor& t, const char* what) {
  TORCH_CHECK(t.is_contiguous(), "moodist: ", what, " tensor must be contiguous");
}

std::string random_name() {
  std::random_device rd;
  uint64_t v = ((uint64_t)rd() << 32) ^ rd();
  char buf[32];
  snprintf(buf, sizeof(buf), "%016llx", (unsigned long long)v);
  return buf;
}

CUstream_st* raw(const c10::cuda::CUDAStream& s) { return reinterpret_cast<CUstream_st*>(s.stream()); }

}  // namespace

namespace {
std::mutex g_registry_mu;
std::map<std::string, MoodistBackend*>& registry() {
  static auto* m = new std::map<std::string, MoodistBackend*>();
  return *m;
}
}  // namespace

static std::atomic<int> g_default_prefer_kernel_less{0};
void MoodistBackend::setDefaultPreferKernelLess(bool v) { g_default_prefer_kernel_less = v ? 1 : 0; }

c10::intrusive_ptr<MoodistBackend> MoodistBackend::find(const std::string& name) {
  std::lock_guard<std::mutex> lk(g_registry_mu);
  auto it = registry().find(name);
  if (it == registry().end()) return nullptr;
  return c10::intrusive_ptr<MoodistBackend>::reclaim_copy(it->second);
}

MoodistBackend::MoodistBackend(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size)
    : c10d::Backend(rank, size), store_(store), kv_(std::make_unique<C10dStoreAdapter>(store)), rank_(rank),
      size_(size) {
  TORCH_CHECK(rank >= 0 && rank < size, "moodist: bad rank ", rank, " for world size ", size);
  // rank 0 names the group; everyone learns it through the store (reference: core/processgroup.cc:977-1050)
  if (rank == 0) {
    name_ = random_name();
    kv_->set_str("moodist_pg_key", name_);
  } else {
    name_ = kv_->get_str("moodist_pg_key");
  }
  opts_.prefer_kernel_less = g_default_prefer_kernel_less.load();
  // The host engine comes up here, while every rank is inside the (ordered, collective) construction of this
  // group. Left to the first operation, two groups first used from two threads would exchange their addresses
  // through the shared store at the same time, each thread waiting in the store for a key that the other rank's
  // blocked thread has yet to write.
  MOODIST_TRANSLATE(host_ = HostGroup::create(*kv_, name_, rank_, size_);)
  std::lock_guard<std::mutex> lk(g_registry_mu);
  registry()[name_] = this;
}

std::vector<c10::intrusive_ptr<MoodistBackend>> MoodistBackend::live() {
  std::lock_guard<std::mutex> lk(g_registry_mu);
  std::vector<c10::intrusive_ptr<MoodistBackend>> out;
  for (auto& [name, p] : registry()) out.push_back(c10::intrusive_ptr<MoodistBackend>::reclaim_copy(p));
  return out;
}

MoodistBackend::~MoodistBackend() {
  {
    std::lock_guard<std::mutex> lk(g_registry_mu);
    auto it = registry().find(name_);
    if (it != registry().end() && it->second == this) registry().erase(it);
  }
  if (p2p_) {
    // acknowledgements still queued as host callbacks on some stream refer to host_: let them run first
    cudaSetDevice(cuda_->device());
    cudaDeviceSynchronize();
    p2p_.reset();
  }
  try {
    if (host_) host_->shutdown();
  } catch (...) {
  }
}

CudaGroup& MoodistBackend::cudaGroup(int device) {
  std::lock_guard<std::mutex> lk(mu_);
  if (!cuda_) {
    MOODIST_TRANSLATE(cuda_ = CudaGroup::create(*kv_, name_, rank_, size_, device);)
    cuda_->options() = opts_;
    // the host engine thread (if it exists already) moves next to the GPU's memory node
    if (host_ && cuda_->numa_node() >= 0) {
      int node = cuda_->numa_node();
      host_->run_on_engine([node] { bind_thread_to_numa_node(node); });
    }
  }
  TORCH_CHECK(cuda_->device() == device, "moodist: this process group is bound to cuda:", cuda_->device(),
              " but got a tensor on cuda:", device);
  return *cuda_;
}

CudaP2P* MoodistBackend::cudaP2P(int device) {
  {
    std::lock_guard<std::mutex> lk(mu_);
    if (p2p_) return p2p_.get();
    if (!cuda_ || size_ < 2 || cuda_->device() != device) return nullptr;
  }
  HostGroup& h = hostGroup();
  std::lock_guard<std::mutex> lk(mu_);
  if (!p2p_) MOODIST_TRANSLATE(p2p_ = std::make_unique<CudaP2P>(*cuda_, h, device);)
  return p2p_.get();
}

HostGroup& MoodistBackend::hostGroup() {
  std::lock_guard<std::mutex> lk(mu_);
  if (!host_) {
    MOODIST_TRANSLATE(host_ = HostGroup::create(*kv_, name_, rank_, size_);)
    if (cuda_ && cuda_->numa_node() >= 0) {
      int node = cuda_->numa_node();
      host_->run_on_engine([node] { bind_thread_to_numa_node(node); });
    }
  }
  return *host_;
}

QueueManager& MoodistBackend::queues() {
  HostGroup& h = hostGroup();
  std::lock_guard<std::mutex> lk(mu_);
  if (!queues_) queues_ = QueueManager::create(h);
  return *queues_;
}

// ------------------------------------------------------------------------------------------------
// collectives
// ------------------------------------------------------------------------------------------------

c10::intrusive_ptr<c10d::Work> MoodistBackend::_allgather_base(at::Tensor& output, at::Tensor& input,
                                                               const c10d::AllgatherOptions&) {
  check_contig(output, "all_gather output");
  check_contig(input, "all_gather input");
  TORCH_CHECK(output.device() == input.device(), "moodist: all_gather tensors must be on the same device");
  TORCH_CHECK(output.scalar_type() == input.scalar_type(), "moodist: all_gather dtype mismatch");
  TORCH_CHECK(output.numel() == input.numel() * size_, "moodist: all_gather output must be world_size x input");
  if (input.is_cuda()) {
    c10::cuda::CUDAGuard guard(input.device());
    auto stream = c10::cuda::getCurrentCUDAStream();
    int dt = dtype_code(input.scalar_type());
    MOODIST_TRANSLATE(cudaGroup(input.get_device())
                          .all_gather(input.data_ptr(), output.data_ptr(), input.numel(), dt, dt, raw(stream));)
    return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::_ALLGATHER_BASE, std::vector<at::Tensor>{output}, stream);
  }
  MOODIST_TRANSLATE(hostGroup().all_gather(input.data_ptr(), output.data_ptr(), input.nbytes());)
  return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::_ALLGATHER_BASE, std::vector<at::Tensor>{output});
}

void MoodistBackend::allGatherCast(at::Tensor& output, const at::Tensor& input) {
  check_contig(output, "all_gather output");
  check_contig(input, "all_gather input");
  TORCH_CHECK(input.is_cuda() && output.is_cuda(), "moodist: all_gather_cast needs CUDA tensors");
  TORCH_CHECK(output.numel() == input.numel() * size_, "moodist: all_gather output must be world_size x input");
  c10::cuda::CUDAGuard guard(input.device());
  auto stream = c10::cuda::getCurrentCUDAStream();
  MOODIST_TRANSLATE(cudaGroup(input.get_device())
                        .all_gather(input.data_ptr(), output.data_ptr(), input.numel(),
                                    dtype_code(input.scalar_type()), dtype_code(output.scalar_type()), raw(stream));)
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::allgather(std::vector<std::vector<at::Tensor>>& outputs,
                                                         std::vector<at::Tensor>& inputs,
                                                         const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(inputs.size() == 1 && outputs.size() == 1, "moodist: all_gather takes one tensor per rank");
  auto& outs = outputs[0];
  TORCH_CHECK((int)outs.size() == size_, "moodist: all_gather output list must have world_size entries");
  at::Tensor in = inputs[0].contiguous();
  // Ranks may contribute different amounts (the output list says how much each one sends, and is the same on every
  // rank): everybody then gathers slots of the largest size. Checked before anything is sent, so that a wrong
  // list is an exception here and not a rejected transfer on some other rank.
  TORCH_CHECK(outs[rank_].numel() == in.numel(), "moodist: all_gather output ", rank_, " has ", outs[rank_].numel(),
              " elements but this rank's input has ", in.numel());
  int64_t slot = 0;
  for (auto& o : outs) {
    TORCH_CHECK(o.scalar_type() == in.scalar_type() && o.device() == in.device(),
                "moodist: all_gather outputs must have the input's dtype and device");
    slot = std::max<int64_t>(slot, o.numel());
  }
  at::Tensor padded = in.reshape({-1});
  if (in.numel() != slot) {
    padded = at::empty({slot}, in.options());
    padded.narrow(0, 0, in.numel()).copy_(in.reshape({-1}), in.is_cuda());
  }
  // gather into one buffer, then hand the pieces out (reference: wrapper/processgroup_wrapper.cc:111-129)
  at::Tensor flat = at::empty({size_ * slot}, in.options());
  auto work = _allgather_base(flat, padded, opts);
  if (in.is_cuda()) {
    c10::cuda::CUDAGuard guard(in.device());
    for (int r = 0; r < size_; ++r) outs[r].copy_(flat.narrow(0, r * slot, outs[r].numel()).view_as(outs[r]), true);
    return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::ALLGATHER, outs, c10::cuda::getCurrentCUDAStream());
  }
  for (int r = 0; r < size_; ++r) outs[r].copy_(flat.narrow(0, r * slot, outs[r].numel()).view_as(outs[r]));
  return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::ALLGATHER, outs);
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::allgather_coalesced(std::vector<std::vector<at::Tensor>>& output_lists,
                                                                   std::vector<at::Tensor>& inputs,
                                                                   const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(output_lists.size() == inputs.size(), "moodist: all_gather_coalesced list size mismatch");
  c10::intrusive_ptr<c10d::Work> last;
  for (size_t i = 0; i < inputs.size(); ++i) {
    std::vector<std::vector<at::Tensor>> outs{output_lists[i]};
    std::vector<at::Tensor> in{inputs[i]};
    last = allgather(outs, in, opts);
  }
  if (!last) return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::ALLGATHER_COALESCED, std::vector<at::Tensor>{});
  return last;
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::endCoalescing() {
  bool on_gpu = false;
  {
    std::lock_guard<std::mutex> lk(mu_);
    on_gpu = cuda_ != nullptr;
  }
  if (on_gpu) {
    c10::cuda::CUDAGuard guard((c10::DeviceIndex)cuda_->device());
    return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::COALESCED, std::vector<at::Tensor>{},
                                         c10::cuda::getCurrentCUDAStream());
  }
  return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::COALESCED, std::vector<at::Tensor>{});
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::allgather_into_tensor_coalesced(std::vector<at::Tensor>& outputs,
                                                                               std::vector<at::Tensor>& inputs,
                                                                               const c10d::AllgatherOptions& opts) {
  TORCH_CHECK(outputs.size() == inputs.size(), "moodist: coalesced all_gather list size mismatch");
  c10::intrusive_ptr<c10d::Work> last;
  for (size_t i = 0; i < inputs.size(); ++i) last = _allgather_base(outputs[i], inputs[i], opts);
  if (!last) return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::ALLGATHER_COALESCED, outputs);
  return last;
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::_reduce_scatter_base(at::Tensor& output, at::Tensor& input,
                                                                    const c10d::ReduceScatterOptions& opts) {
  check_contig(output, "reduce_scatter output");
  check_contig(input, "reduce_scatter input");
  TORCH_CHECK(output.device() == input.device(), "moodist: reduce_scatter tensors must be on the same device");
  TORCH_CHECK(output.scalar_type() == input.scalar_type(), "moodist: reduce_scatter dtype mismatch");
  TORCH_CHECK(input.numel() == output.numel() * size_, "moodist: reduce_scatter input must be world_size x output");
  auto [op, premul] = reduce_code(opts.reduceOp);
  op = bool_op(input.scalar_type(), op);
  int dt = dtype_code(input.scalar_type());
  if (input.is_cuda()) {
    check_cuda_op(op);
    c10::cuda::CUDAGuard guard(input.device());
    auto stream = c10::cuda::getCurrentCUDAStream();
    MOODIST_TRANSLATE(cudaGroup(input.get_device())
                          .reduce_scatter(input.data_ptr(), output.data_ptr(), output.numel(), dt, dt, op,
                                          (float)premul, raw(stream));)
    return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::_REDUCE_SCATTER_BASE, std::vector<at::Tensor>{output},
                                         stream);
  }
  MOODIST_TRANSLATE(hostGroup().reduce_scatter(input.data_ptr(), output.data_ptr(), output.numel(), dt, op, premul);)
  return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::_REDUCE_SCATTER_BASE, std::vector<at::Tensor>{output});
}

void MoodistBackend::reduceScatterCast(at::Tensor& output, const at::Tensor& input, int op, double premul) {
  check_contig(output, "reduce_scatter output");
  check_contig(input, "reduce_scatter input");
  TORCH_CHECK(input.is_cuda() && output.is_cuda(), "moodist: reduce_scatter_cast needs CUDA tensors");
  check_cuda_op(op);
  TORCH_CHECK(input.numel() == output.numel() * size_, "moodist: reduce_scatter input must be world_size x output");
  c10::cuda::CUDAGuard guard(input.device());
  auto stream = c10::cuda::getCurrentCUDAStream();
  MOODIST_TRANSLATE(cudaGroup(input.get_device())
                        .reduce_scatter(input.data_ptr(), output.data_ptr(), output.numel(),
                                        dtype_code(input.scalar_type()), dtype_code(output.scalar_type()), op,
                                        (float)premul, raw(stream));)
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::reduce_scatter(std::vector<at::Tensor>& outputs,
                                                              std::vector<std::vector<at::Tensor>>& inputs,
                                                              const c10d::ReduceScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == 1 && inputs.size() == 1, "moodist: reduce_scatter takes one output per rank");
  TORCH_CHECK((int)inputs[0].size() == size_, "moodist: reduce_scatter input list must have world_size entries");
  std::vector<at::Tensor> flat_list;
  for (auto& t : inputs[0]) flat_list.push_back(t.reshape({-1}));
  at::Tensor flat = at::cat(flat_list);
  at::Tensor out = outputs[0];
  check_contig(out, "reduce_scatter output");
  return _reduce_scatter_base(out, flat, opts);
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::reduce_scatter_tensor_coalesced(
    std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs, const c10d::ReduceScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == inputs.size(), "moodist: coalesced reduce_scatter list size mismatch");
  c10::intrusive_ptr<c10d::Work> last;
  for (size_t i = 0; i < inputs.size(); ++i) last = _reduce_scatter_base(outputs[i], inputs[i], opts);
  if (!last) return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::REDUCE_SCATTER, outputs);
  return last;
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::allreduce(std::vector<at::Tensor>& tensors,
                                                         const c10d::AllreduceOptions& opts) {
  TORCH_CHECK(tensors.size() == 1, "moodist: all_reduce takes one tensor");
  at::Tensor& t = tensors[0];
  check_contig(t, "all_reduce");
  auto [op, premul] = reduce_code(opts.reduceOp);
  op = bool_op(t.scalar_type(), op);
  int dt = dtype_code(t.scalar_type());
  if (t.is_cuda()) {
    check_cuda_op(op);
    c10::cuda::CUDAGuard guard(t.device());
    auto stream = c10::cuda::getCurrentCUDAStream();
    MOODIST_TRANSLATE(cudaGroup(t.get_device())
                          .all_reduce(t.data_ptr(), t.data_ptr(), t.numel(), dt, op, (float)premul, raw(stream));)
    return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::ALLREDUCE, tensors, stream);
  }
  MOODIST_TRANSLATE(hostGroup().all_reduce(t.data_ptr(), t.data_ptr(), t.numel(), dt, op, premul);)
  return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::ALLREDUCE, tensors);
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::allreduce_coalesced(std::vector<at::Tensor>& tensors,
                                                                   const c10d::AllreduceCoalescedOptions& opts) {
  c10::intrusive_ptr<c10d::Work> last;
  for (auto& t : tensors) {
    std::vector<at::Tensor> one{t};
    last = allreduce(one, opts);
  }
  if (!last) return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::ALLREDUCE_COALESCED, tensors);
  return last;
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::broadcast(std::vector<at::Tensor>& tensors,
                                                         const c10d::BroadcastOptions& opts) {
  TORCH_CHECK(tensors.size() == 1, "moodist: broadcast takes one tensor");
  at::Tensor& t = tensors[0];
  check_contig(t, "broadcast");
  int root = (int)opts.rootRank;
  TORCH_CHECK(root >= 0 && root < size_, "moodist: bad broadcast root");
  if (t.is_cuda()) {
    c10::cuda::CUDAGuard guard(t.device());
    auto stream = c10::cuda::getCurrentCUDAStream();
    MOODIST_TRANSLATE(cudaGroup(t.get_device()).broadcast(t.data_ptr(), t.nbytes(), root, raw(stream));)
    return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::BROADCAST, tensors, stream);
  }
  MOODIST_TRANSLATE(hostGroup().broadcast(t.data_ptr(), t.nbytes(), root);)
  return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::BROADCAST, tensors);
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& opts) {
  // reduce = all_reduce into a temporary, root keeps it (the reference supports CUDA SUM only,
  // core/processgroup.cc:1937-1956; every op the kernels know works here)
  TORCH_CHECK(tensors.size() == 1, "moodist: reduce takes one tensor");
  at::Tensor& t = tensors[0];
  check_contig(t, "reduce");
  at::Tensor tmp = t.clone();
  std::vector<at::Tensor> one{tmp};
  c10d::AllreduceOptions ao;
  ao.reduceOp = opts.reduceOp;
  auto w = allreduce(one, ao);
  if (rank_ == (int)opts.rootRank) {
    if (t.is_cuda()) {
      c10::cuda::CUDAGuard guard(t.device());
      t.copy_(tmp, true);
      return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::REDUCE, tensors, c10::cuda::getCurrentCUDAStream());
    }
    t.copy_(tmp);
  }
  return w;
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::gather(std::vector<std::vector<at::Tensor>>& outputs,
                                                      std::vector<at::Tensor>& inputs, const c10d::GatherOptions& opts) {
  TORCH_CHECK(inputs.size() == 1, "moodist: gather takes one input tensor");
  at::Tensor in = inputs[0].contiguous();
  int root = (int)opts.rootRank;
  if (in.is_cuda()) {
    // CUDA gather = all_gather, root keeps the result (the reference throws for CUDA, core/processgroup.cc:2198-2262)
    c10::cuda::CUDAGuard guard(in.device());
    at::Tensor flat = at::empty({size_ * in.numel()}, in.options());
    _allgather_base(flat, in);
    if (rank_ == root) {
      TORCH_CHECK(outputs.size() == 1 && (int)outputs[0].size() == size_, "moodist: gather output list size");
      for (int r = 0; r < size_; ++r)
        outputs[0][r].copy_(flat.narrow(0, r * in.numel(), in.numel()).view_as(in), true);
    }
    return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::GATHER, std::vector<at::Tensor>{},
                                         c10::cuda::getCurrentCUDAStream());
  }
  at::Tensor flat;
  if (rank_ == root) flat = at::empty({size_ * in.numel()}, in.options());
  MOODIST_TRANSLATE(hostGroup().gather(in.data_ptr(), rank_ == root ? flat.data_ptr() : nullptr, in.nbytes(), root);)
  if (rank_ == root) {
    TORCH_CHECK(outputs.size() == 1 && (int)outputs[0].size() == size_, "moodist: gather output list size");
    for (int r = 0; r < size_; ++r) outputs[0][r].copy_(flat.narrow(0, r * in.numel(), in.numel()).view_as(in));
  }
  return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::GATHER, std::vector<at::Tensor>{});
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::scatter(std::vector<at::Tensor>& outputs,
                                                       std::vector<std::vector<at::Tensor>>& inputs,
                                                       const c10d::ScatterOptions& opts) {
  TORCH_CHECK(outputs.size() == 1, "moodist: scatter takes one output tensor");
  at::Tensor& out = outputs[0];
  check_contig(out, "scatter output");
  int root = (int)opts.rootRank;
  at::Tensor flat;
  if (rank_ == root) {
    TORCH_CHECK(inputs.size() == 1 && (int)inputs[0].size() == size_, "moodist: scatter input list size");
    std::vector<at::Tensor> fl;
    for (auto& t : inputs[0]) {
      TORCH_CHECK(t.numel() == out.numel() && t.scalar_type() == out.scalar_type(),
                  "moodist: scatter inputs must have the output's size and dtype");
      fl.push_back(t.reshape({-1}));
    }
    flat = at::cat(fl);
  }
  if (out.is_cuda()) {
    // CUDA scatter rides on the uneven all-to-all: only the root sends
    c10::cuda::CUDAGuard guard(out.device());
    auto stream = c10::cuda::getCurrentCUDAStream();
    std::vector<uint64_t> so(size_, 0), sb(size_, 0), ro(size_, 0), rb(size_, 0);
    if (rank_ == root)
      for (int r = 0; r < size_; ++r) {
        so[r] = (uint64_t)r * out.nbytes();
        sb[r] = out.nbytes();
      }
    rb[root] = out.nbytes();
    if (rank_ != root) flat = at::empty({1}, out.options());
    MOODIST_TRANSLATE(cudaGroup(out.get_device())
                          .all_to_all(flat.data_ptr(), out.data_ptr(), so.data(), sb.data(), ro.data(), rb.data(),
                                      raw(stream));)
    return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::SCATTER, outputs, stream);
  }
  MOODIST_TRANSLATE(hostGroup().scatter(rank_ == root ? flat.data_ptr() : nullptr, out.data_ptr(), out.nbytes(), root);)
  return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::SCATTER, outputs);
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::alltoall_base(at::Tensor& output, at::Tensor& input,
                                                             std::vector<int64_t>& outputSplitSizes,
                                                             std::vector<int64_t>& inputSplitSizes,
                                                             const c10d::AllToAllOptions&) {
  // Split sizes count rows of dim 0. The reference ignores them (wrapper/processgroup_wrapper.cc:265-283);
  // here uneven splits are the point (MoE dispatch / combine).
  check_contig(output, "all_to_all output");
  check_contig(input, "all_to_all input");
  TORCH_CHECK(output.scalar_type() == input.scalar_type(), "moodist: all_to_all dtype mismatch");
  auto row_bytes = [](const at::Tensor& t) -> uint64_t {
    return t.dim() == 0 || t.size(0) == 0 ? t.element_size() : (uint64_t)t.nbytes() / t.size(0);
  };
  std::vector<uint64_t> so(size_), sb(size_), ro(size_), rb(size_);
  uint64_t irb = row_bytes(input), orb = row_bytes(output);
  uint64_t acc = 0;
  for (int r = 0; r < size_; ++r) {
    uint64_t rows;
    if (inputSplitSizes.empty()) {
      TORCH_CHECK(input.size(0) % size_ == 0, "moodist: all_to_all input dim 0 must divide by world size");
      rows = input.size(0) / size_;
    } else {
      TORCH_CHECK((int)inputSplitSizes.size() == size_, "moodist: input split sizes must have world_size entries");
      rows = inputSplitSizes[r];
    }
    so[r] = acc;
    sb[r] = rows * irb;
    acc += sb[r];
  }
  TORCH_CHECK(acc == (uint64_t)input.nbytes(), "moodist: input split sizes do not add up to the input size");
  acc = 0;
  for (int r = 0; r < size_; ++r) {
    uint64_t rows;
    if (outputSplitSizes.empty()) {
      TORCH_CHECK(output.size(0) % size_ == 0, "moodist: all_to_all output dim 0 must divide by world size");
      rows = output.size(0) / size_;
    } else {
      TORCH_CHECK((int)outputSplitSizes.size() == size_, "moodist: output split sizes must have world_size entries");
      rows = outputSplitSizes[r];
    }
    ro[r] = acc;
    rb[r] = rows * orb;
    acc += rb[r];
  }
  TORCH_CHECK(acc == (uint64_t)output.nbytes(), "moodist: output split sizes do not add up to the output size");
  if (input.is_cuda()) {
    c10::cuda::CUDAGuard guard(input.device());
    auto stream = c10::cuda::getCurrentCUDAStream();
    MOODIST_TRANSLATE(cudaGroup(input.get_device())
                          .all_to_all(input.data_ptr(), output.data_ptr(), so.data(), sb.data(), ro.data(), rb.data(),
                                      raw(stream));)
    return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::ALLTOALL_BASE, std::vector<at::Tensor>{output}, stream);
  }
  MOODIST_TRANSLATE(
      hostGroup().all_to_all(input.data_ptr(), output.data_ptr(), so.data(), sb.data(), ro.data(), rb.data());)
  return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::ALLTOALL_BASE, std::vector<at::Tensor>{output});
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::alltoall(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
                                                        const c10d::AllToAllOptions& opts) {
  TORCH_CHECK((int)outputs.size() == size_ && (int)inputs.size() == size_, "moodist: all_to_all list sizes");
  std::vector<at::Tensor> fl;
  std::vector<int64_t> in_split, out_split;
  for (auto& t : inputs) {
    fl.push_back(t.reshape({-1}));
    in_split.push_back(t.numel());
  }
  at::Tensor in = at::cat(fl);
  int64_t total = 0;
  for (auto& t : outputs) {
    out_split.push_back(t.numel());
    total += t.numel();
  }
  at::Tensor out = at::empty({total}, outputs[0].options());
  auto w = alltoall_base(out, in, out_split, in_split, opts);
  int64_t off = 0;
  bool cuda = out.is_cuda();
  c10::optional<c10::cuda::CUDAGuard> guard;
  if (cuda) guard.emplace(out.device());
  for (auto& t : outputs) {
    t.copy_(out.narrow(0, off, t.numel()).view_as(t), cuda);
    off += t.numel();
  }
  if (cuda) return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::ALLTOALL, outputs, c10::cuda::getCurrentCUDAStream());
  return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::ALLTOALL, outputs);
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::barrier(const c10d::BarrierOptions& opts) {
  // CPU-side barrier through the engine, plus a device barrier when this group already runs on a GPU
  bool use_cuda = false;
  {
    std::lock_guard<std::mutex> lk(mu_);
    use_cuda = cuda_ != nullptr;
  }
  if (use_cuda || (opts.device.has_value() && opts.device->is_cuda())) {
    cudaBarrier();
    return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::BARRIER, std::vector<at::Tensor>{});
  }
  MOODIST_TRANSLATE(hostGroup().barrier();)
  return c10::make_intrusive<DoneWork>(rank_, c10d::OpType::BARRIER, std::vector<at::Tensor>{});
}

// CUDA descriptors and host payloads of one (source, tag) pair must never be mistaken for one another
static constexpr uint32_t kCudaTagBit = 0x80000000u;

c10::intrusive_ptr<c10d::Work> MoodistBackend::send(std::vector<at::Tensor>& tensors, int dstRank, int tag) {
  TORCH_CHECK(tensors.size() == 1, "moodist: send takes one tensor");
  TORCH_CHECK(dstRank >= 0 && dstRank < size_ && dstRank != rank_, "moodist: send: bad destination rank ", dstRank);
  at::Tensor t = tensors[0];
  check_contig(t, "send");
  if (t.is_cuda()) {
    if (CudaP2P* p2p = cudaP2P(t.get_device())) {
      // Nothing here waits for the GPU: the bytes become readable to the receiver in stream order, a flag kernel
      // tells it when, and only the small descriptor travels through the host path.
      c10::cuda::CUDAGuard guard(t.device());
      auto stream = c10::cuda::getCurrentCUDAStream();
      MOODIST_TRANSLATE(CudaItemDescriptor d = p2p->publish(t, 1, stream.stream());
                        hostGroup().send(&d, sizeof(d), dstRank, (uint32_t)tag ^ kCudaTagBit);)
      return c10::make_intrusive<CudaWork>(rank_, c10d::OpType::SEND, tensors, stream);
    }
  }
  at::Tensor host = t.is_cuda() ? t.cpu() : t;  // .cpu() synchronises with the producing stream
  // posted, not waited for: a large payload stays where it is until the receiver fetches it, and a rank that posts
  // its sends before its receives (isend, then irecv) must not sit here until the other side gets to its receive
  std::shared_ptr<void> posted;
  MOODIST_TRANSLATE(posted = hostGroup().send_post(host.data_ptr(), (size_t)host.nbytes(), dstRank, (uint32_t)tag,
                                                   std::make_shared<at::Tensor>(host));)
  auto self = c10::intrusive_ptr<MoodistBackend>::unsafe_reclaim_from_nonowning(this);
  return c10::make_intrusive<RecvWork>(rank_, tensors, self, posted, nullptr, true);
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::recv(std::vector<at::Tensor>& tensors, int srcRank, int tag) {
  TORCH_CHECK(tensors.size() == 1, "moodist: recv takes one tensor");
  TORCH_CHECK(srcRank >= 0 && srcRank < size_ && srcRank != rank_, "moodist: recv: bad source rank ", srcRank);
  at::Tensor t = tensors[0];
  check_contig(t, "recv");
  auto self = c10::intrusive_ptr<MoodistBackend>::unsafe_reclaim_from_nonowning(this);
  if (t.is_cuda()) {
    if (CudaP2P* p2p = cudaP2P(t.get_device())) {
      // The host part is the descriptor only (the sender posts it when it calls send, whatever its stream is still
      // busy with); once wait() has it, the data follows in stream order on the stream that was current here.
      auto stream = c10::cuda::getCurrentCUDAStream(t.get_device());
      auto d = std::make_shared<CudaItemDescriptor>();
      std::shared_ptr<void> posted;
      MOODIST_TRANSLATE(posted = hostGroup().recv_post(d.get(), sizeof(*d), srcRank, (uint32_t)tag ^ kCudaTagBit, d);)
      auto after = [p2p, d, t, stream]() {
        c10::cuda::CUDAGuard guard(t.device());
        TORCH_CHECK(d->magic == kCudaItemMagic && d->bytes == (uint64_t)t.nbytes(), "moodist: recv: the sender's tensor has ",
                    d->bytes, " bytes, this one ", t.nbytes());
        MOODIST_TRANSLATE(p2p->fetch(*d, t.data_ptr(), stream.stream());)
        // whoever waits may be on another stream: order it behind the copy
        at::cuda::CUDAEvent landed;
        landed.record(stream);
        landed.block(c10::cuda::getCurrentCUDAStream(t.get_device()));
      };
      return c10::make_intrusive<RecvWork>(rank_, tensors, self, posted, after);
    }
    // no device path between the two ranks yet: through pinned host memory
    at::Tensor host = at::empty(t.sizes(), t.options().device(at::kCPU).pinned_memory(true));
    std::shared_ptr<void> posted;
    MOODIST_TRANSLATE(posted = hostGroup().recv_post(host.data_ptr(), (size_t)host.nbytes(), srcRank, (uint32_t)tag,
                                                     std::make_shared<at::Tensor>(host));)
    auto after = [t, host]() mutable { t.copy_(host); };  // blocking copy: `host` may be released afterwards
    return c10::make_intrusive<RecvWork>(rank_, tensors, self, posted, after);
  }
  std::shared_ptr<void> posted;
  MOODIST_TRANSLATE(posted = hostGroup().recv_post(t.data_ptr(), (size_t)t.nbytes(), srcRank, (uint32_t)tag,
                                                   std::make_shared<at::Tensor>(t));)
  return c10::make_intrusive<RecvWork>(rank_, tensors, self, posted, nullptr);
}

c10::intrusive_ptr<c10d::Work> MoodistBackend::recvAnysource(std::vector<at::Tensor>& tensors, int tag) {
  TORCH_CHECK(tensors.size() == 1, "moodist: recv takes one tensor");
  at::Tensor t = tensors[0];
  check_contig(t, "recv");
  TORCH_CHECK(!t.is_cuda(), "moodist: a receive from any rank is served for CPU tensors (name the source for a CUDA tensor)");
  auto self = c10::intrusive_ptr<MoodistBackend>::unsafe_reclaim_from_nonowning(this);
  std::shared_ptr<void> posted;
  MOODIST_TRANSLATE(posted = hostGroup().recv_post(t.data_ptr(), (size_t)t.nbytes(), -1, (uint32_t)tag,
                                                   std::make_shared<at::Tensor>(t));)
  return c10::make_intrusive<RecvWork>(rank_, tensors, self, posted, nullptr);
}

void MoodistBackend::cudaBarrier() {
  int dev = cuda_ ? cuda_->device() : (int)c10::cuda::current_device();
  c10::cuda::CUDAGuard guard((c10::DeviceIndex)dev);
  auto stream = c10::cuda::getCurrentCUDAStream();
  MOODIST_TRANSLATE(auto& g = cudaGroup(dev); g.barrier(raw(stream)); stream.synchronize(); g.check_status();)
}

int64_t MoodistBackend::getOption(const std::string& name) {
  GroupOptions& o = opts_;
  if (name == "prefer_kernel_less") return o.prefer_kernel_less;
  if (name == "force_kernel_less") return o.force_kernel_less;
  if (name == "num_chunks") return o.num_chunks;
  if (name == "chunk_size") return o.chunk_size;
  if (name == "method") return o.method;
  TORCH_CHECK(false, "moodist: unknown option ", name);
}

void MoodistBackend::setOption(const std::string& name, int64_t value) {
  GroupOptions& o = opts_;
  if (name == "prefer_kernel_less") o.prefer_kernel_less = (int)value;
  else if (name == "force_kernel_less") o.force_kernel_less = (int)value;
  else if (name == "num_chunks") o.num_chunks = (int)value;
  else if (name == "chunk_size") o.chunk_size = (int)value;
  else if (name == "method") o.method = (int)value;
  else TORCH_CHECK(false, "moodist: unknown option ", name);
  if (cuda_) cuda_->options() = opts_;
}

uint64_t MoodistBackend::kernelLaunches() { return cuda_ ? cuda_->launches() : 0; }

std::vector<OpStat> MoodistBackend::cudaStats(bool wait) { return cuda_ ? cuda_->stats(wait) : std::vector<OpStat>{}; }

std::string MoodistBackend::describe() {
  std::string s = "MoodistBackend(name=" + name_ + ", rank=" + std::to_string(rank_) + "/" + std::to_string(size_);
  if (cuda_) s += ", " + cuda_->describe();
  return s + ")";
}

}  // namespace moodist
