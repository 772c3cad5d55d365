// c10d::Backend for the "moodist" process group: CUDA tensors go to the sm_100a kernels through
// CudaGroup, CPU tensors to the host engine. One object serves both device types, like the
// reference's wrapper::ProcessGroup / wrapper::Backend pair (wrapper/processgroup_wrapper.cc:91-95,
// wrapper/backend.h:14-125).
#pragma once

#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

#include <memory>
#include <mutex>
#include <string>

#include "core/cuda_group.h"
#include "core/host_group.h"
#include "core/kvstore.h"
#include "core/queue.h"
#include "cuda_p2p.h"

namespace moodist {

// KVStore view of any c10d::Store
class C10dStoreAdapter final : public KVStore {
 public:
  explicit C10dStoreAdapter(c10::intrusive_ptr<c10d::Store> s) : store_(std::move(s)) {}
  void set(const std::string& key, const std::vector<uint8_t>& value) override { store_->set(key, value); }
  std::vector<uint8_t> get(const std::string& key) override { return store_->get(key); }
  bool check(const std::vector<std::string>& keys) override { return store_->check(keys); }
  void wait(const std::vector<std::string>& keys) override { store_->wait(keys); }
  const c10::intrusive_ptr<c10d::Store>& store() const { return store_; }

 private:
  c10::intrusive_ptr<c10d::Store> store_;
};

class MoodistBackend final : public c10d::Backend {
 public:
  MoodistBackend(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size);
  ~MoodistBackend() override;

  const std::string getBackendName() const override { return "moodist"; }
  bool supportsCoalescing() const override { return false; }

  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors,
                                           const c10d::BroadcastOptions& opts = c10d::BroadcastOptions()) override;
  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors,
                                           const c10d::AllreduceOptions& opts = c10d::AllreduceOptions()) override;
  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(
      std::vector<at::Tensor>& tensors,
      const c10d::AllreduceCoalescedOptions& opts = c10d::AllreduceCoalescedOptions()) override;
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors,
                                        const c10d::ReduceOptions& opts = c10d::ReduceOptions()) override;
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputs,
                                           std::vector<at::Tensor>& inputs,
                                           const c10d::AllgatherOptions& opts = c10d::AllgatherOptions()) override;
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& output, at::Tensor& input,
                                                 const c10d::AllgatherOptions& opts = c10d::AllgatherOptions()) override;
  c10::intrusive_ptr<c10d::Work> allgather_coalesced(std::vector<std::vector<at::Tensor>>& output_lists,
                                                     std::vector<at::Tensor>& inputs,
                                                     const c10d::AllgatherOptions& opts = c10d::AllgatherOptions()) override;
  // Operations run as they are issued (in stream order on a GPU), so a coalescing block has nothing to hold back:
  // it starts nothing and ends with a completed work.
  void startCoalescing() override {}
  c10::intrusive_ptr<c10d::Work> endCoalescing() override;
  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(
      std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
      const c10d::AllgatherOptions& opts = c10d::AllgatherOptions()) override;
  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                        const c10d::GatherOptions& opts = c10d::GatherOptions()) override;
  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& outputs,
                                         std::vector<std::vector<at::Tensor>>& inputs,
                                         const c10d::ScatterOptions& opts = c10d::ScatterOptions()) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter(
      std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs,
      const c10d::ReduceScatterOptions& opts = c10d::ReduceScatterOptions()) override;
  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(
      at::Tensor& output, at::Tensor& input,
      const c10d::ReduceScatterOptions& opts = c10d::ReduceScatterOptions()) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(
      std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
      const c10d::ReduceScatterOptions& opts = c10d::ReduceScatterOptions()) override;
  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& output, at::Tensor& input,
                                               std::vector<int64_t>& outputSplitSizes,
                                               std::vector<int64_t>& inputSplitSizes,
                                               const c10d::AllToAllOptions& opts = c10d::AllToAllOptions()) override;
  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
                                          const c10d::AllToAllOptions& opts = c10d::AllToAllOptions()) override;
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& opts = c10d::BarrierOptions()) override;
  // point-to-point: CPU tensors through the host engine; CUDA tensors over NVLink without blocking the sender's
  // host thread (cuda_p2p.h) once the group has run a CUDA collective, through host memory before that
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dstRank, int tag) override;
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int srcRank, int tag) override;
  c10::intrusive_ptr<c10d::Work> recvAnysource(std::vector<at::Tensor>& tensors, int tag) override;

  // ---- moodist-specific surface (reference: wrapper/module.cc:836-849) ----
  std::string moodistName() const { return name_; }
  // Live group with that name in this process, or null (groups register themselves on construction).
  static c10::intrusive_ptr<MoodistBackend> find(const std::string& name);
  // Default of the prefer_kernel_less option for groups created afterwards (moodist.set_prefer_kernel_less).
  static void setDefaultPreferKernelLess(bool v);
  static std::vector<c10::intrusive_ptr<MoodistBackend>> live();
  void cudaBarrier();
  int64_t getOption(const std::string& name);
  void setOption(const std::string& name, int64_t value);
  bool getPreferKernelLess() { return getOption("prefer_kernel_less") != 0; }
  void setPreferKernelLess(bool v) { setOption("prefer_kernel_less", v ? 1 : 0); }
  uint64_t kernelLaunches();
  std::vector<OpStat> cudaStats(bool wait);
  uint32_t nextCustomOpId() { return ++custom_ops_; }  // compile_op is collective: same ids on every rank
  std::string describe();

  // dtype-converting variants used by the sharded-training helpers (fused cast / mixed-precision reduce)
  void allGatherCast(at::Tensor& output, const at::Tensor& input);
  void reduceScatterCast(at::Tensor& output, const at::Tensor& input, int op, double premul);

  CudaGroup& cudaGroup(int device);
  // The NVLink hand-over path for single CUDA tensors (Queue items, send / recv), or null while the group has
  // not run a CUDA collective yet: creating the CUDA group is itself a collective, which a put or a send
  // between two ranks must not start. Until then such tensors are staged through host memory.
  CudaP2P* cudaP2P(int device);
  HostGroup& hostGroup();
  QueueManager& queues();
  KVStore& kv() { return *kv_; }
  int rank() const { return rank_; }
  int size() const { return size_; }

 private:
  c10::intrusive_ptr<c10d::Store> store_;
  std::unique_ptr<C10dStoreAdapter> kv_;
  int rank_, size_;
  std::string name_;
  std::mutex mu_;
  GroupOptions opts_;
  uint32_t custom_ops_ = 0;
  std::unique_ptr<CudaGroup> cuda_;
  std::unique_ptr<HostGroup> host_;
  std::unique_ptr<QueueManager> queues_;  // declared after host_: destroyed first
  std::unique_ptr<CudaP2P> p2p_;          // uses cuda_ and host_: destroyed before both
};

}  // namespace moodist
