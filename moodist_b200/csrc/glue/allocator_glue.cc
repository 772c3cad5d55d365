// enable_cpu_allocator / cpu_allocator_debug / cuda_copy / enable_profiling / set_prefer_kernel_less.
// The CUDA allocator is torch's CUDAPluggableAllocator built here over the mb_cuda_* hooks of the core library
// (alloc, free, record_stream, base allocation) and handed to Python as an allocator object
// (moodist_b200/allocator.py installs it or wraps it in a MemPool); the reference subclasses
// CUDACachingAllocator::CUDAAllocator itself (wrapper/allocator_wrapper.cc:14-199), an interface that changes
// between torch releases.
#include "core/numa.h"
#include "core/topology.h"
#include <c10/core/Allocator.h>
#include <c10/core/CPUAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime_api.h>
#include <torch/csrc/cuda/CUDAPluggableAllocator.h>
#include <torch/extension.h>

#include <mutex>
#include <set>

#include "bindings.h"
#include "core/cpu_allocator.h"
#include "core/log.h"

extern "C" {
void* mb_cuda_alloc(ssize_t size, int device, cudaStream_t stream);
void mb_cuda_free(void* ptr, ssize_t size, int device, cudaStream_t stream);
void mb_cuda_record_stream(void* ptr, cudaStream_t stream);
void* mb_cuda_base_allocation(void* ptr, size_t* size);
}

namespace moodist {
namespace {

// torch's pluggable CUDA allocator over the symmetric heap, with the hooks Python's CUDAPluggableAllocator
// cannot set: record_stream (a block used on a side stream is not reused before that stream is done with it)
// and the base-allocation query (reference: wrapper/allocator_wrapper.cc:92-100, getBaseAllocation).
std::shared_ptr<c10::cuda::CUDACachingAllocator::CUDAAllocator> cuda_allocator() {
  static std::shared_ptr<c10::cuda::CUDACachingAllocator::CUDAAllocator> alloc = [] {
    auto a = std::make_shared<torch::cuda::CUDAPluggableAllocator::CUDAPluggableAllocator>(
        [](size_t n, int dev, cudaStream_t s) { return mb_cuda_alloc((ssize_t)n, dev, s); },
        [](void* p, size_t n, int dev, cudaStream_t s) { mb_cuda_free(p, (ssize_t)n, dev, s); });
    a->set_record_stream_fn([](void* p, cudaStream_t s) { mb_cuda_record_stream(p, s); });
    a->set_base_alloc_fn([](void* p, size_t* n) { return mb_cuda_base_allocation(p, n); });
    return std::static_pointer_cast<c10::cuda::CUDACachingAllocator::CUDAAllocator>(a);
  }();
  return alloc;
}

void delete_cpu(void* p) { cpu_free(p); }

struct MoodistCpuAllocator final : c10::Allocator {
  c10::DataPtr allocate(size_t n) override {
    void* p = n ? cpu_alloc(n) : nullptr;
    TORCH_CHECK(n == 0 || p, "moodist CPU allocator: out of memory allocating ", n, " bytes");
    return {p, p, &delete_cpu, c10::Device(c10::kCPU)};
  }
  c10::DeleterFnPtr raw_deleter() const override { return &delete_cpu; }
  void copy_data(void* dest, const void* src, std::size_t count) const override { default_copy_data(dest, src, count); }
};

MoodistCpuAllocator g_cpu_allocator;
bool g_cpu_enabled = false;

void enable_cpu_allocator() {
  if (g_cpu_enabled) return;
  c10::SetAllocator(c10::kCPU, &g_cpu_allocator, /*priority=*/10);
  g_cpu_enabled = true;
}

// dst.copy_(src) between host and device where the host side may be pageable memory of the CPU allocator:
// its whole region is pinned once (cudaHostRegister) so the copy is truly asynchronous
// (reference: core/cuda_copy.h:14-41).
void cuda_copy(at::Tensor dst, const at::Tensor& src) {
  TORCH_CHECK(dst.is_contiguous() && src.is_contiguous() && dst.nbytes() == src.nbytes(),
              "moodist.cuda_copy: contiguous tensors of equal byte size");
  const at::Tensor& host = dst.is_cuda() ? src : dst;
  const at::Tensor& devt = dst.is_cuda() ? dst : src;
  TORCH_CHECK(devt.is_cuda() && !host.is_cuda(), "moodist.cuda_copy: one CUDA and one CPU tensor");
  c10::cuda::CUDAGuard guard(devt.device());
  void* base = nullptr;
  size_t size = 0;
  static std::mutex mu;
  static std::set<void*> registered;
  if (cpu_allocator_region(host.data_ptr(), &base, &size)) {
    std::lock_guard<std::mutex> lk(mu);
    if (!registered.count(base)) {
      if (cudaHostRegister(base, size, cudaHostRegisterDefault) == cudaSuccess) registered.insert(base);
      cudaGetLastError();
    }
  }
  auto stream = c10::cuda::getCurrentCUDAStream();
  TORCH_CHECK(cudaMemcpyAsync(dst.data_ptr(), src.data_ptr(), dst.nbytes(),
                              dst.is_cuda() ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost, stream.stream()) == cudaSuccess,
              "moodist.cuda_copy: cudaMemcpyAsync failed");
}

}  // namespace

void bind_allocators(pybind11::module_& m, BackendClass& backend) {
  m.def("enable_cpu_allocator", &enable_cpu_allocator);
  m.def("cpu_allocator_debug", [] { return cpu_allocator_debug(); });
  m.def("cpu_allocator_owns", [](const at::Tensor& t) { return cpu_allocator_owns(t.data_ptr()); });
  m.def("cuda_copy", &cuda_copy, pybind11::arg("dst"), pybind11::arg("src"));
  // what NVML says about this machine: GPUs, NVLink / PCIe reachability between them, NUMA nodes
  m.def("topology", [] {
    const NodeTopology& t = local_topology();
    pybind11::dict d;
    d["node_id"] = t.node_id;
    d["nvswitch"] = t.nvswitch;
    d["all_p2p"] = t.all_p2p;
    pybind11::list gpus;
    for (auto& g : t.gpus) {
      pybind11::dict e;
      e["index"] = g.index;
      e["pci_bus_id"] = g.pci_bus_id;
      e["numa_node"] = g.numa_node;
      e["nvlinks_up"] = g.nvlinks_up;
      e["nvlinks_to_switch"] = g.nvlinks_to_switch;
      gpus.append(e);
    }
    d["gpus"] = gpus;
    static const char* names[] = {"none", "pcie", "nvlink", "self"};
    pybind11::list links;
    for (auto& row : t.link) {
      pybind11::list r;
      for (auto k : row) r.append(names[(int)k]);
      links.append(r);
    }
    d["links"] = links;
    d["text"] = t.describe();
    return d;
  });
  m.def("numa_cpus", [](int node) { return cpus_of_numa_node(node); });
  m.def("bind_thread_to_numa_node", [](int node) { return bind_thread_to_numa_node(node); });
  // profiling is per group in the engine; the module-level switch applies to every live group
  backend.def("enable_profiling", [](c10::intrusive_ptr<MoodistBackend> self, bool on) {
    pybind11::gil_scoped_release nogil;
    self->hostGroup().set_profiling(on);
    return self->hostGroup().last_trace_path();
  });
  m.def("set_prefer_kernel_less", [](bool v) { MoodistBackend::setDefaultPreferKernelLess(v); });
  m.def("cuda_allocator", &cuda_allocator,
        "the symmetric-heap CUDA allocator as a torch allocator object (for torch.cuda.MemPool or "
        "torch.cuda.memory.change_current_allocator), with record_stream and base-allocation hooks");
  m.def("enable_cuda_allocator", [] {
    // also records the allocator as torch's "current custom allocator", which its deleters go through
    torch::cuda::CUDAPluggableAllocator::changeCurrentAllocator(cuda_allocator());
  });
}

}  // namespace moodist
