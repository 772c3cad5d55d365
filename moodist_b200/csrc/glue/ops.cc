// Tensor-level entry points of the compute kernels (tcgen05 GEMM and the fused collective GEMMs).
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "bindings.h"
#include "kernels/kernels_api.h"

namespace moodist {
namespace {

struct DeviceStatus {
  uint32_t* host = nullptr;
  uint32_t* dev = nullptr;
};

// one host-mapped status word per device for kernels launched outside a process group
DeviceStatus& status_word(int device) {
  static DeviceStatus words[64];
  DeviceStatus& w = words[device];
  if (!w.host) {
    TORCH_CHECK(cudaHostAlloc((void**)&w.host, 64, cudaHostAllocMapped) == cudaSuccess, "cudaHostAlloc failed");
    *w.host = 0;
    void* d = nullptr;
    TORCH_CHECK(cudaHostGetDevicePointer(&d, w.host, 0) == cudaSuccess, "cudaHostGetDevicePointer failed");
    w.dev = (uint32_t*)d;
  }
  return w;
}

void check_status(int device) {
  DeviceStatus& w = status_word(device);
  uint32_t st = *(volatile uint32_t*)w.host;
  if (st) {
    *(volatile uint32_t*)w.host = 0;
    TORCH_CHECK(false, "moodist: a GEMM kernel gave up waiting (status 0x", std::hex, st, ")");
  }
}

// out[M,N] = a · b^T. trans_a: `a` is stored [K,M]; trans_b: `b` is stored [K,N].
at::Tensor gemm(const at::Tensor& a, const at::Tensor& b, bool trans_a, bool trans_b, c10::optional<at::Tensor> out,
                bool out_fp32, int64_t epilogue) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda(), "moodist gemm: CUDA tensors required");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "moodist gemm: bf16 inputs");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "moodist gemm: 2-D tensors");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1, "moodist gemm: innermost stride must be 1");
  int64_t M = trans_a ? a.size(1) : a.size(0);
  int64_t K = trans_a ? a.size(0) : a.size(1);
  int64_t N = trans_b ? b.size(1) : b.size(0);
  int64_t Kb = trans_b ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb, "moodist gemm: inner dimensions differ (", K, " vs ", Kb, ")");
  c10::cuda::CUDAGuard guard(a.device());
  at::Tensor c = out.has_value() ? *out
                                 : at::empty({M, N}, a.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  TORCH_CHECK(c.size(0) == M && c.size(1) == N && c.stride(1) == 1, "moodist gemm: bad output tensor");
  TORCH_CHECK(c.scalar_type() == (out_fp32 ? at::kFloat : at::kBFloat16), "moodist gemm: bad output dtype");
  int dev = a.get_device();
  check_status(dev);
  auto stream = c10::cuda::getCurrentCUDAStream();
  int rc = mb_gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0),
                        c.stride(0), trans_a, trans_b, out_fp32, (int)epilogue, status_word(dev).dev, 0,
                        stream.stream());
  TORCH_CHECK(rc == MB_OK, "moodist gemm: launch failed with code ", rc, " (M=", M, " N=", N, " K=", K, ")");
  return c;
}

}  // namespace

void bind_ops(pybind11::module_& m, BackendClass& backend) {
  m.def("gemm", &gemm, pybind11::arg("a"), pybind11::arg("b"), pybind11::arg("trans_a") = false,
        pybind11::arg("trans_b") = false, pybind11::arg("out") = pybind11::none(), pybind11::arg("out_fp32") = false,
        pybind11::arg("epilogue") = 0);
  (void)backend;
}

}  // namespace moodist
