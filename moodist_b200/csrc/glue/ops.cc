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
  m.def("gemm_variant", [](int v) { mb_gemm_set_variant(v); }, pybind11::arg("variant"),
        "0: kernel chosen by shape (two-SM cta_group::2 kernel from 256 rows up); 1: always the one-SM kernel");
  m.def("get_gemm_variant", []() { return mb_gemm_get_variant(); });
  (void)backend;
}

}  // namespace moodist

// ------------------------------------------------------------------------------------------------
// fused collective GEMMs (need a process group)
// ------------------------------------------------------------------------------------------------
namespace moodist {
namespace {

void run_rc(int rc, const char* what) {
  TORCH_CHECK(rc == MB_OK, "moodist ", what, ": ",
              rc == MB_ERR_TOO_BIG ? "operands do not fit the staging area (raise MOODIST_STAGING_MB)"
              : rc == MB_ERR_ARG   ? "unsupported shape (rows must divide by world_size x tile, K and N by 8)"
                                   : "launch failed",
              " (code ", rc, ")");
}

// y = all_gather(x_shard) @ w.T  (gather_weight=false: x_shard [M/world, K], w [N, K])
// y = x @ all_gather(w_shard).T  (gather_weight=true:  x [M, K], w_shard [N/world, K])
// Returns (y, gathered): `gathered` is a view of the staging area holding the gathered operand; it stays
// valid until the collective after next on this group.
std::tuple<at::Tensor, at::Tensor> ag_gemm(c10::intrusive_ptr<MoodistBackend> pg, const at::Tensor& shard,
                                           const at::Tensor& other, bool gather_weight, bool out_fp32, int64_t epilogue,
                                           int64_t comm_ctas, c10::optional<at::Tensor> out) {
  TORCH_CHECK(shard.is_cuda() && other.is_cuda() && shard.scalar_type() == at::kBFloat16 &&
                  other.scalar_type() == at::kBFloat16 && shard.dim() == 2 && other.dim() == 2,
              "moodist ag_gemm: 2-D bf16 CUDA tensors");
  TORCH_CHECK(shard.is_contiguous() && other.stride(1) == 1, "moodist ag_gemm: shard contiguous, other row-contiguous");
  const int world = pg->size();
  const int64_t K = shard.size(1);
  TORCH_CHECK(other.size(1) == K, "moodist ag_gemm: inner dimensions differ");
  const int64_t M = gather_weight ? other.size(0) : shard.size(0) * world;
  const int64_t N = gather_weight ? shard.size(0) * world : other.size(0);
  c10::cuda::CUDAGuard guard(shard.device());
  auto stream = c10::cuda::getCurrentCUDAStream();
  at::Tensor y = out.has_value() ? *out : at::empty({M, N}, shard.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  TORCH_CHECK(y.dim() == 2 && y.size(0) == M && y.size(1) == N && y.is_contiguous() &&
                  y.scalar_type() == (out_fp32 ? at::kFloat : at::kBFloat16),
              "moodist ag_gemm: bad output tensor");
  CudaGroup& g = pg->cudaGroup(shard.get_device());
  const mb_comm_t* comm = static_cast<const mb_comm_t*>(g.comm_struct());
  CUstream_st* raw = reinterpret_cast<CUstream_st*>(stream.stream());
  at::Tensor gathered;
  if (world == 1 && comm->staging_bytes == 0) {
    int rc = mb_gemm_bf16(gather_weight ? other.data_ptr() : shard.data_ptr(), gather_weight ? shard.data_ptr() : other.data_ptr(),
                          y.data_ptr(), (int)M, (int)N, (int)K, gather_weight ? other.stride(0) : K,
                          gather_weight ? K : other.stride(0), N, 0, 0, out_fp32, (int)epilogue, comm->status, 0, raw);
    run_rc(rc, "ag_gemm");
    return {y, shard};
  }
  uint32_t seq = g.next_seq(raw);
  int rc = mb_ag_gemm(comm, seq, shard.data_ptr(), other.data_ptr(), y.data_ptr(), (int)M, (int)N, (int)K, other.stride(0),
                      N, gather_weight ? 1 : 0, 0, out_fp32, (int)epilogue, (int)comm_ctas, raw);
  g.finish_op(raw);
  g.note_op("ag_gemm", gather_weight ? "fused_gather_b" : "fused_gather_a", (size_t)shard.nbytes());
  run_rc(rc, "ag_gemm");
  const int64_t rows = gather_weight ? N : M;
  gathered = at::from_blob(mb_stage_pointer(comm, seq), {rows, K}, shard.options());
  return {y, gathered};
}

// out[M/world, N] = reduce_scatter over rows of (a @ b.T), fp32 accumulation across ranks.
at::Tensor gemm_rs(c10::intrusive_ptr<MoodistBackend> pg, const at::Tensor& a, const at::Tensor& b, bool trans_b,
                   bool out_fp32, double scale) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 &&
                  a.dim() == 2 && b.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1,
              "moodist gemm_rs: 2-D row-contiguous bf16 CUDA tensors");
  const int world = pg->size();
  const int64_t M = a.size(0), K = a.size(1);
  const int64_t N = trans_b ? b.size(1) : b.size(0);
  TORCH_CHECK((trans_b ? b.size(0) : b.size(1)) == K, "moodist gemm_rs: inner dimensions differ");
  c10::cuda::CUDAGuard guard(a.device());
  auto stream = c10::cuda::getCurrentCUDAStream();
  CUstream_st* raw = reinterpret_cast<CUstream_st*>(stream.stream());
  CudaGroup& g = pg->cudaGroup(a.get_device());
  const mb_comm_t* comm = static_cast<const mb_comm_t*>(g.comm_struct());
  at::Tensor out = at::empty({M / world, N}, a.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  if (world == 1 && comm->staging_bytes == 0) {
    TORCH_CHECK(scale == 1.0, "moodist gemm_rs: scale needs more than one rank");
    int rc = mb_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0), N, 0,
                          trans_b, out_fp32, 0, comm->status, 0, raw);
    run_rc(rc, "gemm_rs");
    return out;
  }
  uint32_t seq = g.next_seq(raw);
  int rc = mb_gemm_rs(comm, seq, a.data_ptr(), b.data_ptr(), out.data_ptr(), (int)M, (int)N, (int)K, a.stride(0), b.stride(0),
                      N, trans_b, out_fp32, (float)scale, scale != 1.0, raw);
  g.finish_op(raw);
  g.note_op("gemm_rs", "fused", (size_t)out.nbytes() * world);
  run_rc(rc, "gemm_rs");
  return out;
}

}  // namespace

void bind_fused(pybind11::module_& m) {
  m.def("ag_gemm", &ag_gemm, pybind11::arg("group"), pybind11::arg("shard"), pybind11::arg("other"),
        pybind11::arg("gather_weight") = false, pybind11::arg("out_fp32") = false, pybind11::arg("epilogue") = 0,
        pybind11::arg("comm_ctas") = 0, pybind11::arg("out") = pybind11::none());
  m.def("gemm_rs", &gemm_rs, pybind11::arg("group"), pybind11::arg("a"), pybind11::arg("b"),
        pybind11::arg("trans_b") = false, pybind11::arg("out_fp32") = false, pybind11::arg("scale") = 1.0);
}

}  // namespace moodist
