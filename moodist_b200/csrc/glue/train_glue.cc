// Tensor-level entry points of the memory-bound training kernels (rotary embedding, SwiGLU,
// cross-entropy, AdamW). CUDA bf16 tensors only; each call is one kernel launch on the current stream.
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "bindings.h"
#include "kernels/kernels_api.h"

namespace moodist {
namespace {

void need_bf16_rows(const at::Tensor& t, const char* what) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1, "moodist ", what,
              ": a CUDA bf16 matrix with contiguous rows is required");
}

void run(int rc, const char* what) {
  TORCH_CHECK(rc == MB_OK, "moodist ", what, ": ",
              rc == MB_ERR_ALIGN ? "pointers and row pitches must be 16-byte aligned"
              : rc == MB_ERR_ARG ? "unsupported shape"
                                 : "launch failed",
              " (code ", rc, ")");
}

void* cur_stream() { return c10::cuda::getCurrentCUDAStream().stream(); }

// x[tokens, >= n_heads*head_dim]: rotate the first n_heads heads in place.
void rope_(at::Tensor x, const at::Tensor& cos, const at::Tensor& sin, int64_t seq, int64_t n_heads, int64_t head_dim,
           bool inverse) {
  need_bf16_rows(x, "rope");
  TORCH_CHECK(cos.is_cuda() && sin.is_cuda() && cos.scalar_type() == at::kFloat && sin.scalar_type() == at::kFloat &&
                  cos.is_contiguous() && sin.is_contiguous(),
              "moodist rope: fp32 contiguous tables required");
  TORCH_CHECK(cos.size(0) >= seq && cos.size(1) == head_dim / 2 && sin.sizes() == cos.sizes(),
              "moodist rope: tables must be [>= seq, head_dim/2]");
  TORCH_CHECK(x.size(1) >= n_heads * head_dim, "moodist rope: rows shorter than n_heads*head_dim");
  c10::cuda::CUDAGuard guard(x.device());
  run(mb_rope_bf16(x.data_ptr(), cos.data_ptr<float>(), sin.data_ptr<float>(), x.size(0), (int)seq, (int)n_heads,
                   (int)head_dim, x.stride(0), inverse, cur_stream()),
      "rope");
}

at::Tensor swiglu_fwd(const at::Tensor& gu) {
  need_bf16_rows(gu, "swiglu");
  TORCH_CHECK(gu.size(1) % 2 == 0, "moodist swiglu: even number of columns required");
  int64_t F = gu.size(1) / 2;
  c10::cuda::CUDAGuard guard(gu.device());
  at::Tensor out = at::empty({gu.size(0), F}, gu.options());
  run(mb_swiglu_fwd_bf16(gu.data_ptr(), out.data_ptr(), gu.size(0), (int)F, gu.stride(0), out.stride(0), cur_stream()),
      "swiglu");
  return out;
}

at::Tensor swiglu_bwd(const at::Tensor& gu, const at::Tensor& dout) {
  need_bf16_rows(gu, "swiglu backward");
  need_bf16_rows(dout, "swiglu backward");
  int64_t F = gu.size(1) / 2;
  TORCH_CHECK(dout.size(0) == gu.size(0) && dout.size(1) == F, "moodist swiglu backward: shape mismatch");
  c10::cuda::CUDAGuard guard(gu.device());
  at::Tensor dgu = at::empty({gu.size(0), 2 * F}, gu.options());
  run(mb_swiglu_bwd_bf16(gu.data_ptr(), dout.data_ptr(), dgu.data_ptr(), gu.size(0), (int)F, gu.stride(0),
                         dout.stride(0), dgu.stride(0), cur_stream()),
      "swiglu backward");
  return dgu;
}

// returns (per-row loss fp32 [rows], lse fp32 [rows])
std::tuple<at::Tensor, at::Tensor> cross_entropy_fwd(const at::Tensor& logits, const at::Tensor& targets,
                                                     int64_t ignore_index) {
  need_bf16_rows(logits, "cross_entropy");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() &&
                  targets.numel() == logits.size(0),
              "moodist cross_entropy: int64 contiguous targets, one per row");
  c10::cuda::CUDAGuard guard(logits.device());
  at::Tensor loss = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  at::Tensor lse = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  run(mb_cross_entropy_fwd_bf16(logits.data_ptr(), targets.data_ptr<int64_t>(), lse.data_ptr<float>(),
                                loss.data_ptr<float>(), logits.size(0), (int)logits.size(1), logits.stride(0),
                                ignore_index, cur_stream()),
      "cross_entropy");
  return {loss, lse};
}

// overwrites logits with d loss / d logits; gscale is a 1-element fp32 CUDA tensor (the incoming gradient)
void cross_entropy_bwd_(at::Tensor logits, const at::Tensor& targets, const at::Tensor& lse, const at::Tensor& gscale,
                        double inv_count, int64_t ignore_index) {
  need_bf16_rows(logits, "cross_entropy backward");
  TORCH_CHECK(gscale.is_cuda() && gscale.scalar_type() == at::kFloat && gscale.numel() == 1,
              "moodist cross_entropy backward: fp32 scalar gradient required");
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.numel() == logits.size(0) && targets.numel() == logits.size(0),
              "moodist cross_entropy backward: shape mismatch");
  c10::cuda::CUDAGuard guard(logits.device());
  run(mb_cross_entropy_bwd_bf16(logits.data_ptr(), targets.data_ptr<int64_t>(), lse.data_ptr<float>(),
                                gscale.data_ptr<float>(), (float)inv_count, logits.size(0), (int)logits.size(1),
                                logits.stride(0), ignore_index, cur_stream()),
      "cross_entropy backward");
}

void adamw_(at::Tensor p, const at::Tensor& g, at::Tensor m, at::Tensor v, double lr, double b1, double b2, double eps,
            double wd, int64_t step, double grad_scale) {
  TORCH_CHECK(p.is_cuda() && p.scalar_type() == at::kBFloat16 && m.scalar_type() == at::kBFloat16 &&
                  v.scalar_type() == at::kBFloat16 && p.is_contiguous() && g.is_contiguous() && m.is_contiguous() &&
                  v.is_contiguous(),
              "moodist adamw: contiguous bf16 parameters and moments required");
  TORCH_CHECK(g.numel() == p.numel() && m.numel() == p.numel() && v.numel() == p.numel(), "moodist adamw: size mismatch");
  int gd = g.scalar_type() == at::kFloat ? MB_F32 : g.scalar_type() == at::kBFloat16 ? MB_BF16 : -1;
  TORCH_CHECK(gd >= 0, "moodist adamw: gradient must be fp32 or bf16");
  c10::cuda::CUDAGuard guard(p.device());
  run(mb_adamw_bf16(p.data_ptr(), g.data_ptr(), gd, m.data_ptr(), v.data_ptr(), p.numel(), (float)lr, (float)b1,
                    (float)b2, (float)eps, (float)wd, (int)step, (float)grad_scale, cur_stream()),
      "adamw");
}

// returns (y, rstd)
std::tuple<at::Tensor, at::Tensor> rmsnorm_fwd(const at::Tensor& x, const at::Tensor& w, double eps) {
  need_bf16_rows(x, "rmsnorm");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kBFloat16 && w.is_contiguous() && w.numel() == x.size(1),
              "moodist rmsnorm: bf16 weight of the row length required");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor y = at::empty({x.size(0), x.size(1)}, x.options());
  at::Tensor rstd = at::empty({x.size(0)}, x.options().dtype(at::kFloat));
  run(mb_rmsnorm_fwd_bf16(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), x.size(0), (int)x.size(1),
                          x.stride(0), y.stride(0), (float)eps, cur_stream()),
      "rmsnorm");
  return {y, rstd};
}

// returns (dx, dw)
std::tuple<at::Tensor, at::Tensor> rmsnorm_bwd(const at::Tensor& x, const at::Tensor& w, const at::Tensor& dy,
                                               const at::Tensor& rstd) {
  need_bf16_rows(x, "rmsnorm backward");
  need_bf16_rows(dy, "rmsnorm backward");
  TORCH_CHECK(dy.sizes() == x.sizes() && rstd.numel() == x.size(0) && rstd.scalar_type() == at::kFloat,
              "moodist rmsnorm backward: shape mismatch");
  c10::cuda::CUDAGuard guard(x.device());
  at::Tensor dx = at::empty({x.size(0), x.size(1)}, x.options());
  at::Tensor dw = at::empty({x.size(1)}, x.options());
  at::Tensor part = at::empty({(int64_t)mb_rmsnorm_bwd_parts(x.size(0)), x.size(1)}, x.options().dtype(at::kFloat));
  run(mb_rmsnorm_bwd_bf16(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(),
                          part.data_ptr<float>(), dw.data_ptr(), x.size(0), (int)x.size(1), x.stride(0), dy.stride(0),
                          dx.stride(0), cur_stream()),
      "rmsnorm backward");
  return {dx, dw};
}

}  // namespace

void bind_train_ops(pybind11::module_& m) {
  namespace py = pybind11;
  m.def("rope_", &rope_, py::arg("x"), py::arg("cos"), py::arg("sin"), py::arg("seq"), py::arg("n_heads"),
        py::arg("head_dim"), py::arg("inverse") = false);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("cross_entropy_fwd", &cross_entropy_fwd, py::arg("logits"), py::arg("targets"), py::arg("ignore_index") = -100);
  m.def("cross_entropy_bwd_", &cross_entropy_bwd_);
  m.def("adamw_", &adamw_);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("rmsnorm_max_dim", [] { return mb_rmsnorm_max_dim(); });
}

}  // namespace moodist
