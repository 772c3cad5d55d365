// compile_op_full / CustomOp bindings (reference: wrapper/module.cc:689-804 and CustomOp :1284-1320).
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime_api.h>
#include <torch/extension.h>

#include "bindings.h"
#include "core/compile_plan.h"
#include "core/log.h"
#include "kernels/kernels_api.h"

namespace moodist {
namespace {

namespace py = pybind11;

at::ScalarType parse_dtype(const py::object& dtype) {
  // torch.dtype objects do not convert through pybind here; their str() is stable ("torch.float32")
  std::string s = py::str(dtype).cast<std::string>();
  static const std::pair<const char*, at::ScalarType> table[] = {
      {"torch.float32", at::kFloat},   {"torch.float", at::kFloat},   {"torch.float16", at::kHalf},
      {"torch.half", at::kHalf},       {"torch.bfloat16", at::kBFloat16}, {"torch.float64", at::kDouble},
      {"torch.double", at::kDouble},   {"torch.int32", at::kInt},     {"torch.int", at::kInt},
      {"torch.int64", at::kLong},      {"torch.long", at::kLong},     {"torch.int16", at::kShort},
      {"torch.int8", at::kChar},       {"torch.uint8", at::kByte},    {"torch.bool", at::kBool},
  };
  for (auto& [name, t] : table)
    if (s == name) return t;
  throw std::runtime_error("moodist.compile_op: unsupported dtype " + s);
}

struct PyFuture {
  // All work is finished (CPU) or stream-ordered (CUDA) when the call returns, like the reference's
  // Future whose wait() only orders the stream (core/processgroup.cc:3247-3253).
  std::vector<at::Tensor> outputs;
  void wait() {}
  std::vector<at::Tensor> result() { return outputs; }
};

struct PyCustomOp {
  c10::intrusive_ptr<MoodistBackend> owner;
  std::shared_ptr<RedistributionPlan> plan;
  at::ScalarType dtype;
  uint32_t op_id = 0;
  std::unique_ptr<HostRedistribution> host;

  void check(const std::vector<at::Tensor>& ts, const std::vector<BoxSpec>& specs, const char* what) {
    TORCH_CHECK(ts.size() == specs.size(), "moodist custom op: expected ", specs.size(), " ", what, " tensors, got ",
                ts.size());
    for (size_t i = 0; i < ts.size(); ++i) {
      TORCH_CHECK(ts[i].scalar_type() == dtype, "moodist custom op: ", what, " ", i, " has dtype ", ts[i].scalar_type(),
                  ", the op was compiled for ", dtype);
      TORCH_CHECK(ts[i].is_contiguous(), "moodist custom op: ", what, " ", i, " must be contiguous");
      TORCH_CHECK(ts[i].numel() == specs[i].numel(), "moodist custom op: ", what, " ", i, " has ", ts[i].numel(),
                  " elements, the op was compiled for ", specs[i].numel());
    }
  }

  std::shared_ptr<PyFuture> call(std::vector<at::Tensor> inputs, std::vector<at::Tensor> outputs) {
    const RedistributionPlan& p = *plan;
    check(inputs, p.inputs[p.rank], "input");
    check(outputs, p.outputs[p.rank], "output");
    bool any_cuda = false, any_cpu = false;
    for (auto* list : {&inputs, &outputs})
      for (auto& t : *list) (t.is_cuda() ? any_cuda : any_cpu) = true;
    TORCH_CHECK(!(any_cuda && any_cpu), "moodist custom op: all tensors must be on the same kind of device");
    auto fut = std::make_shared<PyFuture>();
    fut->outputs = outputs;
    try {
      if (any_cuda)
        run_cuda(inputs, outputs);
      else
        run_host(inputs, outputs);
    } catch (const Error& e) {
      throw std::runtime_error(e.what());
    }
    return fut;
  }

  void run_host(std::vector<at::Tensor>& inputs, std::vector<at::Tensor>& outputs) {
    std::vector<const void*> in;
    std::vector<void*> out;
    for (auto& t : inputs) in.push_back(t.data_ptr());
    for (auto& t : outputs) out.push_back(t.data_ptr());
    if (!host) host = HostRedistribution::create(owner->hostGroup(), plan, op_id);
    py::gil_scoped_release nogil;
    host->run(in, out);
  }

  void run_cuda(std::vector<at::Tensor>& inputs, std::vector<at::Tensor>& outputs) {
    const RedistributionPlan& p = *plan;
    int device = -1;
    for (auto* list : {&inputs, &outputs})
      for (auto& t : *list) device = t.get_device();
    if (device < 0) device = (int)c10::cuda::current_device();  // a rank with no tensors still takes part
    c10::cuda::CUDAGuard guard((c10::DeviceIndex)device);
    auto stream = c10::cuda::getCurrentCUDAStream();
    CudaGroup& g = owner->cudaGroup(device);
    const mb_comm_t* comm = static_cast<const mb_comm_t*>(g.comm_struct());
    uint64_t need = 0;
    for (uint64_t b : p.stage_bytes) need = std::max(need, b);
    if (p.world > 1 && need > comm->staging_bytes / 2)
      fail(strf("compile_op: the largest rank stages %llu bytes, the staging area holds %llu per op; raise MOODIST_STAGING_MB",
                (unsigned long long)need, (unsigned long long)(comm->staging_bytes / 2)));
    std::vector<mb_stage_copy_t> stage;
    std::vector<mb_piece_t> pieces;
    bool remote_readers = false;
    for (auto& rd : p.readers) remote_readers |= !rd.empty();
    if (remote_readers)
      for (size_t i = 0; i < inputs.size(); ++i)
        stage.push_back(mb_stage_copy_t{inputs[i].data_ptr(), p.stage_offset[p.rank][i], (uint64_t)inputs[i].nbytes()});
    // The kernel's grid must be the same on every rank (each CTA waits for the READY word of the same CTA index
    // of every peer), so it is sized from the largest box of ANY rank, which all ranks know from the plan;
    // what this rank alone stages or copies may be far smaller (or nothing).
    uint64_t biggest = 1;
    for (auto* side : {&p.inputs, &p.outputs})
      for (auto& per_rank : *side)
        for (const BoxSpec& bx : per_rank) biggest = std::max<uint64_t>(biggest, (uint64_t)bx.numel() * p.elem_size);
    for (const CopyPiece& pc : p.pieces) {
      mb_piece_t q{};
      q.src_rank = pc.src_rank;
      q.rows = (uint32_t)pc.rows;
      q.src_off = p.stage_offset[pc.src_rank][pc.src_input] + pc.src_offset;
      q.src_local = pc.src_rank == p.rank ? (const uint8_t*)inputs[pc.src_input].data_ptr() + pc.src_offset : nullptr;
      q.dst = (uint8_t*)outputs[pc.dst_output].data_ptr() + pc.dst_offset;
      q.row_bytes = pc.row_bytes;
      q.src_pitch = pc.src_pitch;
      q.dst_pitch = pc.dst_pitch;
      pieces.push_back(q);
    }
    CUstream_st* raw = reinterpret_cast<CUstream_st*>(stream.stream());
    uint32_t seq = g.next_seq(raw);  // orders this op after the group's earlier ones before scratch is reused
    size_t sbytes = stage.size() * sizeof(mb_stage_copy_t), pbytes = pieces.size() * sizeof(mb_piece_t);
    uint8_t* scratch = static_cast<uint8_t*>(g.scratch(sbytes + pbytes + 64));
    size_t poff = (sbytes + 15) & ~(size_t)15;
    if (sbytes) TORCH_CHECK(cudaMemcpyAsync(scratch, stage.data(), sbytes, cudaMemcpyHostToDevice, stream.stream()) == cudaSuccess);
    if (pbytes) TORCH_CHECK(cudaMemcpyAsync(scratch + poff, pieces.data(), pbytes, cudaMemcpyHostToDevice, stream.stream()) == cudaSuccess);
    // (a one-rank group runs the same kernel: all its pieces are local, no peer is waited for)
    int rc = mb_gather_scatter(comm, seq, reinterpret_cast<mb_stage_copy_t*>(scratch), (int)stage.size(),
                               reinterpret_cast<mb_piece_t*>(scratch + poff), (int)pieces.size(), biggest, stream.stream());
    g.finish_op(raw);
    if (rc != MB_OK) fail("compile_op: the gather/scatter kernel could not be launched");
  }
};

}  // namespace

void bind_custom_op(pybind11::module_& m, BackendClass& backend) {
  py::class_<PyFuture, std::shared_ptr<PyFuture>>(m, "Future").def("wait", &PyFuture::wait).def("result", &PyFuture::result);
  py::class_<PyCustomOp, std::shared_ptr<PyCustomOp>>(m, "CustomOp")
      .def("__call__", &PyCustomOp::call, py::arg("inputs"), py::arg("outputs"))
      .def("num_pieces", [](PyCustomOp& s) { return s.plan->pieces.size(); })
      .def("pieces", [](PyCustomOp& s) {
        py::list out;
        for (const CopyPiece& p : s.plan->pieces)
          out.append(py::make_tuple(p.src_rank, p.src_input, p.dst_output, p.rows, p.row_bytes, p.src_offset, p.src_pitch,
                                    p.dst_offset, p.dst_pitch));
        return out;
      });

  backend.def(
      "compile_op_full",
      [](c10::intrusive_ptr<MoodistBackend> self, std::vector<int64_t> shape, py::object dtype,
         std::vector<std::tuple<int, std::vector<int64_t>, std::vector<int64_t>>> inputs,
         std::vector<std::tuple<int, std::vector<int64_t>, std::vector<int64_t>>> outputs) {
        auto op = std::make_shared<PyCustomOp>();
        op->owner = self;
        op->dtype = parse_dtype(dtype);
        op->op_id = self->nextCustomOpId();
        std::vector<BoxSpec> in, out;
        for (auto& [r, o, s] : inputs) in.push_back(BoxSpec{r, o, s});
        for (auto& [r, o, s] : outputs) out.push_back(BoxSpec{r, o, s});
        try {
          op->plan = std::make_shared<RedistributionPlan>(
              plan_redistribution(shape, c10::elementSize(op->dtype), in, out, self->rank(), self->size()));
        } catch (const Error& e) {
          throw std::runtime_error(e.what());
        }
        return op;
      },
      py::arg("shape"), py::arg("dtype"), py::arg("inputs"), py::arg("outputs"));
}

}  // namespace moodist
