// Hooks through which the other glue translation units add their bindings to the module.
#pragma once

#include <torch/extension.h>

#include "backend.h"

namespace moodist {

using BackendClass = pybind11::class_<MoodistBackend, c10d::Backend, c10::intrusive_ptr<MoodistBackend>>;

// ops.cc: GEMM and fused ops
void bind_ops(pybind11::module_& m, BackendClass& backend);
void bind_fused(pybind11::module_& m);
void bind_train_ops(pybind11::module_& m);

// store_glue.cc: TcpStore
void bind_store(pybind11::module_& m);

// queue_glue.cc: Queue, QueueWork, MoodistBackend.Queue
void bind_queue(pybind11::module_& m, BackendClass& backend);

// custom_op.cc: compile_op_full, CustomOp, Future
void bind_custom_op(pybind11::module_& m, BackendClass& backend);

// allocator_glue.cc: CPU allocator, cuda_copy, profiling switch
void bind_allocators(pybind11::module_& m, BackendClass& backend);

inline void bind_extras(pybind11::module_& m, BackendClass& backend) {
  bind_ops(m, backend);
  bind_fused(m);
  bind_train_ops(m);
  bind_store(m);
  bind_queue(m, backend);
  bind_custom_op(m, backend);
  bind_allocators(m, backend);
}

}  // namespace moodist
