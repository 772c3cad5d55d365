// moodist.Queue bindings: tensors in, tensors out (reference: wrapper/queue_wrapper.cc, wrapper/module.cc:921-1320).
#include <torch/extension.h>

#include "bindings.h"
#include "core/log.h"
#include "core/queue.h"

namespace moodist {
namespace {

namespace py = pybind11;

struct PyQueueWork {
  std::unique_ptr<QueueWork> work;
  bool wait_on_destroy = false;
  ~PyQueueWork() {
    if (work && wait_on_destroy) {
      py::gil_scoped_release nogil;
      try {
        work->wait();
      } catch (...) {
      }
    }
  }
  void wait() {
    if (!work) return;
    py::gil_scoped_release nogil;
    try {
      work->wait();
    } catch (const Error& e) {
      throw std::runtime_error(e.what());
    }
  }
};

struct PyQueue {
  std::shared_ptr<Queue> q;
  c10::intrusive_ptr<MoodistBackend> owner;  // the group must outlive its queues

  std::shared_ptr<PyQueueWork> put(const at::Tensor& tensor, uint32_t transaction, bool wait_on_destroy) {
    // CUDA tensors are staged to host memory here (synchronises with the producing stream); the receiving
    // side always gets a CPU tensor.
    at::Tensor t = tensor.is_cuda() ? tensor.cpu() : tensor;
    t = t.contiguous();
    auto keep = std::make_shared<at::Tensor>(t);
    std::vector<int64_t> shape(t.sizes().begin(), t.sizes().end());
    auto w = std::make_shared<PyQueueWork>();
    w->wait_on_destroy = wait_on_destroy;
    {
      py::gil_scoped_release nogil;
      try {
        w->work = q->put(t.data_ptr(), t.nbytes(), (int32_t)t.scalar_type(), shape, transaction, keep);
      } catch (const Error& e) {
        throw std::runtime_error(e.what());
      }
    }
    return w;
  }

  py::tuple get(bool block, py::object timeout) {
    double t = timeout.is_none() ? -1.0 : timeout.cast<double>();
    std::optional<QueueItem> item;
    size_t size = 0;
    {
      py::gil_scoped_release nogil;
      try {
        // wake up regularly so Ctrl-C reaches Python (the reference slices its futex waits the same way)
        if (block && t < 0) {
          while (!item) {
            item = q->get(true, 0.5, &size);
            if (!item) {
              py::gil_scoped_acquire gil;
              if (PyErr_CheckSignals() != 0) throw py::error_already_set();
            }
          }
        } else {
          item = q->get(block, t, &size);
        }
      } catch (const Error& e) {
        throw std::runtime_error(e.what());
      }
    }
    if (!item) return py::make_tuple(py::none(), size);
    auto* holder = new Bytes(std::move(item->data));
    auto options = at::TensorOptions().dtype((at::ScalarType)item->dtype).device(at::kCPU);
    at::Tensor out = at::from_blob(holder->data(), item->shape, [holder](void*) { delete holder; }, options);
    return py::make_tuple(out, size);
  }

  size_t qsize() {
    py::gil_scoped_release nogil;
    return q->qsize();
  }
  bool wait(py::object timeout) {
    double t = timeout.is_none() ? -1.0 : timeout.cast<double>();
    py::gil_scoped_release nogil;
    return q->wait(t);
  }
};

}  // namespace

void bind_queue(pybind11::module_& m, BackendClass& backend) {
  py::class_<PyQueueWork, std::shared_ptr<PyQueueWork>>(m, "QueueWork").def("wait", &PyQueueWork::wait);
  py::class_<PyQueue, std::shared_ptr<PyQueue>>(m, "Queue")
      .def("put", &PyQueue::put, py::arg("tensor"), py::arg("transaction") = 0, py::arg("wait_on_destroy") = true)
      .def("get", &PyQueue::get, py::arg("block") = true, py::arg("timeout") = py::none())
      .def("qsize", &PyQueue::qsize)
      .def("wait", &PyQueue::wait, py::arg("timeout") = py::none())
      .def("transaction_begin", [](PyQueue& s) { return s.q->transaction_begin(); })
      .def("transaction_commit", [](PyQueue& s, uint32_t id) { s.q->transaction_commit(id); })
      .def("transaction_cancel", [](PyQueue& s, uint32_t id) { s.q->transaction_cancel(id); })
      .def("name", [](PyQueue& s) { return s.q->name(); });

  backend.def(
      "Queue",
      [](c10::intrusive_ptr<MoodistBackend> self, py::object location, bool streaming, py::object name) {
        std::vector<int> locations;
        if (py::isinstance<py::int_>(location)) {
          locations.push_back(location.cast<int>());
        } else {
          for (auto h : location) locations.push_back(h.cast<int>());
        }
        std::optional<std::string> nm;
        if (!name.is_none()) nm = name.cast<std::string>();
        auto out = std::make_shared<PyQueue>();
        out->owner = self;
        {
          py::gil_scoped_release nogil;
          try {
            out->q = self->queues().make_queue(locations, streaming, nm);
          } catch (const Error& e) {
            throw std::runtime_error(e.what());
          }
        }
        return out;
      },
      py::arg("location"), py::arg("streaming") = false, py::arg("name") = py::none());
}

}  // namespace moodist
