// moodist.Queue bindings: tensors in, tensors out (reference: wrapper/queue_wrapper.cc, wrapper/module.cc:921-1320).
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
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

// dtype code of a queue item that is the descriptor of a CUDA tensor: this offset plus the tensor's own dtype
constexpr int32_t kCudaItemDtypeBase = 1000;

struct PyQueue {
  std::shared_ptr<Queue> q;
  c10::intrusive_ptr<MoodistBackend> owner;  // the group must outlive its queues
  int readers = 1;                           // locations of the queue: each of them fetches a CUDA item once
  std::mutex tx_mu;
  std::map<uint32_t, std::vector<CudaItemDescriptor>> tx_items;  // CUDA items of open transactions

  std::shared_ptr<PyQueueWork> put(const at::Tensor& tensor, uint32_t transaction, bool wait_on_destroy) {
    TORCH_CHECK(tensor.layout() == at::kStrided, "moodist.Queue: only dense tensors can be queued, not ", tensor.layout(),
                " (use put_object for anything else)");
    if (tensor.is_cuda()) {
      if (CudaP2P* p2p = owner->cudaP2P(tensor.get_device())) {
        // Stream-ordered: nothing waits for the GPU here. The item that travels is a descriptor; whoever gets it
        // copies the bytes over NVLink on its own stream and receives a CUDA tensor.
        at::Tensor t = tensor.contiguous();
        c10::cuda::CUDAGuard guard(t.device());
        auto stream = c10::cuda::getCurrentCUDAStream();
        auto desc = std::make_shared<CudaItemDescriptor>();
        try {
          *desc = p2p->publish(t, readers, stream.stream());
        } catch (const Error& e) {
          throw std::runtime_error(e.what());
        }
        if (transaction) {
          std::lock_guard<std::mutex> lk(tx_mu);
          tx_items[transaction].push_back(*desc);
        }
        std::vector<int64_t> shape(t.sizes().begin(), t.sizes().end());
        auto w = std::make_shared<PyQueueWork>();
        w->wait_on_destroy = wait_on_destroy;
        py::gil_scoped_release nogil;
        try {
          w->work = q->put(desc.get(), sizeof(CudaItemDescriptor), kCudaItemDtypeBase + (int32_t)t.scalar_type(), shape,
                           transaction, desc);
        } catch (const Error& e) {
          throw std::runtime_error(e.what());
        }
        return w;
      }
    }
    // Before the group has mapped its peers' memory (its first CUDA collective does that), CUDA tensors are
    // staged to host memory here, which waits for the producing stream; the receiver then gets a CPU tensor.
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
    if (item->dtype >= kCudaItemDtypeBase) {
      // the descriptor of a CUDA tensor: fetch the bytes on this rank's current stream
      TORCH_CHECK(item->data.size() == sizeof(CudaItemDescriptor), "moodist queue: malformed CUDA item");
      CudaItemDescriptor d;
      memcpy(&d, item->data.data(), sizeof(d));
      int device = (int)c10::cuda::current_device();
      CudaP2P* p2p = owner->cudaP2P(device);
      TORCH_CHECK(p2p != nullptr, "moodist queue: received a CUDA tensor but this rank's group has no CUDA side yet "
                                  "(run a CUDA collective on the group first)");
      auto options = at::TensorOptions().dtype((at::ScalarType)(item->dtype - kCudaItemDtypeBase)).device(at::kCUDA, device);
      at::Tensor out = at::empty(item->shape, options);
      TORCH_CHECK((uint64_t)out.nbytes() == d.bytes, "moodist queue: CUDA item size mismatch");
      auto stream = c10::cuda::getCurrentCUDAStream();
      try {
        p2p->fetch(d, out.data_ptr(), stream.stream());
      } catch (const Error& e) {
        throw std::runtime_error(e.what());
      }
      return py::make_tuple(out, size);
    }
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
      .def("transaction_commit",
           [](PyQueue& s, uint32_t id) {
             s.q->transaction_commit(id);
             std::lock_guard<std::mutex> lk(s.tx_mu);
             s.tx_items.erase(id);
           })
      .def("transaction_cancel",
           [](PyQueue& s, uint32_t id) {
             s.q->transaction_cancel(id);
             // nobody will ever fetch the CUDA items of a cancelled transaction: release their buffers
             std::vector<CudaItemDescriptor> items;
             {
               std::lock_guard<std::mutex> lk(s.tx_mu);
               auto it = s.tx_items.find(id);
               if (it != s.tx_items.end()) {
                 items = std::move(it->second);
                 s.tx_items.erase(it);
               }
             }
             if (!items.empty())
               if (CudaP2P* p2p = s.owner->cudaP2P((int)c10::cuda::current_device()))
                 for (auto& d : items) p2p->drop(d);
           })
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
        out->readers = (int)std::max<size_t>(1, locations.size());
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
