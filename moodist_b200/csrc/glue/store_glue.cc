// moodist.TcpStore as a c10d::Store (reference: wrapper/store_wrapper.cc:43-106, wrapper/store.h:18-39).
// add / deleteKey / getNumKeys / compareSet work here; the reference throws for them.
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <pybind11/chrono.h>
#include <torch/extension.h>

#include "bindings.h"
#include "core/log.h"
#include "core/store.h"

namespace moodist {
namespace {

class TcpStoreGlue final : public c10d::Store {
 public:
  TcpStoreGlue(const std::string& hostname, int port, const std::string& key, int world, int rank,
               std::chrono::milliseconds timeout)
      : c10d::Store(timeout) {
    try {
      impl_ = TcpStore::create(hostname, port, key, world, rank, timeout);
    } catch (const Error& e) {
      TORCH_CHECK(false, e.what());
    }
  }
  explicit TcpStoreGlue(std::shared_ptr<TcpStore> impl) : c10d::Store(impl->timeout()), impl_(std::move(impl)) {}

  c10::intrusive_ptr<c10d::Store> clone() override { return c10::make_intrusive<TcpStoreGlue>(impl_); }

#define GUARD(expr)                \
  try {                            \
    expr;                          \
  } catch (const Error& e) {       \
    throw std::runtime_error(e.what()); \
  }
  void set(const std::string& key, const std::vector<uint8_t>& value) override { GUARD(impl_->set(key, value)) }
  std::vector<uint8_t> get(const std::string& key) override { GUARD(return impl_->get(key)) }
  std::vector<uint8_t> compareSet(const std::string& key, const std::vector<uint8_t>& expected,
                                  const std::vector<uint8_t>& desired) override {
    GUARD(return impl_->compare_set(key, expected, desired))
  }
  int64_t add(const std::string& key, int64_t value) override { GUARD(return impl_->add(key, value)) }
  bool deleteKey(const std::string& key) override { GUARD(return impl_->delete_key(key)) }
  bool check(const std::vector<std::string>& keys) override { GUARD(return impl_->check(keys)) }
  int64_t getNumKeys() override { GUARD(return impl_->num_keys()) }
  void wait(const std::vector<std::string>& keys) override { GUARD(impl_->wait_for(keys, timeout_)) }
  void wait(const std::vector<std::string>& keys, const std::chrono::milliseconds& timeout) override {
    GUARD(impl_->wait_for(keys, timeout))
  }
  void setTimeout(const std::chrono::milliseconds& timeout) override {
    c10d::Store::setTimeout(timeout);
    impl_->set_timeout(timeout);
  }
#undef GUARD
  void shutdown() { impl_->shutdown(); }
  std::string describe() const { return impl_->describe(); }
  std::vector<int> edges() const { return impl_->edges(); }
  void injectFaults(int break_every) { impl_->inject_faults(break_every); }
  uint64_t injectedBreaks() { return impl_->injected_breaks(); }

 private:
  std::shared_ptr<TcpStore> impl_;
};

}  // namespace

void bind_store(pybind11::module_& m) {
  namespace py = pybind11;
  py::class_<TcpStoreGlue, c10d::Store, c10::intrusive_ptr<TcpStoreGlue>>(m, "TcpStore")
      .def(py::init([](const std::string& hostname, int port, const std::string& key, int world_size, int rank,
                       std::chrono::milliseconds timeout) {
             return c10::make_intrusive<TcpStoreGlue>(hostname, port, key, world_size, rank, timeout);
           }),
           py::arg("hostname"), py::arg("port"), py::arg("key"), py::arg("world_size"), py::arg("rank"),
           py::arg("timeout") = std::chrono::milliseconds(300000), py::call_guard<py::gil_scoped_release>())
      .def("shutdown", &TcpStoreGlue::shutdown, py::call_guard<py::gil_scoped_release>(),
           "coordinated shutdown now (otherwise when the last handle goes, or when the interpreter exits)")
      .def("describe", &TcpStoreGlue::describe)
      .def("edges", &TcpStoreGlue::edges)
      .def("_inject_faults", &TcpStoreGlue::injectFaults, py::arg("break_every"),
           "test hook: every N-th message this rank sends over a mesh edge is lost with its connection (0: off)")
      .def("_injected_breaks", &TcpStoreGlue::injectedBreaks);
  m.def("_shutdown_all_stores", [] { TcpStore::shutdown_all(); }, py::call_guard<py::gil_scoped_release>());
  m.def("store_string_hash", &store_string_hash);
  m.def("store_mesh", &store_mesh);
}

}  // namespace moodist
