// Python bindings of the torch-facing objects (module `moodist_b200._C`).
//
// Exposes the same Python-visible names as the reference's hand-written CPython module
// (wrapper/module.cc:1355-1428): MoodistProcessGroup / MoodistBackend with moodist_name, cuda_barrier,
// _get_option/_set_option, get/set_prefer_kernel_less, Queue, compile_op_full; TcpStore; Queue objects;
// serialize/deserialize live in the separate _serialize module. pybind11 (shipped with torch) replaces
// the reference's manual subclassing of torch's pybind types since a single torch version is targeted.
#include <torch/extension.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>

#include "backend.h"
#include "bindings.h"
#include "core/log.h"

namespace py = pybind11;
using namespace moodist;

PYBIND11_MODULE(_C, m) {
  // Long waits of the core call this between slices (none of its locks held, the GIL released): pending signal
  // handlers run, and if one raised (KeyboardInterrupt) the wait ends with that exception.
  moodist::interrupt_hook() = [] {
    if (!Py_IsInitialized()) return;
    pybind11::gil_scoped_acquire gil;
    if (PyErr_CheckSignals() != 0) throw pybind11::error_already_set();
  };
  m.doc() = "moodist_b200 native extension";
  py::module::import("torch.distributed");

  auto backend =
      py::class_<MoodistBackend, c10d::Backend, c10::intrusive_ptr<MoodistBackend>>(m, "MoodistBackend")
          .def(py::init([](const c10::intrusive_ptr<c10d::Store>& store, int rank, int size) {
                 return c10::make_intrusive<MoodistBackend>(store, rank, size);
               }),
               py::arg("store"), py::arg("rank"), py::arg("size"), py::call_guard<py::gil_scoped_release>())
          .def("moodist_name", &MoodistBackend::moodistName)
          .def("cuda_barrier", &MoodistBackend::cudaBarrier, py::call_guard<py::gil_scoped_release>())
          .def("_get_option", &MoodistBackend::getOption)
          .def("_set_option", &MoodistBackend::setOption)
          .def("get_prefer_kernel_less", &MoodistBackend::getPreferKernelLess)
          .def("set_prefer_kernel_less", &MoodistBackend::setPreferKernelLess)
          .def("kernel_launches", &MoodistBackend::kernelLaunches)
          .def("describe", &MoodistBackend::describe)
          .def(
              "_inject_faults",
              [](MoodistBackend& self, int drop_every, int duplicate_every, int delay_ms) {
                self.hostGroup().inject_faults(drop_every, duplicate_every, delay_ms);
              },
              py::arg("drop_every") = 0, py::arg("duplicate_every") = 0, py::arg("delay_ms") = 0,
              "test hook (host engine): drop / duplicate every N-th two-sided message this rank sends, delay each one")
          .def(
              "host_stats",
              [](MoodistBackend& self) {
                std::vector<uint64_t> c;
                {
                  py::gil_scoped_release nogil;
                  c = self.hostGroup().transport_counters();
                }
                py::dict out;
                out["tcp_bytes_sent"] = c.at(0);
                out["tcp_bytes_received"] = c.at(1);
                out["direct_bytes"] = c.at(2);
                out["direct_peers"] = c.at(3);
                out["unix_socket_peers"] = c.at(4);
                return out;
              },
              "traffic of the host engine: bytes over its sockets, bytes copied directly between processes of this machine, "
              "and how many peers are reached that way / over a unix-domain socket")
          .def(
              "stats",
              [](MoodistBackend& self, bool wait) {
                // {"all_gather/nvls": {"calls": .., "bytes": .., "timed_calls": .., "device_us": ..}, ...}
                py::dict out;
                for (const OpStat& st : self.cudaStats(wait)) {
                  py::dict row;
                  row["calls"] = st.calls;
                  row["bytes"] = st.bytes;
                  row["timed_calls"] = st.timed_calls;
                  row["device_us"] = st.device_us;
                  out[py::str(st.name)] = row;
                }
                return out;
              },
              py::arg("wait") = true,
              "per operation and kernel family: calls, payload bytes, and the device time of the sampled calls")
          .def("all_gather_cast", &MoodistBackend::allGatherCast, py::arg("output"), py::arg("input"),
               py::call_guard<py::gil_scoped_release>())
          .def("reduce_scatter_cast", &MoodistBackend::reduceScatterCast, py::arg("output"), py::arg("input"),
               py::arg("op") = 0, py::arg("premul") = 1.0, py::call_guard<py::gil_scoped_release>());
  m.attr("MoodistProcessGroup") = backend;
  m.def("load_variant_table", &load_variant_table, py::arg("path"), py::arg("world"),
        "thresholds a group of `world` ranks would take from a MOODIST_VARIANT_TABLE file");
  // the reference's module has the same liveness probe (wrapper/module.cc:1355-1428, `hello`)
  m.def("hello", [] { return std::string("moodist_b200 native extension (sm_100a kernels, host engine, TcpStore)"); });
  m.def("live_process_groups", &MoodistBackend::live, "every moodist group alive in this process");
  m.def("find_process_group", &MoodistBackend::find, "the live moodist group with this name, or None");

  bind_extras(m, backend);
}
