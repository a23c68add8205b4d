// Python bindings of the tensor engine's controller bookkeeping (csrc/tensor/controller_history.h).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "mesh/tree_manifest.h"
#include "tensor/controller_history.h"

namespace py = pybind11;
using namespace mb;

void bind_controller(py::module_& m) {
  // workspace synchronisation: {relative path: content hash} of a directory tree, hashed by
  // a few threads with the GIL released
  m.def(
      "tree_manifest",
      [](const std::string& root, const std::vector<std::string>& skip_dirs,
         const std::vector<std::string>& skip_suffixes, uint64_t max_file_bytes, int threads) {
        std::vector<ManifestEntry> entries;
        {
          py::gil_scoped_release rel;
          entries = tree_manifest(root, skip_dirs, skip_suffixes, max_file_bytes, threads);
        }
        py::dict out;
        for (auto& e : entries) out[py::str(e.rel)] = py::str(e.hash);
        return out;
      },
      py::arg("root"), py::arg("skip_dirs"), py::arg("skip_suffixes"),
      py::arg("max_file_bytes") = (uint64_t)64 << 20, py::arg("threads") = 4);
  m.def("hash_file_128", [](const std::string& path) -> py::object {
    bool ok = false;
    std::string h;
    {
      py::gil_scoped_release rel;
      h = hash_file_128(path, &ok);
    }
    if (!ok) return py::none();
    return py::str(h);
  });

  py::class_<ControllerHistory, std::shared_ptr<ControllerHistory>>(m, "ControllerHistory")
      .def(py::init<int>(), py::arg("world"))
      .def("next_seq", &ControllerHistory::next_seq)
      .def("next_ref", &ControllerHistory::next_ref)
      .def("world", &ControllerHistory::world)
      .def("add_invocation", &ControllerHistory::add_invocation, py::arg("seq"), py::arg("name"),
           py::arg("defs"), py::arg("uses"))
      .def("rank_progress", &ControllerHistory::rank_progress)
      .def("min_completed", &ControllerHistory::min_completed)
      .def("live_invocations", &ControllerHistory::live_invocations)
      .def("fail", &ControllerHistory::fail, py::arg("seq"), py::arg("rank"), py::arg("name"),
           py::arg("text"))
      .def("ref_failed", &ControllerHistory::ref_failed)
      .def("failure",
           [](const ControllerHistory& h, int64_t seq) -> py::object {
             FailureInfo f;
             if (!h.failure(seq, &f)) return py::none();
             return py::make_tuple(f.seq, f.rank, f.name, f.text);
           })
      .def("forget_refs", &ControllerHistory::forget_refs)
      .def("describe",
           [](const ControllerHistory& h, int64_t seq) -> py::object {
             std::string name;
             int64_t failed_by = -1;
             if (!h.describe(seq, &name, &failed_by)) return py::none();
             return py::make_tuple(name, failed_by);
           })
      .def("ping_sent", &ControllerHistory::ping_sent)
      .def("ping_outstanding", &ControllerHistory::ping_outstanding)
      .def("ping_answered", &ControllerHistory::ping_answered)
      .def("stalled", [](ControllerHistory& h, double now, double timeout_s) -> py::object {
        StallReport r;
        if (!h.stalled(now, timeout_s, &r)) return py::none();
        py::dict d;
        d["ranks"] = r.ranks;
        d["waited_s"] = r.waited_s;
        d["controller_seq"] = r.ping_seq;
        d["last_seq_of_responders"] = r.last_seq_of_responders;
        return d;
      });
}
