// Python bindings of the tensor engine's controller bookkeeping (csrc/tensor/controller_history.h).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "tensor/controller_history.h"

namespace py = pybind11;
using namespace mb;

void bind_controller(py::module_& m) {
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
