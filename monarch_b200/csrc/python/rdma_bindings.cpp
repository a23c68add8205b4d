// Python bindings of the native RDMA manager (csrc/rdma/rdma_manager.h).
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <unistd.h>

#include "rdma/rdma_manager.h"

namespace py = pybind11;
using namespace mb;

namespace {

struct PyRdmaManager {
  std::shared_ptr<RdmaRegistry> reg = std::make_shared<RdmaRegistry>();
  std::shared_ptr<Instance> instance;
};

py::dict info_to_dict(const RdmaBufferInfo& b) {
  py::dict d;
  d["id"] = b.id;
  d["addr"] = b.addr;
  d["nbytes"] = b.nbytes;
  d["cuda"] = b.cuda;
  d["device"] = b.device;
  d["pid"] = b.pid;
  d["host"] = b.host;
  d["ipc_handle"] = py::bytes(b.ipc_handle);
  d["ipc_offset"] = b.ipc_offset;
  d["valid_addr"] = b.valid_addr;
  return d;
}

}  // namespace

void bind_rdma(py::module_& m) {
  py::class_<PyRdmaManager, std::shared_ptr<PyRdmaManager>>(m, "RdmaManager")
      .def(py::init([](std::shared_ptr<Proc> proc, const std::string& name, py::object cuda_fallback) {
             auto mgr = std::make_shared<PyRdmaManager>();
             RdmaCudaFallback fb;
             if (!cuda_fallback.is_none()) {
               auto cell = std::shared_ptr<py::object>(new py::object(cuda_fallback),
                                                       [](py::object* p) {
                                                         if (Py_IsInitialized()) {
                                                           py::gil_scoped_acquire g;
                                                           delete p;
                                                         }
                                                       });
               fb = [cell](const RdmaBufferInfo& b, const std::string& op, uint64_t off,
                           uint64_t len, const std::string* payload) -> std::string {
                 py::gil_scoped_acquire g;
                 try {
                   py::object r = (*cell)(info_to_dict(b), op, off, len,
                                          payload ? py::object(py::bytes(*payload)) : py::none());
                   return r.is_none() ? std::string() : std::string(r.cast<py::bytes>());
                 } catch (py::error_already_set& e) {
                   throw std::runtime_error(e.what());
                 }
               };
             }
             auto hooks = make_rdma_manager(mgr->reg, std::move(fb));
             {
               py::gil_scoped_release rel;
               mgr->instance = proc->spawn(name, std::move(hooks));
             }
             rdma_allow_peer_access();
             return mgr;
           }),
           py::arg("proc"), py::arg("name") = "rdma_manager", py::arg("cuda_fallback") = py::none())
      .def_property_readonly("actor_id", [](PyRdmaManager& m) { return m.instance->id().to_string(); })
      .def_property_readonly("instance", [](PyRdmaManager& m) { return m.instance; })
      .def("register",
           [](PyRdmaManager& m, uint64_t addr, uint64_t nbytes, bool cuda, int device,
              py::bytes ipc_handle, int64_t ipc_offset, const std::string& host) {
             RdmaBufferInfo b;
             b.addr = addr;
             b.nbytes = nbytes;
             b.cuda = cuda;
             b.device = device;
             b.pid = (int64_t)::getpid();
             b.host = host;
             b.ipc_handle = std::string(ipc_handle);
             b.ipc_offset = ipc_offset;
             return m.reg->add(std::move(b));
           },
           py::arg("addr"), py::arg("nbytes"), py::arg("cuda") = false, py::arg("device") = -1,
           py::arg("ipc_handle") = py::bytes(""), py::arg("ipc_offset") = 0, py::arg("host") = "")
      .def("drop", [](PyRdmaManager& m, uint64_t id) { return m.reg->drop(id); })
      .def("get",
           [](PyRdmaManager& m, uint64_t id) -> py::object {
             auto b = m.reg->get(id);
             if (!b) return py::none();
             return info_to_dict(*b);
           })
      .def("__len__", [](PyRdmaManager& m) { return m.reg->size(); });

  m.def("rdma_decode_info", [](py::bytes b) { return info_to_dict(RdmaBufferInfo::decode(std::string(b))); });
  m.def("rdma_allow_peer_access", &rdma_allow_peer_access);
  m.def("rdma_host_read",
        [](int64_t pid, uint64_t remote_addr, uint64_t local_addr, uint64_t n, uint64_t valid_addr,
           uint64_t id) {
          py::gil_scoped_release rel;
          return rdma_host_read(pid, remote_addr, reinterpret_cast<void*>(local_addr), n,
                                valid_addr, id);
        },
        py::arg("pid"), py::arg("remote_addr"), py::arg("local_addr"), py::arg("n"),
        py::arg("valid_addr") = 0, py::arg("id") = 0,
        "process_vm_readv: n bytes at remote_addr of process pid -> local_addr.  0, -2 when the "
        "buffer's validity word no longer holds id, or errno.");
  m.def("rdma_host_write",
        [](int64_t pid, uint64_t remote_addr, uint64_t local_addr, uint64_t n, uint64_t valid_addr,
           uint64_t id) {
          py::gil_scoped_release rel;
          return rdma_host_write(pid, remote_addr, reinterpret_cast<const void*>(local_addr), n,
                                 valid_addr, id);
        },
        py::arg("pid"), py::arg("remote_addr"), py::arg("local_addr"), py::arg("n"),
        py::arg("valid_addr") = 0, py::arg("id") = 0,
        "process_vm_writev: n bytes at local_addr -> remote_addr of process pid.  0, -2 (stale "
        "handle) or errno.");
}
