// pybind11 bindings of the native runtime (`monarch_b200._native`).
//
// Parity: monarch_hyperactor (PyProcMesh, PythonActor, PyMailbox/ports, shape/selection
// wrappers, config, telemetry) and monarch_extension (module registry).  Blocking calls
// release the GIL; callbacks from runtime threads take it.  Ids cross the boundary in
// their text form (`world[rank].actor[pid][port]`).
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "actor/runtime.h"
#include "channel/channel.h"
#include "actor/durable.h"
#include "mesh/mesh.h"
#include "ndslice/ndslice.h"
#include "telemetry/telemetry.h"

namespace py = pybind11;
using namespace mb;

namespace {

struct PyEnvelope {
  std::string sender, dest;
  std::map<std::string, std::string> headers;
  py::bytes data;
  std::vector<py::bytes> parts;
};

PyEnvelope to_py(Envelope& e) {
  PyEnvelope p;
  p.sender = e.sender.to_string();
  p.dest = e.dest.to_string();
  p.headers = e.headers;
  p.data = py::bytes(e.data);
  for (auto& x : e.parts) p.parts.emplace_back(x);
  return p;
}

std::string py_error_text(py::error_already_set& e) {
  std::string msg = e.what();
  e.discard_as_unraisable("monarch_b200 actor handler");
  return msg;
}

// Wrap a Python callable so it can be stored in runtime structures and destroyed from
// any thread (the destructor takes the GIL).
struct PyCallable {
  py::object fn;
  explicit PyCallable(py::object f) : fn(std::move(f)) {}
  ~PyCallable() {
    if (!Py_IsInitialized() || _Py_IsFinalizing()) {
      fn.release();  // leak rather than touch a dying interpreter
      return;
    }
    py::gil_scoped_acquire g;
    fn = py::object();
  }
};
using PyFn = std::shared_ptr<PyCallable>;
PyFn wrap(py::object o) { return o.is_none() ? nullptr : std::make_shared<PyCallable>(std::move(o)); }

bool interp_alive() { return Py_IsInitialized() && !_Py_IsFinalizing(); }

ActorHooks hooks_from_python(PyFn on_message, PyFn on_supervision, PyFn on_undeliverable,
                             PyFn on_stop) {
  ActorHooks h;
  if (on_message)
    h.on_message = [on_message](Instance& self, Envelope& env) {
      if (!interp_alive()) return;
      py::gil_scoped_acquire g;
      try {
        PyEnvelope pe = to_py(env);
        on_message->fn(self.shared_from_this(), pe);
      } catch (py::error_already_set& e) {
        throw std::runtime_error(py_error_text(e));
      }
    };
  if (on_supervision)
    h.on_supervision = [on_supervision](Instance& self, const ActorSupervisionEvent& ev) {
      if (!interp_alive()) return true;
      py::gil_scoped_acquire g;
      try {
        return on_supervision->fn(self.shared_from_this(), ev.actor_id.to_string(), ev.status,
                                  ev.message).cast<bool>();
      } catch (py::error_already_set& e) {
        throw std::runtime_error(py_error_text(e));
      }
    };
  if (on_undeliverable)
    h.on_undeliverable = [on_undeliverable](Instance& self, Envelope& env, const std::string& why) {
      if (!interp_alive()) return true;
      py::gil_scoped_acquire g;
      try {
        PyEnvelope pe = to_py(env);
        return on_undeliverable->fn(self.shared_from_this(), pe, why).cast<bool>();
      } catch (py::error_already_set& e) {
        throw std::runtime_error(py_error_text(e));
      }
    };
  if (on_stop)
    h.on_stop = [on_stop](Instance& self) {
      if (!interp_alive()) return;
      py::gil_scoped_acquire g;
      try {
        on_stop->fn(self.shared_from_this());
      } catch (py::error_already_set& e) {
        py_error_text(e);
      }
    };
  return h;
}

// One client context per process: the router every mesh binds into, the client proc and
// (lazily) the unix-socket server child procs talk back to.
struct ClientContext {
  std::shared_ptr<Router> router = std::make_shared<Router>();
  std::shared_ptr<Proc> proc;
  std::mutex mu;
  ClientContext() {
    proc = Proc::create(ProcId{"client_" + std::to_string(getpid()), 0}, router);
    router->bind_local(proc);
    router->set_home(proc);
  }
};
ClientContext& client_ctx() {
  static ClientContext* c = new ClientContext();  // intentionally leaked: outlives atexit
  return *c;
}

std::vector<std::string> to_strings(const std::vector<py::bytes>& parts) {
  std::vector<std::string> out;
  for (auto& p : parts) out.push_back(p);
  return out;
}

// Parts given as bytes or as any C-contiguous buffer (memoryview of a tensor's storage, numpy
// array, bytearray): one copy, from the object's memory into the string that travels.
std::vector<std::string> to_strings(const std::vector<py::object>& parts) {
  std::vector<std::string> out;
  out.reserve(parts.size());
  for (auto& p : parts) {
    if (PyBytes_Check(p.ptr())) {
      char* buf = nullptr;
      Py_ssize_t len = 0;
      PyBytes_AsStringAndSize(p.ptr(), &buf, &len);
      out.emplace_back(buf, (size_t)len);
      continue;
    }
    Py_buffer view;
    if (PyObject_GetBuffer(p.ptr(), &view, PyBUF_C_CONTIGUOUS) != 0) throw py::error_already_set();
    out.emplace_back(static_cast<const char*>(view.buf), (size_t)view.len);
    PyBuffer_Release(&view);
  }
  return out;
}

}  // namespace

void bind_tasks(py::module_& m);   // tasks.cpp
void bind_rdma(py::module_& m);    // rdma_bindings.cpp
void bind_controller(py::module_& m);  // controller_bindings.cpp

PYBIND11_MODULE(_native, m) {
  m.doc() = "monarch_b200 native runtime";
  bind_tasks(m);
  bind_rdma(m);
  bind_controller(m);

  // ------------------------------------------------------------------ ndslice ----
  py::register_exception<NdError>(m, "NdSliceError", PyExc_ValueError);
  py::register_exception<ChannelError>(m, "ChannelError", PyExc_RuntimeError);
  py::register_exception<CodecError>(m, "CodecError", PyExc_ValueError);

  py::class_<Slice>(m, "Slice")
      .def(py::init<size_t, std::vector<size_t>, std::vector<size_t>>(), py::arg("offset"),
           py::arg("sizes"), py::arg("strides"))
      .def_static("new_row_major", &Slice::row_major)
      .def_static("from_list", &Slice::from_list)
      .def_property_readonly("offset", &Slice::offset)
      .def_property_readonly("sizes", &Slice::sizes)
      .def_property_readonly("strides", &Slice::strides)
      .def_property_readonly("ndim", &Slice::ndim)
      .def("__len__", &Slice::len)
      .def("index", &Slice::index)
      .def("coordinates", &Slice::coordinates)
      .def("nditem", &Slice::location)
      .def("get", &Slice::get)
      .def("contains", &Slice::contains)
      .def("ranks", &Slice::ranks)
      .def("at", &Slice::at)
      .def("select", &Slice::select)
      .def("view", &Slice::view)
      .def("is_contiguous", &Slice::is_contiguous)
      .def("__getitem__",
           [](const Slice& s, py::object i) -> py::object {
             if (py::isinstance<py::slice>(i)) {
               size_t start, stop, step, n;
               if (!i.cast<py::slice>().compute(s.len(), &start, &stop, &step, &n))
                 throw py::error_already_set();
               py::tuple t(n);
               for (size_t k = 0; k < n; ++k) t[k] = s.get(start + k * step);
               return std::move(t);
             }
             long idx = i.cast<long>();
             if (idx < 0) idx += (long)s.len();
             if (idx < 0 || (size_t)idx >= s.len()) throw py::index_error();
             return py::int_(s.get((size_t)idx));
           })
      .def("__iter__",
           [](const Slice& s) {
             py::list l;
             for (size_t r : s.ranks()) l.append(r);
             return py::iter(l);
           })
      .def("__eq__", [](const Slice& a, py::object o) {
        return py::isinstance<Slice>(o) && a == o.cast<Slice>();
      })
      .def("__hash__", [](const Slice& s) { return py::hash(py::str(s.to_string())); })
      .def("__repr__", &Slice::to_string)
      .def(py::pickle(
          [](const Slice& s) { return py::make_tuple(s.offset(), s.sizes(), s.strides()); },
          [](py::tuple t) {
            return Slice(t[0].cast<size_t>(), t[1].cast<std::vector<size_t>>(),
                         t[2].cast<std::vector<size_t>>());
          }));

  m.def("reshape_with_limit", &reshape_with_limit);

  py::class_<Selection, std::shared_ptr<Selection>>(m, "Selection")
      .def_static("from_string",
                  [](const std::string& s) { return std::const_pointer_cast<Selection>(Selection::parse(s)); })
      .def_static("all", [] { return std::const_pointer_cast<Selection>(Selection::t()); })
      .def_static("any",
                  [] { return std::const_pointer_cast<Selection>(Selection::any(Selection::t())); })
      .def_static("of_ranks",
                  [](const Slice& sl, const std::vector<size_t>& r) {
                    return std::const_pointer_cast<Selection>(Selection::of_ranks(sl, r));
                  })
      .def("eval",
           [](std::shared_ptr<Selection> s, const Slice& sl, uint64_t seed) {
             return eval(s, sl, seed);
           },
           py::arg("slice"), py::arg("seed") = 4)
      .def("__repr__", [](const Selection& s) { return s.to_string(); });

  // Routing simulation for tests: runs the cast tree to completion and returns
  // (delivered ranks in arrival order, {rank: hop count}, max fan-out seen).
  m.def("simulate_cast", [](std::shared_ptr<Selection> sel, const Slice& slice) {
    std::vector<size_t> delivered;
    std::map<size_t, size_t> hops;
    size_t max_fanout = 0;
    std::vector<size_t> zero(slice.ndim(), 0);
    size_t root = slice.location(zero);
    std::deque<std::tuple<size_t, std::vector<RoutingFrame>, size_t>> q;
    q.emplace_back(root, std::vector<RoutingFrame>{RoutingFrame::root(sel, slice)}, 0);
    while (!q.empty()) {
      auto [rank, frames, h] = std::move(q.front());
      q.pop_front();
      Resolved r = resolve_routing(rank, slice, std::move(frames));
      if (r.deliver_here) {
        delivered.push_back(rank);
        hops[rank] = h;
      }
      max_fanout = std::max(max_fanout, r.next.size());
      for (auto& kv : r.next) q.emplace_back(kv.first, std::move(kv.second), h + 1);
    }
    return py::make_tuple(delivered, hops, max_fanout);
  });

  // ---------------------------------------------------------- config / telemetry ----
  m.def("config_get", [](const std::string& k) { return Config::global().get(k); });
  m.def("config_set", [](const std::string& k, const std::string& v) { Config::global().set(k, v); });
  m.def("config_unset", [](const std::string& k) { Config::global().unset(k); });
  m.def("config_override",
        [](const std::string& k, const std::string& v) { return Config::global().override_key(k, v); });
  m.def("config_snapshot", [] { return Config::global().snapshot(); });
  m.def("config_to_yaml", [] { return Config::global().to_yaml(); });
  m.def("config_load_yaml", [](const std::string& t) { Config::global().load_yaml(t); });
  m.def("log", [](int lvl, const std::string& msg) {
    log_write((LogLevel)lvl, "python", 0, msg);
  });
  m.def("log_file_path", &log_file_path);
  m.def("metrics_snapshot", [] { return Metrics::global().snapshot(); });
  m.def("metrics_counter_add", [](const std::string& n, int64_t v) { Metrics::global().counter_add(n, v); });
  m.def("metrics_counter", [](const std::string& n) { return Metrics::global().counter(n); });
  m.def("metrics_gauge_set", [](const std::string& n, double v) { Metrics::global().gauge_set(n, v); });
  m.def("metrics_histogram_record",
        [](const std::string& n, double v) { Metrics::global().histogram_record(n, v); });
  m.def("metrics_histogram", [](const std::string& n) {
    auto h = Metrics::global().histogram(n);
    py::dict d;
    d["count"] = h.count;
    d["sum"] = h.sum;
    d["min"] = h.min;
    d["max"] = h.max;
    d["recent"] = h.recent;
    return d;
  });
  m.def("metrics_reset", [] { Metrics::global().reset(); });
  m.def("trace_enable", [](bool on) { TraceWriter::global().enable(on); });
  m.def("trace_complete", [](const std::string& n, const std::string& c, double ts, double dur,
                             int64_t pid, int64_t tid) {
    TraceWriter::global().complete(n, c, ts, dur, pid, tid);
  });
  m.def("trace_json", [] { return TraceWriter::global().to_json(); });
  m.def("trace_clear", [] { TraceWriter::global().clear(); });
  m.def("span_enter", [](const std::string& n, const std::string& a) { return span_enter(n, a); },
        py::arg("name"), py::arg("actor_id") = "");
  m.def("span_exit", &span_exit);
  m.def("current_span_id", &current_span_id);
  m.def("use_sim_clock", &use_sim_clock);
  m.def("use_real_clock", &use_real_clock);
  m.def("sim_clock_advance_us", &sim_clock_advance_us);
  m.def("telemetry_now_us", &telemetry_now_us);
  m.def("execution_id", [] { return execution_id(); });
  m.def("events_enable", [](bool on) { EventCollector::global().enable(on); });
  m.def("events_enabled", [] { return EventCollector::global().enabled(); });
  m.def("trace_enabled", [] { return TraceWriter::global().enabled(); });
  m.def("events_dropped", [] { return EventCollector::global().dropped(); });
  m.def("events_drain", [] {
    py::list out;
    for (auto& e : EventCollector::global().drain())
      out.append(py::make_tuple(e.kind, e.t_us, e.level, e.file, e.line, e.message, e.actor_id,
                                e.span_id, e.parent_id, e.thread));
    return out;
  });
  m.def("log_event", [](int level, const std::string& file, int line, const std::string& msg) {
    LogLevel l = level < 0 ? LogLevel::Trace : level > 4 ? LogLevel::Error : (LogLevel)level;
    // captured for readers even when below the file/stderr thresholds
    if (log_enabled(l) || EventCollector::global().enabled()) log_write(l, file.c_str(), line, msg);
  });
  m.def("now_us", &now_us);
  m.def("channel_stats", [] {
    auto& s = channel_stats();
    py::dict d;
    d["connects"] = s.connects.load();
    d["reconnects"] = s.reconnects.load();
    d["frames_sent"] = s.frames_sent.load();
    d["frames_resent"] = s.frames_resent.load();
    d["frames_received"] = s.frames_received.load();
    d["duplicates_dropped"] = s.duplicates_dropped.load();
    d["acks_sent"] = s.acks_sent.load();
    d["undeliverable"] = s.undeliverable.load();
    return d;
  });

  // --------------------------------------------------------------------- channels ----
  py::class_<Rx, std::shared_ptr<Rx>>(m, "ChannelRx")
      .def_property_readonly("addr", [](Rx& r) { return r.addr().to_string(); })
      .def("recv",
           [](Rx& r, int64_t timeout_ms) -> py::object {
             std::optional<Frame> f;
             {
               py::gil_scoped_release rel;
               f = r.recv(timeout_ms);
             }
             if (!f) return py::none();
             py::list parts;
             for (auto& p : f->parts) parts.append(py::bytes(p));
             return py::make_tuple(py::bytes(f->head), parts);
           },
           py::arg("timeout_ms") = -1)
      .def("close", &Rx::close, py::call_guard<py::gil_scoped_release>());
  py::class_<Tx, std::shared_ptr<Tx>>(m, "ChannelTx")
      .def_property_readonly("addr", [](Tx& t) { return t.addr().to_string(); })
      .def("post",
           [](Tx& t, py::bytes head, std::vector<py::bytes> parts, py::object on_fail) {
             Frame f;
             f.head = head;
             f.parts = to_strings(parts);
             PyFn cb = wrap(on_fail);
             py::gil_scoped_release rel;
             if (cb)
               t.post(std::move(f), [cb](Frame&& fr) {
                 if (!interp_alive()) return;
                 py::gil_scoped_acquire g;
                 try {
                   cb->fn(py::bytes(fr.head));
                 } catch (py::error_already_set& e) {
                   py_error_text(e);
                 }
               });
             else
               t.post(std::move(f));
           },
           py::arg("head"), py::arg("parts") = std::vector<py::bytes>{},
           py::arg("on_undeliverable") = py::none())
      .def("is_closed", [](Tx& t) { return t.status() == TxStatus::Closed; })
      .def("close", &Tx::close, py::call_guard<py::gil_scoped_release>());
  m.def("channel_serve", [](const std::string& a) { return serve(ChannelAddr::parse(a)); });
  m.def("channel_serve_any", [](const std::string& kind) {
    return serve(ChannelAddr::any(kind == "tcp" ? ChannelAddr::Tcp
                                  : kind == "unix" ? ChannelAddr::Unix
                                                   : ChannelAddr::Local));
  });
  m.def("channel_dial", [](const std::string& a) { return dial(ChannelAddr::parse(a)); });
  m.def("channel_debug_drop_connections",
        [](const std::string& a) { debug_drop_connections(ChannelAddr::parse(a)); });
  m.def("parse_channel_addr", [](const std::string& a) { return ChannelAddr::parse(a).to_string(); });

  // --------------------------------------------------------------------- runtime ----
  m.def("parse_actor_id", [](const std::string& s) {
    ActorId a = ActorId::parse(s);
    return py::make_tuple(a.proc.world, a.proc.rank, a.name, a.pid);
  });
  m.def("parse_port_id", [](const std::string& s) {
    PortId p = PortId::parse(s);
    return py::make_tuple(p.actor.proc.world, p.actor.proc.rank, p.actor.name, p.actor.pid, p.port);
  });

  py::class_<PyEnvelope>(m, "Envelope")
      .def_readonly("sender", &PyEnvelope::sender)
      .def_readonly("dest", &PyEnvelope::dest)
      .def_readonly("headers", &PyEnvelope::headers)
      .def_readonly("data", &PyEnvelope::data)
      .def_readonly("parts", &PyEnvelope::parts);

  py::class_<QueueSink, std::shared_ptr<QueueSink>>(m, "QueueReceiver")
      .def("recv",
           [](QueueSink& q, int64_t timeout_ms) -> py::object {
             std::optional<Envelope> e;
             {
               py::gil_scoped_release rel;
               e = q.recv(timeout_ms);
             }
             if (!e) return py::none();
             return py::cast(to_py(*e));
           },
           py::arg("timeout_ms") = -1)
      .def("try_recv",
           [](QueueSink& q) -> py::object {
             auto e = q.try_recv();
             if (!e) return py::none();
             return py::cast(to_py(*e));
           })
      .def("set_notify",
           [](QueueSink& q, py::object fn) {
             PyFn cb = wrap(fn);
             if (!cb) {
               q.set_notify({});
               return;
             }
             q.set_notify([cb] {
               if (!interp_alive()) return;
               py::gil_scoped_acquire g;
               try {
                 cb->fn();
               } catch (py::error_already_set& e) {
                 py_error_text(e);
               }
             });
           })
      .def("close", &QueueSink::close)
      .def("__len__", &QueueSink::size);

  py::class_<AccumSink, std::shared_ptr<AccumSink>>(m, "AccumReceiver")
      .def("state", [](AccumSink& a) { return py::bytes(a.state()); })
      .def("count", &AccumSink::count)
      .def("wait_count", &AccumSink::wait_count, py::call_guard<py::gil_scoped_release>());

  py::class_<Instance, std::shared_ptr<Instance>>(m, "Instance")
      .def_property_readonly("actor_id", [](Instance& i) { return i.id().to_string(); })
      .def_property_readonly("proc_id", [](Instance& i) { return i.id().proc.to_string(); })
      .def_property_readonly("rank", [](Instance& i) { return i.id().proc.rank; })
      .def_property_readonly("name", [](Instance& i) { return i.id().name; })
      .def_property_readonly("status", [](Instance& i) { return status_name(i.status()); })
      .def_property_readonly("failure", &Instance::failure)
      .def_property_readonly("messages_handled", &Instance::messages_handled)
      .def_property_readonly("proc", &Instance::proc)
      .def("send",
           [](Instance& i, const std::string& dest, py::bytes data,
              std::map<std::string, std::string> headers, std::vector<py::object> parts) {
             PortId d = PortId::parse(dest);
             std::string body = data;
             auto ps = to_strings(parts);
             py::gil_scoped_release rel;
             i.send(d, std::move(body), std::move(headers), std::move(ps));
           },
           py::arg("dest"), py::arg("data"), py::arg("headers") = std::map<std::string, std::string>{},
           py::arg("parts") = std::vector<py::object>{})
      .def("open_port",
           [](Instance& i, bool once) {
             auto q = std::make_shared<QueueSink>(once);
             PortId p = i.bind(q);
             return py::make_tuple(p.to_string(), q);
           },
           py::arg("once") = false)
      .def("open_accum_port",
           [](Instance& i, py::object reducer, py::bytes init) {
             ReduceFn fn;
             if (py::isinstance<py::str>(reducer)) {
               fn = builtin_reducer(reducer.cast<std::string>());
             } else {
               PyFn cb = wrap(reducer);
               fn = [cb](const std::string& acc, const std::string& upd) -> std::string {
                 py::gil_scoped_acquire g;
                 try {
                   return cb->fn(py::bytes(acc), py::bytes(upd)).cast<std::string>();
                 } catch (py::error_already_set& e) {
                   throw std::runtime_error(py_error_text(e));
                 }
               };
             }
             auto a = std::make_shared<AccumSink>(std::move(fn), (std::string)init);
             PortId p = i.bind(a);
             return py::make_tuple(p.to_string(), a);
           },
           py::arg("reducer"), py::arg("init") = py::bytes(""))
      .def("close_port", [](Instance& i, const std::string& port) { i.unbind(PortId::parse(port).port); })
      .def("undeliverable_receiver", &Instance::undeliverable_queue)
      .def("stop", [](Instance& i) { i.signal(Signal::Stop); })
      .def("drain_and_stop", [](Instance& i) { i.signal(Signal::DrainAndStop); })
      .def("fail", &Instance::fail)
      .def("join", &Instance::join, py::arg("timeout_ms") = -1,
           py::call_guard<py::gil_scoped_release>())
      .def("events", [](Instance& i) {
        py::list l;
        for (auto& e : i.recorder().tail()) l.append(py::make_tuple(e.t_us, e.name, e.detail));
        return l;
      });

  py::class_<Proc, std::shared_ptr<Proc>>(m, "Proc")
      .def_static("local",
                  [](const std::string& world, int64_t rank) {
                    auto& c = client_ctx();
                    auto p = Proc::create(ProcId{world, rank}, c.router);
                    c.router->bind_local(p);
                    return p;
                  },
                  py::arg("world") = "local", py::arg("rank") = 0)
      .def_property_readonly("proc_id", [](Proc& p) { return p.id().to_string(); })
      .def_property_readonly("rank", [](Proc& p) { return p.id().rank; })
      .def_property_readonly("world", [](Proc& p) { return p.id().world; })
      .def("spawn",
           [](std::shared_ptr<Proc> p, const std::string& name, py::object on_message,
              py::object on_supervision, py::object on_undeliverable, py::object on_stop,
              std::shared_ptr<Instance> parent) {
             ActorHooks h = hooks_from_python(wrap(on_message), wrap(on_supervision),
                                              wrap(on_undeliverable), wrap(on_stop));
             py::gil_scoped_release rel;
             return p->spawn(name, std::move(h), parent);
           },
           py::arg("name"), py::arg("on_message"), py::arg("on_supervision") = py::none(),
           py::arg("on_undeliverable") = py::none(), py::arg("on_stop") = py::none(),
           py::arg("parent") = nullptr)
      .def("attach", &Proc::attach)
      .def("find", &Proc::find)
      .def("set_supervision_coordinator",
           [](Proc& p, py::object port) {
             if (port.is_none())
               p.set_supervision_coordinator(std::nullopt);
             else
               p.set_supervision_coordinator(PortId::parse(port.cast<std::string>()));
           })
      .def("ledger_snapshot",
           [](Proc& p) {
             py::list out;
             for (auto& s : p.ledger_snapshot()) {
               py::dict d;
               d["actor_id"] = s.actor_id;
               d["status"] = s.status;
               d["failure"] = s.failure;
               d["messages_handled"] = s.messages_handled;
               d["children"] = s.children;
               py::list ev;
               for (auto& e : s.events) ev.append(py::make_tuple(e.t_us, e.name, e.detail));
               d["events"] = ev;
               out.append(d);
             }
             return out;
           })
      .def("stop_all", &Proc::stop_all, py::arg("timeout_ms") = 1000,
           py::call_guard<py::gil_scoped_release>());

  // Python actors spawned through a MeshAgent: the agent looks up type "python" and calls
  // this factory with (proc, actor name, pickled params); it returns the four hooks.
  m.def("register_python_actor_type", [](const std::string& type, py::object factory) {
    PyFn f = wrap(factory);
    register_actor_type(type, [f](const std::shared_ptr<Proc>& proc, const std::string& name,
                                  const std::string& params) {
      py::gil_scoped_acquire g;
      try {
        py::tuple t = f->fn(proc, name, py::bytes(params)).cast<py::tuple>();
        return hooks_from_python(wrap(t[0]), wrap(t[1]), wrap(t[2]), wrap(t[3]));
      } catch (py::error_already_set& e) {
        throw std::runtime_error(py_error_text(e));
      }
    });
  });

  // ------------------------------------------------------------------------ mesh ----
  // Cast from any actor instance (client or remote): the message enters the cast tree at
  // the comm actor of the proc holding the first element of `slice`.
  m.def("cast", [](std::shared_ptr<Instance> inst, const std::string& world,
                   const std::string& name, const Slice& slice, std::shared_ptr<Selection> sel,
                   py::bytes data, std::map<std::string, std::string> headers,
                   std::vector<py::object> parts, const Slice& cast_shape) {
    static std::atomic<uint64_t> seq{0};
    CastRequest c;
    c.mesh_id = name;
    c.slice = slice;
    c.selection = sel;
    c.sender = inst->id();
    c.data = data;
    c.headers = std::move(headers);
    c.cast_shape = cast_shape;
    c.seq = seq++;
    auto ps = to_strings(parts);
    py::gil_scoped_release rel;
    auto proc = inst->proc();
    if (!proc) throw std::runtime_error("cast from an instance whose proc is gone");
    std::vector<size_t> zero(slice.ndim(), 0);
    int64_t root = (int64_t)slice.location(zero);
    Envelope e;
    e.sender = inst->id();
    e.dest = PortId{ActorId{ProcId{world, root}, "comm", 0}, kPortMessage};
    e.data = encode_cast_root(c, ps);
    e.parts = std::move(ps);
    Metrics::global().counter_add("cast.messages");
    proc->post(std::move(e));
  });
  // ---- durable sender, checkpoints, preemptible lock --------------------------------
  py::class_<MessageLog, std::shared_ptr<MessageLog>>(m, "MessageLog")
      .def(py::init<const std::string&>())
      .def("append",
           [](MessageLog& l, const std::string& sender, const std::string& dest, py::bytes data,
              std::map<std::string, std::string> headers, std::vector<py::bytes> parts) {
             Envelope e;
             e.sender = ActorId::parse(sender);
             e.dest = PortId::parse(dest);
             e.data = data;
             e.headers = std::move(headers);
             e.parts = to_strings(parts);
             return l.append(e);
           },
           py::arg("sender"), py::arg("dest"), py::arg("data"),
           py::arg("headers") = std::map<std::string, std::string>{},
           py::arg("parts") = std::vector<py::bytes>{})
      .def("flush", &MessageLog::flush, py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("next_seq", &MessageLog::next_seq)
      .def_property_readonly("path", &MessageLog::path)
      .def("read",
           [](MessageLog& l, uint64_t from) {
             py::list out;
             for (auto& r : l.read(from)) out.append(py::make_tuple(r.first, to_py(r.second)));
             return out;
           },
           py::arg("from_seq") = 0);
  py::class_<DurableMailboxSender, std::shared_ptr<DurableMailboxSender>>(m, "DurableSender")
      .def(py::init([](std::shared_ptr<MessageLog> log, std::shared_ptr<Proc> proc) {
             return std::make_shared<DurableMailboxSender>(
                 std::move(log), std::make_shared<ProcSender>(proc),
                 [](Envelope env, const std::string& why) {
                   MB_LOG(Error, "message to " + env.dest.to_string() + " dropped: " + why);
                 });
           }),
           py::arg("log"), py::arg("proc"))
      .def("post",
           [](DurableMailboxSender& d, const std::string& sender, const std::string& dest,
              py::bytes data, std::map<std::string, std::string> headers,
              std::vector<py::bytes> parts) {
             Envelope e;
             e.sender = ActorId::parse(sender);
             e.dest = PortId::parse(dest);
             e.data = data;
             e.headers = std::move(headers);
             e.parts = to_strings(parts);
             py::gil_scoped_release rel;
             d.post(std::move(e));
           },
           py::arg("sender"), py::arg("dest"), py::arg("data"),
           py::arg("headers") = std::map<std::string, std::string>{},
           py::arg("parts") = std::vector<py::bytes>{})
      .def("replay", &DurableMailboxSender::replay, py::arg("from_seq") = 0,
           py::call_guard<py::gil_scoped_release>());
  m.def("write_checkpoint", [](const std::string& path, py::bytes blob) {
    std::string b = blob;
    py::gil_scoped_release rel;
    write_checkpoint(path, b);
  });
  m.def("read_checkpoint", [](const std::string& path) -> py::object {
    std::string b;
    if (!read_checkpoint(path, &b)) return py::none();
    return py::bytes(b);
  });
  struct PyRwLock {
    PreemptibleRwLock lock;
    std::mutex mu;
    std::map<uint64_t, std::unique_ptr<PreemptibleRwLock::ReadGuard>> reads;
    std::unique_ptr<PreemptibleRwLock::WriteGuard> write;
    uint64_t next = 1;
  };
  py::class_<PyRwLock, std::shared_ptr<PyRwLock>>(m, "PreemptibleRwLock")
      .def(py::init<>())
      .def("read_acquire",
           [](PyRwLock& l, int64_t timeout_ms) -> py::object {
             std::unique_ptr<PreemptibleRwLock::ReadGuard> g;
             bool ok;
             {
               py::gil_scoped_release rel;
               ok = l.lock.try_read_for(timeout_ms, &g);
             }
             if (!ok) return py::none();
             std::lock_guard<std::mutex> lk(l.mu);
             uint64_t id = l.next++;
             l.reads[id] = std::move(g);
             return py::int_(id);
           },
           py::arg("timeout_ms") = -1)
      .def("preempted",
           [](PyRwLock& l, uint64_t id) {
             std::lock_guard<std::mutex> lk(l.mu);
             auto it = l.reads.find(id);
             return it != l.reads.end() && it->second->preempted();
           })
      .def("read_release",
           [](PyRwLock& l, uint64_t id) {
             std::unique_ptr<PreemptibleRwLock::ReadGuard> g;
             {
               std::lock_guard<std::mutex> lk(l.mu);
               auto it = l.reads.find(id);
               if (it == l.reads.end()) return;
               g = std::move(it->second);
               l.reads.erase(it);
             }
             g->release();
           })
      .def("write_acquire",
           [](PyRwLock& l) {
             py::gil_scoped_release rel;
             auto g = std::make_unique<PreemptibleRwLock::WriteGuard>(l.lock.write());
             std::lock_guard<std::mutex> lk(l.mu);
             l.write = std::move(g);
           })
      .def("write_release",
           [](PyRwLock& l) {
             std::unique_ptr<PreemptibleRwLock::WriteGuard> g;
             {
               std::lock_guard<std::mutex> lk(l.mu);
               g = std::move(l.write);
             }
             if (g) g->release();
           })
      .def_property_readonly("readers", [](PyRwLock& l) { return l.lock.readers(); })
      .def_property_readonly("writers_waiting",
                             [](PyRwLock& l) { return l.lock.writers_waiting(); });
  m.def("client_proc", [] { return client_ctx().proc; });
  m.def("bootstrap_main", [] {
    py::gil_scoped_release rel;
    return bootstrap_main();
  });
  m.def("simnet_configure", &simnet_configure, py::arg("latency_us_by_distance"),
        py::arg("bandwidth_gbs") = 0.0,
        "Latency (microseconds) per node distance 0, 1, 2, ... and the link bandwidth of the "
        "simulated network behind sim: channels.");
  m.def("simnet_stats", [] {
    SimNetStats s = simnet_stats();
    py::dict d;
    d["frames"] = s.frames;
    d["bytes"] = s.bytes;
    d["latency_us_total"] = s.latency_us_total;
    py::list by;
    for (int i = 0; i < 8; ++i) by.append(s.by_distance[i]);
    d["frames_by_distance"] = by;
    return d;
  });
  m.def("simnet_reset_stats", &simnet_reset_stats);
  m.def("simnet_distance", &simnet_distance);
  m.def("bootstrap_attach", [](const std::string& addr, int64_t index) {
    py::gil_scoped_release rel;
    return bootstrap_attach(addr, index);
  }, py::arg("addr"), py::arg("index"),
  "Host proc `index` of the attach allocation listening at `addr` in this process; returns "
  "when the mesh is stopped.");
  py::class_<AttachAlloc, std::shared_ptr<AttachAlloc>>(m, "AttachAlloc")
      .def(py::init([](const std::string& world, size_t n, const std::string& transport) {
             return make_attach_alloc(world, n, transport);
           }),
           py::arg("world"), py::arg("n"), py::arg("transport") = "unix")
      .def_property_readonly("bootstrap_addr", &AttachAlloc::bootstrap_addr)
      .def("stop", [](AttachAlloc& a) {
        py::gil_scoped_release rel;
        a.stop();
      });

  py::class_<ProcMesh, std::shared_ptr<ProcMesh>>(m, "ProcMesh")
      .def_static(
          "allocate_local",
          [](const std::string& world, size_t n, int64_t timeout_ms) {
            py::gil_scoped_release rel;
            auto& c = client_ctx();
            return ProcMesh::allocate(make_local_alloc(world, n, c.router), c.router, c.proc,
                                      timeout_ms);
          },
          py::arg("world"), py::arg("n"), py::arg("timeout_ms") = 30000)
      .def_static(
          "allocate_sim",
          [](const std::string& world, std::vector<std::string> nodes, int64_t timeout_ms) {
            py::gil_scoped_release rel;
            auto& c = client_ctx();
            return ProcMesh::allocate(make_sim_alloc(world, std::move(nodes)), c.router, c.proc,
                                      timeout_ms);
          },
          py::arg("world"), py::arg("nodes"), py::arg("timeout_ms") = 60000)
      .def_static(
          "allocate_attached",
          [](std::shared_ptr<AttachAlloc> alloc, int64_t timeout_ms) {
            py::gil_scoped_release rel;
            auto& c = client_ctx();
            return ProcMesh::allocate(alloc, c.router, c.proc, timeout_ms);
          },
          py::arg("alloc"), py::arg("timeout_ms") = 120000)
      .def_static(
          "allocate_process",
          [](const std::string& world, size_t n, std::vector<std::string> argv,
             std::map<std::string, std::string> env, bool per_rank_gpu_env, py::object log_sink,
             const std::string& transport, int64_t timeout_ms) {
            ProcessAllocOptions o;
            o.argv = std::move(argv);
            o.env = std::move(env);
            o.per_rank_gpu_env = per_rank_gpu_env;
            o.transport = transport;
            PyFn cb = wrap(log_sink);
            if (cb)
              o.log_sink = [cb](int64_t rank, bool is_err, const std::string& line) {
                if (!interp_alive()) return;
                py::gil_scoped_acquire g;
                try {
                  cb->fn(rank, is_err, line);
                } catch (py::error_already_set& e) {
                  py_error_text(e);
                }
              };
            py::gil_scoped_release rel;
            auto& c = client_ctx();
            return ProcMesh::allocate(make_process_alloc(world, n, std::move(o)), c.router, c.proc,
                                      timeout_ms);
          },
          py::arg("world"), py::arg("n"), py::arg("argv"),
          py::arg("env") = std::map<std::string, std::string>{},
          py::arg("per_rank_gpu_env") = false, py::arg("log_sink") = py::none(),
          py::arg("transport") = "unix", py::arg("timeout_ms") = 120000)
      .def_property_readonly("world", &ProcMesh::world)
      .def("__len__", &ProcMesh::size)
      .def_property_readonly("client", &ProcMesh::client)
      .def("local_procs", &ProcMesh::local_procs)
      .def("spawn",
           [](ProcMesh& pm, const std::string& name, const std::string& type, py::bytes params,
              int64_t timeout_ms) {
             std::string p = params;
             std::vector<SpawnResult> res;
             {
               py::gil_scoped_release rel;
               res = pm.spawn(name, type, p, timeout_ms);
             }
             py::list out;
             for (auto& r : res) out.append(py::make_tuple(r.rank, r.ok, r.actor_id_or_error));
             return out;
           },
           py::arg("name"), py::arg("actor_type"), py::arg("params"),
           py::arg("timeout_ms") = 60000)
      .def("cast",
           [](ProcMesh& pm, const std::string& name, const Slice& slice,
              std::shared_ptr<Selection> sel, const std::string& sender, py::bytes data,
              std::map<std::string, std::string> headers, std::vector<py::object> parts,
              const Slice& cast_shape) {
             ActorId s = ActorId::parse(sender);
             std::string body = data;
             auto ps = to_strings(parts);
             py::gil_scoped_release rel;
             pm.cast(name, slice, sel, s, std::move(body), std::move(headers), std::move(ps),
                     cast_shape);
           },
           py::arg("name"), py::arg("slice"), py::arg("selection"), py::arg("sender"),
           py::arg("data"), py::arg("headers") = std::map<std::string, std::string>{},
           py::arg("parts") = std::vector<py::object>{}, py::arg("cast_shape") = Slice())
      .def("stop_actor", &ProcMesh::stop_actor, py::arg("name"), py::arg("timeout_ms") = 5000,
           py::call_guard<py::gil_scoped_release>())
      .def("ledger", &ProcMesh::ledger, py::arg("timeout_ms") = 5000,
           py::call_guard<py::gil_scoped_release>())
      .def("next_event",
           [](ProcMesh& pm, int64_t timeout_ms) -> py::object {
             std::optional<ProcMesh::Event> e;
             {
               py::gil_scoped_release rel;
               e = pm.next_event(timeout_ms);
             }
             if (!e) return py::none();
             py::dict d;
             d["kind"] = e->kind;
             d["rank"] = e->rank;
             d["reason"] = e->reason;
             d["actor_id"] = e->kind == "supervision" ? e->sup.actor_id.to_string() : "";
             d["status"] = e->sup.status;
             d["message"] = e->sup.message;
             return std::move(d);
           },
           py::arg("timeout_ms") = -1)
      .def("kill_rank", &ProcMesh::kill_rank, py::arg("rank"), py::arg("sig") = 9)
      .def("stop", &ProcMesh::stop, py::call_guard<py::gil_scoped_release>())
      .def_property_readonly("stopped", &ProcMesh::stopped);
}
