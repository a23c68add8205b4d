// Native executor core of the tensor worker.
//
// Holds the worker's environment (controller-assigned ref id -> tensor | error | other
// Python value) and executes ATen operator calls against it without returning to Python:
// refs in the arguments are resolved from the environment, a poisoned input poisons the
// results (dependent error), the operator is looked up once in the c10 dispatcher and
// called boxed on the requested CUDA stream, outputs are stored under the result refs.
// Recordings (the worker half of compile()) are parsed once into native call lists and
// replayed with ref rebinding in one call; messages that are not operator calls (UDFs,
// collectives, borrows) are handed back to a Python callback in order.
//
// Parity: monarch_tensor_worker/src/stream.rs:701-784 (try_define, call_torch_op),
// :1771-2026 (recordings), borrow.rs:27-68 (borrow state machine, here CUDA events),
// torch-sys/src/call_op.rs:169 (boxed dispatcher call), torch-sys/src/cell.rs (alias
// tracking is left to ATen: results that alias inputs share storage as usual).
#include <torch/csrc/jit/python/pybind_utils.h>
#include <torch/extension.h>
#include <torch/csrc/Dtype.h>

#include "messages.h"

#include <ATen/core/dispatch/Dispatcher.h>
#include <c10/core/Stream.h>
#include <c10/core/impl/VirtualGuardImpl.h>

#include <atomic>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <thread>
#include <unordered_map>
#include <variant>
#include <vector>

namespace py = pybind11;
using namespace mb::tensor;

namespace {


// One OS thread per named stream (monarch_tensor_worker/src/stream.rs:542-588 gives every
// StreamActor a dedicated thread): the worker actor only routes messages; each stream's
// commands run in arrival order on its own thread, so a command that blocks on the host
// (a user function waiting for something another stream produces, a collective's
// bootstrap) holds up its own stream only.  A task is either a Python callable, executed
// with the GIL held, or a native closure (an operator call parsed into an OpCall, a
// deletion), executed without ever taking the GIL: the actor's thread can unpickle and
// parse the next batch while this one computes.
class StreamThread {
 public:
  StreamThread(int64_t id, py::object on_start) : id_(id) {
    auto* cell = new py::object(std::move(on_start));
    thr_ = std::thread([this, cell] { loop(cell); });
  }
  ~StreamThread() { stop(); }

  struct Task {
    py::object* fn = nullptr;          // owned; released under the GIL
    std::function<void()> native;      // used when fn is null
  };

  // GIL held by the caller; the callable is released under the GIL on the stream thread.
  void submit(py::object fn) {
    Task t;
    t.fn = new py::object(std::move(fn));
    push(std::move(t));
  }
  void submit_native(std::function<void()> fn) {
    Task t;
    t.native = std::move(fn);
    push(std::move(t));
  }

  // GIL released by the caller.
  void drain() {
    std::unique_lock<std::mutex> lk(mu_);
    idle_cv_.wait(lk, [&] { return pending_ == 0 || stop_; });
  }

  void stop() {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (stop_) return;
      stop_ = true;
    }
    cv_.notify_all();
    idle_cv_.notify_all();
    if (thr_.joinable()) {
      if (thr_.get_id() == std::this_thread::get_id())
        thr_.detach();
      else {
        py::gil_scoped_release rel;
        thr_.join();
      }
    }
  }

  int64_t pending() {
    std::lock_guard<std::mutex> g(mu_);
    return pending_;
  }

 private:
  void run_cell(py::object* cell) {
    py::gil_scoped_acquire g;
    std::unique_ptr<py::object> own(cell);
    try {
      (*own)();
    } catch (py::error_already_set& e) {
      e.discard_as_unraisable("tensor worker stream thread");
    }
    own.reset();
  }
  void push(Task t) {
    {
      std::lock_guard<std::mutex> g(mu_);
      q_.push_back(std::move(t));
      ++pending_;
    }
    cv_.notify_all();
  }
  void loop(py::object* on_start) {
    if (!Py_IsInitialized()) return;
    run_cell(on_start);
    while (true) {
      Task task;
      {
        std::unique_lock<std::mutex> lk(mu_);
        cv_.wait(lk, [&] { return stop_ || !q_.empty(); });
        if (q_.empty()) break;       // stop requested and nothing left
        task = std::move(q_.front());
        q_.pop_front();
      }
      if (!Py_IsInitialized()) break;
      if (task.fn != nullptr) {
        run_cell(task.fn);
      } else {
        try {
          task.native();
        } catch (const std::exception&) {
          // native tasks report their own failures; nothing may escape the thread
        }
        task.native = nullptr;
      }
      {
        std::lock_guard<std::mutex> g(mu_);
        --pending_;
      }
      idle_cv_.notify_all();
    }
  }
  int64_t id_;
  std::thread thr_;
  std::mutex mu_;
  std::condition_variable cv_, idle_cv_;
  std::deque<Task> q_;
  int64_t pending_ = 0;
  bool stop_ = false;
};

// Rendezvous of all stream threads: every stream runs `arrive()` in its queue position; the
// last to arrive performs the action; with hold=true the others wait for it to finish
// (a barrier across streams), otherwise they carry on at once.
struct Fence {
  std::mutex mu;
  std::condition_variable cv;
  int remaining;
  bool done = false;
  explicit Fence(int n) : remaining(n) {}
};

class WorkerCore {
 public:
  WorkerCore(int64_t rank, py::object ref_type) : rank_(rank), ref_type_(std::move(ref_type)) {}
  ~WorkerCore() { stop_threads(); }

  // ------------------------------------------------------------------ stream threads
  // Start the thread of stream `id`; `on_start` runs first on it (device, current stream).
  void start_stream_thread(int64_t id, py::object on_start) {
    if (threads_.count(id)) return;
    threads_[id] = std::make_unique<StreamThread>(id, std::move(on_start));
  }
  bool has_stream_thread(int64_t id) const { return threads_.count(id) != 0; }
  void submit(int64_t id, py::object fn) {
    auto it = threads_.find(id);
    if (it == threads_.end()) throw py::key_error("stream " + std::to_string(id) + " has no thread");
    it->second->submit(std::move(fn));
  }
  // `action` (may be None) runs once every stream has reached this point of its queue.
  void fence(py::object action, bool hold) {
    if (threads_.empty()) {
      if (!action.is_none()) action();
      return;
    }
    auto f = std::make_shared<Fence>((int)threads_.size());
    auto act = std::make_shared<py::object>(std::move(action));
    for (auto& kv : threads_) {
      kv.second->submit(py::cpp_function([f, act, hold]() {
        bool last;
        {
          std::lock_guard<std::mutex> g(f->mu);
          last = --f->remaining == 0;
        }
        if (last) {
          if (!act->is_none()) {
            try {
              (*act)();
            } catch (py::error_already_set& e) {
              e.discard_as_unraisable("tensor worker fence action");
            }
          }
          *act = py::none();
          {
            std::lock_guard<std::mutex> g(f->mu);
            f->done = true;
          }
          f->cv.notify_all();
        } else if (hold) {
          py::gil_scoped_release rel;
          std::unique_lock<std::mutex> lk(f->mu);
          f->cv.wait(lk, [&] { return f->done; });
        }
      }));
    }
  }
  // Wait until every stream has run everything submitted so far.
  void drain() {
    py::gil_scoped_release rel;
    for (auto& kv : threads_) kv.second->drain();
  }
  void stop_threads() {
    for (auto& kv : threads_) kv.second->stop();
    threads_.clear();
  }
  int64_t pending() {
    int64_t n = 0;
    for (auto& kv : threads_) n += kv.second->pending();
    return n;
  }

  // ------------------------------------------------------------------ environment
  // The table is shared by the actor's thread and the stream threads.  Native tasks touch it
  // without the GIL, so `env_mu_` guards it; the methods below are called from Python (GIL
  // held) and take the mutex inside.  Values that own a Python reference are never destroyed
  // by a native task: it parks them in `graveyard_`, emptied by the next GIL-holding call.
  void set(int64_t id, py::object v) {
    Value nv;
    if (v.is_none()) {
      nv = std::monostate{};
    } else if (THPVariable_Check(v.ptr())) {
      nv = THPVariable_Unpack(v.ptr());
    } else {
      nv = std::move(v);
    }
    Value old;
    std::vector<Value> dead;
    {
      std::lock_guard<std::mutex> g(env_mu_);
      auto& slot = env_[id];
      old = std::move(slot);
      slot = std::move(nv);
      dead.swap(graveyard_);
    }
  }
  void set_error(int64_t id, int64_t seq, int64_t rank, std::string func, std::string text,
                 std::string tb, int64_t dep) {
    Value old;
    std::lock_guard<std::mutex> g(env_mu_);
    auto& slot = env_[id];
    old = std::move(slot);
    slot = std::make_shared<RemoteErr>(RemoteErr{seq, rank, std::move(func), std::move(text),
                                                 std::move(tb), dep});
  }
  // The index of the GPU this worker owns (-1: a CPU worker).
  void set_cuda_index(int64_t idx) { cuda_index_ = idx; }
  bool contains(int64_t id) {
    std::lock_guard<std::mutex> g(env_mu_);
    return env_.count(id) != 0;
  }
  py::object get(int64_t id) {
    Value v;
    {
      std::lock_guard<std::mutex> g(env_mu_);
      auto it = env_.find(id);
      if (it == env_.end()) throw py::key_error("Ref(" + std::to_string(id) + ")");
      v = it->second;
    }
    return to_py(v);
  }
  py::object pop(int64_t id) {
    Value v;
    {
      std::lock_guard<std::mutex> g(env_mu_);
      auto it = env_.find(id);
      if (it == env_.end()) return py::none();
      v = std::move(it->second);
      env_.erase(it);
    }
    return to_py(v);
  }
  void erase(const std::vector<int64_t>& ids) {
    std::vector<Value> dead;     // destroyed after the mutex is released (GIL held here)
    std::lock_guard<std::mutex> g(env_mu_);
    dead.swap(graveyard_);
    for (auto i : ids) {
      auto it = env_.find(i);
      if (it == env_.end()) continue;
      dead.push_back(std::move(it->second));
      env_.erase(it);
    }
  }
  size_t size() {
    std::lock_guard<std::mutex> g(env_mu_);
    return env_.size();
  }
  int64_t live_bytes() {
    std::lock_guard<std::mutex> g(env_mu_);
    int64_t n = 0;
    for (auto& kv : env_)
      if (auto* t = std::get_if<at::Tensor>(&kv.second))
        if (t->defined()) n += (int64_t)t->numel() * t->element_size();
    return n;
  }

  // ------------------------------------------------------------------ message batches
  // `report(err_tuple)` is called (GIL taken for it) when a native task fails on its own.
  void set_report(py::object report) { report_ = std::move(report); }
  void set_null_device(bool on) { null_device_ = on; }
  int64_t last_seq() const { return last_seq_.load(); }

  // Route one batch of worker messages (monarch_messages/src/worker.rs WorkerMessage:
  // CallFunction, DeleteRefs, ...).  Operator calls are decoded here into native OpCall
  // structs and queued on the thread of their stream, deletions into a native rendezvous of
  // all streams; both then run without the GIL.  Every other message, and any call whose
  // arguments the native decoder does not take, goes to `fallback(msg)` (the Python router),
  // in order.
  int64_t route_batch(py::list msgs, py::object fallback) {
    int64_t native = 0;
    for (auto h : msgs) {
      py::tuple m = py::reinterpret_borrow<py::tuple>(h);
      bool done = false;
      if (!threads_.empty() && m.size() >= 2 && PyUnicode_Check(m[0].ptr())) {
        switch (kind_of(PyUnicode_AsUTF8(m[0].ptr()))) {
          case MessageKind::Call:
            if (m.size() == 8)
              done = route_call(m);
            else if (m.size() == 9 && null_device_ && !m[8].is_none())
              done = route_null_call(m);
            break;
          case MessageKind::Delete:
            if (m.size() == 2) {
              auto del = std::make_shared<DeleteRefs>();
              del->ids = m[1].cast<std::vector<int64_t>>();
              fence_native([this, del]() { erase_nogil(del->ids); });
              done = true;
            }
            break;
          default:
            break;   // named and handled by the Python router
        }
      }
      if (done)
        ++native;
      else
        fallback(m);
    }
    return native;
  }

  // ------------------------------------------------------------------ operator calls
  // Returns None on success, or (seq, rank, func, text, tb, dependent_of) of the error that
  // now poisons the result refs (dependent_of >= 0: inherited, nothing new to report).
  py::object call_op(int64_t seq, std::vector<int64_t> results, std::vector<int64_t> mutates,
                     const std::string& qualname, py::tuple args, py::dict kwargs,
                     int64_t stream) {
    auto call = parse_call(seq, std::move(results), std::move(mutates), qualname, args, kwargs,
                           stream);
    return run(*call, nullptr);
  }

  // ---------------------------------------------------------------------- recordings
  // msgs: the recorded worker messages.  ("call", seq, results, mutates, ("op", name), args,
  // kwargs, stream) items become native calls; everything else stays with Python.
  void define_recording(int64_t rec_id, py::list msgs,
                        const std::unordered_map<int64_t, std::vector<int64_t>>& drop_after) {
    std::vector<RecItem> items;
    size_t idx = 0;
    for (auto h : msgs) {
      py::tuple m = py::reinterpret_borrow<py::tuple>(h);
      RecItem it;
      it.index = idx++;
      if (py::str(m[0]).cast<std::string>() == "call") {
        py::tuple spec = m[4];
        if (py::str(spec[0]).cast<std::string>() == "op") {
          try {
            it.call = parse_call(m[1].cast<int64_t>(), refs_of(m[2]), refs_of(m[3]),
                                 spec[1].cast<std::string>(), m[5], m[6],
                                 m[7].cast<int64_t>());
          } catch (const std::exception&) {
            it.call.reset();  // unusual argument structure: let Python run this one
          }
        }
      }
      auto d = drop_after.find((int64_t)it.index);
      if (d != drop_after.end()) it.drop = d->second;
      items.push_back(std::move(it));
    }
    recordings_[rec_id] = std::move(items);
  }

  // Replays recording `rec_id` with ref ids rebound through `bind`.  `fallback(index, bind)`
  // runs the non-native messages; `report(err_tuple)` is called for each new failure.
  int64_t call_recording(int64_t rec_id, const std::unordered_map<int64_t, int64_t>& bind,
                         py::object fallback, py::object report) {
    auto rit = recordings_.find(rec_id);
    if (rit == recordings_.end()) throw py::key_error("recording " + std::to_string(rec_id));
    int64_t native = 0;
    for (auto& it : rit->second) {
      if (it.call) {
        py::object err = run(*it.call, &bind);
        ++native;
        if (!err.is_none() && !report.is_none() &&
            err.cast<py::tuple>()[5].cast<int64_t>() < 0)
          report(err);
      } else {
        fallback(it.index, bind);
      }
      // temporaries of the recording die after their last use
      if (!it.drop.empty()) erase(it.drop);
    }
    return native;
  }
  bool has_recording(int64_t id) const { return recordings_.count(id) != 0; }

  // ------------------------------------------------------------------------- streams
  void create_stream(int64_t id, py::object torch_stream) { streams_[id] = std::move(torch_stream); }

 private:
  int64_t rank_;
  int64_t cuda_index_ = -1;
  py::object ref_type_;
  std::unordered_map<int64_t, Value> env_;
  std::unordered_map<int64_t, std::vector<RecItem>> recordings_;
  std::unordered_map<int64_t, py::object> streams_;
  std::unordered_map<int64_t, std::unique_ptr<StreamThread>> threads_;
  std::mutex env_mu_;
  std::vector<Value> graveyard_;     // guarded by env_mu_
  py::object report_ = py::none();
  std::atomic<int64_t> last_seq_{-1};
  bool null_device_ = false;

  // An operator call of a batch: parse with the GIL, run on the stream's thread without.
  bool route_call(const py::tuple& m) {
    py::handle spec = m[4];
    if (!PyTuple_Check(spec.ptr()) || PyTuple_GET_SIZE(spec.ptr()) != 2) return false;
    py::handle tag = PyTuple_GET_ITEM(spec.ptr(), 0), name = PyTuple_GET_ITEM(spec.ptr(), 1);
    if (!PyUnicode_Check(tag.ptr()) || !PyUnicode_Check(name.ptr())) return false;
    if (std::strcmp(PyUnicode_AsUTF8(tag.ptr()), "op") != 0) return false;
    std::shared_ptr<OpCall> call;
    StreamThread* thr = nullptr;
    try {
      const int64_t stream = m[7].cast<int64_t>();
      auto it = threads_.find(stream);
      if (it == threads_.end()) return false;
      thr = it->second.get();
      call = parse_call(m[1].cast<int64_t>(), refs_of(m[2]), refs_of(m[3]),
                        name.cast<std::string>(), m[5], m[6], stream);
    } catch (py::error_already_set& e) {
      e.restore();
      PyErr_Clear();
      return false;
    } catch (const std::exception&) {
      return false;            // unusual argument structure: Python runs this one
    }
    thr->submit_native([this, call]() {
      int64_t prev = last_seq_.load();
      while (prev < call->seq && !last_seq_.compare_exchange_weak(prev, call->seq)) {
      }
      ErrPtr e = run_impl(*call, nullptr, false);
      if (e && e->dependent_of < 0) {
        py::gil_scoped_acquire g;
        if (!report_.is_none()) {
          try {
            report_(err_tuple(*e, false));
          } catch (py::error_already_set& ex) {
            ex.discard_as_unraisable("tensor worker error report");
          }
        }
      }
    });
    return true;
  }

  // Shape-only workers: the controller announces the results' metadata and nothing is
  // executed; zero tensors of those shapes stand in.
  bool route_null_call(const py::tuple& m) {
    auto call = std::make_shared<ShapeOnlyCall>();
    StreamThread* thr = nullptr;
    try {
      call->seq = m[1].cast<int64_t>();
      call->results = refs_of(m[2]);
      call->stream = m[7].cast<int64_t>();
      auto it = threads_.find(call->stream);
      if (it == threads_.end()) return false;
      thr = it->second.get();
      for (auto h : m[8]) {
        py::tuple mt = py::reinterpret_borrow<py::tuple>(h);
        if (!THPDtype_Check(mt[1].ptr())) return false;
        call->metas.push_back(ShapeOnlyCall::Meta{
            mt[0].cast<std::vector<int64_t>>(),
            reinterpret_cast<THPDtype*>(mt[1].ptr())->scalar_type});
      }
    } catch (py::error_already_set& e) {
      e.restore();
      PyErr_Clear();
      return false;
    } catch (const std::exception&) {
      return false;
    }
    if (call->metas.size() != call->results.size()) return false;
    thr->submit_native([this, call]() {
      int64_t prev = last_seq_.load();
      while (prev < call->seq && !last_seq_.compare_exchange_weak(prev, call->seq)) {
      }
      for (size_t i = 0; i < call->results.size(); ++i)
        assign(call->results[i], at::zeros(call->metas[i].shape,
                                           at::TensorOptions().dtype(call->metas[i].dtype)));
    });
    return true;
  }

  // `action` runs (without the GIL) once every stream has reached this point of its queue;
  // no stream waits for it.
  void fence_native(std::function<void()> action) {
    auto remaining = std::make_shared<std::atomic<int>>((int)threads_.size());
    auto act = std::make_shared<std::function<void()>>(std::move(action));
    for (auto& kv : threads_) {
      kv.second->submit_native([remaining, act]() {
        if (remaining->fetch_sub(1) == 1) (*act)();
      });
    }
  }

  void erase_nogil(const std::vector<int64_t>& ids) {
    std::vector<Value> dead;   // tensors: freed here, after the mutex is released
    {
      std::lock_guard<std::mutex> g(env_mu_);
      for (auto i : ids) {
        auto it = env_.find(i);
        if (it == env_.end()) continue;
        if (std::holds_alternative<py::object>(it->second))
          graveyard_.push_back(std::move(it->second));
        else
          dead.push_back(std::move(it->second));
        env_.erase(it);
      }
    }
  }

  // Store `v` under `id`; callable without the GIL.
  void assign(int64_t id, Value v) {
    Value old;
    std::lock_guard<std::mutex> g(env_mu_);
    auto& slot = env_[id];
    if (std::holds_alternative<py::object>(slot))
      graveyard_.push_back(std::move(slot));
    else
      old = std::move(slot);
    slot = std::move(v);
  }

  static py::object to_py(const Value& v) {
    if (std::holds_alternative<std::monostate>(v)) return py::none();
    if (auto* t = std::get_if<at::Tensor>(&v))
      return py::reinterpret_steal<py::object>(THPVariable_Wrap(*t));
    if (auto* e = std::get_if<ErrPtr>(&v)) return err_tuple(**e, true);
    return std::get<py::object>(v);
  }
  static py::object err_tuple(const RemoteErr& e, bool tagged) {
    py::object dep = e.dependent_of >= 0 ? py::cast(e.dependent_of) : py::cast(int64_t(-1));
    if (tagged)
      return py::make_tuple("__remote_error__", e.seq, e.rank, e.func, e.text, e.tb, dep);
    return py::make_tuple(e.seq, e.rank, e.func, e.text, e.tb, dep);
  }

  bool is_ref(py::handle h) const { return py::isinstance(h, ref_type_); }
  std::vector<int64_t> refs_of(py::handle seq) const {
    std::vector<int64_t> out;
    for (auto h : seq) out.push_back(h.attr("id").cast<int64_t>());
    return out;
  }

  std::unique_ptr<OpCall> parse_call(int64_t seq, std::vector<int64_t> results,
                                     std::vector<int64_t> mutates, const std::string& qualname,
                                     py::handle args, py::handle kwargs, int64_t stream) {
    // "aten.add.Tensor" -> ("aten::add", "Tensor")
    auto p1 = qualname.find('.');
    auto p2 = qualname.rfind('.');
    if (p1 == std::string::npos || p2 == p1) throw std::runtime_error("bad op name " + qualname);
    std::string name = qualname.substr(0, p1) + "::" + qualname.substr(p1 + 1, p2 - p1 - 1);
    std::string overload = qualname.substr(p2 + 1);
    if (overload == "default") overload = "";
    auto call = std::make_unique<OpCall>(
        c10::Dispatcher::singleton().findSchemaOrThrow(name.c_str(), overload.c_str()));
    call->seq = seq;
    call->results = std::move(results);
    call->mutates = std::move(mutates);
    call->name = qualname;
    call->stream = stream;
    auto sit = streams_.find(stream);
    if (sit != streams_.end() && !sit->second.is_none()) call->py_stream = sit->second.ptr();
    const auto& schema = call->op.schema();
    const auto& sargs = schema.arguments();
    size_t pos = 0;
    for (auto h : args) {
      if (pos >= sargs.size()) throw std::runtime_error("too many arguments for " + qualname);
      call->args.push_back(parse_arg(h, sargs[pos].type(), ""));
      ++pos;
    }
    if (kwargs && !kwargs.is_none()) {
      for (auto kv : py::reinterpret_borrow<py::dict>(kwargs)) {
        std::string k = py::str(kv.first).cast<std::string>();
        auto idx = schema.argumentIndexWithName(k);
        if (!idx) throw std::runtime_error("unknown keyword " + k + " for " + qualname);
        call->args.push_back(parse_arg(kv.second, sargs[*idx].type(), k));
      }
    }
    return call;
  }

  Arg parse_arg(py::handle h, const c10::TypePtr& type, std::string name) const {
    Arg a;
    a.name = std::move(name);
    if (is_ref(h)) {
      a.kind = Arg::RefOne;
      a.refs.push_back(h.attr("id").cast<int64_t>());
      return a;
    }
    if ((py::isinstance<py::list>(h) || py::isinstance<py::tuple>(h)) && py::len(h) > 0) {
      bool all_refs = true, any_ref = false;
      for (auto x : h) {
        bool r = is_ref(x);
        all_refs = all_refs && r;
        any_ref = any_ref || r;
      }
      if (all_refs) {
        a.kind = Arg::RefList;
        for (auto x : h) a.refs.push_back(x.attr("id").cast<int64_t>());
        return a;
      }
      if (any_ref) throw std::runtime_error("mixed ref/value list");
    }
    a.kind = Arg::Const;
    // A Python number in a Tensor slot (`x + 1.0` reaches the dispatcher as
    // add.Tensor(x, 1.0)): a 0-dim "wrapped number" tensor, which takes part in type
    // promotion like the scalar it stands for.
    const bool tensor_slot =
        type->kind() == c10::TypeKind::TensorType ||
        (type->kind() == c10::TypeKind::OptionalType &&
         type->expectRef<c10::OptionalType>().getElementType()->kind() == c10::TypeKind::TensorType);
    if (tensor_slot && (py::isinstance<py::float_>(h) || py::isinstance<py::int_>(h) ||
                        py::isinstance<py::bool_>(h))) {
      at::Tensor t;
      if (py::isinstance<py::bool_>(h))
        t = at::scalar_to_tensor(c10::Scalar(h.cast<bool>()));
      else if (py::isinstance<py::int_>(h))
        t = at::scalar_to_tensor(c10::Scalar(h.cast<int64_t>()));
      else
        t = at::scalar_to_tensor(c10::Scalar(h.cast<double>()));
      t.unsafeGetTensorImpl()->set_wrapped_number(true);
      a.constant = c10::IValue(t);
      return a;
    }
    a.constant = torch::jit::toIValue(h, type);
    // The controller names "the worker's GPU" as cuda or cuda:<its own current index>; every
    // worker owns exactly one GPU, so any CUDA device in an argument means that one (the
    // reference gets the same effect by showing each worker process a single device).
    if (cuda_index_ >= 0 && a.constant.isDevice() && a.constant.toDevice().is_cuda())
      a.constant = c10::IValue(c10::Device(c10::DeviceType::CUDA, (c10::DeviceIndex)cuda_index_));

    return a;
  }

  // Resolve one ref; records the first poisoned input in `dep`.
  bool resolve(int64_t id, const std::unordered_map<int64_t, int64_t>* bind, at::Tensor& out,
               ErrPtr& dep, bool& is_none) {
    if (bind) {
      auto b = bind->find(id);
      if (b != bind->end()) id = b->second;
    }
    std::lock_guard<std::mutex> g(env_mu_);
    auto it = env_.find(id);
    if (it == env_.end()) throw std::runtime_error("Ref(" + std::to_string(id) + ") is not defined");
    is_none = false;
    if (auto* t = std::get_if<at::Tensor>(&it->second)) {
      out = *t;
      return true;
    }
    if (auto* e = std::get_if<ErrPtr>(&it->second)) {
      if (!dep) dep = *e;
      return false;
    }
    if (std::holds_alternative<std::monostate>(it->second)) {
      is_none = true;
      return true;
    }
    throw std::runtime_error("Ref(" + std::to_string(id) + ") does not hold a tensor");
  }

  static int64_t rebound(int64_t id, const std::unordered_map<int64_t, int64_t>* bind) {
    if (!bind) return id;
    auto b = bind->find(id);
    return b == bind->end() ? id : b->second;
  }

  ErrPtr poison(const OpCall& c, const std::unordered_map<int64_t, int64_t>* bind, ErrPtr e) {
    for (auto r : c.results) assign(rebound(r, bind), e);
    for (auto r : c.mutates) assign(rebound(r, bind), e);
    return e;
  }

  // GIL held by the caller.
  py::object run(const OpCall& c, const std::unordered_map<int64_t, int64_t>* bind) {
    ErrPtr e = run_impl(c, bind, true);
    if (!e) return py::none();
    return err_tuple(*e, false);
  }

  // Executes one operator call; null on success, else the error that now poisons its
  // results.  `gil_held` says whether the calling thread holds the GIL (it is released
  // around the dispatcher call); a native task passes false and never takes it, except to
  // enter a torch.cuda.Stream context where the call names one.
  ErrPtr run_impl(const OpCall& c, const std::unordered_map<int64_t, int64_t>* bind,
                  bool gil_held) {
    ErrPtr dep;
    try {
      const auto& schema = c.op.schema();
      const auto& sargs = schema.arguments();
      std::vector<c10::IValue> slots(sargs.size());
      std::vector<bool> filled(sargs.size(), false);
      size_t pos = 0;
      for (const auto& a : c.args) {
        size_t idx = pos;
        if (!a.name.empty()) {
          idx = *schema.argumentIndexWithName(a.name);
        } else {
          ++pos;
        }
        if (a.kind == Arg::Const) {
          slots[idx] = a.constant;
        } else if (a.kind == Arg::RefOne) {
          at::Tensor t;
          bool none = false;
          if (resolve(a.refs[0], bind, t, dep, none)) slots[idx] = none ? c10::IValue() : c10::IValue(t);
        } else {
          c10::List<at::Tensor> l;
          for (auto id : a.refs) {
            at::Tensor t;
            bool none = false;
            if (resolve(id, bind, t, dep, none)) l.push_back(t);
          }
          slots[idx] = c10::IValue(l);
        }
        filled[idx] = true;
      }
      if (dep) {
        auto e = std::make_shared<RemoteErr>(
            RemoteErr{c.seq, rank_, c.name, dep->text, dep->tb, dep->seq});
        return poison(c, bind, e);
      }
      for (size_t i = 0; i < sargs.size(); ++i) {
        if (filled[i]) continue;
        if (!sargs[i].default_value())
          throw std::runtime_error("missing argument " + sargs[i].name() + " of " + c.name);
        slots[i] = *sargs[i].default_value();
      }
      torch::jit::Stack stack(slots.begin(), slots.end());
      if (c.py_stream == nullptr && !gil_held) {
        c.op.callBoxed(stack);       // the thread's current stream is the call's stream
      } else {
        std::optional<py::gil_scoped_acquire> take;
        if (!gil_held) take.emplace();
        py::object guard;
        const bool has_stream = c.py_stream != nullptr;
        if (has_stream) {
          // torch.cuda.stream(s) context: enter/exit around the launch
          guard = py::module_::import("torch").attr("cuda").attr("stream")(
              py::reinterpret_borrow<py::object>(c.py_stream));
          guard.attr("__enter__")();
        }
        try {
          py::gil_scoped_release nogil;
          c.op.callBoxed(stack);
        } catch (...) {
          if (has_stream) guard.attr("__exit__")(py::none(), py::none(), py::none());
          throw;
        }
        if (has_stream) guard.attr("__exit__")(py::none(), py::none(), py::none());
      }
      // flatten tensor outputs (tensors and tensor lists) in return order
      std::vector<at::Tensor> flat;
      for (auto& v : stack) {
        if (v.isTensor()) {
          // an undefined tensor is an optional output that is absent (None on the
          // controller, which counts only the tensors it saw during propagation)
          if (v.toTensor().defined()) flat.push_back(v.toTensor());
        } else if (v.isTensorList()) {
          for (const at::Tensor& t : v.toTensorList()) flat.push_back(t);
        }
      }
      if (c.results.empty() && !c.mutates.empty()) flat.clear();  // in-place: aliases an arg
      if (flat.size() != c.results.size())
        throw std::runtime_error(c.name + " returned " + std::to_string(flat.size()) +
                                 " tensors, controller expected " +
                                 std::to_string(c.results.size()));
      for (size_t i = 0; i < flat.size(); ++i) assign(rebound(c.results[i], bind), flat[i]);
      return nullptr;
    } catch (const std::exception& ex) {
      auto e = std::make_shared<RemoteErr>(
          RemoteErr{c.seq, rank_, c.name, std::string("RuntimeError: ") + ex.what(), "", -1});
      return poison(c, bind, e);
    }
  }
};

}  // namespace

PYBIND11_MODULE(_tensor_worker, m) {
  m.doc() = "native executor core of the tensor worker";
  py::class_<WorkerCore>(m, "WorkerCore")
      .def(py::init<int64_t, py::object>(), py::arg("rank"), py::arg("ref_type"))
      .def("set", &WorkerCore::set)
      .def("set_error", &WorkerCore::set_error)
      .def("set_cuda_index", &WorkerCore::set_cuda_index)
      .def("get", &WorkerCore::get)
      .def("pop", &WorkerCore::pop)
      .def("contains", &WorkerCore::contains)
      .def("erase", &WorkerCore::erase)
      .def("__len__", &WorkerCore::size)
      .def("live_bytes", &WorkerCore::live_bytes)
      .def("call_op", &WorkerCore::call_op)
      .def("define_recording", &WorkerCore::define_recording, py::arg("rec_id"), py::arg("msgs"),
           py::arg("drop_after") = std::unordered_map<int64_t, std::vector<int64_t>>{})
      .def("call_recording", &WorkerCore::call_recording)
      .def("has_recording", &WorkerCore::has_recording)
      .def("create_stream", &WorkerCore::create_stream)
      .def("start_stream_thread", &WorkerCore::start_stream_thread)
      .def("has_stream_thread", &WorkerCore::has_stream_thread)
      .def("submit", &WorkerCore::submit)
      .def("route_batch", &WorkerCore::route_batch)
      .def("set_report", &WorkerCore::set_report)
      .def("set_null_device", &WorkerCore::set_null_device)
      .def("last_seq", &WorkerCore::last_seq)
      .def("fence", &WorkerCore::fence, py::arg("action"), py::arg("hold") = true)
      .def("drain", &WorkerCore::drain)
      .def("pending", &WorkerCore::pending)
      .def("stop_threads", &WorkerCore::stop_threads);
}
