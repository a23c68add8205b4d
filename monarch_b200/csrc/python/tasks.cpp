// Task runtime behind monarch_b200.actor.pytokio and Future: a native thread pool that
// runs Python callables, completion objects that can be waited on without the GIL, waited
// on in groups (select), and observed through callbacks (event-loop integration).
//
// Parity: monarch_hyperactor/src/pytokio.rs:61-295 (PythonTask / Shared over the tokio
// runtime: block_on, spawn, spawn_blocking, with_timeout, select_one, is_tokio_thread) and
// runtime.rs:36-155 (signal_safe_block_on).  The reference schedules Rust futures; here
// the unit of scheduling is a callable on a pool thread and a completion that continuations
// hang off, which is all the Python layer needs.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace {

std::atomic<bool> g_shutdown{false};
thread_local bool t_in_pool = false;

// A one-shot result slot.  The Python value is only touched with the GIL held; waiting
// happens on the native condition variable with the GIL released.
struct Completion : std::enable_shared_from_this<Completion> {
  std::mutex mu;
  std::condition_variable cv;
  bool done = false;
  bool is_err = false;
  py::object value;                                // guarded by the GIL
  std::vector<py::object> py_callbacks;            // guarded by the GIL (+ mu for the swap)
  std::vector<std::function<void()>> native_callbacks;

  // GIL held.
  void finish(py::object v, bool err) {
    std::vector<py::object> pcbs;
    std::vector<std::function<void()>> ncbs;
    {
      std::lock_guard<std::mutex> g(mu);
      if (done) return;
      value = std::move(v);
      is_err = err;
      done = true;
      pcbs.swap(py_callbacks);
      ncbs.swap(native_callbacks);
    }
    cv.notify_all();
    for (auto& f : ncbs) f();
    for (auto& cb : pcbs) {
      try {
        cb();
      } catch (py::error_already_set& e) {
        e.discard_as_unraisable("monarch_b200 completion callback");
      }
    }
  }

  // GIL released by the caller.  timeout_ms < 0: forever.
  bool wait(int64_t timeout_ms) {
    std::unique_lock<std::mutex> lk(mu);
    if (timeout_ms < 0) {
      cv.wait(lk, [&] { return done; });
      return true;
    }
    return cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return done; });
  }

  bool is_done() {
    std::lock_guard<std::mutex> g(mu);
    return done;
  }

  // Runs fn now if already complete, else when it completes (on the completing thread).
  void on_done_native(std::function<void()> fn) {
    {
      std::lock_guard<std::mutex> g(mu);
      if (!done) {
        native_callbacks.push_back(std::move(fn));
        return;
      }
    }
    fn();
  }
};

class TaskPool {
 public:
  static TaskPool& get() {
    static TaskPool* p = new TaskPool();  // leaked: threads may outlive static destruction
    return *p;
  }

  void submit(std::function<void()> job) {
    {
      std::lock_guard<std::mutex> g(mu_);
      q_.push_back({std::move(job), std::chrono::steady_clock::now()});
      if (idle_ == 0 && threads_ < kCoreThreads) add_thread();
      if (!watchdog_started_) {
        watchdog_started_ = true;
        std::thread([this] { watchdog(); }).detach();
      }
    }
    cv_.notify_one();
  }

  int threads() {
    std::lock_guard<std::mutex> g(mu_);
    return threads_;
  }

 private:
  // A few threads serve short jobs (coroutine steps, callbacks).  Jobs may also block --
  // on I/O, or on the result of a job that is still queued -- so when work has waited
  // with every thread busy, the watchdog adds a thread; no queued job starves.
  static constexpr int kCoreThreads = 4;
  static constexpr int kMaxThreads = 512;
  struct Item {
    std::function<void()> job;
    std::chrono::steady_clock::time_point at;
  };
  void add_thread() {  // mu_ held
    ++threads_;
    std::thread([this] { run(); }).detach();
  }
  void watchdog() {
    while (!g_shutdown) {
      std::this_thread::sleep_for(std::chrono::milliseconds(5));
      std::lock_guard<std::mutex> g(mu_);
      if (!q_.empty() && idle_ == 0 && threads_ < kMaxThreads &&
          std::chrono::steady_clock::now() - q_.front().at > std::chrono::milliseconds(20))
        add_thread();
    }
  }
  void run() {
    t_in_pool = true;
    while (!g_shutdown) {
      std::function<void()> job;
      {
        std::unique_lock<std::mutex> lk(mu_);
        ++idle_;
        cv_.wait_for(lk, std::chrono::milliseconds(200), [&] { return !q_.empty() || g_shutdown; });
        --idle_;
        if (q_.empty()) continue;
        job = std::move(q_.front().job);
        q_.pop_front();
      }
      job();
    }
  }
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Item> q_;
  int threads_ = 0, idle_ = 0;
  bool watchdog_started_ = false;
};

// Run a Python callable on the pool; its return value (or exception) completes `c`.
void spawn_py(std::shared_ptr<Completion> c, py::object fn) {
  // The callable and the completion travel in a heap cell that is released under the GIL
  // on the pool thread: dropping the last reference to either may free Python objects.
  struct Cell {
    py::object fn;
    std::shared_ptr<Completion> c;
  };
  auto* cell = new Cell{std::move(fn), std::move(c)};
  TaskPool::get().submit([cell] {
    if (g_shutdown || !Py_IsInitialized()) return;   // interpreter is going away: drop it
    py::gil_scoped_acquire g;
    std::unique_ptr<Cell> own(cell);
    try {
      py::object r = own->fn();
      own->c->finish(std::move(r), false);
    } catch (py::error_already_set& e) {
      py::object exc = e.value();
      own->c->finish(std::move(exc), true);
    }
    own.reset();   // still under the GIL
  });
}

}  // namespace

void bind_tasks(py::module_& m) {
  py::class_<Completion, std::shared_ptr<Completion>>(m, "Completion")
      .def(py::init([] { return std::make_shared<Completion>(); }))
      .def("set_result", [](Completion& c, py::object v) { c.finish(std::move(v), false); })
      .def("set_exception", [](Completion& c, py::object e) { c.finish(std::move(e), true); })
      .def("done", &Completion::is_done)
      .def("wait",
           [](Completion& c, int64_t timeout_ms) {
             py::gil_scoped_release rel;
             return c.wait(timeout_ms);
           },
           py::arg("timeout_ms") = -1,
           "Block (GIL released) until complete; False when the timeout ran out.")
      .def("failed", [](Completion& c) {
        std::lock_guard<std::mutex> g(c.mu);
        return c.done && c.is_err;
      })
      .def("value",
           [](Completion& c) -> py::object {
             std::lock_guard<std::mutex> g(c.mu);
             if (!c.done) throw std::runtime_error("completion is not done");
             return c.value;
           },
           "The result or the exception object (see failed()).")
      .def("add_done_callback",
           [](std::shared_ptr<Completion> c, py::object fn) {
             {
               std::lock_guard<std::mutex> g(c->mu);
               if (!c->done) {
                 c->py_callbacks.push_back(std::move(fn));
                 return;
               }
             }
             fn();
           },
           "Call fn() once the completion is done (at once if it already is); fn runs on the "
           "completing thread and must not block.");

  m.def("task_spawn",
        [](py::object fn) {
          auto c = std::make_shared<Completion>();
          spawn_py(c, std::move(fn));
          return c;
        },
        "Run fn() on the native task pool; returns its Completion.");
  m.def("is_task_thread", [] { return t_in_pool; });
  m.def("task_pool_threads", [] { return TaskPool::get().threads(); });
  m.def("task_shutdown", [] { g_shutdown = true; },
        "Stop handing work to pool threads (called at interpreter exit).");
  m.def("wait_any",
        [](std::vector<std::shared_ptr<Completion>> cs, int64_t timeout_ms) -> int {
          struct Waiter {
            std::mutex mu;
            std::condition_variable cv;
            int fired = -1;
          };
          auto w = std::make_shared<Waiter>();
          for (size_t i = 0; i < cs.size(); ++i) {
            int idx = (int)i;
            cs[i]->on_done_native([w, idx] {
              {
                std::lock_guard<std::mutex> g(w->mu);
                if (w->fired < 0) w->fired = idx;
              }
              w->cv.notify_all();
            });
          }
          py::gil_scoped_release rel;
          std::unique_lock<std::mutex> lk(w->mu);
          if (timeout_ms < 0)
            w->cv.wait(lk, [&] { return w->fired >= 0; });
          else
            w->cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return w->fired >= 0; });
          return w->fired;
        },
        py::arg("completions"), py::arg("timeout_ms") = -1,
        "Index of the first completion to finish (-1 on timeout); waits without the GIL.");
}
