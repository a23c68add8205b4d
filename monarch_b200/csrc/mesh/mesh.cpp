#include "mesh/mesh.h"

#include <fcntl.h>
#include <signal.h>
#include <spawn.h>
#include <sys/prctl.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstring>
#include <sstream>

extern char** environ;

namespace mb {

// ------------------------------------------------------------------ selection codec --
void encode_selection(Writer& w, const Sel& s) {
  w.u8((uint8_t)s->kind);
  switch (s->kind) {
    case Selection::False_:
    case Selection::True_: break;
    case Selection::All:
    case Selection::First:
    case Selection::Any: encode_selection(w, s->a); break;
    case Selection::RangeK:
      w.u64(s->range.begin);
      w.u8(s->range.end ? 1 : 0);
      w.u64(s->range.end.value_or(0));
      w.u64(s->range.step);
      encode_selection(w, s->a);
      break;
    case Selection::Label:
      w.u32((uint32_t)s->labels.size());
      for (auto& l : s->labels) w.str(l);
      encode_selection(w, s->a);
      break;
    case Selection::Intersection:
    case Selection::Union:
      encode_selection(w, s->a);
      encode_selection(w, s->b);
      break;
  }
}

Sel decode_selection(Reader& r) {
  auto k = (Selection::Kind)r.u8();
  switch (k) {
    case Selection::False_: return Selection::f();
    case Selection::True_: return Selection::t();
    case Selection::All: return Selection::all(decode_selection(r));
    case Selection::First: return Selection::first(decode_selection(r));
    case Selection::Any: return Selection::any(decode_selection(r));
    case Selection::RangeK: {
      Range rg;
      rg.begin = r.u64();
      bool has_end = r.u8() != 0;
      uint64_t e = r.u64();
      if (has_end) rg.end = e;
      rg.step = r.u64();
      return Selection::range_of(rg, decode_selection(r));
    }
    case Selection::Label: {
      uint32_t n = r.u32();
      std::vector<std::string> l(n);
      for (auto& x : l) x = r.str();
      return Selection::label(l, decode_selection(r));
    }
    case Selection::Intersection: {
      Sel a = decode_selection(r);
      Sel b = decode_selection(r);
      return Selection::intersection(a, b);
    }
    case Selection::Union: {
      Sel a = decode_selection(r);
      Sel b = decode_selection(r);
      return Selection::union_(a, b);
    }
  }
  throw CodecError("bad selection kind");
}

void encode_slice(Writer& w, const Slice& s) {
  w.u64(s.offset());
  w.u32((uint32_t)s.ndim());
  for (size_t i = 0; i < s.ndim(); ++i) {
    w.u64(s.sizes()[i]);
    w.u64(s.strides()[i]);
  }
}
Slice decode_slice(Reader& r) {
  size_t off = r.u64();
  uint32_t n = r.u32();
  std::vector<size_t> sz(n), st(n);
  for (uint32_t i = 0; i < n; ++i) {
    sz[i] = r.u64();
    st[i] = r.u64();
  }
  return Slice(off, sz, st);
}

// --------------------------------------------------------------- actor type registry --
namespace {
std::mutex g_reg_mu;
std::map<std::string, ActorFactory>& registry() {
  static std::map<std::string, ActorFactory> r;
  return r;
}
}  // namespace
void register_actor_type(const std::string& type, ActorFactory f) {
  std::lock_guard<std::mutex> g(g_reg_mu);
  registry()[type] = std::move(f);
}
std::optional<ActorFactory> lookup_actor_type(const std::string& type) {
  std::lock_guard<std::mutex> g(g_reg_mu);
  auto it = registry().find(type);
  if (it == registry().end()) return std::nullopt;
  return it->second;
}

// --------------------------------------------------------------------- log tailer ----
LogTailer::LogTailer(int fd, size_t keep, std::function<void(const std::string&)> sink)
    : fd_(fd), keep_(keep), sink_(std::move(sink)) {
  thr_ = std::thread([this] {
    std::string buf;
    char tmp[4096];
    while (true) {
      ssize_t n = ::read(fd_, tmp, sizeof(tmp));
      if (n < 0 && errno == EINTR) continue;
      if (n <= 0) break;
      buf.append(tmp, (size_t)n);
      size_t pos;
      while ((pos = buf.find('\n')) != std::string::npos) {
        std::string line = buf.substr(0, pos);
        buf.erase(0, pos + 1);
        {
          std::lock_guard<std::mutex> g(mu_);
          if (lines_.size() >= keep_) lines_.pop_front();
          lines_.push_back(line);
        }
        if (sink_) sink_(line);
      }
    }
    if (!buf.empty()) {
      std::lock_guard<std::mutex> g(mu_);
      lines_.push_back(buf);
      if (sink_) sink_(buf);
    }
    ::close(fd_);
  });
}
LogTailer::~LogTailer() { join(); }
void LogTailer::join() {
  if (thr_.joinable()) thr_.join();
}
std::vector<std::string> LogTailer::tail() const {
  std::lock_guard<std::mutex> g(mu_);
  return std::vector<std::string>(lines_.begin(), lines_.end());
}

// ------------------------------------------------------------------- event queue ----
namespace {
class EventQueue {
 public:
  void push(ProcEvent e) {
    {
      std::lock_guard<std::mutex> g(mu_);
      q_.push_back(std::move(e));
    }
    cv_.notify_all();
  }
  std::optional<ProcEvent> pop(int64_t timeout_ms) {
    std::unique_lock<std::mutex> g(mu_);
    auto ready = [&] { return !q_.empty(); };
    if (timeout_ms < 0)
      cv_.wait(g, ready);
    else if (!cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), ready))
      return std::nullopt;
    ProcEvent e = std::move(q_.front());
    q_.pop_front();
    return e;
  }

 private:
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<ProcEvent> q_;
};

// -------------------------------------------------------------------- local alloc ----
class LocalAlloc : public Alloc {
 public:
  LocalAlloc(std::string world, size_t n, std::shared_ptr<Router> router)
      : world_(std::move(world)), n_(n), router_(std::move(router)) {
    for (size_t i = 0; i < n_; ++i) {
      auto p = Proc::create(ProcId{world_, (int64_t)i}, router_);
      router_->bind_local(p);
      p->spawn("mesh_agent", make_mesh_agent(p, router_));
      procs_.push_back(p);
      ProcEvent e;
      e.kind = ProcEvent::Running;
      e.rank = (int64_t)i;
      e.proc_id = p->id().to_string();
      events_.push(std::move(e));
    }
  }
  ~LocalAlloc() override { stop(); }
  std::string world() const override { return world_; }
  size_t size() const override { return n_; }
  std::optional<ProcEvent> next(int64_t t) override { return events_.pop(t); }
  std::string transport() const override { return "local"; }
  std::vector<std::shared_ptr<Proc>> local_procs() const override { return procs_; }
  void stop() override {
    if (stopped_.exchange(true)) return;
    for (size_t i = 0; i < procs_.size(); ++i) {
      procs_[i]->stop_all(Config::global().get_int("STOP_ACTOR_TIMEOUT_MS"));
      router_->unbind_local(procs_[i]->id());
      ProcEvent e;
      e.kind = ProcEvent::Stopped;
      e.rank = (int64_t)i;
      e.proc_id = procs_[i]->id().to_string();
      e.reason = "stopped";
      events_.push(std::move(e));
    }
  }
  void kill_rank(int64_t rank, int) override {
    if (rank < 0 || (size_t)rank >= procs_.size()) return;
    procs_[rank]->stop_all(100);
    router_->unbind_local(procs_[rank]->id());
    ProcEvent e;
    e.kind = ProcEvent::Stopped;
    e.rank = rank;
    e.proc_id = procs_[rank]->id().to_string();
    e.reason = "killed";
    events_.push(std::move(e));
  }

 private:
  std::string world_;
  size_t n_;
  std::shared_ptr<Router> router_;
  std::vector<std::shared_ptr<Proc>> procs_;
  EventQueue events_;
  std::atomic<bool> stopped_{false};
};

// ---------------------------------------------------------------------- sim alloc ----
class SimAlloc : public Alloc {
 public:
  SimAlloc(std::string world, std::vector<std::string> nodes)
      : world_(std::move(world)), nodes_(std::move(nodes)) {
    for (size_t i = 0; i < nodes_.size(); ++i) {
      auto router = std::make_shared<Router>();
      auto p = Proc::create(ProcId{world_, (int64_t)i}, router);
      router->bind_local(p);
      router->set_home(p);
      ChannelAddr a = ChannelAddr::any(ChannelAddr::Sim);
      a.node = nodes_[i];
      auto rx = serve(a);
      std::string addr = rx->addr().to_string();
      servers_.push_back(std::make_unique<MailboxServer>(rx, std::make_shared<ProcSender>(p)));
      p->spawn("mesh_agent", make_mesh_agent(p, router));
      procs_.push_back(p);
      routers_.push_back(router);
      ProcEvent e;
      e.kind = ProcEvent::Running;
      e.rank = (int64_t)i;
      e.proc_id = p->id().to_string();
      e.addr = addr;
      events_.push(std::move(e));
    }
  }
  ~SimAlloc() override { stop(); }
  std::string world() const override { return world_; }
  size_t size() const override { return nodes_.size(); }
  std::optional<ProcEvent> next(int64_t t) override { return events_.pop(t); }
  std::string transport() const override { return "sim"; }
  void stop() override {
    if (stopped_.exchange(true)) return;
    for (size_t i = 0; i < procs_.size(); ++i) {
      procs_[i]->stop_all(Config::global().get_int("STOP_ACTOR_TIMEOUT_MS"));
      ProcEvent e;
      e.kind = ProcEvent::Stopped;
      e.rank = (int64_t)i;
      e.proc_id = procs_[i]->id().to_string();
      e.reason = "stopped";
      events_.push(std::move(e));
    }
    servers_.clear();
  }

 private:
  std::string world_;
  std::vector<std::string> nodes_;
  std::vector<std::shared_ptr<Proc>> procs_;
  std::vector<std::shared_ptr<Router>> routers_;
  std::vector<std::unique_ptr<MailboxServer>> servers_;
  EventQueue events_;
  std::atomic<bool> stopped_{false};
};

// ------------------------------------------------------------------ process alloc ----
std::string describe_wait_status(int st, int* code) {
  if (WIFEXITED(st)) {
    *code = WEXITSTATUS(st);
    return "exited(" + std::to_string(*code) + ")";
  }
  if (WIFSIGNALED(st)) {
    *code = 128 + WTERMSIG(st);
    return "killed(" + std::to_string(WTERMSIG(st)) + ")";
  }
  *code = -1;
  return "unknown";
}

class ProcessAlloc : public Alloc {
 public:
  ProcessAlloc(std::string world, size_t n, ProcessAllocOptions opts)
      : world_(std::move(world)), n_(n), opts_(std::move(opts)) {
    ChannelAddr a = ChannelAddr::any(opts_.transport == "tcp" ? ChannelAddr::Tcp : ChannelAddr::Unix);
    rx_ = serve(a);
    children_.resize(n_);
    for (size_t i = 0; i < n_; ++i) spawn_child(i);
    ctrl_thr_ = std::thread([this] { control_loop(); });
  }
  ~ProcessAlloc() override { stop(); }
  std::string world() const override { return world_; }
  size_t size() const override { return n_; }
  std::optional<ProcEvent> next(int64_t t) override { return events_.pop(t); }
  std::string transport() const override { return opts_.transport; }

  void kill_rank(int64_t rank, int sig) override {
    if (rank < 0 || (size_t)rank >= children_.size()) return;
    pid_t pid = children_[rank].pid;
    if (pid > 0) ::kill(pid, sig);
  }

  void stop() override {
    if (stopped_.exchange(true)) return;
    // Ask politely, then insist.
    for (auto& c : children_) {
      if (c.ctrl) {
        Frame f;
        f.head = "X";
        c.ctrl->post(std::move(f));
      }
    }
    auto deadline = std::chrono::steady_clock::now() +
                    std::chrono::milliseconds(Config::global().get_int("PROCESS_EXIT_TIMEOUT_MS"));
    for (auto& c : children_) {
      while (!c.exited && std::chrono::steady_clock::now() < deadline)
        std::this_thread::sleep_for(std::chrono::milliseconds(5));
      if (!c.exited && c.pid > 0) ::kill(c.pid, SIGKILL);
    }
    for (auto& c : children_)
      if (c.waiter.joinable()) c.waiter.join();
    rx_->close();
    if (ctrl_thr_.joinable()) ctrl_thr_.join();
    for (auto& c : children_) {
      if (c.ctrl) c.ctrl->close();
      c.out.reset();
      c.err.reset();
    }
  }

 private:
  struct Child {
    pid_t pid = -1;
    std::shared_ptr<Tx> ctrl;
    std::unique_ptr<LogTailer> out, err;
    std::thread waiter;
    std::atomic<bool> exited{false};
    Child() = default;
    Child(Child&&) = delete;
  };

  void spawn_child(size_t i) {
    int po[2], pe[2];
    if (::pipe2(po, O_CLOEXEC) < 0 || ::pipe2(pe, O_CLOEXEC) < 0)
      throw std::runtime_error("pipe() failed");
    posix_spawn_file_actions_t fa;
    posix_spawn_file_actions_init(&fa);
    posix_spawn_file_actions_adddup2(&fa, po[1], 1);
    posix_spawn_file_actions_adddup2(&fa, pe[1], 2);
    std::vector<std::string> envs;
    std::map<std::string, std::string> extra = opts_.env;
    extra["HYPERACTOR_MESH_BOOTSTRAP_ADDR"] = rx_->addr().to_string();
    extra["HYPERACTOR_MESH_INDEX"] = std::to_string(i);
    extra["HYPERACTOR_MESH_WORLD"] = world_;
    if (opts_.per_rank_gpu_env) {
      extra["LOCAL_RANK"] = std::to_string(i);
      extra["MB200_PROC_RANK"] = std::to_string(i);
    }
    for (char** e = environ; *e; ++e) {
      std::string kv(*e);
      std::string k = kv.substr(0, kv.find('='));
      if (!extra.count(k)) envs.push_back(kv);
    }
    for (auto& kv : extra) envs.push_back(kv.first + "=" + kv.second);
    std::vector<char*> envp, argv;
    for (auto& s : envs) envp.push_back(s.data());
    envp.push_back(nullptr);
    for (auto& s : opts_.argv) argv.push_back(const_cast<char*>(s.c_str()));
    argv.push_back(nullptr);
    pid_t pid = -1;
    int rc = posix_spawnp(&pid, argv[0], &fa, nullptr, argv.data(), envp.data());
    posix_spawn_file_actions_destroy(&fa);
    ::close(po[1]);
    ::close(pe[1]);
    if (rc != 0) {
      ::close(po[0]);
      ::close(pe[0]);
      throw std::runtime_error(std::string("cannot spawn ") + argv[0] + ": " + std::strerror(rc));
    }
    Child& c = children_[i];
    c.pid = pid;
    auto sink = opts_.log_sink;
    int64_t rank = (int64_t)i;
    c.out = std::make_unique<LogTailer>(po[0], opts_.tail_lines, [sink, rank](const std::string& l) {
      if (sink) sink(rank, false, l);
    });
    c.err = std::make_unique<LogTailer>(pe[0], opts_.tail_lines, [sink, rank](const std::string& l) {
      if (sink) sink(rank, true, l);
    });
    ProcEvent ev;
    ev.kind = ProcEvent::Created;
    ev.rank = rank;
    events_.push(std::move(ev));
    c.waiter = std::thread([this, i, pid] {
      int st = 0;
      while (::waitpid(pid, &st, 0) < 0 && errno == EINTR) {
      }
      Child& ch = children_[i];
      ch.exited = true;
      ProcEvent e;
      int code = 0;
      e.reason = describe_wait_status(st, &code);
      e.exit_code = code;
      e.kind = (code == 0) ? ProcEvent::Stopped : ProcEvent::Failed;
      if (stopped_) e.kind = ProcEvent::Stopped;
      e.rank = (int64_t)i;
      e.proc_id = ProcId{world_, (int64_t)i}.to_string();
      if (ch.err) {
        ch.err->join();
        e.stderr_tail = ch.err->tail();
      }
      events_.push(std::move(e));
    });
  }

  void control_loop() {
    while (!rx_->closed()) {
      auto f = rx_->recv(100);
      if (!f) continue;
      if (f->head.empty()) continue;
      try {
        Reader r(std::string_view(f->head).substr(1));
        if (f->head[0] == 'H') {
          int64_t idx = r.i64();
          std::string ctrl = r.str();
          if (idx < 0 || (size_t)idx >= n_) continue;
          children_[idx].ctrl = dial(ChannelAddr::parse(ctrl));
          Writer w;
          w.buf = "S";
          w.str(ProcId{world_, idx}.to_string());
          w.str(opts_.transport);
          Frame s;
          s.head = std::move(w.buf);
          children_[idx].ctrl->post(std::move(s));
        } else if (f->head[0] == 'R') {
          ProcEvent e;
          e.kind = ProcEvent::Running;
          e.rank = r.i64();
          e.proc_id = r.str();
          e.addr = r.str();
          events_.push(std::move(e));
        }
      } catch (const std::exception& ex) {
        MB_LOG(Warn, std::string("process alloc: bad control frame: ") + ex.what());
      }
    }
  }

  std::string world_;
  size_t n_;
  ProcessAllocOptions opts_;
  std::shared_ptr<Rx> rx_;
  std::deque<Child> children_;
  EventQueue events_;
  std::thread ctrl_thr_;
  std::atomic<bool> stopped_{false};
};

// Allocation whose procs are hosted by processes someone else started.
class AttachAllocImpl : public AttachAlloc {
 public:
  AttachAllocImpl(std::string world, size_t n, std::string transport)
      : world_(std::move(world)), n_(n), transport_(std::move(transport)) {
    rx_ = serve(ChannelAddr::any(transport_ == "tcp" ? ChannelAddr::Tcp : ChannelAddr::Unix));
    ctrl_.resize(n_);
    thr_ = std::thread([this] { control_loop(); });
  }
  ~AttachAllocImpl() override { stop(); }
  std::string world() const override { return world_; }
  size_t size() const override { return n_; }
  std::optional<ProcEvent> next(int64_t t) override { return events_.pop(t); }
  std::string transport() const override { return transport_; }
  std::string bootstrap_addr() const override { return rx_->addr().to_string(); }

  void stop() override {
    if (stopped_.exchange(true)) return;
    rx_->close();
    if (thr_.joinable()) thr_.join();   // the control thread owned ctrl_ until here
    for (auto& c : ctrl_) {
      if (c) {
        Frame f;
        f.head = "X";
        c->post(std::move(f));
      }
    }
    // the hosts stop their actors and drop the connection; give the frames time to leave
    std::this_thread::sleep_for(std::chrono::milliseconds(50));
    for (auto& c : ctrl_)
      if (c) c->close();
  }

 private:
  void control_loop() {
    auto last_check = std::chrono::steady_clock::now();
    while (!rx_->closed()) {
      auto f = rx_->recv(100);
      auto now = std::chrono::steady_clock::now();
      if (now - last_check > std::chrono::milliseconds(500)) {
        last_check = now;
        for (size_t i = 0; i < n_; ++i) {   // a host that went away took its proc with it
          if (ctrl_[i] && !gone_[i] && !stopped_ && ctrl_[i]->status() == TxStatus::Closed) {
            gone_[i] = true;
            ProcEvent e;
            e.kind = ProcEvent::Failed;
            e.rank = (int64_t)i;
            e.proc_id = ProcId{world_, (int64_t)i}.to_string();
            e.reason = "lost the connection to the process hosting it";
            events_.push(std::move(e));
          }
        }
      }
      if (!f || f->head.empty()) continue;
      try {
        Reader r(std::string_view(f->head).substr(1));
        if (f->head[0] == 'H') {
          int64_t idx = r.i64();
          std::string ctrl = r.str();
          if (idx < 0 || (size_t)idx >= n_ || ctrl_[idx]) continue;   // unknown or duplicate
          ctrl_[idx] = dial(ChannelAddr::parse(ctrl));
          ProcEvent c;
          c.kind = ProcEvent::Created;
          c.rank = idx;
          events_.push(std::move(c));
          Writer w;
          w.buf = "S";
          w.str(ProcId{world_, idx}.to_string());
          w.str(transport_);
          Frame s;
          s.head = std::move(w.buf);
          ctrl_[idx]->post(std::move(s));
        } else if (f->head[0] == 'R') {
          ProcEvent e;
          e.kind = ProcEvent::Running;
          e.rank = r.i64();
          e.proc_id = r.str();
          e.addr = r.str();
          events_.push(std::move(e));
        }
      } catch (const std::exception& ex) {
        MB_LOG(Warn, std::string("attach alloc: bad control frame: ") + ex.what());
      }
    }
  }

  std::string world_;
  size_t n_;
  std::string transport_;
  std::shared_ptr<Rx> rx_;
  std::deque<std::shared_ptr<Tx>> ctrl_;
  std::map<size_t, bool> gone_;
  EventQueue events_;
  std::thread thr_;
  std::atomic<bool> stopped_{false};
};

}  // namespace

std::shared_ptr<AttachAlloc> make_attach_alloc(const std::string& world, size_t n,
                                               const std::string& transport) {
  return std::make_shared<AttachAllocImpl>(world, n, transport);
}

std::shared_ptr<Alloc> make_sim_alloc(const std::string& world, std::vector<std::string> nodes) {
  return std::make_shared<SimAlloc>(world, std::move(nodes));
}

std::shared_ptr<Alloc> make_local_alloc(const std::string& world, size_t n,
                                        std::shared_ptr<Router> router) {
  return std::make_shared<LocalAlloc>(world, n, std::move(router));
}
std::shared_ptr<Alloc> make_process_alloc(const std::string& world, size_t n,
                                          ProcessAllocOptions opts) {
  return std::make_shared<ProcessAlloc>(world, n, std::move(opts));
}

// ----------------------------------------------------------------- child bootstrap ----
namespace {
// The proc-hosting side of the bootstrap protocol.  `child`: this process was started by
// the allocator for this purpose (it dies with the allocator and exits when told to stop);
// otherwise the process only hosts the proc and the function returns when the mesh stops.
int bootstrap_loop(const std::string& addr_s, int64_t index, bool child) {
  const pid_t parent = ::getppid();
  auto to_parent = dial(ChannelAddr::parse(addr_s));
  ChannelAddr::Kind kind = ChannelAddr::parse(addr_s).kind;
  auto ctrl = serve(ChannelAddr::any(kind == ChannelAddr::Tcp ? ChannelAddr::Tcp : ChannelAddr::Unix));
  {
    Writer w;
    w.buf = "H";
    w.i64(index);
    w.str(ctrl->addr().to_string());
    Frame f;
    f.head = std::move(w.buf);
    to_parent->post(std::move(f));
  }
  std::shared_ptr<Router> router;
  std::shared_ptr<Proc> proc;
  std::unique_ptr<MailboxServer> server;
  const int64_t hb_ms = Config::global().get_int("BOOTSTRAP_HEARTBEAT_INTERVAL_MS");
  auto last_check = std::chrono::steady_clock::now();
  while (true) {
    auto f = ctrl->recv(200);
    auto now = std::chrono::steady_clock::now();
    if (now - last_check > std::chrono::milliseconds(hb_ms)) {
      last_check = now;
      if ((child && ::getppid() != parent) || to_parent->status() == TxStatus::Closed) {
        MB_LOG(Warn, "bootstrap: allocator is gone");
        if (child) ::_exit(1);
        if (proc) proc->stop_all(Config::global().get_int("STOP_ACTOR_TIMEOUT_MS"));
        server.reset();
        ctrl->close();
        return 1;
      }
    }
    if (!f || f->head.empty()) continue;
    Reader r(std::string_view(f->head).substr(1));
    if (f->head[0] == 'S') {
      ProcId pid = ProcId::parse(r.str());
      std::string transport = r.str();
      router = std::make_shared<Router>();
      proc = Proc::create(pid, router);
      router->bind_local(proc);
      router->set_home(proc);
      auto rx = serve(ChannelAddr::any(transport == "tcp" ? ChannelAddr::Tcp : ChannelAddr::Unix));
      std::string maddr = rx->addr().to_string();
      server = std::make_unique<MailboxServer>(rx, std::make_shared<ProcSender>(proc));
      proc->spawn("mesh_agent", make_mesh_agent(proc, router));
      Writer w;
      w.buf = "R";
      w.i64(index);
      w.str(pid.to_string());
      w.str(maddr);
      Frame out;
      out.head = std::move(w.buf);
      to_parent->post(std::move(out));
    } else if (f->head[0] == 'X') {
      if (proc) proc->stop_all(Config::global().get_int("STOP_ACTOR_TIMEOUT_MS"));
      std::fflush(stdout);
      std::fflush(stderr);
      if (child) ::_exit(0);
      server.reset();
      ctrl->close();
      to_parent->close();
      return 0;
    }
  }
}
}  // namespace

int bootstrap_main() {
  const char* addr_s = std::getenv("HYPERACTOR_MESH_BOOTSTRAP_ADDR");
  const char* idx_s = std::getenv("HYPERACTOR_MESH_INDEX");
  if (!addr_s || !idx_s) return 1;
  ::prctl(PR_SET_PDEATHSIG, SIGKILL);  // never outlive the allocator
  if (std::getenv("MONARCH_ERROR_DURING_BOOTSTRAP_FOR_TESTING")) {
    std::fprintf(stderr, "bootstrap: injected failure (MONARCH_ERROR_DURING_BOOTSTRAP_FOR_TESTING)\n");
    ::_exit(17);
  }
  return bootstrap_loop(addr_s, std::stoll(idx_s), true);
}

int bootstrap_attach(const std::string& addr, int64_t index) {
  return bootstrap_loop(addr, index, false);
}

// --------------------------------------------------------------------- mesh agent ----
ActorHooks make_mesh_agent(const std::shared_ptr<Proc>& proc_sp, std::shared_ptr<Router> router) {
  std::weak_ptr<Proc> wproc = proc_sp;
  ActorHooks h;
  h.on_message = [wproc, router](Instance& self, Envelope& env) {
    auto proc = wproc.lock();
    if (!proc) return;
    const std::string kind = env.headers.count(kHdrKind) ? env.headers[kHdrKind] : "";
    Reader r(env.data);
    if (kind == "configure") {
      int64_t rank = r.i64();
      uint32_t n = r.u32();
      for (uint32_t i = 0; i < n; ++i) {
        std::string prefix = r.str();
        std::string addr = r.str();
        if (addr.empty() || prefix == proc->id().to_string()) continue;
        if (prefix == "*")
          router->set_default(std::make_shared<MailboxClient>(dial(ChannelAddr::parse(addr)), proc));
        else
          router->bind_addr(prefix, ChannelAddr::parse(addr));
      }
      PortId supervisor = read_port(r);
      PortId reply = read_port(r);
      proc->set_supervision_coordinator(supervisor);
      if (!proc->find("comm", 0)) proc->spawn("comm", make_comm_actor(proc));
      Writer w;
      w.i64(rank);
      self.send(reply, std::move(w.buf), {{kHdrKind, "configured"}});
    } else if (kind == "gspawn") {
      std::string type = r.str();
      std::string name = r.str();
      std::string params = r.str();
      PortId reply = read_port(r);
      Writer w;
      w.i64(proc->id().rank);
      auto f = lookup_actor_type(type);
      if (!f) {
        w.u8(0);
        w.str("unknown actor type: " + type);
      } else {
        try {
          auto inst = proc->spawn(name, (*f)(proc, name, params));
          w.u8(1);
          w.str(inst->id().to_string());
        } catch (const std::exception& e) {
          w.u8(0);
          w.str(std::string("spawn failed: ") + e.what());
        }
      }
      self.send(reply, std::move(w.buf), {{kHdrKind, "gspawn_result"}});
    } else if (kind == "stop_actor") {
      std::string name = r.str();
      PortId reply = read_port(r);
      int64_t timeout = Config::global().get_int("STOP_ACTOR_TIMEOUT_MS");
      bool ok = true;
      for (int64_t pid = 0;; ++pid) {
        auto inst = proc->find(name, pid);
        if (!inst) break;
        inst->signal(Signal::DrainAndStop);
        if (!inst->join(timeout)) {
          inst->signal(Signal::Stop);
          ok = inst->join(timeout) && ok;
        }
      }
      Writer w;
      w.i64(proc->id().rank);
      w.u8(ok ? 1 : 0);
      self.send(reply, std::move(w.buf), {{kHdrKind, "stopped"}});
    } else if (kind == "ledger") {
      PortId reply = read_port(r);
      std::ostringstream os;
      // one line per actor: id, status, messages handled, failure, children (comma
      // separated), newest recorded event
      auto flat = [](std::string v) {
        for (auto& c : v)
          if (c == '\t' || c == '\n') c = ' ';
        return v;
      };
      for (auto& s : proc->ledger_snapshot()) {
        os << s.actor_id << "\t" << s.status << "\t" << s.messages_handled << "\t"
           << flat(s.failure) << "\t";
        for (size_t i = 0; i < s.children.size(); ++i) os << (i ? "," : "") << s.children[i];
        os << "\t";
        if (!s.events.empty())
          os << s.events.back().t_us << " " << flat(s.events.back().name) << " "
             << flat(s.events.back().detail);
        os << "\n";
      }
      self.send(reply, os.str(), {{kHdrKind, "ledger"}});
    }
  };
  // The agent never dies because some message it relayed bounced.
  h.on_undeliverable = [](Instance&, Envelope&, const std::string&) { return true; };
  return h;
}

// --------------------------------------------------------------------- comm actor ----
namespace {
struct CastWire {
  std::string mesh_id;
  Slice slice, cast_shape;
  ActorId sender;
  uint64_t seq = 0;
  std::map<std::string, std::string> headers;
  std::vector<RoutingFrame> frames;
  std::string body;
  bool body_in_parts = false;  // the body is the last part of the carrying envelope
};

std::string encode_cast(const CastWire& c) {
  Writer w;
  w.str(c.mesh_id);
  encode_slice(w, c.slice);
  encode_slice(w, c.cast_shape);
  write_actor(w, c.sender);
  w.u64(c.seq);
  w.u32((uint32_t)c.headers.size());
  for (auto& kv : c.headers) {
    w.str(kv.first);
    w.str(kv.second);
  }
  w.u32((uint32_t)c.frames.size());
  for (auto& f : c.frames) {
    w.u32((uint32_t)f.here.size());
    for (size_t x : f.here) w.u64(x);
    w.u64(f.dim);
    encode_selection(w, f.sel);
  }
  w.u8(c.body_in_parts ? 1 : 0);
  if (!c.body_in_parts) w.str(c.body);
  return std::move(w.buf);
}

CastWire decode_cast(std::string_view b) {
  Reader r(b);
  CastWire c;
  c.mesh_id = r.str();
  c.slice = decode_slice(r);
  c.cast_shape = decode_slice(r);
  c.sender = read_actor(r);
  c.seq = r.u64();
  uint32_t nh = r.u32();
  for (uint32_t i = 0; i < nh; ++i) {
    std::string k = r.str();
    c.headers[k] = r.str();
  }
  uint32_t nf = r.u32();
  c.frames.resize(nf);
  for (auto& f : c.frames) {
    uint32_t nd = r.u32();
    f.here.resize(nd);
    for (auto& x : f.here) x = r.u64();
    f.dim = r.u64();
    f.sel = decode_selection(r);
  }
  c.body_in_parts = r.u8() != 0;
  if (!c.body_in_parts) c.body = r.str();
  return c;
}
}  // namespace

std::string encode_cast_root(CastRequest& c, std::vector<std::string>& parts) {
  CastWire w;
  w.mesh_id = c.mesh_id;
  w.slice = c.slice;
  w.cast_shape = c.cast_shape;
  w.sender = c.sender;
  w.seq = c.seq;
  w.headers = c.headers;
  w.frames.push_back(RoutingFrame::root(c.selection, c.slice));
  if (c.data.size() >= kCastBodyAsPartBytes) {
    w.body_in_parts = true;
    parts.push_back(std::move(c.data));
  } else {
    w.body = c.data;
  }
  return encode_cast(w);
}

namespace {
// Partial results of the casts whose replies are reduced along the tree.
struct PendingReduce {
  PortId parent;            // where the folded result of this subtree goes
  bool parent_is_comm = false;
  std::string final_port;   // the caller's accumulating port
  ReduceFn fn;
  size_t expected = 0;      // local actor (if any) + one part per child hop
  size_t received = 0;
  uint64_t contributions = 0;
  std::string state;
  // "gather": replies are not folded but collected -- `state` holds one record per reply
  // (u32 part count, u64 body length, body) and `parts` every reply's parts in order
  bool gather = false;
  std::vector<std::string> parts;
  double t_us = 0;
};

void append_u32(std::string& s, uint32_t v) { s.append(reinterpret_cast<const char*>(&v), 4); }
void append_u64(std::string& s, uint64_t v) { s.append(reinterpret_cast<const char*>(&v), 8); }
struct ReduceTable {
  std::map<std::string, PendingReduce> pending;
};
}  // namespace

ActorHooks make_comm_actor(const std::shared_ptr<Proc>& proc_sp) {
  std::weak_ptr<Proc> wproc = proc_sp;
  auto reduces = std::make_shared<ReduceTable>();  // touched only by this actor's handler
  ActorHooks h;
  // a relay without state: routed on the delivering thread (forwards go down the tree of
  // the mesh's spawn-time slice, so nested deliveries cannot form a cycle)
  h.inline_messages = Config::global().get_bool("COMM_ACTOR_INLINE");
  h.on_message = [wproc, reduces](Instance& self, Envelope& env) {
    auto proc = wproc.lock();
    if (!proc) return;
    double t0 = now_us();
    auto kind_it = env.headers.find(kHdrKind);
    if (kind_it != env.headers.end() && kind_it->second == "reduce_part") {
      // a partial result from the local actor or from a child hop
      const std::string key = env.headers[kHdrReduceKey];
      uint64_t n = 1;
      if (auto it = env.headers.find(kHdrReduceCount); it != env.headers.end())
        n = std::stoull(it->second);
      auto pit = reduces->pending.find(key);
      if (pit == reduces->pending.end()) {
        // no record (expired, or the cast never passed here): hand it to the caller as is
        Envelope e;
        e.sender = self.id();
        e.dest = PortId::parse(env.headers[kHdrReducePort]);
        const bool item = env.headers.count("gather_item") != 0;
        e.headers = {{kHdrKind, item ? "reply" : (env.headers.count("gather") ? "batch" : "reduce")},
                     {"no_return", "1"},
                     {kHdrReduceCount, std::to_string(n)}};
        e.data = std::move(env.data);
        e.parts = std::move(env.parts);
        proc->post(std::move(e));
        return;
      }
      PendingReduce& pr = pit->second;
      if (pr.gather) {
        if (env.headers.count("gather_item")) {  // one reply of the local actor: make a record
          append_u32(pr.state, (uint32_t)env.parts.size());
          append_u64(pr.state, (uint64_t)env.data.size());
          pr.state += env.data;
        } else {                                 // records collected by a child hop
          pr.state += env.data;
        }
        for (auto& p : env.parts) pr.parts.push_back(std::move(p));
      } else {
        pr.state = pr.fn(pr.state, env.data);
      }
      pr.contributions += n;
      if (++pr.received < pr.expected) return;
      Envelope e;
      e.sender = self.id();
      e.dest = pr.parent;
      e.headers = {{kHdrKind, pr.parent_is_comm ? "reduce_part" : (pr.gather ? "batch" : "reduce")},
                   {"no_return", "1"},
                   {kHdrReduceKey, key},
                   {kHdrReducePort, pr.final_port},
                   {kHdrReduceCount, std::to_string(pr.contributions)}};
      if (pr.gather) e.headers["gather"] = "1";
      e.data = std::move(pr.state);
      e.parts = std::move(pr.parts);
      reduces->pending.erase(pit);
      proc->post(std::move(e));
      return;
    }
    CastWire c = decode_cast(env.data);
    const size_t my_rank = (size_t)proc->id().rank;
    Resolved res = resolve_routing(my_rank, c.slice, std::move(c.frames), /*seed=*/4 + c.seq);
    // Forward first so the subtree makes progress while we deliver locally.  The parts
    // (with a large body among them) are copied for every consumer but the last, which
    // takes them over.
    size_t consumers = res.next.size() + (res.deliver_here ? 1 : 0);
    std::string reduce_key;
    if (auto rt = c.headers.find(kHdrReduceTree); rt != c.headers.end() && consumers > 0) {
      reduce_key = c.sender.to_string() + "/" + c.mesh_id + "/" + std::to_string(c.seq);
      PendingReduce pr;
      pr.gather = rt->second == "gather";
      if (!pr.gather) pr.fn = builtin_reducer(rt->second);
      pr.final_port = c.headers[kHdrReducePort];
      pr.expected = consumers;
      pr.t_us = t0;
      // the previous hop is a comm actor unless this is the root of the tree
      pr.parent_is_comm = env.sender.name == "comm" && env.sender.proc.world == proc->id().world;
      pr.parent = pr.parent_is_comm ? PortId{env.sender, kPortMessage}
                                    : PortId::parse(pr.final_port);
      if (reduces->pending.size() > 256) {  // forget what was abandoned long ago
        for (auto it = reduces->pending.begin(); it != reduces->pending.end();)
          it = (t0 - it->second.t_us > 600e6) ? reduces->pending.erase(it) : std::next(it);
      }
      reduces->pending[reduce_key] = std::move(pr);
    }
    for (auto& kv : res.next) {
      CastWire fwd;
      fwd.mesh_id = c.mesh_id;
      fwd.slice = c.slice;
      fwd.cast_shape = c.cast_shape;
      fwd.sender = c.sender;
      fwd.seq = c.seq;
      fwd.headers = c.headers;
      fwd.frames = std::move(kv.second);
      fwd.body_in_parts = c.body_in_parts;
      if (!c.body_in_parts) fwd.body = c.body;
      Envelope e;
      e.sender = self.id();
      e.dest = PortId{ActorId{ProcId{proc->id().world, (int64_t)kv.first}, "comm", 0}, kPortMessage};
      e.data = encode_cast(fwd);
      if (--consumers == 0)
        e.parts = std::move(env.parts);
      else
        e.parts = env.parts;
      proc->post(std::move(e));
    }
    if (res.deliver_here) {
      Envelope e;
      e.sender = c.sender;
      e.dest = PortId{ActorId{proc->id(), c.mesh_id, 0}, kPortMessage};
      e.headers = c.headers;
      size_t cast_rank = 0;
      try {
        cast_rank = c.cast_shape.index(my_rank);
      } catch (const NdError&) {
        cast_rank = c.slice.index(my_rank);
      }
      e.headers[kHdrCastRank] = std::to_string(cast_rank);
      e.headers[kHdrCastSender] = c.sender.to_string();
      e.headers[kHdrCastMesh] = c.mesh_id;
      if (!reduce_key.empty()) {
        e.headers[kHdrReduceKey] = reduce_key;
        e.headers[kHdrReduceVia] = PortId{self.id(), kPortMessage}.to_string();
      }
      e.parts = std::move(env.parts);
      if (c.body_in_parts && !e.parts.empty()) {
        e.data = std::move(e.parts.back());
        e.parts.pop_back();
      } else {
        e.data = std::move(c.body);
      }
      proc->post(std::move(e));
    }
    Metrics::global().histogram_record("comm.cast_hop_us", now_us() - t0);
  };
  h.on_undeliverable = [wproc](Instance& self, Envelope& returned, const std::string& reason) {
    // A hop of the tree (or the final actor) was unreachable: tell the originator.
    auto proc = wproc.lock();
    if (!proc) return true;
    try {
      if (returned.dest.actor.name == "comm") {
        CastWire c = decode_cast(returned.data);
        Envelope lost;
        lost.sender = c.sender;
        lost.dest = PortId{ActorId{returned.dest.actor.proc, c.mesh_id, 0}, kPortMessage};
        lost.headers = c.headers;
        proc->return_undeliverable(std::move(lost), "cast hop unreachable: " + reason);
      } else {
        proc->return_undeliverable(std::move(returned), reason);
      }
    } catch (const std::exception&) {
    }
    (void)self;
    return true;
  };
  return h;
}

// ----------------------------------------------------------------------- proc mesh ----
// The client proc is served on one socket per transport, shared by every mesh.
static std::string client_server_addr(const std::shared_ptr<Proc>& client,
                                      const std::string& transport) {
  static std::mutex mu;
  static std::map<std::string, std::unique_ptr<MailboxServer>>* servers =
      new std::map<std::string, std::unique_ptr<MailboxServer>>();
  std::lock_guard<std::mutex> g(mu);
  std::string key = client->id().to_string() + "/" + transport;
  auto it = servers->find(key);
  if (it == servers->end()) {
    ChannelAddr any = ChannelAddr::any(transport == "tcp"   ? ChannelAddr::Tcp
                                       : transport == "sim" ? ChannelAddr::Sim
                                                            : ChannelAddr::Unix);
    if (transport == "sim") any.node = "client";
    auto rx = serve(any);
    it = servers->emplace(key, std::make_unique<MailboxServer>(
                                   rx, std::make_shared<ProcSender>(client))).first;
  }
  return it->second->addr().to_string();
}

std::shared_ptr<ProcMesh> ProcMesh::allocate(std::shared_ptr<Alloc> alloc,
                                             std::shared_ptr<Router> router,
                                             std::shared_ptr<Proc> client, int64_t timeout_ms) {
  auto pm = std::shared_ptr<ProcMesh>(new ProcMesh());
  pm->alloc_ = alloc;
  pm->world_ = alloc->world();
  pm->n_ = alloc->size();
  const bool local = alloc->transport() == "local";
  pm->router_ = router;
  pm->client_ = client;
  pm->client_inst_ = pm->client_->attach("mesh_client");
  pm->supervisor_q_ = std::make_shared<QueueSink>();
  pm->supervisor_port_ = pm->client_inst_->bind(pm->supervisor_q_);

  // Wait for every rank to be running.
  std::map<int64_t, std::string> addrs;
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  size_t running = 0;
  while (running < pm->n_) {
    int64_t left = std::chrono::duration_cast<std::chrono::milliseconds>(
                       deadline - std::chrono::steady_clock::now()).count();
    if (left <= 0) {
      alloc->stop();
      throw std::runtime_error("proc mesh allocation timed out (" + std::to_string(running) +
                               " of " + std::to_string(pm->n_) + " procs running)");
    }
    auto ev = alloc->next(std::min<int64_t>(left, 200));
    if (!ev) continue;
    if (ev->kind == ProcEvent::Running) {
      addrs[ev->rank] = ev->addr;
      ++running;
    } else if (ev->kind == ProcEvent::Failed || ev->kind == ProcEvent::Stopped) {
      std::string tail;
      for (auto& l : ev->stderr_tail) tail += "\n    " + l;
      alloc->stop();
      throw std::runtime_error("proc " + std::to_string(ev->rank) + " " + ev->reason +
                               " during allocation" + (tail.empty() ? "" : "; stderr:" + tail));
    }
  }
  std::string client_addr;
  const bool sim = alloc->transport() == "sim";
  // on sim channels the latency depends on who dials: every address handed out names the
  // dialling node as its source
  auto from_node = [&](const std::string& addr, const std::string& src_node) {
    if (!sim) return addr;
    ChannelAddr a = ChannelAddr::parse(addr);
    a.src_node = src_node;
    return a.to_string();
  };
  if (!local) {
    client_addr = client_server_addr(pm->client_, alloc->transport());
    for (auto& kv : addrs)
      pm->router_->bind_addr(pm->proc_id(kv.first).to_string(),
                             ChannelAddr::parse(from_node(kv.second, "client")));
  }
  // Configure agents: full address book, supervision sink.
  auto replies = std::make_shared<QueueSink>();
  PortId reply_port = pm->client_inst_->bind(replies);
  for (size_t rank = 0; rank < pm->n_; ++rank) {
    Writer w;
    w.i64((int64_t)rank);
    w.u32((uint32_t)(addrs.size() + 2));
    const std::string my_node = sim ? ChannelAddr::parse(addrs[(int64_t)rank]).node : "";
    for (auto& kv : addrs) {
      w.str(pm->proc_id(kv.first).to_string());
      w.str(from_node(kv.second, my_node));
    }
    w.str(pm->client_->id().to_string());
    w.str(from_node(client_addr, my_node));
    w.str("*");  // default route: anything unknown goes through the client's router
    w.str(from_node(client_addr, my_node));
    write_port(w, pm->supervisor_port_);
    write_port(w, reply_port);
    pm->client_inst_->send(PortId{ActorId{pm->proc_id((int64_t)rank), "mesh_agent", 0}, kPortMessage},
                           std::move(w.buf), {{kHdrKind, "configure"}});
  }
  for (size_t got = 0; got < pm->n_;) {
    int64_t left = std::chrono::duration_cast<std::chrono::milliseconds>(
                       deadline - std::chrono::steady_clock::now()).count();
    if (left <= 0) {
      alloc->stop();
      throw std::runtime_error("proc mesh configuration timed out");
    }
    if (replies->recv(std::min<int64_t>(left, 200))) ++got;
  }
  pm->client_inst_->unbind(reply_port.port);

  std::weak_ptr<ProcMesh> weak = pm;
  auto* raw = pm.get();
  pm->pump_thr_ = std::thread([raw] {
    while (!raw->stopped_) {
      auto e = raw->supervisor_q_->recv(100);
      if (!e) continue;
      Event ev;
      ev.kind = "supervision";
      try {
        ev.sup = ActorSupervisionEvent::decode(e->data);
        ev.rank = ev.sup.actor_id.proc.rank;
      } catch (const std::exception&) {
        continue;
      }
      {
        std::lock_guard<std::mutex> g(raw->mu_);
        raw->events_.push_back(std::move(ev));
      }
      raw->ev_cv_.notify_all();
    }
  });
  pm->alloc_thr_ = std::thread([raw] { raw->pump_alloc_events(); });
  Metrics::global().counter_add("proc_mesh.allocations");
  return pm;
}

void ProcMesh::pump_alloc_events() {
  while (!stopped_) {
    auto ev = alloc_->next(100);
    if (!ev) continue;
    if (ev->kind != ProcEvent::Stopped && ev->kind != ProcEvent::Failed) continue;
    if (stopped_) break;
    Event e;
    e.kind = "proc_stopped";
    e.rank = ev->rank;
    e.reason = ev->reason;
    for (auto& l : ev->stderr_tail) e.reason += "\n" + l;
    Metrics::global().counter_add("proc_mesh.proc_failures");
    {
      std::lock_guard<std::mutex> g(mu_);
      events_.push_back(std::move(e));
    }
    ev_cv_.notify_all();
  }
}

std::optional<ProcMesh::Event> ProcMesh::next_event(int64_t timeout_ms) {
  std::unique_lock<std::mutex> g(mu_);
  auto ready = [&] { return !events_.empty() || stopped_.load(); };
  if (timeout_ms < 0)
    ev_cv_.wait(g, ready);
  else if (!ev_cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), ready))
    return std::nullopt;
  if (events_.empty()) return std::nullopt;
  Event e = std::move(events_.front());
  events_.pop_front();
  return e;
}

std::vector<SpawnResult> ProcMesh::spawn(const std::string& name, const std::string& actor_type,
                                         const std::string& params, int64_t timeout_ms) {
  auto replies = std::make_shared<QueueSink>();
  PortId reply_port = client_inst_->bind(replies);
  for (size_t rank = 0; rank < n_; ++rank) {
    Writer w;
    w.str(actor_type);
    w.str(name);
    w.str(params);
    write_port(w, reply_port);
    client_inst_->send(PortId{ActorId{proc_id((int64_t)rank), "mesh_agent", 0}, kPortMessage},
                       std::move(w.buf), {{kHdrKind, "gspawn"}});
  }
  std::vector<SpawnResult> out;
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  while (out.size() < n_) {
    int64_t left = std::chrono::duration_cast<std::chrono::milliseconds>(
                       deadline - std::chrono::steady_clock::now()).count();
    if (left <= 0) break;
    auto e = replies->recv(std::min<int64_t>(left, 200));
    if (!e) continue;
    Reader r(e->data);
    SpawnResult s;
    s.rank = r.i64();
    s.ok = r.u8() != 0;
    s.actor_id_or_error = r.str();
    out.push_back(std::move(s));
  }
  client_inst_->unbind(reply_port.port);
  if (out.size() < n_)
    throw std::runtime_error("spawn of '" + name + "' timed out: " + std::to_string(out.size()) +
                             " of " + std::to_string(n_) + " procs answered");
  std::sort(out.begin(), out.end(), [](auto& a, auto& b) { return a.rank < b.rank; });
  return out;
}

void ProcMesh::cast(const std::string& name, const Slice& slice, const Sel& selection,
                    const ActorId& sender, std::string data,
                    std::map<std::string, std::string> headers, std::vector<std::string> parts,
                    const Slice& cast_shape) {
  ScopedTimer timer("proc_mesh.cast_us");
  CastRequest c;
  c.mesh_id = name;
  c.slice = slice;
  c.selection = selection;
  c.sender = sender;
  c.data = std::move(data);
  c.headers = std::move(headers);
  c.cast_shape = cast_shape;
  {
    std::lock_guard<std::mutex> g(mu_);
    c.seq = cast_seq_[name + "/" + sender.to_string()]++;
  }
  // Root of the tree = the proc holding the first element of the slice.
  std::vector<size_t> zero(slice.ndim(), 0);
  int64_t root = (int64_t)slice.location(zero);
  Envelope e;
  e.sender = sender;
  e.dest = PortId{ActorId{proc_id(root), "comm", 0}, kPortMessage};
  e.data = encode_cast_root(c, parts);
  e.parts = std::move(parts);
  client_->post(std::move(e));
}

void ProcMesh::stop_actor(const std::string& name, int64_t timeout_ms) {
  auto replies = std::make_shared<QueueSink>();
  PortId reply_port = client_inst_->bind(replies);
  for (size_t rank = 0; rank < n_; ++rank) {
    Writer w;
    w.str(name);
    write_port(w, reply_port);
    client_inst_->send(PortId{ActorId{proc_id((int64_t)rank), "mesh_agent", 0}, kPortMessage},
                       std::move(w.buf), {{kHdrKind, "stop_actor"}});
  }
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (size_t got = 0; got < n_;) {
    int64_t left = std::chrono::duration_cast<std::chrono::milliseconds>(
                       deadline - std::chrono::steady_clock::now()).count();
    if (left <= 0) break;
    if (replies->recv(std::min<int64_t>(left, 200))) ++got;
  }
  client_inst_->unbind(reply_port.port);
}

std::vector<std::pair<int64_t, std::string>> ProcMesh::ledger(int64_t timeout_ms) {
  auto replies = std::make_shared<QueueSink>();
  PortId reply_port = client_inst_->bind(replies);
  for (size_t rank = 0; rank < n_; ++rank) {
    Writer w;
    write_port(w, reply_port);
    client_inst_->send(PortId{ActorId{proc_id((int64_t)rank), "mesh_agent", 0}, kPortMessage},
                       std::move(w.buf), {{kHdrKind, "ledger"}});
  }
  std::vector<std::pair<int64_t, std::string>> out;
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  while (out.size() < n_) {
    int64_t left = std::chrono::duration_cast<std::chrono::milliseconds>(
                       deadline - std::chrono::steady_clock::now()).count();
    if (left <= 0) break;
    auto env = replies->recv(std::min<int64_t>(left, 200));
    if (env) out.emplace_back(env->sender.proc.rank, env->data);
  }
  client_inst_->unbind(reply_port.port);
  std::sort(out.begin(), out.end());
  return out;
}

void ProcMesh::stop() {
  if (stopped_.exchange(true)) return;
  ev_cv_.notify_all();
  alloc_->stop();
  if (pump_thr_.joinable()) pump_thr_.join();
  if (alloc_thr_.joinable()) alloc_thr_.join();
  supervisor_q_->close();
}

ProcMesh::~ProcMesh() { stop(); }

}  // namespace mb
