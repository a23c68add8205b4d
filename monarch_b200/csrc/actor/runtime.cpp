#include "actor/runtime.h"

#include <algorithm>
#include <cstring>

namespace mb {

// ------------------------------------------------------------------- supervision --
std::string ActorSupervisionEvent::encode() const {
  Writer w;
  write_actor(w, actor_id);
  w.str(status);
  w.str(message);
  w.str(mesh);
  return std::move(w.buf);
}
ActorSupervisionEvent ActorSupervisionEvent::decode(std::string_view b) {
  Reader r(b);
  ActorSupervisionEvent e;
  e.actor_id = read_actor(r);
  e.status = r.str();
  e.message = r.str();
  e.mesh = r.str();
  return e;
}

const char* status_name(ActorStatus s) {
  switch (s) {
    case ActorStatus::Created: return "created";
    case ActorStatus::Idle: return "idle";
    case ActorStatus::Processing: return "processing";
    case ActorStatus::Stopping: return "stopping";
    case ActorStatus::Stopped: return "stopped";
    case ActorStatus::Failed: return "failed";
  }
  return "?";
}

// ----------------------------------------------------------------------- frames ----
Frame envelope_to_frame(Envelope&& env) {
  Frame f;
  f.head = env.encode_head();
  f.head.append(env.data);
  f.parts = std::move(env.parts);
  return f;
}

Envelope frame_to_envelope(Frame&& f) {
  Reader r(f.head);
  Envelope e;
  e.sender = read_actor(r);
  e.dest = read_port(r);
  uint32_t nh = r.u32();
  for (uint32_t i = 0; i < nh; ++i) {
    std::string k = r.str();
    e.headers[k] = r.str();
  }
  uint64_t dn = r.u64();
  uint32_t np = r.u32();
  for (uint32_t i = 0; i < np; ++i) (void)r.u64();
  size_t pos = r.pos();
  if (pos + dn > f.head.size()) throw CodecError("truncated envelope frame");
  if (np != f.parts.size()) throw CodecError("envelope part count mismatch");
  e.data.assign(f.head, pos, dn);
  e.parts = std::move(f.parts);
  return e;
}

// ------------------------------------------------------------------------ sinks ----
void QueueSink::deliver(Envelope&& env) {
  std::function<void()> n;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (closed_) return;
    q_.push_back(std::move(env));
    n = notify_;
  }
  cv_.notify_one();
  if (n) n();
}
std::optional<Envelope> QueueSink::recv(int64_t timeout_ms) {
  std::unique_lock<std::mutex> g(mu_);
  auto ready = [&] { return !q_.empty() || closed_; };
  if (timeout_ms < 0)
    cv_.wait(g, ready);
  else if (!cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), ready))
    return std::nullopt;
  if (q_.empty()) return std::nullopt;
  Envelope e = std::move(q_.front());
  q_.pop_front();
  return e;
}
std::optional<Envelope> QueueSink::try_recv() {
  std::lock_guard<std::mutex> g(mu_);
  if (q_.empty()) return std::nullopt;
  Envelope e = std::move(q_.front());
  q_.pop_front();
  return e;
}
void QueueSink::close() {
  {
    std::lock_guard<std::mutex> g(mu_);
    closed_ = true;
  }
  cv_.notify_all();
}
size_t QueueSink::size() const {
  std::lock_guard<std::mutex> g(mu_);
  return q_.size();
}
void QueueSink::set_notify(std::function<void()> fn) {
  std::lock_guard<std::mutex> g(mu_);
  notify_ = std::move(fn);
}

template <typename T, typename Op>
static std::string reduce_arrays(const std::string& a, const std::string& b, Op op) {
  if (a.empty()) return b;
  if (a.size() != b.size()) throw std::runtime_error("reducer: operand sizes differ");
  std::string out = a;
  size_t n = a.size() / sizeof(T);
  for (size_t i = 0; i < n; ++i) {
    T x, y;
    std::memcpy(&x, a.data() + i * sizeof(T), sizeof(T));
    std::memcpy(&y, b.data() + i * sizeof(T), sizeof(T));
    T z = op(x, y);
    std::memcpy(out.data() + i * sizeof(T), &z, sizeof(T));
  }
  return out;
}

ReduceFn builtin_reducer(const std::string& name) {
  if (name == "sum_f64")
    return [](const std::string& a, const std::string& b) {
      return reduce_arrays<double>(a, b, [](double x, double y) { return x + y; });
    };
  if (name == "sum_f32")
    return [](const std::string& a, const std::string& b) {
      return reduce_arrays<float>(a, b, [](float x, float y) { return x + y; });
    };
  if (name == "max_f64")
    return [](const std::string& a, const std::string& b) {
      return reduce_arrays<double>(a, b, [](double x, double y) { return std::max(x, y); });
    };
  if (name == "min_f64")
    return [](const std::string& a, const std::string& b) {
      return reduce_arrays<double>(a, b, [](double x, double y) { return std::min(x, y); });
    };
  if (name == "sum_i64")
    return [](const std::string& a, const std::string& b) {
      return reduce_arrays<int64_t>(a, b, [](int64_t x, int64_t y) { return x + y; });
    };
  if (name == "max_i64" || name == "low_watermark")
    return [name](const std::string& a, const std::string& b) {
      return reduce_arrays<int64_t>(a, b, [&](int64_t x, int64_t y) {
        return name == "max_i64" ? std::max(x, y) : std::min(x, y);
      });
    };
  throw std::runtime_error("unknown reducer: " + name);
}

void AccumSink::deliver(Envelope&& env) {
  // an update folded along a reduction tree stands for several senders
  uint64_t n = 1;
  if (auto it = env.headers.find(kHdrReduceCount); it != env.headers.end()) {
    try {
      n = std::stoull(it->second);
    } catch (const std::exception&) {
      n = 1;
    }
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    state_ = fn_(state_, env.data);
    count_ += n;
  }
  Metrics::global().counter_add("accum.messages");
  cv_.notify_all();
}
std::string AccumSink::state() const {
  std::lock_guard<std::mutex> g(mu_);
  return state_;
}
uint64_t AccumSink::count() const {
  std::lock_guard<std::mutex> g(mu_);
  return count_;
}
bool AccumSink::wait_count(uint64_t n, int64_t timeout_ms) {
  std::unique_lock<std::mutex> g(mu_);
  auto ready = [&] { return count_ >= n; };
  if (timeout_ms < 0) {
    cv_.wait(g, ready);
    return true;
  }
  return cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), ready);
}

// --------------------------------------------------------------------- instance ----
Instance::Instance(std::shared_ptr<Proc> proc, ActorId id, ActorHooks hooks,
                   std::shared_ptr<Instance> parent, bool has_loop)
    : proc_(proc), id_(std::move(id)), hooks_(std::move(hooks)), parent_(parent),
      has_loop_(has_loop) {
  if (!has_loop_) {
    undeliverable_q_ = std::make_shared<QueueSink>();
    status_ = ActorStatus::Idle;
  }
}

Instance::~Instance() {
  if (thr_.joinable()) {
    if (std::this_thread::get_id() == thr_.get_id())
      thr_.detach();
    else {
      signal(Signal::Stop);
      thr_.join();
    }
  }
}

std::string Instance::failure() const {
  std::lock_guard<std::mutex> g(mu_);
  return failure_;
}

PortId Instance::bind(std::shared_ptr<PortSink> sink) {
  std::lock_guard<std::mutex> g(mu_);
  uint64_t p = next_port_++;
  ports_[p] = std::move(sink);
  return PortId{id_, p};
}
void Instance::unbind(uint64_t port) {
  std::lock_guard<std::mutex> g(mu_);
  ports_.erase(port);
}

void Instance::send(const PortId& dest, std::string data,
                    std::map<std::string, std::string> headers, std::vector<std::string> parts) {
  auto p = proc();
  if (!p) return;
  Envelope e;
  e.sender = id_;
  e.dest = dest;
  e.headers = std::move(headers);
  e.data = std::move(data);
  e.parts = std::move(parts);
  Metrics::global().counter_add("mailbox.posts");
  p->post(std::move(e));
}

void Instance::enqueue(Work w) {
  {
    std::lock_guard<std::mutex> g(mu_);
    work_.push_back(std::move(w));
    Metrics::global().gauge_set("actor.queue_size." + id_.name, (double)work_.size());
  }
  cv_.notify_one();
}

bool Instance::deliver(Envelope&& env) {
  const uint64_t port = env.dest.port;
  if (port >= kPortUserBase) {
    std::shared_ptr<PortSink> sink;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = ports_.find(port);
      if (it == ports_.end()) return false;
      sink = it->second;
      if (sink->once()) ports_.erase(it);
    }
    sink->deliver(std::move(env));
    return true;
  }
  if (port == kPortUndeliverable && !has_loop_) {
    undeliverable_q_->deliver(std::move(env));
    return true;
  }
  if (!has_loop_) return false;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (!accepting_) return false;
  }
  if (port == kPortMessage && hooks_.inline_messages && hooks_.on_message) {
    std::lock_guard<std::mutex> one_at_a_time(inline_mu_);
    try {
      status_ = ActorStatus::Processing;
      hooks_.on_message(*this, env);
      handled_++;
      status_ = ActorStatus::Idle;
    } catch (const std::exception& e) {
      // fail on the actor's own thread, through the same path as a throwing loop handler
      ActorSupervisionEvent ev;
      ev.mesh = "__self__";
      ev.message = e.what();
      post_supervision(ev);
    }
    return true;
  }
  Work w;
  switch (port) {
    case kPortMessage:
      w.kind = Work::Message;
      w.env = std::move(env);
      break;
    case kPortSignal:
      w.kind = Work::Sig;
      w.sig = env.data.empty() ? Signal::Stop : (Signal)(uint8_t)env.data[0];
      break;
    case kPortSupervision:
      w.kind = Work::Supervision;
      w.ev = ActorSupervisionEvent::decode(env.data);
      break;
    case kPortUndeliverable:
      w.kind = Work::Undeliverable;
      w.env = std::move(env);
      break;
    default: return false;
  }
  enqueue(std::move(w));
  return true;
}

void Instance::post_supervision(const ActorSupervisionEvent& ev) {
  Work w;
  w.kind = Work::Supervision;
  w.ev = ev;
  enqueue(std::move(w));
}

void Instance::signal(Signal s) {
  if (!has_loop_) return;
  Work w;
  w.kind = Work::Sig;
  w.sig = s;
  {
    std::lock_guard<std::mutex> g(mu_);
    if (done_) return;
    // Stop jumps the queue; DrainAndStop waits its turn.
    if (s == Signal::Stop)
      work_.push_front(std::move(w));
    else
      work_.push_back(std::move(w));
  }
  cv_.notify_one();
}

void Instance::fail(const std::string& why) {
  Work w;
  w.kind = Work::Supervision;
  w.ev.actor_id = id_;
  w.ev.status = "failed";
  w.ev.message = why;
  w.ev.mesh = "__self__";
  {
    std::lock_guard<std::mutex> g(mu_);
    if (done_) return;
    work_.push_front(std::move(w));
  }
  cv_.notify_one();
}

bool Instance::join(int64_t timeout_ms) {
  std::unique_lock<std::mutex> g(mu_);
  auto ready = [&] { return done_.load(); };
  if (!has_loop_) return true;
  if (timeout_ms < 0) {
    done_cv_.wait(g, ready);
    return true;
  }
  return done_cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), ready);
}

std::vector<std::shared_ptr<Instance>> Instance::children() const {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<std::shared_ptr<Instance>> out;
  for (auto& w : children_)
    if (auto c = w.lock()) out.push_back(c);
  return out;
}

void Instance::handle_returned(Envelope& outer) {
  std::string reason = outer.headers.count("reason") ? outer.headers["reason"] : "undeliverable";
  Envelope inner;
  try {
    inner = Envelope::decode(outer.data);
  } catch (const std::exception&) {
  }
  Metrics::global().counter_add("mailbox.undeliverable");
  recorder_.record("undeliverable", inner.dest.to_string() + ": " + reason);
  bool handled = false;
  if (hooks_.on_undeliverable) handled = hooks_.on_undeliverable(*this, inner, reason);
  if (!handled)
    throw std::runtime_error("undeliverable message to " + inner.dest.to_string() + ": " + reason);
}

void Instance::finish(ActorStatus final_status, const std::string& why) {
  std::deque<Work> rest;
  {
    std::lock_guard<std::mutex> g(mu_);
    accepting_ = false;
    failure_ = why;
    rest.swap(work_);
  }
  status_ = final_status;
  recorder_.record(status_name(final_status), why);
  if (hooks_.on_stop) {
    try {
      hooks_.on_stop(*this);
    } catch (const std::exception& e) {
      MB_LOG(Warn, id_.to_string() + ": on_stop raised: " + e.what());
    }
  }
  for (auto& c : children()) c->signal(Signal::Stop);
  auto p = proc();
  if (p) {
    for (auto& w : rest)
      if (w.kind == Work::Message) p->return_undeliverable(std::move(w.env), "actor " + std::string(status_name(final_status)));
  }
  if (final_status == ActorStatus::Failed) {
    MB_LOG(Warn, "actor " + id_.to_string() + " failed: " + why);
    ActorSupervisionEvent ev;
    ev.actor_id = id_;
    ev.status = "failed";
    ev.message = why;
    if (auto par = parent())
      par->post_supervision(ev);
    else if (p)
      p->report_supervision(ev, this);
  }
  {
    std::lock_guard<std::mutex> g(mu_);
    done_ = true;
    for (auto& kv : ports_) {
      if (auto q = std::dynamic_pointer_cast<QueueSink>(kv.second)) q->close();
    }
  }
  done_cv_.notify_all();
}

void Instance::run() {
  status_ = ActorStatus::Idle;
  bool draining = false;
  while (true) {
    Work w;
    {
      std::unique_lock<std::mutex> g(mu_);
      if (draining && work_.empty()) {
        g.unlock();
        finish(ActorStatus::Stopped, "");
        return;
      }
      cv_.wait(g, [&] { return !work_.empty(); });
      w = std::move(work_.front());
      work_.pop_front();
    }
    try {
      switch (w.kind) {
        case Work::Message: {
          status_ = ActorStatus::Processing;
          double t0 = now_us();
          if (hooks_.on_message) hooks_.on_message(*this, w.env);
          handled_++;
          Metrics::global().histogram_record("actor.handler_us", now_us() - t0);
          if (TraceWriter::global().enabled())
            TraceWriter::global().complete(id_.name + ".handle", "actor", t0, now_us() - t0,
                                           id_.proc.rank, id_.pid);
          status_ = ActorStatus::Idle;
          break;
        }
        case Work::Sig:
          if (w.sig == Signal::Stop) {
            finish(ActorStatus::Stopped, "");
            return;
          }
          draining = true;
          {
            std::lock_guard<std::mutex> g(mu_);
            accepting_ = false;
          }
          status_ = ActorStatus::Stopping;
          break;
        case Work::Supervision: {
          if (w.ev.mesh == "__self__") throw std::runtime_error(w.ev.message);
          bool handled = false;
          if (hooks_.on_supervision) handled = hooks_.on_supervision(*this, w.ev);
          if (!handled)
            throw std::runtime_error("supervision: child " + w.ev.actor_id.to_string() +
                                     " failed: " + w.ev.message);
          break;
        }
        case Work::Undeliverable: handle_returned(w.env); break;
      }
    } catch (const std::exception& e) {
      finish(ActorStatus::Failed, e.what());
      return;
    }
  }
}

// ------------------------------------------------------------------------- proc ----
std::shared_ptr<Proc> Proc::create(ProcId id, std::shared_ptr<MailboxSender> forwarder) {
  return std::shared_ptr<Proc>(new Proc(std::move(id), std::move(forwarder)));
}

Proc::~Proc() { stop_all(200); }

std::shared_ptr<Instance> Proc::spawn(const std::string& name, ActorHooks hooks,
                                      std::shared_ptr<Instance> parent) {
  std::shared_ptr<Instance> inst;
  {
    std::lock_guard<std::mutex> g(mu_);
    auto& v = actors_[name];
    ActorId id{id_, name, (int64_t)v.size()};
    inst = std::make_shared<Instance>(shared_from_this(), id, std::move(hooks), parent, true);
    v.push_back(inst);
  }
  if (parent) {
    std::lock_guard<std::mutex> g(parent->mu_);
    parent->children_.push_back(inst);
  }
  Instance* raw = inst.get();
  inst->thr_ = std::thread([raw] { raw->run(); });
  Metrics::global().counter_add("proc.actors_spawned");
  return inst;
}

std::shared_ptr<Instance> Proc::attach(const std::string& name) {
  std::lock_guard<std::mutex> g(mu_);
  auto& v = actors_[name];
  ActorId id{id_, name, (int64_t)v.size()};
  auto inst = std::make_shared<Instance>(shared_from_this(), id, ActorHooks{}, nullptr, false);
  v.push_back(inst);
  return inst;
}

std::shared_ptr<Instance> Proc::find(const std::string& name, int64_t pid) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = actors_.find(name);
  if (it == actors_.end() || pid < 0 || (size_t)pid >= it->second.size()) return nullptr;
  return it->second[(size_t)pid];
}

void Proc::set_forwarder(std::shared_ptr<MailboxSender> f) {
  std::lock_guard<std::mutex> g(mu_);
  forwarder_ = std::move(f);
}
std::shared_ptr<MailboxSender> Proc::forwarder() const {
  std::lock_guard<std::mutex> g(mu_);
  return forwarder_;
}

void Proc::post(Envelope env) {
  if (env.dest.actor.proc == id_) {
    auto inst = find(env.dest.actor.name, env.dest.actor.pid);
    if (inst) {
      // deliver() moves from the envelope only when it accepts it
      if (inst->deliver(std::move(env))) return;
      return_undeliverable(std::move(env), "actor or port is gone");
      return;
    }
    return_undeliverable(std::move(env), "no such actor");
    return;
  }
  auto f = forwarder();
  if (f)
    f->post(std::move(env));
  else
    return_undeliverable(std::move(env), "no route to " + env.dest.actor.proc.to_string());
}

void Proc::return_undeliverable(Envelope env, const std::string& reason) {
  Metrics::global().counter_add("mailbox.returned");
  // Returned messages never bounce again; replies ("no_return") to a port the caller has
  // already closed are dropped rather than failing the replying actor.
  if (env.headers.count("undeliverable") || env.headers.count("no_return") ||
      env.sender.name.empty()) {
    MB_LOG(Debug, "dropping undeliverable message to " + env.dest.to_string() + ": " + reason);
    return;
  }
  Envelope r;
  r.sender = env.dest.actor;
  r.dest = PortId{env.sender, kPortUndeliverable};
  r.headers["undeliverable"] = "1";
  r.headers["reason"] = reason;
  r.data = env.encode();
  post(std::move(r));
}

void Proc::set_supervision_coordinator(std::optional<PortId> port) {
  std::lock_guard<std::mutex> g(mu_);
  coordinator_ = std::move(port);
}

void Proc::report_supervision(const ActorSupervisionEvent& ev, Instance* from) {
  std::optional<PortId> c;
  {
    std::lock_guard<std::mutex> g(mu_);
    c = coordinator_;
  }
  Metrics::global().counter_add("proc.supervision_events");
  if (!c) {
    MB_LOG(Error, "unhandled supervision event on " + id_.to_string() + ": " +
                      ev.actor_id.to_string() + " " + ev.status + ": " + ev.message);
    return;
  }
  Envelope e;
  e.sender = ev.actor_id;
  e.dest = *c;
  e.headers[kHdrKind] = "supervision";
  e.headers["undeliverable"] = "1";  // never bounce supervision reports
  e.data = ev.encode();
  post(std::move(e));
}

std::vector<ActorSnapshot> Proc::ledger_snapshot() const {
  std::vector<std::shared_ptr<Instance>> all;
  {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : actors_)
      for (auto& i : kv.second) all.push_back(i);
  }
  std::vector<ActorSnapshot> out;
  for (auto& i : all) {
    ActorSnapshot s;
    s.actor_id = i->id().to_string();
    s.status = status_name(i->status());
    s.failure = i->failure();
    s.messages_handled = i->messages_handled();
    for (auto& c : i->children()) s.children.push_back(c->id().to_string());
    s.events = i->recorder().tail(16);
    out.push_back(std::move(s));
  }
  return out;
}

std::vector<std::string> Proc::stop_all(int64_t timeout_ms) {
  std::vector<std::shared_ptr<Instance>> all;
  {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : actors_)
      for (auto& i : kv.second) all.push_back(i);
  }
  for (auto& i : all) i->signal(Signal::Stop);
  std::vector<std::string> alive;
  for (auto& i : all)
    if (!i->join(timeout_ms)) alive.push_back(i->id().to_string());
  return alive;
}

// ---------------------------------------------------------------------- senders ----
void MailboxClient::post(Envelope env) {
  auto home = home_;
  Metrics::global().histogram_record("channel.send_bytes", (double)env.data.size());
  tx_->post(envelope_to_frame(std::move(env)), [home](Frame&& f) {
    auto p = home.lock();
    if (!p) return;
    try {
      p->return_undeliverable(frame_to_envelope(std::move(f)), "delivery failed");
    } catch (const std::exception& e) {
      MB_LOG(Warn, std::string("cannot return undeliverable frame: ") + e.what());
    }
  });
}

MailboxServer::MailboxServer(std::shared_ptr<Rx> rx, std::shared_ptr<MailboxSender> target)
    : rx_(std::move(rx)), target_(std::move(target)) {
  thr_ = std::thread([this] {
    while (!stop_) {
      auto f = rx_->recv(100);
      if (!f) {
        if (rx_->closed()) break;
        continue;
      }
      try {
        target_->post(frame_to_envelope(std::move(*f)));
      } catch (const std::exception& e) {
        MB_LOG(Warn, std::string("mailbox server: bad frame: ") + e.what());
      }
    }
  });
}
MailboxServer::~MailboxServer() { stop(); }
void MailboxServer::stop() {
  if (stop_.exchange(true)) return;
  if (thr_.joinable()) thr_.join();
  rx_->close();
}

void Router::bind_local(const std::shared_ptr<Proc>& proc) {
  std::lock_guard<std::mutex> g(mu_);
  local_[proc->id().to_string()] = proc;
}
void Router::unbind_local(const ProcId& id) {
  std::lock_guard<std::mutex> g(mu_);
  local_.erase(id.to_string());
}
void Router::bind_addr(const std::string& prefix, const ChannelAddr& addr) {
  std::lock_guard<std::mutex> g(mu_);
  book_[prefix] = addr;
}
void Router::unbind_addr(const std::string& prefix) {
  std::lock_guard<std::mutex> g(mu_);
  book_.erase(prefix);
}
void Router::set_default(std::shared_ptr<MailboxSender> s) {
  std::lock_guard<std::mutex> g(mu_);
  default_ = std::move(s);
}
void Router::set_home(std::weak_ptr<Proc> home) {
  std::lock_guard<std::mutex> g(mu_);
  home_ = std::move(home);
}
std::map<std::string, std::string> Router::address_book() const {
  std::lock_guard<std::mutex> g(mu_);
  std::map<std::string, std::string> out;
  for (auto& kv : book_) out[kv.first] = kv.second.to_string();
  return out;
}

void Router::post(Envelope env) {
  const std::string key = env.dest.actor.proc.to_string();
  std::shared_ptr<Proc> local;
  std::shared_ptr<MailboxSender> next;
  std::shared_ptr<Proc> home;
  {
    std::lock_guard<std::mutex> g(mu_);
    home = home_.lock();
    auto li = local_.find(key);
    if (li != local_.end()) local = li->second.lock();
    if (!local) {
      const ChannelAddr* addr = nullptr;
      auto bi = book_.find(key);
      if (bi != book_.end())
        addr = &bi->second;
      else {
        bi = book_.find(env.dest.actor.proc.world);
        if (bi != book_.end()) addr = &bi->second;
      }
      if (addr) {
        std::string as = addr->to_string();
        auto ci = clients_.find(as);
        if (ci == clients_.end() || ci->second->status() == TxStatus::Closed) {
          auto c = std::make_shared<MailboxClient>(dial(*addr), home_);
          clients_[as] = c;
          next = c;
        } else {
          next = ci->second;
        }
      } else {
        next = default_;
      }
    }
  }
  if (local) {
    local->post(std::move(env));
  } else if (next) {
    next->post(std::move(env));
  } else if (home) {
    home->return_undeliverable(std::move(env), "no route to " + key);
  } else {
    MB_LOG(Warn, "router: no route to " + key + " and nowhere to return the message");
  }
}

}  // namespace mb
