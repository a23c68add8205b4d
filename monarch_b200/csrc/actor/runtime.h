// Actor runtime: procs, actor instances, mailboxes/ports, message routing, supervision.
//
// Parity: hyperactor/src/proc.rs (Proc, Instance, the per-actor serve loop, supervision
// bubbling, ledger snapshot), hyperactor/src/mailbox.rs (ports, once ports, accumulating
// ports, MailboxSender family: client/server/muxer/router/dial-router, undeliverable
// returns), hyperactor/src/actor.rs (Signal, ActorStatus), hyperactor/src/accum.rs
// (reducers), hyperactor/src/supervision.rs (ActorSupervisionEvent).
//
// Design: every actor instance owns one OS thread that drains a single work queue holding
// messages, signals, supervision events and returned (undeliverable) envelopes, so an
// actor handles one thing at a time and per-sender FIFO order is preserved end to end.
// User-opened ports deliver straight into their sink from the posting thread.
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#include "actor/reference.h"
#include "channel/channel.h"
#include "telemetry/telemetry.h"

namespace mb {

// ------------------------------------------------------------------- supervision --
struct ActorSupervisionEvent {
  ActorId actor_id;
  std::string status;   // "failed", "stopped"
  std::string message;  // failure text (exception text / traceback)
  std::string mesh;     // actor-mesh id when the failing message came from a cast
  std::string encode() const;
  static ActorSupervisionEvent decode(std::string_view b);
};

enum class ActorStatus { Created, Idle, Processing, Stopping, Stopped, Failed };
const char* status_name(ActorStatus s);

enum class Signal : uint8_t { Stop = 1, DrainAndStop = 2 };

// --------------------------------------------------------------------- senders ----
class MailboxSender {
 public:
  virtual ~MailboxSender() = default;
  virtual void post(Envelope env) = 0;
};

// --------------------------------------------------------------------------- ports --
class PortSink {
 public:
  virtual ~PortSink() = default;
  virtual void deliver(Envelope&& env) = 0;
  virtual bool once() const { return false; }
};

// Blocking FIFO a caller can wait on (backs Port/OncePort receivers).
class QueueSink : public PortSink {
 public:
  explicit QueueSink(bool once = false) : once_(once) {}
  void deliver(Envelope&& env) override;
  bool once() const override { return once_; }
  // nullopt on timeout (timeout_ms < 0 waits forever) or when closed and drained.
  std::optional<Envelope> recv(int64_t timeout_ms);
  std::optional<Envelope> try_recv();
  void close();
  size_t size() const;
  // Callback invoked (from the delivering thread) after each delivery: lets an event
  // loop be woken without polling.
  void set_notify(std::function<void()> fn);

 private:
  bool once_;
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Envelope> q_;
  bool closed_ = false;
  std::function<void()> notify_;
};

// Reducers of accumulating / split ports.  Payloads are fixed-layout numeric blobs
// ("f64:<n>" headers) or opaque bytes combined by a user callback.
using ReduceFn = std::function<std::string(const std::string& acc, const std::string& update)>;
ReduceFn builtin_reducer(const std::string& name);  // "sum_f64", "max_f64", "min_f64", "sum_i64"

class AccumSink : public PortSink {
 public:
  AccumSink(ReduceFn fn, std::string init) : fn_(std::move(fn)), state_(std::move(init)) {}
  void deliver(Envelope&& env) override;
  std::string state() const;
  uint64_t count() const;
  // Wait until at least `n` updates were folded in; false on timeout.
  bool wait_count(uint64_t n, int64_t timeout_ms);

 private:
  ReduceFn fn_;
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::string state_;
  uint64_t count_ = 0;
};

// ------------------------------------------------------------------------ instance --
class Proc;
class Instance;

struct ActorHooks {
  // Handle one message addressed to the actor (port 0).  Throwing fails the actor.
  std::function<void(Instance&, Envelope&)> on_message;
  // Return true if the child failure was handled; false propagates it upward.
  std::function<bool(Instance&, const ActorSupervisionEvent&)> on_supervision;
  // Return true if handled; false fails this actor (the default for returned messages).
  std::function<bool(Instance&, Envelope& returned, const std::string& reason)> on_undeliverable;
  std::function<void(Instance&)> on_stop;
  // Run on_message on the thread that delivers the message (one at a time, under a lock)
  // instead of waking the actor's own thread.  For stateless relays such as the comm actors
  // of the cast tree, where the hand-over to another thread is most of the hop's cost.  The
  // handler must not block and must only deliver "downstream" (no cycles between inline
  // actors), since deliveries nest.
  bool inline_messages = false;
};

class Instance : public std::enable_shared_from_this<Instance> {
 public:
  Instance(std::shared_ptr<Proc> proc, ActorId id, ActorHooks hooks,
           std::shared_ptr<Instance> parent, bool has_loop);
  ~Instance();

  const ActorId& id() const { return id_; }
  std::shared_ptr<Proc> proc() const { return proc_.lock(); }
  ActorStatus status() const { return status_.load(); }
  std::string failure() const;

  // Ports ---------------------------------------------------------------------------
  PortId bind(std::shared_ptr<PortSink> sink);
  void unbind(uint64_t port);
  PortId port_id(uint64_t port) const { return PortId{id_, port}; }

  // Sending -------------------------------------------------------------------------
  void send(const PortId& dest, std::string data, std::map<std::string, std::string> headers = {},
            std::vector<std::string> parts = {});

  // Lifecycle -----------------------------------------------------------------------
  void signal(Signal s);
  // Block until the actor thread has exited (or timeout). True if stopped.
  bool join(int64_t timeout_ms);
  // Fail the actor from outside its handler (e.g. a panic side channel).
  void fail(const std::string& why);

  // Delivery entry (called by Proc). Returns false if the port does not exist or the
  // actor no longer accepts messages.
  bool deliver(Envelope&& env);
  // Used by Proc to hand a child failure / returned message to this actor.
  void post_supervision(const ActorSupervisionEvent& ev);

  Recorder& recorder() { return recorder_; }
  std::vector<std::shared_ptr<Instance>> children() const;
  std::shared_ptr<Instance> parent() const { return parent_.lock(); }
  uint64_t messages_handled() const { return handled_.load(); }
  // For client ("attached") instances: returned envelopes queue here.
  std::shared_ptr<QueueSink> undeliverable_queue() const { return undeliverable_q_; }

 private:
  friend class Proc;
  struct Work {
    enum Kind { Message, Sig, Supervision, Undeliverable } kind;
    Envelope env;
    Signal sig = Signal::Stop;
    ActorSupervisionEvent ev;
  };
  void run();
  void enqueue(Work w);
  void finish(ActorStatus final_status, const std::string& why);
  void handle_returned(Envelope& outer);

  std::weak_ptr<Proc> proc_;
  ActorId id_;
  ActorHooks hooks_;
  std::weak_ptr<Instance> parent_;
  bool has_loop_;

  std::mutex inline_mu_;  // serialises inline_messages handlers
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Work> work_;
  bool accepting_ = true;
  std::unordered_map<uint64_t, std::shared_ptr<PortSink>> ports_;
  uint64_t next_port_ = kPortUserBase;
  std::vector<std::weak_ptr<Instance>> children_;
  std::string failure_;
  std::atomic<ActorStatus> status_{ActorStatus::Created};
  std::atomic<uint64_t> handled_{0};
  std::thread thr_;
  std::atomic<bool> done_{false};
  std::condition_variable done_cv_;
  Recorder recorder_;
  std::shared_ptr<QueueSink> undeliverable_q_;
};

// ---------------------------------------------------------------------------- proc --
struct ActorSnapshot {
  std::string actor_id, status, failure;
  uint64_t messages_handled = 0;
  std::vector<std::string> children;
  std::vector<RecordedEvent> events;
};

class Proc : public std::enable_shared_from_this<Proc> {
 public:
  static std::shared_ptr<Proc> create(ProcId id, std::shared_ptr<MailboxSender> forwarder);
  ~Proc();
  const ProcId& id() const { return id_; }

  // Spawn an actor with its own message loop.  pid is assigned per name (0, 1, ...).
  std::shared_ptr<Instance> spawn(const std::string& name, ActorHooks hooks,
                                  std::shared_ptr<Instance> parent = nullptr);
  // A loop-less instance whose ports a client thread reads directly.
  std::shared_ptr<Instance> attach(const std::string& name);

  // Route an envelope: local actors directly, everything else through the forwarder.
  void post(Envelope env);
  // Send `env` back to its sender's undeliverable port.
  void return_undeliverable(Envelope env, const std::string& reason);

  void set_forwarder(std::shared_ptr<MailboxSender> f);
  std::shared_ptr<MailboxSender> forwarder() const;
  // Root-actor failures (and unhandled bubbled failures) are reported here.
  void set_supervision_coordinator(std::optional<PortId> port);
  void report_supervision(const ActorSupervisionEvent& ev, Instance* from);

  std::shared_ptr<Instance> find(const std::string& name, int64_t pid) const;
  std::vector<ActorSnapshot> ledger_snapshot() const;
  // Stop every actor (Stop signal, then wait up to timeout). Returns actors still alive.
  std::vector<std::string> stop_all(int64_t timeout_ms);

 private:
  Proc(ProcId id, std::shared_ptr<MailboxSender> fwd) : id_(std::move(id)), forwarder_(std::move(fwd)) {}
  ProcId id_;
  mutable std::mutex mu_;
  std::shared_ptr<MailboxSender> forwarder_;
  std::map<std::string, std::vector<std::shared_ptr<Instance>>> actors_;
  std::optional<PortId> coordinator_;
};

// ---------------------------------------------------------- senders (implementations) --
// Sends envelopes over a dialled channel; returns them to `home` when undeliverable.
class MailboxClient : public MailboxSender {
 public:
  MailboxClient(std::shared_ptr<Tx> tx, std::weak_ptr<Proc> home) : tx_(std::move(tx)), home_(home) {}
  void post(Envelope env) override;
  TxStatus status() const { return tx_->status(); }

 private:
  std::shared_ptr<Tx> tx_;
  std::weak_ptr<Proc> home_;
};

// Serves a channel: every received frame is decoded and handed to `target`.
class MailboxServer {
 public:
  MailboxServer(std::shared_ptr<Rx> rx, std::shared_ptr<MailboxSender> target);
  ~MailboxServer();
  ChannelAddr addr() const { return rx_->addr(); }
  void stop();

 private:
  std::shared_ptr<Rx> rx_;
  std::shared_ptr<MailboxSender> target_;
  std::atomic<bool> stop_{false};
  std::thread thr_;
};

// Routes by destination proc: in-process procs first (muxer), then the longest matching
// address-book prefix ("world[3]" or "world") dialled on demand, then an optional default.
class Router : public MailboxSender, public std::enable_shared_from_this<Router> {
 public:
  void bind_local(const std::shared_ptr<Proc>& proc);
  void unbind_local(const ProcId& id);
  void bind_addr(const std::string& prefix, const ChannelAddr& addr);
  void unbind_addr(const std::string& prefix);
  void set_default(std::shared_ptr<MailboxSender> s);
  void set_home(std::weak_ptr<Proc> home);  // where undeliverables are returned
  void post(Envelope env) override;
  std::map<std::string, std::string> address_book() const;

 private:
  mutable std::mutex mu_;
  std::map<std::string, std::weak_ptr<Proc>> local_;
  std::map<std::string, ChannelAddr> book_;
  std::map<std::string, std::shared_ptr<MailboxClient>> clients_;  // by address string
  std::shared_ptr<MailboxSender> default_;
  std::weak_ptr<Proc> home_;
};

// Adapts a Proc to the MailboxSender interface (target of a MailboxServer).
class ProcSender : public MailboxSender {
 public:
  explicit ProcSender(std::weak_ptr<Proc> p) : p_(std::move(p)) {}
  void post(Envelope env) override {
    if (auto p = p_.lock()) p->post(std::move(env));
  }

 private:
  std::weak_ptr<Proc> p_;
};

Frame envelope_to_frame(Envelope&& env);
Envelope frame_to_envelope(Frame&& f);

}  // namespace mb
