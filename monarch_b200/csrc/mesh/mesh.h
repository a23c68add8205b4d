// Mesh layer: proc allocation + bootstrap, the per-proc MeshAgent, the cast tree
// (CommActor) and the client-side ProcMesh.
//
// Parity: hyperactor_mesh/src/alloc.rs (Alloc, ProcState, ProcStopReason),
// alloc/local.rs (in-process procs), alloc/process.rs (fork/exec children with
// HYPERACTOR_MESH_BOOTSTRAP_ADDR / HYPERACTOR_MESH_INDEX, piped stdio, exit monitoring),
// alloc/logtailer.rs, bootstrap.rs (Hello -> StartProc -> StartedProc, heartbeat,
// StopAndExit), proc_mesh/mesh_agent.rs (Configure / Gspawn / StopActor, supervision
// forwarding), comm.rs + comm/multicast.rs (cast tree over ndslice routing frames with
// CAST_* headers), proc_mesh.rs (router, client proc, supervision sink, events),
// actor_mesh.rs (cast / sliced cast).
#pragma once
#include <sys/types.h>

#include <atomic>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <thread>
#include <vector>

#include "actor/runtime.h"
#include "ndslice/ndslice.h"

namespace mb {

// ------------------------------------------------------------------ selection codec --
void encode_selection(Writer& w, const Sel& s);
Sel decode_selection(Reader& r);
void encode_slice(Writer& w, const Slice& s);
Slice decode_slice(Reader& r);

// --------------------------------------------------------------- actor type registry --
// A factory builds the hooks of a new actor from its spawn parameters.
using ActorFactory =
    std::function<ActorHooks(const std::shared_ptr<Proc>&, const std::string& name,
                             const std::string& params)>;
void register_actor_type(const std::string& type, ActorFactory f);
std::optional<ActorFactory> lookup_actor_type(const std::string& type);

// ------------------------------------------------------------------------- alloc ----
struct ProcEvent {
  enum Kind { Created, Running, Stopped, Failed } kind;
  int64_t rank = 0;
  std::string proc_id;
  std::string addr;    // mailbox address when Running
  std::string reason;  // "exited(0)", "killed(9)", "watchdog", ... when Stopped/Failed
  int exit_code = 0;
  std::vector<std::string> stderr_tail;
};

class LogTailer {
 public:
  // Reads `fd` line by line on its own thread; keeps the last `keep` lines and hands
  // every line to `sink` (may be empty).
  LogTailer(int fd, size_t keep, std::function<void(const std::string&)> sink);
  ~LogTailer();
  std::vector<std::string> tail() const;
  void join();

 private:
  int fd_;
  size_t keep_;
  std::function<void(const std::string&)> sink_;
  mutable std::mutex mu_;
  std::deque<std::string> lines_;
  std::thread thr_;
};

class Alloc {
 public:
  virtual ~Alloc() = default;
  virtual std::string world() const = 0;
  virtual size_t size() const = 0;
  // Next lifecycle event (blocks up to timeout_ms; <0 forever). nullopt on timeout.
  virtual std::optional<ProcEvent> next(int64_t timeout_ms) = 0;
  virtual void stop() = 0;
  // In-process allocs expose their procs (for routing without sockets).
  virtual std::vector<std::shared_ptr<Proc>> local_procs() const { return {}; }
  virtual std::string transport() const = 0;  // "local" | "unix" | "tcp"
  // Hard-kill one rank (host-side fault injection for tests).
  virtual void kill_rank(int64_t rank, int sig) { (void)rank; (void)sig; }
};

// N procs inside this process, linked by one Router.
std::shared_ptr<Alloc> make_local_alloc(const std::string& world, size_t n,
                                        std::shared_ptr<Router> router);

// N procs inside this process whose mailboxes are reached through `sim:` channels: every
// message between procs (and between the client and a proc) crosses the simulated network
// (channel.h SimNet) and pays the latency of the distance between the two nodes.
// `nodes[i]` names the node of proc i ("dc0.rack1.host3"); the client sits on node "client".
// (hyperactor_mesh/src/alloc/sim.rs in the reference.)
std::shared_ptr<Alloc> make_sim_alloc(const std::string& world, std::vector<std::string> nodes);

struct ProcessAllocOptions {
  std::vector<std::string> argv;             // bootstrap command
  std::map<std::string, std::string> env;    // extra environment for every child
  bool per_rank_gpu_env = false;             // export LOCAL_RANK / rank index to children
  std::function<void(int64_t rank, bool is_stderr, const std::string&)> log_sink;
  size_t tail_lines = 100;
  std::string transport = "unix";
};
std::shared_ptr<Alloc> make_process_alloc(const std::string& world, size_t n,
                                          ProcessAllocOptions opts);

// Child side of the bootstrap protocol: never returns (exits the process) unless the
// environment does not describe a bootstrap, in which case it returns 1.
int bootstrap_main();

// Procs that are NOT started by the allocator: processes launched by something else (an
// SPMD launcher such as torchrun, a batch scheduler) join the mesh by dialling
// `bootstrap_addr()` with their rank (`bootstrap_attach`).  The allocator waits for `n` of
// them; a joined proc that drops its control connection is reported as failed.
// (The reference gets externally started procs through its allocator daemons,
// hyperactor_mesh/src/alloc/remoteprocess.rs; this is the in-box form of the same idea.)
class AttachAlloc : public Alloc {
 public:
  virtual std::string bootstrap_addr() const = 0;
};
std::shared_ptr<AttachAlloc> make_attach_alloc(const std::string& world, size_t n,
                                               const std::string& transport);

// Host one proc of an attach allocation inside the calling process: announces `index` to
// the allocator at `addr`, creates the proc with its mesh agent when told to and serves it
// until the allocator stops the mesh or goes away; then stops the proc's actors and
// RETURNS (the hosting process lives on).  0 on an orderly stop, 1 when the allocator vanished.
int bootstrap_attach(const std::string& addr, int64_t index);

// --------------------------------------------------------------------- comm actor ----
ActorHooks make_comm_actor(const std::shared_ptr<Proc>& proc);
ActorHooks make_mesh_agent(const std::shared_ptr<Proc>& proc, std::shared_ptr<Router> router);

struct CastRequest {
  std::string mesh_id;     // name of the actor mesh (also the destination actor name)
  Slice slice;             // proc ranks of the mesh (root = first element)
  Sel selection;           // which of them receive the message
  ActorId sender;          // originating sender
  std::string data;        // message body delivered to each actor's port 0
  std::map<std::string, std::string> headers;
  std::vector<std::string> parts;
  uint64_t seq = 0;        // per (sender, mesh) sequence number
  Slice cast_shape;        // shape reported to receivers (CAST_SHAPE); cast_rank = index in it
};
// Bodies of this size or more travel as the last part of the envelope instead of inside the
// routing header, so that the hops of the cast tree never re-encode (copy) them.
constexpr size_t kCastBodyAsPartBytes = 4096;
// Encodes the routing header.  A large body is moved out of `c.data` and appended to
// `parts` (the envelope's parts).
std::string encode_cast_root(CastRequest& c, std::vector<std::string>& parts);

// ----------------------------------------------------------------------- proc mesh ----
struct SpawnResult {
  int64_t rank;
  bool ok;
  std::string actor_id_or_error;
};

class ProcMesh : public std::enable_shared_from_this<ProcMesh> {
 public:
  // Bring up a mesh over `alloc`: waits until every rank is Running, wires routing,
  // spawns mesh agents' peers (comm actors) and installs the supervision sink.
  static std::shared_ptr<ProcMesh> allocate(std::shared_ptr<Alloc> alloc,
                                            std::shared_ptr<Router> router,
                                            std::shared_ptr<Proc> client, int64_t timeout_ms);
  ~ProcMesh();

  const std::string& world() const { return world_; }
  size_t size() const { return n_; }
  std::shared_ptr<Proc> client_proc() const { return client_; }
  std::shared_ptr<Instance> client() const { return client_inst_; }
  std::shared_ptr<Router> router() const { return router_; }
  ProcId proc_id(int64_t rank) const { return ProcId{world_, rank}; }
  std::vector<std::shared_ptr<Proc>> local_procs() const { return alloc_->local_procs(); }

  // Spawn `actor_type` named `name` on every proc. Blocks until all ranks answered.
  std::vector<SpawnResult> spawn(const std::string& name, const std::string& actor_type,
                                 const std::string& params, int64_t timeout_ms);
  // Cast `data` to actor `name` on the procs of `slice` selected by `selection`.
  void cast(const std::string& name, const Slice& slice, const Sel& selection,
            const ActorId& sender, std::string data, std::map<std::string, std::string> headers,
            std::vector<std::string> parts, const Slice& cast_shape);
  void stop_actor(const std::string& name, int64_t timeout_ms);
  // Actor-tree snapshot of every proc (rank, tab-separated lines as written by the mesh
  // agent); procs that do not answer within the timeout are missing from the result.
  std::vector<std::pair<int64_t, std::string>> ledger(int64_t timeout_ms);

  // Supervision / lifecycle events for Python monitors: blocks up to timeout.
  struct Event {
    std::string kind;  // "supervision" | "proc_stopped"
    int64_t rank = -1;
    ActorSupervisionEvent sup;
    std::string reason;
  };
  std::optional<Event> next_event(int64_t timeout_ms);
  void stop();
  bool stopped() const { return stopped_; }
  void kill_rank(int64_t rank, int sig) { alloc_->kill_rank(rank, sig); }

 private:
  ProcMesh() = default;
  void pump_alloc_events();

  std::shared_ptr<Alloc> alloc_;
  std::string world_;
  size_t n_ = 0;
  std::shared_ptr<Router> router_;
  std::shared_ptr<Proc> client_;
  std::shared_ptr<Instance> client_inst_;
  std::shared_ptr<QueueSink> supervisor_q_;
  PortId supervisor_port_;
  std::mutex mu_;
  std::map<std::string, uint64_t> cast_seq_;
  std::deque<Event> events_;
  std::condition_variable ev_cv_;
  std::thread pump_thr_, alloc_thr_;
  std::atomic<bool> stopped_{false};
};

}  // namespace mb
