// One-way, ordered, reliable message channels.
//
// Parity: hyperactor/src/channel.rs (ChannelAddr syntax `tcp:host:port`, `unix:/path`,
// `local:n`; `dial` / `serve`; Tx/Rx), channel/net.rs (frames = 8-byte big-endian length +
// payload; Init / Message(seq) frames; Ack responses; outbox + unacked queue; reconnect
// with exponential backoff; delivery timeout after which messages are returned),
// channel/local.rs (in-process transport), channel/sim.rs + simnet.rs (`sim:` addresses:
// in-process delivery after a simulated network latency, see SimNet below).
//
// Design: one sender thread per dialled channel (owns the socket, the outbox and the
// unacked queue) and one reader thread per accepted connection.  A multi-part message
// (head + parts) is written with a single writev so large payloads are never copied into
// a contiguous frame.
#pragma once
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <mutex>
#include <optional>
#include <string>
#include <thread>
#include <vector>

namespace mb {

struct ChannelAddr {
  enum Kind { Tcp, Unix, Local, Sim } kind = Local;
  std::string host;  // tcp
  int port = 0;      // tcp (0 = any)
  std::string path;  // unix ("" = any: an abstract/temporary path is chosen)
  uint64_t id = 0;   // local, sim (0 = any)
  // sim: `sim:<node>/<id>`; a dialled address may name the sender's node as well,
  // `sim:<src>-><node>/<id>` -- the latency of a frame depends on both.  Nodes are dotted
  // paths ("dc0.rack1.host3"); the distance of two nodes is the number of trailing
  // components in which they differ.
  std::string node, src_node;

  static ChannelAddr parse(const std::string& s);
  static ChannelAddr any(Kind k);
  std::string to_string() const;
  bool operator==(const ChannelAddr& o) const { return to_string() == o.to_string(); }
};

struct ChannelError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

// A message: `head` plus optional out-of-band parts, delivered as one unit.
struct Frame {
  std::string head;
  std::vector<std::string> parts;
  size_t size() const {
    size_t n = head.size();
    for (auto& p : parts) n += p.size();
    return n;
  }
};

enum class TxStatus { Active, Closed };

class Tx {
 public:
  virtual ~Tx() = default;
  // Queue a frame.  `on_undeliverable` (may be empty) is invoked with the frame if it
  // could not be delivered within the delivery timeout or the channel is closed.
  virtual void post(Frame f, std::function<void(Frame&&)> on_undeliverable = {}) = 0;
  virtual TxStatus status() const = 0;
  virtual ChannelAddr addr() const = 0;
  virtual void close() = 0;
};

class Rx {
 public:
  virtual ~Rx() = default;
  // Blocks up to `timeout_ms` (<0: forever).  nullopt on timeout or when closed.
  virtual std::optional<Frame> recv(int64_t timeout_ms = -1) = 0;
  virtual ChannelAddr addr() const = 0;
  virtual void close() = 0;
  virtual bool closed() const = 0;
};

std::shared_ptr<Rx> serve(const ChannelAddr& addr);
std::shared_ptr<Tx> dial(const ChannelAddr& addr);

// Simulated network behind `sim:` channels: every frame is delivered after
//   latency_us[distance(src, dst)] + bytes / bandwidth
// in simulated time.  While the telemetry sim clock is in use (use_sim_clock) the scheduler
// jumps the clock to each delivery's time, so a run costs no wall-clock waiting and the
// clock reads the critical-path latency of what was sent; with the real clock, deliveries
// are delayed in real time.  Frames of one channel stay in order.
struct SimNetStats {
  uint64_t frames = 0, bytes = 0;
  double latency_us_total = 0;   // sum of the simulated latencies of all delivered frames
  uint64_t by_distance[8] = {0, 0, 0, 0, 0, 0, 0, 0};
};
void simnet_configure(const std::vector<double>& latency_us_by_distance, double bandwidth_gbs);
SimNetStats simnet_stats();
void simnet_reset_stats();
int simnet_distance(const std::string& a, const std::string& b);

// Counters for tests / metrics (process-wide).
struct ChannelStats {
  std::atomic<uint64_t> connects{0}, reconnects{0}, frames_sent{0}, frames_resent{0},
      frames_received{0}, duplicates_dropped{0}, acks_sent{0}, undeliverable{0};
};
ChannelStats& channel_stats();

// Test hook: forcibly drop every live connection of dialled channels to `addr` (the
// senders reconnect and resend what was not acknowledged).
void debug_drop_connections(const ChannelAddr& addr);

}  // namespace mb
