// Identifiers and the wire codec of the actor runtime.
//
// Parity: hyperactor/src/reference.rs (WorldId/ProcId/ActorId/PortId and their text
// syntax `world[rank].actor[pid][port]`), hyperactor/src/data.rs (Serialized),
// serde_multipart (multi-part frames: a header part plus payload parts that are written
// with scatter-gather IO instead of being copied into one buffer).
#pragma once
#include <cstdint>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <string_view>
#include <vector>

namespace mb {

struct CodecError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

class Writer {
 public:
  std::string buf;
  void u8(uint8_t v) { buf.push_back((char)v); }
  void u32(uint32_t v) {
    char b[4];
    for (int i = 0; i < 4; ++i) b[i] = (char)(v >> (8 * i));
    buf.append(b, 4);
  }
  void u64(uint64_t v) {
    char b[8];
    for (int i = 0; i < 8; ++i) b[i] = (char)(v >> (8 * i));
    buf.append(b, 8);
  }
  void i64(int64_t v) { u64((uint64_t)v); }
  void str(std::string_view s) {
    u64(s.size());
    buf.append(s.data(), s.size());
  }
};

class Reader {
 public:
  explicit Reader(std::string_view d) : d_(d) {}
  uint8_t u8() {
    need(1);
    return (uint8_t)d_[pos_++];
  }
  uint32_t u32() {
    need(4);
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) v |= (uint32_t)(uint8_t)d_[pos_ + i] << (8 * i);
    pos_ += 4;
    return v;
  }
  uint64_t u64() {
    need(8);
    uint64_t v = 0;
    for (int i = 0; i < 8; ++i) v |= (uint64_t)(uint8_t)d_[pos_ + i] << (8 * i);
    pos_ += 8;
    return v;
  }
  int64_t i64() { return (int64_t)u64(); }
  std::string str() {
    uint64_t n = u64();
    need(n);
    std::string s(d_.substr(pos_, n));
    pos_ += n;
    return s;
  }
  bool done() const { return pos_ == d_.size(); }
  size_t pos() const { return pos_; }

 private:
  void need(uint64_t n) {
    if (pos_ + n > d_.size()) throw CodecError("truncated message");
  }
  std::string_view d_;
  size_t pos_ = 0;
};

struct ProcId {
  std::string world;
  int64_t rank = 0;
  std::string to_string() const { return world + "[" + std::to_string(rank) + "]"; }
  bool operator==(const ProcId& o) const { return world == o.world && rank == o.rank; }
  bool operator<(const ProcId& o) const {
    return world != o.world ? world < o.world : rank < o.rank;
  }
  static ProcId parse(const std::string& s);
};

struct ActorId {
  ProcId proc;
  std::string name;
  int64_t pid = 0;
  std::string to_string() const {
    return proc.to_string() + "." + name + "[" + std::to_string(pid) + "]";
  }
  bool operator==(const ActorId& o) const {
    return proc == o.proc && name == o.name && pid == o.pid;
  }
  bool operator<(const ActorId& o) const {
    if (!(proc == o.proc)) return proc < o.proc;
    if (name != o.name) return name < o.name;
    return pid < o.pid;
  }
  static ActorId parse(const std::string& s);
};

struct PortId {
  ActorId actor;
  uint64_t port = 0;
  std::string to_string() const { return actor.to_string() + "[" + std::to_string(port) + "]"; }
  bool operator==(const PortId& o) const { return actor == o.actor && port == o.port; }
  static PortId parse(const std::string& s);
};

// Well-known ports of every actor.
enum : uint64_t {
  kPortMessage = 0,        // the actor's handler port
  kPortSignal = 1,         // Stop / DrainAndStop
  kPortSupervision = 2,    // ActorSupervisionEvent from children
  kPortUndeliverable = 3,  // returned envelopes
  kPortUserBase = 1024,
};

inline void write_proc(Writer& w, const ProcId& p) {
  w.str(p.world);
  w.i64(p.rank);
}
inline ProcId read_proc(Reader& r) {
  ProcId p;
  p.world = r.str();
  p.rank = r.i64();
  return p;
}
inline void write_actor(Writer& w, const ActorId& a) {
  write_proc(w, a.proc);
  w.str(a.name);
  w.i64(a.pid);
}
inline ActorId read_actor(Reader& r) {
  ActorId a;
  a.proc = read_proc(r);
  a.name = r.str();
  a.pid = r.i64();
  return a;
}
inline void write_port(Writer& w, const PortId& p) {
  write_actor(w, p.actor);
  w.u64(p.port);
}
inline PortId read_port(Reader& r) {
  PortId p;
  p.actor = read_actor(r);
  p.port = r.u64();
  return p;
}

// A message in flight.  `data` is the body; `parts` are large out-of-band blobs
// (pickled tensors and the like) that travel as separate iovecs of the same frame.
struct Envelope {
  ActorId sender;
  PortId dest;
  std::map<std::string, std::string> headers;
  std::string data;
  std::vector<std::string> parts;

  // Header part only (ids, headers, sizes); body and parts follow it on the wire.
  std::string encode_head() const;
  std::string encode() const;  // contiguous form (head + data + parts)
  static Envelope decode(std::string_view bytes);
};

// Header keys used by casts (hyperactor_mesh/src/comm/multicast.rs CAST_* headers).
constexpr const char* kHdrCastRank = "cast_rank";
constexpr const char* kHdrCastShape = "cast_shape";
constexpr const char* kHdrCastSender = "cast_originating_sender";
constexpr const char* kHdrCastMesh = "cast_actor_mesh_id";
constexpr const char* kHdrKind = "kind";
// Tree reduction of replies to a cast (the reference's split ports with a reducer): the cast
// names a built-in reducer and the final accumulating port; every comm actor folds the
// partial results of its subtree and passes one message up.
constexpr const char* kHdrReduceTree = "reduce_tree";    // reducer name, on the cast
constexpr const char* kHdrReducePort = "reduce_port";    // final port, on the cast
constexpr const char* kHdrReduceVia = "reduce_via";      // local comm actor, on the delivery
constexpr const char* kHdrReduceKey = "reduce_key";      // identifies the cast
constexpr const char* kHdrReduceCount = "n";             // contributions folded into a part

}  // namespace mb
