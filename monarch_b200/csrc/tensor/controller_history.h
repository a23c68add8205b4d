// Controller-side bookkeeping of the tensor engine: what was issued, how far every worker
// has come, which results are known to be poisoned.
//
// Parity: controller/src/history.rs (History / Invocation: dependents of a failed
// invocation inherit its failure; invocations retire once every rank has passed them) and
// controller/src/lib.rs:263-336 (CheckWorkerProgress: ranks that have not answered a ping
// within the operation timeout are reported as stuck).
#pragma once

#include <cstdint>
#include <deque>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

namespace mb {

struct Invocation {
  int64_t seq = 0;
  uint32_t name_id = 0;
  std::vector<int64_t> defs;   // refs the invocation defines (results and mutated arguments)
  std::vector<int64_t> uses;   // refs it reads
  int64_t failed_by = -1;      // seq of the failure this one carries (itself or inherited)
};

struct FailureInfo {
  int64_t seq = -1;            // the invocation that failed on its own
  int64_t rank = -1;
  std::string name, text;
};

struct StallReport {
  std::vector<int> ranks;      // ranks that did not answer the outstanding ping
  double waited_s = 0;
  int64_t ping_seq = 0;
  std::unordered_map<int, int64_t> last_seq_of_responders;
};

class ControllerHistory {
 public:
  explicit ControllerHistory(int world);

  int64_t next_seq();
  int64_t next_ref();
  int world() const { return world_; }

  // Record an invocation.  If one of `uses` is known to be poisoned the invocation (and the
  // refs it defines) inherit that failure; returns the seq of the original failure or -1.
  int64_t add_invocation(int64_t seq, const std::string& name, std::vector<int64_t> defs,
                         const std::vector<int64_t>& uses);
  // Rank `rank` has executed everything up to `last_seq`.
  void rank_progress(int rank, int64_t last_seq);
  int64_t min_completed() const;
  size_t live_invocations() const;

  // A worker reported that invocation `seq` failed on its own.  Marks it, and every later
  // invocation that used what it defines (transitively, in issue order).  Returns the seqs
  // of those dependents.
  std::vector<int64_t> fail(int64_t seq, int64_t rank, const std::string& name,
                            const std::string& text);
  // -1, or the seq of the original failure that poisons `ref`.
  int64_t ref_failed(int64_t ref) const;
  bool failure(int64_t seq, FailureInfo* out) const;
  void forget_refs(const std::vector<int64_t>& refs);
  // (name, failed_by) of a live invocation; false when it has retired or never existed.
  bool describe(int64_t seq, std::string* name, int64_t* failed_by) const;

  // -- progress watchdog --------------------------------------------------------------
  void ping_sent(int64_t ping_seq, double now);
  bool ping_outstanding() const;
  // True once every rank has answered the outstanding ping (which is then closed).
  bool ping_answered(int rank, int64_t last_seq);
  // Ranks that have not answered within `timeout_s`; reported once per ping.
  bool stalled(double now, double timeout_s, StallReport* out);

 private:
  uint32_t intern(const std::string& name);
  void retire_locked();

  static constexpr size_t kMaxLive = 1u << 20;
  const int world_;
  mutable std::mutex mu_;
  int64_t seq_ = 0, ref_ = 0;
  std::deque<Invocation> live_;                       // in issue order
  std::unordered_map<int64_t, int64_t> poisoned_;     // ref -> seq of the original failure
  std::unordered_map<int64_t, FailureInfo> failures_; // original failures by seq
  std::vector<int64_t> completed_;                    // per rank
  std::unordered_map<std::string, uint32_t> name_ids_;
  std::vector<std::string> names_;
  // outstanding ping
  bool ping_open_ = false, ping_reported_ = false;
  int64_t ping_seq_ = 0;
  double ping_t_ = 0;
  std::unordered_map<int, int64_t> ping_seen_;
};

}  // namespace mb
