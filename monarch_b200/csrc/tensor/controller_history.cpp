#include "tensor/controller_history.h"

#include <algorithm>
#include <limits>

namespace mb {

ControllerHistory::ControllerHistory(int world)
    : world_(world), completed_((size_t)std::max(world, 0), -1) {}

int64_t ControllerHistory::next_seq() {
  std::lock_guard<std::mutex> g(mu_);
  return ++seq_;
}

int64_t ControllerHistory::next_ref() {
  std::lock_guard<std::mutex> g(mu_);
  return ++ref_;
}

uint32_t ControllerHistory::intern(const std::string& name) {
  auto it = name_ids_.find(name);
  if (it != name_ids_.end()) return it->second;
  const uint32_t id = (uint32_t)names_.size();
  names_.push_back(name);
  name_ids_.emplace(name, id);
  return id;
}

int64_t ControllerHistory::add_invocation(int64_t seq, const std::string& name,
                                          std::vector<int64_t> defs,
                                          const std::vector<int64_t>& uses) {
  std::lock_guard<std::mutex> g(mu_);
  Invocation inv;
  inv.seq = seq;
  inv.name_id = intern(name);
  inv.defs = std::move(defs);
  inv.uses = uses;
  if (!poisoned_.empty()) {
    for (int64_t u : uses) {
      auto p = poisoned_.find(u);
      if (p != poisoned_.end()) {
        inv.failed_by = p->second;
        break;
      }
    }
    if (inv.failed_by >= 0)
      for (int64_t d : inv.defs) poisoned_[d] = inv.failed_by;
  }
  const int64_t r = inv.failed_by;
  live_.push_back(std::move(inv));
  // without progress reports (watchdog off, simulated workers) nothing retires: keep the
  // table bounded by forgetting the oldest invocations
  while (live_.size() > kMaxLive) live_.pop_front();
  return r;
}

void ControllerHistory::rank_progress(int rank, int64_t last_seq) {
  std::lock_guard<std::mutex> g(mu_);
  if (rank < 0 || rank >= world_) return;
  if (last_seq > completed_[(size_t)rank]) completed_[(size_t)rank] = last_seq;
  retire_locked();
}

int64_t ControllerHistory::min_completed() const {
  std::lock_guard<std::mutex> g(mu_);
  int64_t m = std::numeric_limits<int64_t>::max();
  for (int64_t c : completed_) m = std::min(m, c);
  return completed_.empty() ? -1 : m;
}

size_t ControllerHistory::live_invocations() const {
  std::lock_guard<std::mutex> g(mu_);
  return live_.size();
}

void ControllerHistory::retire_locked() {
  int64_t m = std::numeric_limits<int64_t>::max();
  for (int64_t c : completed_) m = std::min(m, c);
  if (completed_.empty()) return;
  // an invocation that every rank has passed can no longer fail; what a failed one poisons
  // lives on in `poisoned_` until those refs are forgotten
  while (!live_.empty() && live_.front().seq <= m) live_.pop_front();
}

std::vector<int64_t> ControllerHistory::fail(int64_t seq, int64_t rank, const std::string& name,
                                             const std::string& text) {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<int64_t> dependents;
  if (!failures_.count(seq)) failures_[seq] = FailureInfo{seq, rank, name, text};
  // live_ is sorted by seq: find the invocation, poison what it defines, then walk forward
  auto it = std::lower_bound(live_.begin(), live_.end(), seq,
                             [](const Invocation& a, int64_t s) { return a.seq < s; });
  if (it == live_.end() || it->seq != seq) return dependents;   // retired: nothing live uses it
  if (it->failed_by < 0) it->failed_by = seq;
  const int64_t origin = it->failed_by;
  for (int64_t d : it->defs) poisoned_.emplace(d, origin);
  // invocations issued after it, before the failure was known: whoever read a poisoned ref
  // is poisoned too (one forward pass suffices: live_ is in issue order)
  for (++it; it != live_.end(); ++it) {
    if (it->failed_by >= 0) continue;
    bool hit = false;
    for (int64_t u : it->uses)
      if (poisoned_.count(u)) {
        hit = true;
        break;
      }
    if (!hit) continue;
    it->failed_by = origin;
    for (int64_t d : it->defs) poisoned_.emplace(d, origin);
    dependents.push_back(it->seq);
  }
  return dependents;
}

int64_t ControllerHistory::ref_failed(int64_t ref) const {
  std::lock_guard<std::mutex> g(mu_);
  auto p = poisoned_.find(ref);
  return p == poisoned_.end() ? -1 : p->second;
}

bool ControllerHistory::failure(int64_t seq, FailureInfo* out) const {
  std::lock_guard<std::mutex> g(mu_);
  auto f = failures_.find(seq);
  if (f == failures_.end()) return false;
  *out = f->second;
  return true;
}

void ControllerHistory::forget_refs(const std::vector<int64_t>& refs) {
  std::lock_guard<std::mutex> g(mu_);
  if (poisoned_.empty()) return;
  for (int64_t r : refs) poisoned_.erase(r);
}

bool ControllerHistory::describe(int64_t seq, std::string* name, int64_t* failed_by) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = std::lower_bound(live_.begin(), live_.end(), seq,
                             [](const Invocation& a, int64_t s) { return a.seq < s; });
  if (it == live_.end() || it->seq != seq) return false;
  *name = names_[it->name_id];
  *failed_by = it->failed_by;
  return true;
}

void ControllerHistory::ping_sent(int64_t ping_seq, double now) {
  std::lock_guard<std::mutex> g(mu_);
  ping_open_ = true;
  ping_reported_ = false;
  ping_seq_ = ping_seq;
  ping_t_ = now;
  ping_seen_.clear();
}

bool ControllerHistory::ping_outstanding() const {
  std::lock_guard<std::mutex> g(mu_);
  return ping_open_;
}

bool ControllerHistory::ping_answered(int rank, int64_t last_seq) {
  std::lock_guard<std::mutex> g(mu_);
  if (rank >= 0 && rank < world_) {
    if (last_seq > completed_[(size_t)rank]) completed_[(size_t)rank] = last_seq;
    retire_locked();
  }
  if (!ping_open_) return true;
  ping_seen_[rank] = last_seq;
  if ((int)ping_seen_.size() >= world_) {
    ping_open_ = false;
    return true;
  }
  return false;
}

bool ControllerHistory::stalled(double now, double timeout_s, StallReport* out) {
  std::lock_guard<std::mutex> g(mu_);
  if (!ping_open_ || ping_reported_ || now - ping_t_ <= timeout_s) return false;
  ping_reported_ = true;
  out->ranks.clear();
  for (int r = 0; r < world_; ++r)
    if (!ping_seen_.count(r)) out->ranks.push_back(r);
  out->waited_s = now - ping_t_;
  out->ping_seq = ping_seq_;
  out->last_seq_of_responders = ping_seen_;
  return true;
}

}  // namespace mb
