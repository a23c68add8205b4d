#include "actor/durable.h"

#include <fcntl.h>
#include <unistd.h>

#include <chrono>
#include <cstring>
#include <stdexcept>

namespace mb {

namespace {
uint32_t checksum(const std::string& s) {  // FNV-1a
  uint32_t h = 2166136261u;
  for (unsigned char c : s) {
    h ^= c;
    h *= 16777619u;
  }
  return h;
}
bool read_exact(std::FILE* f, void* p, size_t n) { return std::fread(p, 1, n, f) == n; }
}  // namespace

MessageLog::MessageLog(const std::string& path) : path_(path) {
  // scan what is there, remember where the last complete record ends
  long good_end = 0;
  if (std::FILE* r = std::fopen(path.c_str(), "rb")) {
    for (;;) {
      uint64_t seq;
      uint32_t len, sum;
      if (!read_exact(r, &seq, 8) || !read_exact(r, &len, 4)) break;
      if (len > (1u << 30)) break;
      std::string body(len, '\0');
      if (!read_exact(r, body.data(), len) || !read_exact(r, &sum, 4)) break;
      if (sum != checksum(body)) break;
      next_seq_ = seq + 1;
      good_end = std::ftell(r);
    }
    std::fclose(r);
    if (::truncate(path.c_str(), good_end) != 0) {
      // a torn tail that cannot be cut off would corrupt later appends
      throw std::runtime_error("message log: cannot truncate " + path);
    }
  }
  f_ = std::fopen(path.c_str(), "ab");
  if (!f_) throw std::runtime_error("message log: cannot open " + path);
}

MessageLog::~MessageLog() {
  if (f_) std::fclose(f_);
}

uint64_t MessageLog::append(const Envelope& env) {
  std::string body = env.encode();
  std::lock_guard<std::mutex> g(mu_);
  uint64_t seq = next_seq_;
  uint32_t len = (uint32_t)body.size(), sum = checksum(body);
  if (std::fwrite(&seq, 8, 1, f_) != 1 || std::fwrite(&len, 4, 1, f_) != 1 ||
      (len && std::fwrite(body.data(), 1, len, f_) != len) || std::fwrite(&sum, 4, 1, f_) != 1)
    throw std::runtime_error("message log: write failed on " + path_);
  ++next_seq_;
  return seq;
}

void MessageLog::flush() {
  std::lock_guard<std::mutex> g(mu_);
  if (std::fflush(f_) != 0 || ::fsync(::fileno(f_)) != 0)
    throw std::runtime_error("message log: flush failed on " + path_);
}

std::vector<std::pair<uint64_t, Envelope>> MessageLog::read(uint64_t from) const {
  std::vector<std::pair<uint64_t, Envelope>> out;
  {
    std::lock_guard<std::mutex> g(mu_);
    std::fflush(f_);
  }
  std::FILE* r = std::fopen(path_.c_str(), "rb");
  if (!r) return out;
  for (;;) {
    uint64_t seq;
    uint32_t len, sum;
    if (!read_exact(r, &seq, 8) || !read_exact(r, &len, 4)) break;
    if (len > (1u << 30)) break;
    std::string body(len, '\0');
    if (!read_exact(r, body.data(), len) || !read_exact(r, &sum, 4)) break;
    if (sum != checksum(body)) break;
    if (seq >= from) out.emplace_back(seq, Envelope::decode(body));
  }
  std::fclose(r);
  return out;
}

void DurableMailboxSender::post(Envelope env) {
  std::lock_guard<std::mutex> g(mu_);
  try {
    log_->append(env);
    log_->flush();
  } catch (const std::exception& e) {
    if (on_failed_) on_failed_(std::move(env), std::string("durable sender: ") + e.what());
    return;
  }
  inner_->post(std::move(env));
}

size_t DurableMailboxSender::replay(uint64_t from) {
  std::lock_guard<std::mutex> g(mu_);
  auto records = log_->read(from);
  for (auto& r : records) inner_->post(std::move(r.second));
  return records.size();
}

void write_checkpoint(const std::string& path, const std::string& blob) {
  std::string tmp = path + ".tmp." + std::to_string((long)getpid());
  std::FILE* f = std::fopen(tmp.c_str(), "wb");
  if (!f) throw std::runtime_error("checkpoint: cannot open " + tmp);
  bool ok = blob.empty() || std::fwrite(blob.data(), 1, blob.size(), f) == blob.size();
  ok = ok && std::fflush(f) == 0 && ::fsync(::fileno(f)) == 0;
  std::fclose(f);
  if (!ok || ::rename(tmp.c_str(), path.c_str()) != 0) {
    ::unlink(tmp.c_str());
    throw std::runtime_error("checkpoint: cannot write " + path);
  }
}

bool read_checkpoint(const std::string& path, std::string* blob) {
  std::FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) return false;
  blob->clear();
  char buf[1 << 16];
  size_t n;
  while ((n = std::fread(buf, 1, sizeof(buf), f)) > 0) blob->append(buf, n);
  std::fclose(f);
  return true;
}

// ---------------------------------------------------------------- PreemptibleRwLock --
PreemptibleRwLock::ReadGuard PreemptibleRwLock::read() {
  std::unique_lock<std::mutex> g(mu_);
  cv_.wait(g, [&] { return !writer_ && writers_waiting_ == 0; });
  ++readers_;
  return ReadGuard(this);
}

bool PreemptibleRwLock::try_read_for(int64_t timeout_ms, std::unique_ptr<ReadGuard>* out) {
  std::unique_lock<std::mutex> g(mu_);
  auto ready = [&] { return !writer_ && writers_waiting_ == 0; };
  if (timeout_ms < 0)
    cv_.wait(g, ready);
  else if (!cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), ready))
    return false;
  ++readers_;
  out->reset(new ReadGuard(this));
  return true;
}

PreemptibleRwLock::WriteGuard PreemptibleRwLock::write() {
  std::unique_lock<std::mutex> g(mu_);
  ++writers_waiting_;  // from here on readers see preempted() == true
  cv_.wait(g, [&] { return !writer_ && readers_ == 0; });
  --writers_waiting_;
  writer_ = true;
  return WriteGuard(this);
}

void PreemptibleRwLock::ReadGuard::release() {
  if (!l_) return;
  {
    std::lock_guard<std::mutex> g(l_->mu_);
    --l_->readers_;
  }
  l_->cv_.notify_all();
  l_ = nullptr;
}

void PreemptibleRwLock::WriteGuard::release() {
  if (!l_) return;
  {
    std::lock_guard<std::mutex> g(l_->mu_);
    l_->writer_ = false;
  }
  l_->cv_.notify_all();
  l_ = nullptr;
}

int PreemptibleRwLock::readers() const {
  std::lock_guard<std::mutex> g(mu_);
  return readers_;
}
int PreemptibleRwLock::writers_waiting() const {
  std::lock_guard<std::mutex> g(mu_);
  return writers_waiting_;
}

}  // namespace mb
