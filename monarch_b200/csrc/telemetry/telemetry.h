// Configuration registry, logging, metrics, flight recorder and chrome-trace writer.
//
// Parity: hyperactor/src/config.rs + attrs.rs (typed keys with defaults, HYPERACTOR_*
// environment overrides, scoped overrides for tests), hyperactor_telemetry (glog-style
// file + stderr logs with MONARCH_FILE_LOG / MONARCH_STDERR_LOG levels, static
// counters/gauges/histograms, per-actor in-memory flight recorder),
// monarch_perfetto_trace (trace-event output; here chrome-trace JSON).
#pragma once
#include <atomic>
#include <chrono>
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace mb {

// ------------------------------------------------------------------------- config --
class Config {
 public:
  static Config& global();
  // Keys are upper-case (e.g. "MESSAGE_DELIVERY_TIMEOUT_MS").  Lookup order: scoped
  // override, explicit set(), environment HYPERACTOR_<KEY> then MONARCH_<KEY>, default.
  std::string get(const std::string& key) const;
  int64_t get_int(const std::string& key) const;
  double get_float(const std::string& key) const;
  bool get_bool(const std::string& key) const;
  void set(const std::string& key, const std::string& value);
  void unset(const std::string& key);
  // Returns the previous explicit value ("" + false if none) so a scope can restore it.
  std::pair<std::string, bool> override_key(const std::string& key, const std::string& value);
  std::map<std::string, std::string> snapshot() const;  // effective values of known keys
  std::string to_yaml() const;
  void load_yaml(const std::string& text);

 private:
  Config();
  mutable std::mutex mu_;
  std::map<std::string, std::string> defaults_;
  std::map<std::string, std::string> values_;
};

// ------------------------------------------------------------------------ logging --
enum class LogLevel { Trace = 0, Debug = 1, Info = 2, Warn = 3, Error = 4, Off = 5 };
LogLevel parse_level(const std::string& s, LogLevel dflt);
void log_init();  // idempotent; reads MONARCH_FILE_LOG / MONARCH_STDERR_LOG
void log_write(LogLevel lvl, const char* file, int line, const std::string& msg);
bool log_enabled(LogLevel lvl);
std::string log_file_path();

#define MB_LOG(lvl, msg)                                                  \
  do {                                                                    \
    if (::mb::log_enabled(::mb::LogLevel::lvl))                           \
      ::mb::log_write(::mb::LogLevel::lvl, __FILE__, __LINE__, (msg));    \
  } while (0)

// ------------------------------------------------------------------------ metrics --
class Metrics {
 public:
  static Metrics& global();
  void counter_add(const std::string& name, int64_t v = 1);
  void gauge_set(const std::string& name, double v);
  void histogram_record(const std::string& name, double v);
  int64_t counter(const std::string& name) const;
  double gauge(const std::string& name) const;
  struct Hist {
    uint64_t count = 0;
    double sum = 0, min = 0, max = 0;
    std::vector<double> recent;  // up to 1024 most recent samples for percentiles
  };
  Hist histogram(const std::string& name) const;
  std::map<std::string, double> snapshot() const;
  void reset();

 private:
  mutable std::mutex mu_;
  std::map<std::string, int64_t> counters_;
  std::map<std::string, double> gauges_;
  std::map<std::string, Hist> hists_;
};

struct ScopedTimer {
  std::string name;
  std::chrono::steady_clock::time_point t0 = std::chrono::steady_clock::now();
  explicit ScopedTimer(std::string n) : name(std::move(n)) {}
  ~ScopedTimer() {
    Metrics::global().histogram_record(
        name, std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0)
                  .count());
  }
};

// ---------------------------------------------------------------- flight recorder --
struct RecordedEvent {
  double t_us;
  std::string name;
  std::string detail;
};
class Recorder {
 public:
  explicit Recorder(size_t capacity = 128) : cap_(capacity) {}
  void record(std::string name, std::string detail = "");
  std::vector<RecordedEvent> tail(size_t n = 0) const;

 private:
  size_t cap_;
  mutable std::mutex mu_;
  std::deque<RecordedEvent> q_;
};

// ------------------------------------------------------------------- chrome trace --
class TraceWriter {
 public:
  static TraceWriter& global();
  void enable(bool on) { enabled_ = on; }
  bool enabled() const { return enabled_; }
  void complete(const std::string& name, const std::string& cat, double ts_us, double dur_us,
                int64_t pid, int64_t tid, const std::string& args_json = "");
  void instant(const std::string& name, const std::string& cat, double ts_us, int64_t pid,
               int64_t tid);
  void counter(const std::string& name, double ts_us, int64_t pid, double value);
  std::string to_json() const;
  void clear();

 private:
  std::atomic<bool> enabled_{false};
  mutable std::mutex mu_;
  std::vector<std::string> events_;
};

double now_us();

// ------------------------------------------------------------ spans + event capture --
// Parity: hyperactor_telemetry spans (PySpan, get_current_span_id), the sqlite layer's
// event capture (sqlite.rs: log events and span lifecycles as rows) and the real/sim clock
// switch.  Capture is off until a reader turns it on; a reader drains the rows and stores
// them where it likes (the Python side writes them into a sqlite database).
struct CollectedEvent {
  std::string kind;      // "event" | "span_enter" | "span_exit"
  double t_us = 0;       // telemetry clock (wall time since the epoch, or the sim clock)
  int level = 2;         // LogLevel of an event
  std::string file;
  int line = 0;
  std::string message;   // event text, or span name
  std::string actor_id;
  uint64_t span_id = 0;  // the span itself, or the span an event happened in
  uint64_t parent_id = 0;
  uint64_t thread = 0;
};
class EventCollector {
 public:
  static EventCollector& global();
  void enable(bool on);
  bool enabled() const { return enabled_; }
  void push(CollectedEvent&& e);
  std::vector<CollectedEvent> drain();
  uint64_t dropped() const { return dropped_; }

 private:
  std::atomic<bool> enabled_{false};
  std::atomic<uint64_t> dropped_{0};
  std::mutex mu_;
  std::vector<CollectedEvent> q_;
  static constexpr size_t kMax = 1 << 18;
};
uint64_t span_enter(const std::string& name, const std::string& actor_id = "");
void span_exit(uint64_t id);
uint64_t current_span_id();
// Telemetry timestamps: wall clock by default, a manually advanced clock in simulations.
void use_sim_clock();
void use_real_clock();
void sim_clock_advance_us(double us);
bool sim_clock_in_use();
double telemetry_now_us();
const std::string& execution_id();

}  // namespace mb
