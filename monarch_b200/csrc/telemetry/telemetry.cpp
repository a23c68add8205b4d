#include "telemetry/telemetry.h"

#include <sys/stat.h>
#include <sys/types.h>
#include <unistd.h>

#include <algorithm>
#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <ctime>
#include <sstream>

namespace mb {

double now_us() {
  return std::chrono::duration<double, std::micro>(
             std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

// ------------------------------------------------------------------------- config --
Config::Config() {
  defaults_ = {
      {"CODEC_MAX_FRAME_LENGTH", "1073741824"},
      {"MESSAGE_DELIVERY_TIMEOUT_MS", "30000"},
      {"PROCESS_EXIT_TIMEOUT_MS", "10000"},
      {"MESSAGE_ACK_TIME_INTERVAL_MS", "500"},
      {"MESSAGE_ACK_EVERY_N_MESSAGES", "1000"},
      {"SPLIT_MAX_BUFFER_SIZE", "5"},
      {"STOP_ACTOR_TIMEOUT_MS", "1000"},
      {"REMOTE_ALLOCATOR_HEARTBEAT_INTERVAL_MS", "5000"},
      {"BOOTSTRAP_HEARTBEAT_INTERVAL_MS", "5000"},
      {"CASTING_FANOUT_SIZE", "8"},
      {"CHANNEL_MULTIPART", "true"},
      {"CHANNEL_RECONNECT_BACKOFF_MIN_MS", "10"},
      {"CHANNEL_RECONNECT_BACKOFF_MAX_MS", "1000"},
      {"SHARED_ASYNCIO_RUNTIME", "false"},
      {"KERNEL_SPIN_BUDGET_MS", "1500"},
      {"DDP_BUCKET_BYTES", "26214400"},
      {"NVLS_ENABLE", "true"},
      {"COMM_ACTOR_INLINE", "true"},
  };
}
Config& Config::global() {
  static Config c;
  return c;
}
std::string Config::get(const std::string& key) const {
  {
    std::lock_guard<std::mutex> g(mu_);
    auto it = values_.find(key);
    if (it != values_.end()) return it->second;
  }
  for (const char* prefix : {"HYPERACTOR_", "MONARCH_"}) {
    if (const char* e = std::getenv((std::string(prefix) + key).c_str())) return e;
  }
  std::lock_guard<std::mutex> g(mu_);
  auto it = defaults_.find(key);
  return it == defaults_.end() ? std::string() : it->second;
}
int64_t Config::get_int(const std::string& key) const {
  std::string v = get(key);
  return v.empty() ? 0 : std::stoll(v);
}
double Config::get_float(const std::string& key) const {
  std::string v = get(key);
  return v.empty() ? 0.0 : std::stod(v);
}
bool Config::get_bool(const std::string& key) const {
  std::string v = get(key);
  std::transform(v.begin(), v.end(), v.begin(), [](unsigned char c) { return std::tolower(c); });
  return v == "1" || v == "true" || v == "yes" || v == "on";
}
void Config::set(const std::string& key, const std::string& value) {
  std::lock_guard<std::mutex> g(mu_);
  values_[key] = value;
}
void Config::unset(const std::string& key) {
  std::lock_guard<std::mutex> g(mu_);
  values_.erase(key);
}
std::pair<std::string, bool> Config::override_key(const std::string& key,
                                                  const std::string& value) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = values_.find(key);
  std::pair<std::string, bool> prev{"", false};
  if (it != values_.end()) prev = {it->second, true};
  values_[key] = value;
  return prev;
}
std::map<std::string, std::string> Config::snapshot() const {
  std::map<std::string, std::string> keys;
  {
    std::lock_guard<std::mutex> g(mu_);
    keys = defaults_;
    for (auto& kv : values_) keys[kv.first] = kv.second;
  }
  for (auto& kv : keys) kv.second = get(kv.first);
  return keys;
}
std::string Config::to_yaml() const {
  std::ostringstream os;
  for (auto& kv : snapshot()) os << kv.first << ": " << kv.second << "\n";
  return os.str();
}
void Config::load_yaml(const std::string& text) {
  std::istringstream is(text);
  std::string line;
  while (std::getline(is, line)) {
    auto c = line.find(':');
    if (c == std::string::npos || line[0] == '#') continue;
    auto trim = [](std::string s) {
      size_t a = s.find_first_not_of(" \t\r\"'"), b = s.find_last_not_of(" \t\r\"'");
      return a == std::string::npos ? std::string() : s.substr(a, b - a + 1);
    };
    std::string k = trim(line.substr(0, c)), v = trim(line.substr(c + 1));
    if (!k.empty()) set(k, v);
  }
}

// ------------------------------------------------------------------------ logging --
namespace {
struct LogState {
  std::mutex mu;
  bool inited = false;
  LogLevel file_level = LogLevel::Info, stderr_level = LogLevel::Warn;
  FILE* file = nullptr;
  std::string path;
};
LogState& ls() {
  static LogState s;
  return s;
}
}  // namespace

LogLevel parse_level(const std::string& s, LogLevel dflt) {
  std::string v = s;
  std::transform(v.begin(), v.end(), v.begin(), [](unsigned char c) { return std::tolower(c); });
  if (v == "trace") return LogLevel::Trace;
  if (v == "debug") return LogLevel::Debug;
  if (v == "info") return LogLevel::Info;
  if (v == "warn" || v == "warning") return LogLevel::Warn;
  if (v == "error") return LogLevel::Error;
  if (v == "off" || v == "none") return LogLevel::Off;
  return dflt;
}

void log_init() {
  LogState& s = ls();
  std::lock_guard<std::mutex> g(s.mu);
  if (s.inited) return;
  s.inited = true;
  if (const char* e = std::getenv("MONARCH_FILE_LOG")) s.file_level = parse_level(e, LogLevel::Info);
  if (const char* e = std::getenv("MONARCH_STDERR_LOG"))
    s.stderr_level = parse_level(e, LogLevel::Warn);
  if (s.file_level != LogLevel::Off) {
    const char* user = std::getenv("USER");
    std::string dir = std::string("/tmp/") + (user ? user : "monarch");
    ::mkdir(dir.c_str(), 0755);
    s.path = dir + "/monarch_log.log";
    s.file = std::fopen(s.path.c_str(), "a");
  }
}
bool log_enabled(LogLevel lvl) {
  LogState& s = ls();
  if (!s.inited) log_init();
  return lvl >= s.file_level || lvl >= s.stderr_level ||
         (lvl >= LogLevel::Debug && EventCollector::global().enabled());
}
std::string log_file_path() {
  log_init();
  return ls().path;
}
void log_write(LogLevel lvl, const char* file, int line, const std::string& msg) {
  LogState& s = ls();
  if (!s.inited) log_init();
  static const char tag[] = {'T', 'D', 'I', 'W', 'E', 'O'};
  auto now = std::chrono::system_clock::now();
  std::time_t t = std::chrono::system_clock::to_time_t(now);
  auto us = std::chrono::duration_cast<std::chrono::microseconds>(now.time_since_epoch()).count() %
            1000000;
  std::tm tmv;
  localtime_r(&t, &tmv);
  char head[96];
  const char* base = std::strrchr(file, '/');
  std::snprintf(head, sizeof(head), "%c%02d%02d %02d:%02d:%02d.%06ld %d %s:%d] ", tag[(int)lvl],
                tmv.tm_mon + 1, tmv.tm_mday, tmv.tm_hour, tmv.tm_min, tmv.tm_sec, (long)us,
                (int)getpid(), base ? base + 1 : file, line);
  if (EventCollector::global().enabled()) {
    CollectedEvent ev;
    ev.kind = "event";
    ev.t_us = telemetry_now_us();
    ev.level = (int)lvl;
    ev.file = base ? base + 1 : file;
    ev.line = line;
    ev.message = msg;
    ev.span_id = current_span_id();
    EventCollector::global().push(std::move(ev));
  }
  std::lock_guard<std::mutex> g(s.mu);
  if (s.file && lvl >= s.file_level) {
    std::fputs(head, s.file);
    std::fputs(msg.c_str(), s.file);
    std::fputc('\n', s.file);
    std::fflush(s.file);
  }
  if (lvl >= s.stderr_level) {
    std::fputs(head, stderr);
    std::fputs(msg.c_str(), stderr);
    std::fputc('\n', stderr);
  }
}

// ------------------------------------------------------------------------ metrics --
Metrics& Metrics::global() {
  static Metrics m;
  return m;
}
void Metrics::counter_add(const std::string& name, int64_t v) {
  std::lock_guard<std::mutex> g(mu_);
  counters_[name] += v;
}
void Metrics::gauge_set(const std::string& name, double v) {
  std::lock_guard<std::mutex> g(mu_);
  gauges_[name] = v;
}
void Metrics::histogram_record(const std::string& name, double v) {
  std::lock_guard<std::mutex> g(mu_);
  Hist& h = hists_[name];
  if (h.count == 0) h.min = h.max = v;
  h.count++;
  h.sum += v;
  h.min = std::min(h.min, v);
  h.max = std::max(h.max, v);
  if (h.recent.size() >= 1024) h.recent.erase(h.recent.begin());
  h.recent.push_back(v);
}
int64_t Metrics::counter(const std::string& name) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = counters_.find(name);
  return it == counters_.end() ? 0 : it->second;
}
double Metrics::gauge(const std::string& name) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = gauges_.find(name);
  return it == gauges_.end() ? 0 : it->second;
}
Metrics::Hist Metrics::histogram(const std::string& name) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = hists_.find(name);
  return it == hists_.end() ? Hist{} : it->second;
}
std::map<std::string, double> Metrics::snapshot() const {
  std::lock_guard<std::mutex> g(mu_);
  std::map<std::string, double> out;
  for (auto& kv : counters_) out[kv.first] = (double)kv.second;
  for (auto& kv : gauges_) out[kv.first] = kv.second;
  for (auto& kv : hists_) {
    out[kv.first + ".count"] = (double)kv.second.count;
    out[kv.first + ".sum"] = kv.second.sum;
    out[kv.first + ".max"] = kv.second.max;
  }
  return out;
}
void Metrics::reset() {
  std::lock_guard<std::mutex> g(mu_);
  counters_.clear();
  gauges_.clear();
  hists_.clear();
}

// ----------------------------------------------------------------------- recorder --
void Recorder::record(std::string name, std::string detail) {
  std::lock_guard<std::mutex> g(mu_);
  if (q_.size() >= cap_) q_.pop_front();
  q_.push_back(RecordedEvent{now_us(), std::move(name), std::move(detail)});
}
std::vector<RecordedEvent> Recorder::tail(size_t n) const {
  std::lock_guard<std::mutex> g(mu_);
  size_t k = (n == 0 || n > q_.size()) ? q_.size() : n;
  return std::vector<RecordedEvent>(q_.end() - k, q_.end());
}

// -------------------------------------------------------------------------- trace --
TraceWriter& TraceWriter::global() {
  static TraceWriter t;
  return t;
}
static std::string jesc(const std::string& s) {
  std::string o;
  for (char c : s) {
    if (c == '"' || c == '\\') {
      o.push_back('\\');
      o.push_back(c);
    } else if (c == '\n') {
      o += "\\n";
    } else {
      o.push_back(c);
    }
  }
  return o;
}
void TraceWriter::complete(const std::string& name, const std::string& cat, double ts_us,
                           double dur_us, int64_t pid, int64_t tid, const std::string& args_json) {
  if (!enabled_) return;
  std::ostringstream os;
  os << "{\"name\":\"" << jesc(name) << "\",\"cat\":\"" << jesc(cat) << "\",\"ph\":\"X\",\"ts\":"
     << ts_us << ",\"dur\":" << dur_us << ",\"pid\":" << pid << ",\"tid\":" << tid;
  if (!args_json.empty()) os << ",\"args\":" << args_json;
  os << "}";
  std::lock_guard<std::mutex> g(mu_);
  events_.push_back(os.str());
}
void TraceWriter::instant(const std::string& name, const std::string& cat, double ts_us,
                          int64_t pid, int64_t tid) {
  if (!enabled_) return;
  std::ostringstream os;
  os << "{\"name\":\"" << jesc(name) << "\",\"cat\":\"" << jesc(cat)
     << "\",\"ph\":\"i\",\"s\":\"t\",\"ts\":" << ts_us << ",\"pid\":" << pid << ",\"tid\":" << tid
     << "}";
  std::lock_guard<std::mutex> g(mu_);
  events_.push_back(os.str());
}
void TraceWriter::counter(const std::string& name, double ts_us, int64_t pid, double value) {
  if (!enabled_) return;
  std::ostringstream os;
  os << "{\"name\":\"" << jesc(name) << "\",\"ph\":\"C\",\"ts\":" << ts_us << ",\"pid\":" << pid
     << ",\"args\":{\"value\":" << value << "}}";
  std::lock_guard<std::mutex> g(mu_);
  events_.push_back(os.str());
}
std::string TraceWriter::to_json() const {
  std::lock_guard<std::mutex> g(mu_);
  std::string out = "{\"traceEvents\":[";
  for (size_t i = 0; i < events_.size(); ++i) {
    if (i) out += ",";
    out += events_[i];
  }
  out += "]}";
  return out;
}
void TraceWriter::clear() {
  std::lock_guard<std::mutex> g(mu_);
  events_.clear();
}

// ------------------------------------------------------------ spans + event capture --
namespace {
struct SimClock {
  std::atomic<bool> on{false};
  std::mutex mu;
  double t_us = 0;
};
SimClock& sim_clock() {
  static SimClock c;
  return c;
}
struct OpenSpan {
  uint64_t id;
  std::string name;
  double t0_us;      // telemetry clock
  double t0_mono_us;  // steady clock, for the trace writer
};
thread_local std::vector<OpenSpan> tl_spans;
std::atomic<uint64_t> g_next_span{1};
uint64_t thread_tag() {
  static std::atomic<uint64_t> next{1};
  thread_local uint64_t mine = next.fetch_add(1);
  return mine;
}
}  // namespace

void use_sim_clock() { sim_clock().on = true; }
void use_real_clock() { sim_clock().on = false; }
bool sim_clock_in_use() { return sim_clock().on; }
void sim_clock_advance_us(double us) {
  std::lock_guard<std::mutex> g(sim_clock().mu);
  sim_clock().t_us += us;
}
double telemetry_now_us() {
  SimClock& c = sim_clock();
  if (c.on) {
    std::lock_guard<std::mutex> g(c.mu);
    return c.t_us;
  }
  return std::chrono::duration<double, std::micro>(
             std::chrono::system_clock::now().time_since_epoch())
      .count();
}

const std::string& execution_id() {
  static const std::string id = [] {
    for (const char* k : {"HYPERACTOR_EXECUTION_ID", "MONARCH_EXECUTION_ID"})
      if (const char* e = std::getenv(k))
        if (*e) return std::string(e);
    char buf[64];
    std::snprintf(buf, sizeof(buf), "exec_%ld_%d", (long)std::time(nullptr), (int)getpid());
    return std::string(buf);
  }();
  return id;
}

EventCollector& EventCollector::global() {
  static EventCollector c;
  return c;
}
void EventCollector::enable(bool on) { enabled_ = on; }
void EventCollector::push(CollectedEvent&& e) {
  e.thread = thread_tag();
  std::lock_guard<std::mutex> g(mu_);
  if (q_.size() >= kMax) {
    ++dropped_;
    return;
  }
  q_.push_back(std::move(e));
}
std::vector<CollectedEvent> EventCollector::drain() {
  std::lock_guard<std::mutex> g(mu_);
  std::vector<CollectedEvent> out;
  out.swap(q_);
  return out;
}

uint64_t span_enter(const std::string& name, const std::string& actor_id) {
  const uint64_t id = g_next_span.fetch_add(1);
  const uint64_t parent = tl_spans.empty() ? 0 : tl_spans.back().id;
  const double t = telemetry_now_us();
  tl_spans.push_back(OpenSpan{id, name, t, now_us()});
  if (EventCollector::global().enabled()) {
    CollectedEvent ev;
    ev.kind = "span_enter";
    ev.t_us = t;
    ev.message = name;
    ev.actor_id = actor_id;
    ev.span_id = id;
    ev.parent_id = parent;
    EventCollector::global().push(std::move(ev));
  }
  return id;
}
void span_exit(uint64_t id) {
  // spans close innermost-first; closing an outer span closes what is still open inside it
  while (!tl_spans.empty()) {
    OpenSpan s = tl_spans.back();
    tl_spans.pop_back();
    if (EventCollector::global().enabled()) {
      CollectedEvent ev;
      ev.kind = "span_exit";
      ev.t_us = telemetry_now_us();
      ev.message = s.name;
      ev.span_id = s.id;
      EventCollector::global().push(std::move(ev));
    }
    if (TraceWriter::global().enabled())
      TraceWriter::global().complete(s.name, "span", s.t0_mono_us, now_us() - s.t0_mono_us,
                                     (int64_t)getpid(), (int64_t)thread_tag());
    if (s.id == id) break;
  }
}
uint64_t current_span_id() { return tl_spans.empty() ? 0 : tl_spans.back().id; }

}  // namespace mb
