#include "channel/channel.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <sys/uio.h>
#include <sys/un.h>
#include <unistd.h>

#include <cstring>
#include <map>
#include <random>
#include <set>

#include "telemetry/telemetry.h"

namespace mb {

ChannelStats& channel_stats() {
  static ChannelStats s;
  return s;
}

// -------------------------------------------------------------------- ChannelAddr --
ChannelAddr ChannelAddr::parse(const std::string& s) {
  ChannelAddr a;
  auto starts = [&](const char* p) { return s.rfind(p, 0) == 0; };
  if (starts("tcp:") || starts("tcp!")) {
    a.kind = Tcp;
    std::string rest = s.substr(4);
    auto c = rest.rfind(':');
    if (c == std::string::npos) throw ChannelError("bad tcp address: " + s);
    a.host = rest.substr(0, c);
    if (a.host.size() >= 2 && a.host.front() == '[' && a.host.back() == ']')
      a.host = a.host.substr(1, a.host.size() - 2);
    a.port = std::stoi(rest.substr(c + 1));
  } else if (starts("unix:")) {
    a.kind = Unix;
    a.path = s.substr(5);
  } else if (starts("local:")) {
    a.kind = Local;
    a.id = std::stoull(s.substr(6));
  } else if (starts("sim:")) {
    a.kind = Sim;
    std::string rest = s.substr(4);
    auto arrow = rest.find("->");
    if (arrow != std::string::npos) {
      a.src_node = rest.substr(0, arrow);
      rest = rest.substr(arrow + 2);
    }
    auto slash = rest.rfind('/');
    if (slash == std::string::npos) throw ChannelError("bad sim address: " + s);
    a.node = rest.substr(0, slash);
    a.id = std::stoull(rest.substr(slash + 1));
  } else {
    throw ChannelError("unsupported channel address: " + s);
  }
  return a;
}
ChannelAddr ChannelAddr::any(Kind k) {
  ChannelAddr a;
  a.kind = k;
  if (k == Tcp) a.host = "127.0.0.1";
  return a;
}
std::string ChannelAddr::to_string() const {
  switch (kind) {
    case Tcp: return "tcp:" + host + ":" + std::to_string(port);
    case Unix: return "unix:" + path;
    case Local: return "local:" + std::to_string(id);
    case Sim:
      return "sim:" + (src_node.empty() ? std::string() : src_node + "->") + node + "/" +
             std::to_string(id);
  }
  return "";
}

// ------------------------------------------------------------------ frame queue --
namespace {

class FrameQueue {
 public:
  void push(Frame f) {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (closed_) return;
      q_.push_back(std::move(f));
    }
    cv_.notify_one();
  }
  std::optional<Frame> pop(int64_t timeout_ms) {
    std::unique_lock<std::mutex> g(mu_);
    auto ready = [&] { return !q_.empty() || closed_; };
    if (timeout_ms < 0)
      cv_.wait(g, ready);
    else if (!cv_.wait_for(g, std::chrono::milliseconds(timeout_ms), ready))
      return std::nullopt;
    if (q_.empty()) return std::nullopt;
    Frame f = std::move(q_.front());
    q_.pop_front();
    return f;
  }
  void close() {
    {
      std::lock_guard<std::mutex> g(mu_);
      closed_ = true;
    }
    cv_.notify_all();
  }
  bool closed() const {
    std::lock_guard<std::mutex> g(mu_);
    return closed_;
  }

 private:
  mutable std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Frame> q_;
  bool closed_ = false;
};

// ---------------------------------------------------------------- local transport --
std::mutex g_local_mu;
std::map<uint64_t, std::weak_ptr<FrameQueue>> g_local;
uint64_t g_local_next = 1;

class LocalRx : public Rx {
 public:
  LocalRx(uint64_t id, std::shared_ptr<FrameQueue> q) : id_(id), q_(std::move(q)) {}
  ~LocalRx() override { close(); }
  std::optional<Frame> recv(int64_t t) override { return q_->pop(t); }
  ChannelAddr addr() const override {
    ChannelAddr a;
    a.kind = ChannelAddr::Local;
    a.id = id_;
    return a;
  }
  void close() override {
    q_->close();
    std::lock_guard<std::mutex> g(g_local_mu);
    g_local.erase(id_);
  }
  bool closed() const override { return q_->closed(); }

 private:
  uint64_t id_;
  std::shared_ptr<FrameQueue> q_;
};

class LocalTx : public Tx {
 public:
  explicit LocalTx(uint64_t id) : id_(id) {}
  void post(Frame f, std::function<void(Frame&&)> on_fail) override {
    std::shared_ptr<FrameQueue> q;
    {
      std::lock_guard<std::mutex> g(g_local_mu);
      auto it = g_local.find(id_);
      if (it != g_local.end()) q = it->second.lock();
    }
    if (!q || q->closed() || closed_) {
      channel_stats().undeliverable++;
      if (on_fail) on_fail(std::move(f));
      return;
    }
    channel_stats().frames_sent++;
    q->push(std::move(f));
  }
  TxStatus status() const override {
    std::lock_guard<std::mutex> g(g_local_mu);
    auto it = g_local.find(id_);
    if (closed_ || it == g_local.end()) return TxStatus::Closed;
    auto q = it->second.lock();
    return (q && !q->closed()) ? TxStatus::Active : TxStatus::Closed;
  }
  ChannelAddr addr() const override {
    ChannelAddr a;
    a.kind = ChannelAddr::Local;
    a.id = id_;
    return a;
  }
  void close() override { closed_ = true; }

 private:
  uint64_t id_;
  std::atomic<bool> closed_{false};
};

// ------------------------------------------------------------------ sim transport --
// hyperactor/src/simnet.rs schedules events on a simulated clock; here one scheduler thread
// owns a time-ordered queue of deliveries.
double telemetry_now_us_for_sim();   // defined below: the telemetry clock (sim or real)

class SimNet {
 public:
  static SimNet& get() {
    static SimNet* n = new SimNet();
    return *n;
  }
  void configure(const std::vector<double>& lat, double bw_gbs) {
    std::lock_guard<std::mutex> g(mu_);
    if (!lat.empty()) lat_ = lat;
    if (bw_gbs > 0) bytes_per_us_ = bw_gbs * 1e3;
  }
  double latency_us(const std::string& a, const std::string& b, size_t bytes, int* dist_out) {
    std::lock_guard<std::mutex> g(mu_);
    int d = simnet_distance(a, b);
    if (d >= (int)lat_.size()) d = (int)lat_.size() - 1;
    *dist_out = d;
    return lat_[d] + (double)bytes / bytes_per_us_;
  }
  // `deliver` runs on the scheduler thread once simulated time reaches now + delay.
  // `chan_ready_us` (per channel, owned by the caller under its own lock) keeps one
  // channel's frames in order when a later, smaller frame would otherwise overtake.
  void schedule(double delay_us, size_t bytes, int dist, double* chan_ready_us,
                std::function<void()> deliver) {
    {
      std::lock_guard<std::mutex> g(mu_);
      double at = now_locked() + delay_us;
      if (chan_ready_us) {
        if (at < *chan_ready_us) at = *chan_ready_us;
        *chan_ready_us = at;
      }
      q_.push_back(Ev{at, seq_++, std::move(deliver)});
      std::push_heap(q_.begin(), q_.end(), later);
      stats_.frames++;
      stats_.bytes += bytes;
      stats_.latency_us_total += delay_us;
      stats_.by_distance[dist < 8 ? dist : 7]++;
      if (!started_) {
        started_ = true;
        std::thread([this] { run(); }).detach();
      }
    }
    cv_.notify_all();
  }
  SimNetStats stats() {
    std::lock_guard<std::mutex> g(mu_);
    return stats_;
  }
  void reset_stats() {
    std::lock_guard<std::mutex> g(mu_);
    stats_ = SimNetStats{};
  }

 private:
  struct Ev {
    double at;
    uint64_t seq;
    std::function<void()> fn;
  };
  static bool later(const Ev& a, const Ev& b) {
    return a.at > b.at || (a.at == b.at && a.seq > b.seq);
  }
  double now_locked() { return telemetry_now_us_for_sim(); }
  void run();
  std::mutex mu_;
  std::condition_variable cv_;
  std::vector<Ev> q_;
  uint64_t seq_ = 0;
  bool started_ = false;
  std::vector<double> lat_{2.0, 10.0, 50.0, 500.0, 5000.0};
  double bytes_per_us_ = 50e3;   // 50 GB/s
  SimNetStats stats_;
};

std::mutex g_sim_mu;
std::map<std::string, std::weak_ptr<FrameQueue>> g_sim;   // "node/id" -> queue
uint64_t g_sim_next = 1;

class SimRx : public Rx {
 public:
  SimRx(std::string node, uint64_t id, std::shared_ptr<FrameQueue> q)
      : node_(std::move(node)), id_(id), q_(std::move(q)) {}
  ~SimRx() override { close(); }
  std::optional<Frame> recv(int64_t t) override { return q_->pop(t); }
  ChannelAddr addr() const override {
    ChannelAddr a;
    a.kind = ChannelAddr::Sim;
    a.node = node_;
    a.id = id_;
    return a;
  }
  void close() override {
    q_->close();
    std::lock_guard<std::mutex> g(g_sim_mu);
    g_sim.erase(node_ + "/" + std::to_string(id_));
  }
  bool closed() const override { return q_->closed(); }

 private:
  std::string node_;
  uint64_t id_;
  std::shared_ptr<FrameQueue> q_;
};

class SimTx : public Tx {
 public:
  explicit SimTx(ChannelAddr a) : addr_(std::move(a)) {}
  void post(Frame f, std::function<void(Frame&&)> on_fail) override {
    auto q = lookup();
    if (!q || q->closed() || closed_) {
      channel_stats().undeliverable++;
      if (on_fail) on_fail(std::move(f));
      return;
    }
    channel_stats().frames_sent++;
    int dist = 0;
    const size_t bytes = f.size();
    const double lat = SimNet::get().latency_us(addr_.src_node.empty() ? addr_.node : addr_.src_node,
                                                addr_.node, bytes, &dist);
    auto cell = std::make_shared<Frame>(std::move(f));
    std::lock_guard<std::mutex> g(order_mu_);
    SimNet::get().schedule(lat, bytes, dist, &ready_us_, [q, cell, on_fail] {
      if (q->closed()) {
        channel_stats().undeliverable++;
        if (on_fail) on_fail(std::move(*cell));
        return;
      }
      q->push(std::move(*cell));
    });
  }
  TxStatus status() const override {
    auto q = lookup();
    return (!closed_ && q && !q->closed()) ? TxStatus::Active : TxStatus::Closed;
  }
  ChannelAddr addr() const override { return addr_; }
  void close() override { closed_ = true; }

 private:
  std::shared_ptr<FrameQueue> lookup() const {
    std::lock_guard<std::mutex> g(g_sim_mu);
    auto it = g_sim.find(addr_.node + "/" + std::to_string(addr_.id));
    return it == g_sim.end() ? nullptr : it->second.lock();
  }
  ChannelAddr addr_;
  std::atomic<bool> closed_{false};
  std::mutex order_mu_;
  double ready_us_ = 0;
};

// ------------------------------------------------------------------ socket helpers --
void put_be64(char* b, uint64_t v) {
  for (int i = 0; i < 8; ++i) b[i] = (char)(v >> (56 - 8 * i));
}
uint64_t get_be64(const char* b) {
  uint64_t v = 0;
  for (int i = 0; i < 8; ++i) v = (v << 8) | (uint8_t)b[i];
  return v;
}

bool write_all_iov(int fd, std::vector<iovec>& iov) {
  size_t idx = 0;
  while (idx < iov.size()) {
    int cnt = (int)std::min<size_t>(iov.size() - idx, 64);
    // sendmsg rather than writev: MSG_NOSIGNAL keeps a peer that went away from raising
    // SIGPIPE in hosts that have not ignored it (a plain C++ embedder, unlike Python)
    msghdr mh{};
    mh.msg_iov = &iov[idx];
    mh.msg_iovlen = (size_t)cnt;
    ssize_t n = ::sendmsg(fd, &mh, MSG_NOSIGNAL);
    if (n < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    size_t left = (size_t)n;
    while (left > 0 && idx < iov.size()) {
      if (left >= iov[idx].iov_len) {
        left -= iov[idx].iov_len;
        ++idx;
      } else {
        iov[idx].iov_base = (char*)iov[idx].iov_base + left;
        iov[idx].iov_len -= left;
        left = 0;
      }
    }
    while (idx < iov.size() && iov[idx].iov_len == 0) ++idx;
  }
  return true;
}

bool read_exact(int fd, char* buf, size_t n) {
  size_t got = 0;
  while (got < n) {
    ssize_t r = ::recv(fd, buf + got, n - got, 0);
    if (r == 0) return false;
    if (r < 0) {
      if (errno == EINTR) continue;
      return false;
    }
    got += (size_t)r;
  }
  return true;
}

enum : uint8_t { kFrameInit = 1, kFrameMsg = 2 };

int make_listen_socket(ChannelAddr& a) {
  if (a.kind == ChannelAddr::Tcp) {
    int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) throw ChannelError("socket() failed");
    int one = 1;
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    sockaddr_in sa{};
    sa.sin_family = AF_INET;
    sa.sin_port = htons((uint16_t)a.port);
    std::string host = a.host.empty() || a.host == "localhost" ? "127.0.0.1" : a.host;
    if (host == "0.0.0.0" || host == "*")
      sa.sin_addr.s_addr = INADDR_ANY;
    else if (inet_pton(AF_INET, host.c_str(), &sa.sin_addr) != 1) {
      ::close(fd);
      throw ChannelError("cannot parse tcp host: " + host);
    }
    if (::bind(fd, (sockaddr*)&sa, sizeof(sa)) < 0 || ::listen(fd, 512) < 0) {
      int e = errno;
      ::close(fd);
      throw ChannelError("bind/listen failed on " + a.to_string() + ": " + std::strerror(e));
    }
    socklen_t len = sizeof(sa);
    getsockname(fd, (sockaddr*)&sa, &len);
    a.port = ntohs(sa.sin_port);
    a.host = host;
    return fd;
  }
  // unix
  static std::atomic<uint64_t> counter{0};
  if (a.path.empty())
    a.path = "@mb200_" + std::to_string(getpid()) + "_" + std::to_string(counter++) + "_" +
             std::to_string(std::random_device{}());
  int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) throw ChannelError("socket() failed");
  sockaddr_un sa{};
  sa.sun_family = AF_UNIX;
  if (a.path.size() >= sizeof(sa.sun_path)) {
    ::close(fd);
    throw ChannelError("unix path too long");
  }
  std::memcpy(sa.sun_path, a.path.data(), a.path.size());
  socklen_t len = (socklen_t)(offsetof(sockaddr_un, sun_path) + a.path.size());
  if (a.path[0] == '@')
    sa.sun_path[0] = 0;  // abstract namespace: no filesystem entry to clean up
  else
    ::unlink(a.path.c_str());
  if (::bind(fd, (sockaddr*)&sa, len) < 0 || ::listen(fd, 512) < 0) {
    int e = errno;
    ::close(fd);
    throw ChannelError("bind/listen failed on " + a.to_string() + ": " + std::strerror(e));
  }
  return fd;
}

int connect_socket(const ChannelAddr& a) {
  if (a.kind == ChannelAddr::Tcp) {
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_INET;
    hints.ai_socktype = SOCK_STREAM;
    std::string host = a.host == "localhost" ? "127.0.0.1" : a.host;
    if (getaddrinfo(host.c_str(), std::to_string(a.port).c_str(), &hints, &res) != 0 || !res)
      return -1;
    int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd >= 0 && ::connect(fd, res->ai_addr, res->ai_addrlen) < 0) {
      ::close(fd);
      fd = -1;
    }
    freeaddrinfo(res);
    if (fd >= 0) {
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    }
    return fd;
  }
  int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) return -1;
  sockaddr_un sa{};
  sa.sun_family = AF_UNIX;
  std::memcpy(sa.sun_path, a.path.data(), std::min(a.path.size(), sizeof(sa.sun_path) - 1));
  socklen_t len = (socklen_t)(offsetof(sockaddr_un, sun_path) + a.path.size());
  if (!a.path.empty() && a.path[0] == '@') sa.sun_path[0] = 0;
  if (::connect(fd, (sockaddr*)&sa, len) < 0) {
    ::close(fd);
    return -1;
  }
  return fd;
}

// ----------------------------------------------------------------------- NetRx --
class NetRx : public Rx, public std::enable_shared_from_this<NetRx> {
 public:
  explicit NetRx(ChannelAddr a) : addr_(std::move(a)) {
    listen_fd_ = make_listen_socket(addr_);
    q_ = std::make_shared<FrameQueue>();
    accept_thr_ = std::thread([this] { accept_loop(); });
  }
  ~NetRx() override { close(); }
  std::optional<Frame> recv(int64_t t) override { return q_->pop(t); }
  ChannelAddr addr() const override { return addr_; }
  bool closed() const override { return stop_; }
  void close() override {
    bool was = stop_.exchange(true);
    if (was) return;
    ::shutdown(listen_fd_, SHUT_RDWR);
    ::close(listen_fd_);
    {
      std::lock_guard<std::mutex> g(mu_);
      for (int fd : conns_) ::shutdown(fd, SHUT_RDWR);
    }
    if (accept_thr_.joinable()) accept_thr_.join();
    std::vector<std::thread> readers;
    {
      std::lock_guard<std::mutex> g(mu_);
      readers.swap(readers_);
    }
    for (auto& t : readers)
      if (t.joinable()) t.join();
    q_->close();
    if (addr_.kind == ChannelAddr::Unix && !addr_.path.empty() && addr_.path[0] != '@')
      ::unlink(addr_.path.c_str());
  }

 private:
  void accept_loop() {
    while (!stop_) {
      int fd = ::accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
      if (fd < 0) {
        if (errno == EINTR) continue;
        break;
      }
      if (addr_.kind == ChannelAddr::Tcp) {
        int one = 1;
        setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      }
      std::lock_guard<std::mutex> g(mu_);
      conns_.insert(fd);
      readers_.emplace_back([this, fd] { reader_loop(fd); });
    }
  }

  void reader_loop(int fd) {
    const uint64_t max_frame = (uint64_t)Config::global().get_int("CODEC_MAX_FRAME_LENGTH");
    const uint64_t ack_every = (uint64_t)Config::global().get_int("MESSAGE_ACK_EVERY_N_MESSAGES");
    uint64_t session = 0;
    uint64_t unacked = 0;
    uint64_t last_seq = 0;
    bool have_seq = false;
    auto send_ack = [&]() {
      if (!have_seq || unacked == 0) return true;
      char b[8];
      put_be64(b, last_seq);
      unacked = 0;
      channel_stats().acks_sent++;
      return ::send(fd, b, 8, MSG_NOSIGNAL) == 8;
    };
    constexpr uint64_t kSmallFrame = 64 * 1024;
    std::string small;
    while (!stop_) {
      // frame = len(8) type(1) ...; a message frame continues with seq(8) nparts(8)
      // head_len(8) part_len(8)* head parts*.  Head and parts of a large frame are read
      // straight into the strings that are handed on, so a large part is written once by
      // the kernel and never copied again on this side.
      char lenb[8];
      if (!read_exact(fd, lenb, 8)) break;
      uint64_t len = get_be64(lenb);
      if (len == 0 || len > max_frame) break;
      Frame f;
      uint64_t seq = 0;
      if (len <= kSmallFrame) {
        // small frame: one read, then split
        small.resize(len);
        if (!read_exact(fd, small.data(), len)) break;
        uint8_t type = (uint8_t)small[0];
        if (type == kFrameInit && len >= 9) {
          session = get_be64(small.data() + 1);
          continue;
        }
        if (type != kFrameMsg || len < 25) break;
        const char* p = small.data() + 1;
        seq = get_be64(p);
        uint64_t nparts = get_be64(p + 8);
        uint64_t head_len = get_be64(p + 16);
        p += 24;
        if (25 + 8 * nparts > len) break;
        uint64_t total = 25 + 8 * nparts + head_len;
        std::vector<uint64_t> plens(nparts);
        for (auto& l : plens) {
          l = get_be64(p);
          p += 8;
          total += l;
        }
        if (head_len > len || total != len) break;
        f.head.assign(p, head_len);
        p += head_len;
        for (uint64_t l : plens) {
          f.parts.emplace_back(p, l);
          p += l;
        }
      } else {
        char type_b;
        if (!read_exact(fd, &type_b, 1)) break;
        if ((uint8_t)type_b != kFrameMsg) break;
        char fixed[24];
        if (!read_exact(fd, fixed, 24)) break;
        seq = get_be64(fixed);
        uint64_t nparts = get_be64(fixed + 8);
        uint64_t head_len = get_be64(fixed + 16);
        if (nparts > (1u << 20) || 25 + 8 * nparts > len) break;
        std::vector<uint64_t> plens(nparts);
        {
          std::string lens(8 * nparts, '\0');
          if (nparts && !read_exact(fd, lens.data(), lens.size())) break;
          for (uint64_t i = 0; i < nparts; ++i) plens[i] = get_be64(lens.data() + 8 * i);
        }
        uint64_t total = 25 + 8 * nparts + head_len;
        bool sane = head_len <= len;
        for (uint64_t l : plens) {
          if (l > len) sane = false;
          total += l;
        }
        if (!sane || total != len) break;
        f.head.resize(head_len);
        if (head_len && !read_exact(fd, f.head.data(), head_len)) break;
        bool ok = true;
        f.parts.resize(nparts);
        for (uint64_t i = 0; i < nparts && ok; ++i) {
          f.parts[i].resize(plens[i]);
          if (plens[i] && !read_exact(fd, f.parts[i].data(), plens[i])) ok = false;
        }
        if (!ok) break;
      }
      {
        // The sequence check and the hand-over to the queue are one critical section: after
        // a reconnect the reader of the old connection may still hold frames it had already
        // read while the reader of the new connection delivers the resent tail; checked and
        // queued separately, an older frame could land behind a newer one.
        std::lock_guard<std::mutex> g(mu_);
        uint64_t& next = next_seq_[session];
        if (seq < next) {
          channel_stats().duplicates_dropped++;
        } else {
          next = seq + 1;
          channel_stats().frames_received++;
          q_->push(std::move(f));
        }
      }
      last_seq = seq;
      have_seq = true;
      ++unacked;
      // Ack when the batch limit is reached or the socket has gone quiet.
      pollfd pf{fd, POLLIN, 0};
      if (unacked >= ack_every || ::poll(&pf, 1, 0) == 0) {
        if (!send_ack()) break;
      }
    }
    send_ack();
    ::close(fd);
    std::lock_guard<std::mutex> g(mu_);
    conns_.erase(fd);
  }

  ChannelAddr addr_;
  int listen_fd_ = -1;
  std::shared_ptr<FrameQueue> q_;
  std::atomic<bool> stop_{false};
  std::thread accept_thr_;
  std::mutex mu_;
  std::set<int> conns_;
  std::vector<std::thread> readers_;
  std::map<uint64_t, uint64_t> next_seq_;
};

// ----------------------------------------------------------------------- NetTx --
class NetTx;
std::mutex g_tx_mu;
std::multimap<std::string, NetTx*> g_txs;

class NetTx : public Tx {
 public:
  explicit NetTx(ChannelAddr a) : addr_(std::move(a)) {
    std::random_device rd;
    session_ = ((uint64_t)rd() << 32) ^ rd() ^ ((uint64_t)getpid() << 16);
    wake_fd_ = ::eventfd(0, EFD_CLOEXEC | EFD_NONBLOCK);
    {
      std::lock_guard<std::mutex> g(g_tx_mu);
      g_txs.emplace(addr_.to_string(), this);
    }
    thr_ = std::thread([this] { run(); });
  }
  ~NetTx() override {
    close();
    std::lock_guard<std::mutex> g(g_tx_mu);
    for (auto it = g_txs.begin(); it != g_txs.end(); ++it)
      if (it->second == this) {
        g_txs.erase(it);
        break;
      }
  }
  void post(Frame f, std::function<void(Frame&&)> on_fail) override {
    // Fast path: a small frame on an idle, connected, writable link is written by the
    // caller itself, which saves waking the writer thread (one thread hop per message).
    // io_mu_ serialises everything that writes to or closes the socket and is always taken
    // before mu_; the writer thread moves frames from the outbox to the unacked queue only
    // while holding it, so the wire order equals the sequence order.
    if (f.size() <= kInlineSendBytes) {
      std::unique_lock<std::mutex> io(io_mu_, std::try_to_lock);
      if (io.owns_lock()) {
        Item* it = nullptr;
        int fd = -1;
        {
          std::lock_guard<std::mutex> g(mu_);
          if (!closed_ && !stop_ && fd_ >= 0 && outbox_.empty()) {
            pollfd pf{fd_, POLLOUT, 0};
            if (::poll(&pf, 1, 0) == 1 && (pf.revents & POLLOUT) &&
                !(pf.revents & (POLLERR | POLLHUP))) {
              unacked_.push_back(Item{next_seq_++, std::move(f), std::move(on_fail),
                                      std::chrono::steady_clock::now()});
              it = &unacked_.back();
              fd = fd_;
            }
          }
        }
        if (it) {
          channel_stats().frames_sent++;
          if (!send_item(fd, *it)) ::shutdown(fd, SHUT_RDWR);  // the writer thread reconnects
          return;                                               // and resends what is unacked
        }
      }
    }
    {
      std::lock_guard<std::mutex> g(mu_);
      if (closed_) {
        channel_stats().undeliverable++;
        if (on_fail) on_fail(std::move(f));
        return;
      }
      outbox_.push_back(Item{next_seq_++, std::move(f), std::move(on_fail),
                             std::chrono::steady_clock::now()});
    }
    wake();
  }
  TxStatus status() const override { return closed_ ? TxStatus::Closed : TxStatus::Active; }
  ChannelAddr addr() const override { return addr_; }
  void close() override {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (stop_) return;
      stop_ = true;
    }
    wake();
    if (thr_.joinable()) thr_.join();
    ::close(wake_fd_);
  }
  void drop_connection() {
    std::lock_guard<std::mutex> g(mu_);
    if (fd_ >= 0) ::shutdown(fd_, SHUT_RDWR);
  }

 private:
  struct Item {
    uint64_t seq;
    Frame frame;
    std::function<void(Frame&&)> on_fail;
    std::chrono::steady_clock::time_point t;
  };

  void wake() {
    uint64_t one = 1;
    (void)!::write(wake_fd_, &one, 8);
  }

  bool send_item(int fd, const Item& it) {
    // payload = type(1) seq(8) nparts(8) head_len(8) part_len(8)* head parts*
    std::string meta;
    meta.resize(8 + 1 + 8 + 8 + 8 + 8 * it.frame.parts.size());
    char* p = meta.data();
    uint64_t payload_len = 1 + 8 + 8 + 8 + 8 * it.frame.parts.size() + it.frame.size();
    put_be64(p, payload_len);
    p += 8;
    *p++ = (char)kFrameMsg;
    put_be64(p, it.seq);
    p += 8;
    put_be64(p, it.frame.parts.size());
    p += 8;
    put_be64(p, it.frame.head.size());
    p += 8;
    for (auto& part : it.frame.parts) {
      put_be64(p, part.size());
      p += 8;
    }
    std::vector<iovec> iov;
    iov.push_back({meta.data(), meta.size()});
    if (!it.frame.head.empty())
      iov.push_back({(void*)it.frame.head.data(), it.frame.head.size()});
    for (auto& part : it.frame.parts)
      if (!part.empty()) iov.push_back({(void*)part.data(), part.size()});
    return write_all_iov(fd, iov);
  }

  void fail_all() {
    std::deque<Item> items;
    {
      std::lock_guard<std::mutex> io(io_mu_);  // no caller-side send is using an item
      std::lock_guard<std::mutex> g(mu_);
      closed_ = true;
      for (auto& i : unacked_) items.push_back(std::move(i));
      for (auto& i : outbox_) items.push_back(std::move(i));
      unacked_.clear();
      outbox_.clear();
    }
    for (auto& i : items) {
      channel_stats().undeliverable++;
      if (i.on_fail) i.on_fail(std::move(i.frame));
    }
  }

  void run() {
    const auto timeout =
        std::chrono::milliseconds(Config::global().get_int("MESSAGE_DELIVERY_TIMEOUT_MS"));
    int64_t backoff = Config::global().get_int("CHANNEL_RECONNECT_BACKOFF_MIN_MS");
    const int64_t backoff_max = Config::global().get_int("CHANNEL_RECONNECT_BACKOFF_MAX_MS");
    bool ever_connected = false;
    while (true) {
      {
        std::lock_guard<std::mutex> g(mu_);
        if (stop_ && outbox_.empty() && unacked_.empty()) break;
        if (stop_ && fd_ < 0) break;  // closing while disconnected: give up
      }
      // Expire messages that have waited longer than the delivery timeout.
      {
        bool expired = false;
        {
          std::lock_guard<std::mutex> g(mu_);
          auto now = std::chrono::steady_clock::now();
          const Item* oldest =
              !unacked_.empty() ? &unacked_.front() : (!outbox_.empty() ? &outbox_.front() : nullptr);
          if (oldest && now - oldest->t > timeout) expired = true;
        }
        if (expired) {
          MB_LOG(Warn, "channel " + addr_.to_string() + ": delivery timeout, closing");
          fail_all();
          break;
        }
      }
      if (fd_ < 0) {
        bool idle;
        {
          std::lock_guard<std::mutex> g(mu_);
          idle = outbox_.empty() && unacked_.empty();
        }
        if (idle) {  // nothing to send: do not hammer a peer that is not there yet
          pollfd pf{wake_fd_, POLLIN, 0};
          ::poll(&pf, 1, 200);
          uint64_t junk;
          (void)!::read(wake_fd_, &junk, 8);
          continue;
        }
        int fd = connect_socket(addr_);
        if (fd < 0) {
          std::this_thread::sleep_for(std::chrono::milliseconds(backoff));
          backoff = std::min(backoff * 2, backoff_max);
          continue;
        }
        backoff = Config::global().get_int("CHANNEL_RECONNECT_BACKOFF_MIN_MS");
        channel_stats().connects++;
        if (ever_connected) channel_stats().reconnects++;
        ever_connected = true;
        char init[8 + 9];
        put_be64(init, 9);
        init[8] = (char)kFrameInit;
        put_be64(init + 9, session_);
        bool ok = ::send(fd, init, sizeof(init), MSG_NOSIGNAL) == (ssize_t)sizeof(init);
        // Resend everything not yet acknowledged, in order.
        if (ok) {
          std::lock_guard<std::mutex> io(io_mu_);
          std::lock_guard<std::mutex> g(mu_);
          for (auto& it : unacked_) {
            channel_stats().frames_resent++;
            if (!send_item(fd, it)) {
              ok = false;
              break;
            }
          }
        }
        if (!ok) {
          ::close(fd);
          continue;
        }
        std::lock_guard<std::mutex> io(io_mu_);
        std::lock_guard<std::mutex> g(mu_);
        fd_ = fd;
      }
      // Send new items.
      bool io_ok = true;
      while (io_ok) {
        std::lock_guard<std::mutex> io(io_mu_);
        Item* it = nullptr;
        {
          std::lock_guard<std::mutex> g(mu_);
          if (outbox_.empty()) break;
          unacked_.push_back(std::move(outbox_.front()));
          outbox_.pop_front();
          it = &unacked_.back();
        }
        channel_stats().frames_sent++;
        io_ok = send_item(fd_, *it);
      }
      // Drain acks / wait for work.
      if (io_ok) {
        pollfd pfs[2] = {{fd_, POLLIN, 0}, {wake_fd_, POLLIN, 0}};
        int pr = ::poll(pfs, 2, 100);
        if (pr > 0 && (pfs[1].revents & POLLIN)) {
          uint64_t junk;
          (void)!::read(wake_fd_, &junk, 8);
        }
        if (pr > 0 && (pfs[0].revents & (POLLIN | POLLHUP | POLLERR))) {
          char b[8 * 64];
          ssize_t n = ::recv(fd_, b, sizeof(b), MSG_DONTWAIT);
          if (n == 0 || (n < 0 && errno != EAGAIN && errno != EWOULDBLOCK && errno != EINTR)) {
            io_ok = false;
          } else if (n > 0) {
            ack_buf_.append(b, (size_t)n);
            while (ack_buf_.size() >= 8) {
              uint64_t acked = get_be64(ack_buf_.data());
              ack_buf_.erase(0, 8);
              // io_mu_ first: a caller-side send may still be inside sendmsg with pointers
              // into the item whose acknowledgement has just arrived
              std::lock_guard<std::mutex> io(io_mu_);
              std::lock_guard<std::mutex> g(mu_);
              while (!unacked_.empty() && unacked_.front().seq <= acked) unacked_.pop_front();
            }
          }
        }
      }
      if (!io_ok) {
        std::lock_guard<std::mutex> io(io_mu_);
        std::lock_guard<std::mutex> g(mu_);
        ::close(fd_);
        fd_ = -1;
        ack_buf_.clear();
      }
    }
    {
      std::lock_guard<std::mutex> io(io_mu_);
      std::lock_guard<std::mutex> g(mu_);
      if (fd_ >= 0) {
        ::close(fd_);
        fd_ = -1;
      }
    }
    fail_all();
  }

  ChannelAddr addr_;
  uint64_t session_;
  int wake_fd_ = -1;
  int fd_ = -1;
  static constexpr size_t kInlineSendBytes = 16 * 1024;
  std::mutex io_mu_;  // writers to / closers of fd_; taken before mu_
  std::mutex mu_;
  std::deque<Item> outbox_, unacked_;
  uint64_t next_seq_ = 0;
  bool stop_ = false;
  std::atomic<bool> closed_{false};
  std::string ack_buf_;
  std::thread thr_;
};

}  // namespace

std::shared_ptr<Rx> serve(const ChannelAddr& addr) {
  if (addr.kind == ChannelAddr::Sim) {
    std::lock_guard<std::mutex> g(g_sim_mu);
    uint64_t id = addr.id ? addr.id : g_sim_next++;
    if (addr.id) g_sim_next = std::max(g_sim_next, addr.id + 1);
    std::string node = addr.node.empty() ? "node0" : addr.node;
    std::string key = node + "/" + std::to_string(id);
    auto it = g_sim.find(key);
    if (it != g_sim.end() && !it->second.expired())
      throw ChannelError("sim channel " + key + " already served");
    auto q = std::make_shared<FrameQueue>();
    g_sim[key] = q;
    return std::make_shared<SimRx>(node, id, q);
  }
  if (addr.kind == ChannelAddr::Local) {
    std::lock_guard<std::mutex> g(g_local_mu);
    uint64_t id = addr.id ? addr.id : g_local_next++;
    if (addr.id) g_local_next = std::max(g_local_next, addr.id + 1);
    auto it = g_local.find(id);
    if (it != g_local.end() && !it->second.expired())
      throw ChannelError("local channel " + std::to_string(id) + " already served");
    auto q = std::make_shared<FrameQueue>();
    g_local[id] = q;
    return std::make_shared<LocalRx>(id, q);
  }
  return std::make_shared<NetRx>(addr);
}

std::shared_ptr<Tx> dial(const ChannelAddr& addr) {
  if (addr.kind == ChannelAddr::Local) return std::make_shared<LocalTx>(addr.id);
  if (addr.kind == ChannelAddr::Sim) return std::make_shared<SimTx>(addr);
  return std::make_shared<NetTx>(addr);
}

// ------------------------------------------------------------------------- simnet --
namespace {
double telemetry_now_us_for_sim() { return telemetry_now_us(); }

void SimNet::run() {
  std::unique_lock<std::mutex> lk(mu_);
  while (true) {
    cv_.wait(lk, [&] { return !q_.empty(); });
    std::pop_heap(q_.begin(), q_.end(), later);
    Ev ev = std::move(q_.back());
    q_.pop_back();
    const double now = telemetry_now_us();
    if (ev.at > now) {
      if (sim_clock_in_use()) {
        sim_clock_advance_us(ev.at - now);      // nothing earlier is pending: jump there
      } else {
        // real time: sleep until it is due (an earlier delivery may be scheduled meanwhile)
        const double wait_us = ev.at - now;
        q_.push_back(std::move(ev));
        std::push_heap(q_.begin(), q_.end(), later);
        cv_.wait_for(lk, std::chrono::microseconds((int64_t)wait_us + 1));
        continue;
      }
    }
    lk.unlock();
    ev.fn();
    lk.lock();
  }
}
}  // namespace

int simnet_distance(const std::string& a, const std::string& b) {
  auto split = [](const std::string& s) {
    std::vector<std::string> out;
    size_t i = 0;
    while (i <= s.size()) {
      size_t j = s.find('.', i);
      if (j == std::string::npos) j = s.size();
      out.push_back(s.substr(i, j - i));
      i = j + 1;
    }
    return out;
  };
  auto pa = split(a), pb = split(b);
  size_t common = 0;
  while (common < pa.size() && common < pb.size() && pa[common] == pb[common]) ++common;
  return (int)(std::max(pa.size(), pb.size()) - common);
}
void simnet_configure(const std::vector<double>& lat, double bw) { SimNet::get().configure(lat, bw); }
SimNetStats simnet_stats() { return SimNet::get().stats(); }
void simnet_reset_stats() { SimNet::get().reset_stats(); }

void debug_drop_connections(const ChannelAddr& addr) {
  std::lock_guard<std::mutex> g(g_tx_mu);
  auto range = g_txs.equal_range(addr.to_string());
  for (auto it = range.first; it != range.second; ++it) it->second->drop_connection();
}

}  // namespace mb
