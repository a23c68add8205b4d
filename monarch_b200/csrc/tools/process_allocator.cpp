// Process-allocator daemon (native): runs on a host and starts procs there on behalf of
// remote clients.
//
//   process_allocator_native --addr tcp!127.0.0.1:26600 --program "python -m monarch_b200.actor.bootstrap_main"
//
// The daemon decides WHAT runs: its --program, in its own working directory.  A client only
// asks for one more instance of it: it connects once per proc, sends one JSON line
// {"start": 1, "env": {...}, "token": ...} and then receives JSON lines {"pid": n, "host": s},
// {"out": text} / {"err": text} / {"exit": code}.  Of the client's env only the bootstrap
// variables pass (prefixes HYPERACTOR_, MONARCH_, MB200_, MASTER_ and a few exact names); a
// request that names a program ("argv") or a directory ("cwd") is refused.  With
// MB200_ALLOCATOR_TOKEN set in the daemon's environment, requests without the same token are
// refused.  The client may send {"signal": n}.  Heartbeats {"hb": 1} flow both ways every
// --heartbeat seconds; when the client has been silent for 3 intervals, or its connection
// drops, the proc is killed (SIGTERM to its process group, then SIGKILL): a host never keeps
// orphans of a vanished client.
//
// Parity: monarch_hyperactor/src/bin/process_allocator (the daemon binary; the program is
// fixed by its --program option, common.rs:41), hyperactor_mesh alloc/remoteprocess.rs:73-108
// (RemoteProcessAllocator), :940-1085 (heartbeats and the host watchdog).  The wire protocol is
// the one of tools/process_allocator.py; either daemon serves the same clients.
#include <arpa/inet.h>
#include <fcntl.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <sys/socket.h>
#include <sys/wait.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <set>
#include <string>
#include <thread>
#include <vector>

#include "json_lines.h"

extern char** environ;

using namespace mbtools;

namespace {

// ------------------------------------------------------------------------- the daemon --
bool same_token(const std::string& a, const std::string& b) {   // constant-time compare
  unsigned char d = (unsigned char)(a.size() != b.size());
  for (size_t i = 0; i < b.size(); ++i) d |= (unsigned char)((i < a.size() ? a[i] : 0) ^ b[i]);
  return d == 0;
}

double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

struct Session;
std::mutex g_reg_mu;
std::set<Session*> g_sessions;

struct Session {
  int fd;
  double hb;
  std::vector<std::string> program;
  std::string token;
  std::mutex wmu;
  std::atomic<pid_t> pid{0};
  std::atomic<bool> exited{false}, closed{false};
  std::atomic<double> last_seen{0};

  bool send_line(const std::string& line) {
    std::lock_guard<std::mutex> g(wmu);
    std::string data = line + "\n";
    size_t off = 0;
    while (off < data.size()) {
      ssize_t n = ::send(fd, data.data() + off, data.size() - off, MSG_NOSIGNAL);
      if (n <= 0) return false;
      off += (size_t)n;
    }
    return true;
  }

  void kill_child() {
    pid_t p = pid.load();
    if (p <= 0 || exited.load()) return;
    ::kill(-p, SIGTERM);
    for (int i = 0; i < 30 && !exited.load(); ++i) std::this_thread::sleep_for(std::chrono::milliseconds(100));
    if (!exited.load()) ::kill(-p, SIGKILL);
  }

  // Forward one of the child's pipes line by line.
  void pump(int rfd, const char* key) {
    std::string buf;
    char tmp[4096];
    bool alive = true;
    while (alive) {
      ssize_t n = ::read(rfd, tmp, sizeof tmp);
      if (n <= 0) break;
      buf.append(tmp, (size_t)n);
      size_t nl;
      while ((nl = buf.find('\n')) != std::string::npos) {
        if (!send_line(std::string("{\"") + key + "\": " + quote(buf.substr(0, nl + 1)) + "}")) {
          alive = false;
          break;
        }
        buf.erase(0, nl + 1);
      }
    }
    if (alive && !buf.empty()) send_line(std::string("{\"") + key + "\": " + quote(buf) + "}");
    ::close(rfd);
  }

  bool read_line(std::string& carry, std::string& line) {
    while (true) {
      size_t nl = carry.find('\n');
      if (nl != std::string::npos) {
        line = carry.substr(0, nl);
        carry.erase(0, nl + 1);
        return true;
      }
      char tmp[4096];
      ssize_t n = ::recv(fd, tmp, sizeof tmp, 0);
      if (n <= 0) return false;
      carry.append(tmp, (size_t)n);
      if (carry.size() > (1u << 22)) return false;   // no request line is that long
    }
  }

  void run() {
    {
      std::lock_guard<std::mutex> g(g_reg_mu);
      g_sessions.insert(this);
    }
    serve();
    closed = true;
    kill_child();
    ::shutdown(fd, SHUT_RDWR);
    ::close(fd);
    {
      std::lock_guard<std::mutex> g(g_reg_mu);
      g_sessions.erase(this);
    }
  }

  void serve() {
    std::string carry, line;
    if (!read_line(carry, line)) {
      send_line("{\"exit\": 126, \"error\": \"malformed request\"}");   // or a port probe
      return;
    }
    Parser ps(line);
    Json req = ps.value();
    const Json* start = req.get("start");
    if (!ps.ok || req.kind != Json::Obj || !start || !start->truthy()) {
      send_line("{\"exit\": 126, \"error\": \"malformed request\"}");
      return;
    }
    if (!token.empty()) {
      const Json* t = req.get("token");
      if (!same_token(t && t->kind == Json::Str ? t->str : std::string(), token)) {
        send_line("{\"exit\": 126, \"error\": \"bad or missing allocator token\"}");
        return;
      }
    }
    const Json* argv = req.get("argv");
    const Json* cwd = req.get("cwd");
    if ((argv && argv->truthy()) || (cwd && cwd->truthy())) {
      send_line("{\"exit\": 126, \"error\": \"this daemon runs its own --program; a request may not "
                "name a program or a working directory\"}");
      return;
    }
    // the child's environment: the daemon's own, minus its token, plus what the client may set
    std::map<std::string, std::string> env;
    for (char** e = environ; *e; ++e) {
      std::string kv(*e);
      size_t eq = kv.find('=');
      if (eq == std::string::npos) continue;
      env[kv.substr(0, eq)] = kv.substr(eq + 1);
    }
    env.erase("MB200_ALLOCATOR_TOKEN");
    if (const Json* je = req.get("env"))
      if (je->kind == Json::Obj)
        for (auto& kv : je->obj)
          if (env_allowed(kv.first)) {
            const Json& v = kv.second;
            if (v.kind == Json::Str) env[kv.first] = v.str;
            else if (v.kind == Json::Num) {
              char b[64];
              if (v.num == (double)(long long)v.num) std::snprintf(b, sizeof b, "%lld", (long long)v.num);
              else std::snprintf(b, sizeof b, "%g", v.num);
              env[kv.first] = b;
            } else if (v.kind == Json::Bool) env[kv.first] = v.b ? "True" : "False";
          }
    int out_pipe[2], err_pipe[2];
    if (::pipe(out_pipe) != 0 || ::pipe(err_pipe) != 0) {
      send_line("{\"exit\": 127, \"error\": \"pipe failed\"}");
      return;
    }
    std::vector<std::string> envs;
    for (auto& kv : env) envs.push_back(kv.first + "=" + kv.second);
    std::vector<char*> envp, args;
    for (auto& e : envs) envp.push_back(const_cast<char*>(e.c_str()));
    envp.push_back(nullptr);
    for (auto& a : program) args.push_back(const_cast<char*>(a.c_str()));
    args.push_back(nullptr);
    pid_t child = ::fork();
    if (child < 0) {
      send_line("{\"exit\": 127, \"error\": \"fork failed\"}");
      return;
    }
    if (child == 0) {
      ::setsid();                       // its own process group: signals reach its children too
      ::dup2(out_pipe[1], 1);
      ::dup2(err_pipe[1], 2);
      int devnull = ::open("/dev/null", 0);
      if (devnull >= 0) ::dup2(devnull, 0);
      for (int f = 3; f < 1024; ++f) ::close(f);
      ::execvpe(args[0], args.data(), envp.data());
      std::fprintf(stderr, "exec %s: %s\n", args[0], std::strerror(errno));
      ::_exit(127);
    }
    ::close(out_pipe[1]);
    ::close(err_pipe[1]);
    pid = child;
    last_seen = now_s();
    char host[256] = "localhost";
    ::gethostname(host, sizeof host - 1);
    send_line("{\"pid\": " + std::to_string((long long)child) + ", \"host\": " + quote(host) + "}");
    std::thread t_out([this, r = out_pipe[0]] { pump(r, "out"); });
    std::thread t_err([this, r = err_pipe[0]] { pump(r, "err"); });
    std::thread t_watch([this] {
      while (!closed.load() && !exited.load()) {
        for (int i = 0; i < (int)(hb * 10) && !closed.load() && !exited.load(); ++i)
          std::this_thread::sleep_for(std::chrono::milliseconds(100));
        if (closed.load() || exited.load()) return;
        send_line("{\"hb\": 1}");
        if (now_s() - last_seen.load() > 3 * hb + 1.0) {
          kill_child();   // the client vanished without closing the connection
          return;
        }
      }
    });
    std::thread t_read([this, carry]() mutable {
      std::string line;
      while (read_line(carry, line)) {
        last_seen = now_s();
        Parser p(line);
        Json msg = p.value();
        if (!p.ok || msg.kind != Json::Obj) continue;
        const Json* sig = msg.get("signal");
        pid_t c = pid.load();
        if (sig && sig->kind == Json::Num && c > 0 && !exited.load()) ::kill(-c, (int)sig->num);
      }
      if (!closed.load()) kill_child();   // connection closed by the client
    });
    int status = 0;
    while (::waitpid(child, &status, 0) < 0 && errno == EINTR) {
    }
    exited = true;
    int code = WIFEXITED(status) ? WEXITSTATUS(status) : (WIFSIGNALED(status) ? -WTERMSIG(status) : -1);
    t_out.join();
    t_err.join();
    send_line("{\"exit\": " + std::to_string(code) + "}");
    closed = true;
    ::shutdown(fd, SHUT_RD);           // wakes the reader
    t_read.join();
    t_watch.join();
  }
};

std::vector<std::string> split_command(const std::string& s) {   // shell-like: quotes, backslash
  std::vector<std::string> out;
  std::string cur;
  bool in = false;
  char q = 0;
  for (size_t i = 0; i < s.size(); ++i) {
    char c = s[i];
    if (q) {
      if (c == q) q = 0;
      else if (c == '\\' && q == '"' && i + 1 < s.size()) cur += s[++i];
      else cur += c;
    } else if (c == '\'' || c == '"') {
      q = c;
      in = true;
    } else if (c == '\\' && i + 1 < s.size()) {
      cur += s[++i];
      in = true;
    } else if (c == ' ' || c == '\t') {
      if (in) out.push_back(cur);
      cur.clear();
      in = false;
    } else {
      cur += c;
      in = true;
    }
  }
  if (in) out.push_back(cur);
  return out;
}

void on_term(int) {
  // best effort from a signal handler: children are in their own groups, so signal each
  {
    std::unique_lock<std::mutex> g(g_reg_mu, std::try_to_lock);
    if (g.owns_lock())
      for (Session* s : g_sessions) {
        pid_t p = s->pid.load();
        if (p > 0 && !s->exited.load()) ::kill(-p, SIGTERM);
      }
  }
  ::_exit(0);
}

}  // namespace

int main(int argc, char** argv) {
  std::string addr = "tcp!127.0.0.1:26600", program;
  double hb = 5.0;
  for (int i = 1; i < argc; ++i) {
    std::string a = argv[i];
    auto next = [&]() -> std::string { return i + 1 < argc ? std::string(argv[++i]) : std::string(); };
    if (a == "--addr") addr = next();
    else if (a == "--heartbeat") hb = std::atof(next().c_str());
    else if (a == "--program") program = next();
    else if (a == "-h" || a == "--help") {
      std::printf("usage: %s [--addr tcp!HOST:PORT] [--heartbeat SECONDS] --program \"COMMAND\"\n", argv[0]);
      return 0;
    }
  }
  std::vector<std::string> prog = split_command(program);
  if (prog.empty()) {
    std::fprintf(stderr, "process_allocator: --program is required\n");
    return 2;
  }
  if (addr.compare(0, 4, "tcp!") == 0) addr = addr.substr(4);
  size_t colon = addr.rfind(':');
  std::string host = colon == std::string::npos || colon == 0 ? "127.0.0.1" : addr.substr(0, colon);
  int port = std::atoi(addr.substr(colon == std::string::npos ? 0 : colon + 1).c_str());
  const char* tok = std::getenv("MB200_ALLOCATOR_TOKEN");
  std::string token = tok ? tok : "";

  ::signal(SIGPIPE, SIG_IGN);
  ::signal(SIGTERM, on_term);
  ::signal(SIGINT, on_term);
  int srv = ::socket(AF_INET, SOCK_STREAM, 0);
  int one = 1;
  ::setsockopt(srv, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in sa{};
  sa.sin_family = AF_INET;
  sa.sin_port = htons((uint16_t)port);
  if (::inet_pton(AF_INET, host.c_str(), &sa.sin_addr) != 1) {
    addrinfo hints{}, *res = nullptr;
    hints.ai_family = AF_INET;
    if (::getaddrinfo(host.c_str(), nullptr, &hints, &res) != 0 || !res) {
      std::fprintf(stderr, "process_allocator: cannot resolve %s\n", host.c_str());
      return 2;
    }
    sa.sin_addr = reinterpret_cast<sockaddr_in*>(res->ai_addr)->sin_addr;
    ::freeaddrinfo(res);
  }
  if (::bind(srv, reinterpret_cast<sockaddr*>(&sa), sizeof sa) != 0 || ::listen(srv, 256) != 0) {
    std::perror("process_allocator: bind/listen");
    return 2;
  }
  socklen_t sl = sizeof sa;
  ::getsockname(srv, reinterpret_cast<sockaddr*>(&sa), &sl);
  std::printf("process_allocator listening on tcp!%s:%d\n", host.c_str(), (int)ntohs(sa.sin_port));
  std::fflush(stdout);
  while (true) {
    int c = ::accept(srv, nullptr, nullptr);
    if (c < 0) {
      if (errno == EINTR) continue;
      break;
    }
    ::setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
    auto* s = new Session();
    s->fd = c;
    s->hb = hb;
    s->program = prog;
    s->token = token;
    std::thread([s] {
      s->run();
      delete s;
    }).detach();
  }
  return 0;
}
