// Local stand-in of a proc that runs under another host's process-allocator daemon (native
// form of tools/remote_exec.py; same behaviour, no interpreter per remote proc).
//
// The client's process allocator starts one of these per remote proc.  It picks the daemon
// from MB200_REMOTE_HOSTS (comma-separated tcp!host:port) by the proc's rank
// (HYPERACTOR_MESH_INDEX / MB200_PROCS_PER_HOST), forwards the bootstrap environment (the
// daemon starts its own program; clients cannot name one) and MB200_ALLOCATOR_TOKEN when set,
// relays the remote stdout / stderr to its own (where the allocator's log tailer reads them),
// forwards SIGTERM / SIGINT, sends heartbeats and exits with the remote exit code.  Killing it
// kills the remote proc: the daemon sees the connection drop.
//
// Parity: hyperactor_mesh alloc/remoteprocess.rs (RemoteProcessAlloc: one connection per
// host, heartbeats, forwarded process state).
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <signal.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <cerrno>
#include <chrono>
#include <mutex>
#include <string>
#include <thread>

#include "json_lines.h"

extern char** environ;

using namespace mbtools;

namespace {

int g_fd = -1;
std::mutex g_wmu;

void send_line(const std::string& line) {
  std::lock_guard<std::mutex> g(g_wmu);
  std::string data = line + "\n";
  size_t off = 0;
  while (off < data.size()) {
    ssize_t n = ::send(g_fd, data.data() + off, data.size() - off, MSG_NOSIGNAL);
    if (n <= 0) return;
    off += (size_t)n;
  }
}

void write_all(int fd, const std::string& s) {
  size_t off = 0;
  while (off < s.size()) {
    ssize_t n = ::write(fd, s.data() + off, s.size() - off);
    if (n <= 0) return;
    off += (size_t)n;
  }
}

const char* env_or(const char* k, const char* dflt) {
  const char* v = std::getenv(k);
  return v && *v ? v : dflt;
}

}  // namespace

int main() {
  // the daemon for this proc
  std::vector<std::string> hosts;
  {
    std::string all = env_or("MB200_REMOTE_HOSTS", "");
    size_t pos = 0;
    while (pos <= all.size()) {
      size_t c = all.find(',', pos);
      if (c == std::string::npos) c = all.size();
      if (c > pos) hosts.push_back(all.substr(pos, c - pos));
      pos = c + 1;
    }
  }
  if (hosts.empty()) {
    std::fprintf(stderr, "remote_exec: MB200_REMOTE_HOSTS is empty\n");
    return 2;
  }
  const long rank = std::atol(env_or("HYPERACTOR_MESH_INDEX", "0"));
  long per_host = std::atol(env_or("MB200_PROCS_PER_HOST", "1"));
  if (per_host < 1) per_host = 1;
  size_t hi = (size_t)(rank / per_host);
  if (hi >= hosts.size()) hi = hosts.size() - 1;
  std::string addr = hosts[hi];
  if (addr.compare(0, 4, "tcp!") == 0) addr = addr.substr(4);
  const size_t colon = addr.rfind(':');
  const std::string host = colon == std::string::npos || colon == 0 ? "127.0.0.1" : addr.substr(0, colon);
  const std::string port = addr.substr(colon == std::string::npos ? 0 : colon + 1);
  const double hb = std::atof(env_or("MB200_ALLOCATOR_HEARTBEAT", "5"));

  // SIGTERM / SIGINT are taken by a thread of their own (sigwait) and forwarded
  sigset_t sigs;
  sigemptyset(&sigs);
  sigaddset(&sigs, SIGTERM);
  sigaddset(&sigs, SIGINT);
  pthread_sigmask(SIG_BLOCK, &sigs, nullptr);
  ::signal(SIGPIPE, SIG_IGN);

  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  if (::getaddrinfo(host.c_str(), port.c_str(), &hints, &res) != 0 || !res) {
    std::fprintf(stderr, "remote_exec: cannot resolve allocator %s:%s\n", host.c_str(), port.c_str());
    return 111;
  }
  g_fd = ::socket(res->ai_family, res->ai_socktype, res->ai_protocol);
  timeval tv{10, 0};
  ::setsockopt(g_fd, SOL_SOCKET, SO_SNDTIMEO, &tv, sizeof tv);   // bounds the connect
  if (g_fd < 0 || ::connect(g_fd, res->ai_addr, res->ai_addrlen) != 0) {
    std::fprintf(stderr, "remote_exec: cannot reach allocator %s:%s: %s\n", host.c_str(),
                 port.c_str(), std::strerror(errno));
    ::freeaddrinfo(res);
    return 111;
  }
  ::freeaddrinfo(res);
  timeval none{0, 0};
  ::setsockopt(g_fd, SOL_SOCKET, SO_SNDTIMEO, &none, sizeof none);
  int one = 1;
  ::setsockopt(g_fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);

  // the request: bootstrap environment + token
  std::string req = "{\"start\": 1, \"env\": {";
  bool first = true;
  for (char** e = environ; *e; ++e) {
    std::string kv(*e);
    const size_t eq = kv.find('=');
    if (eq == std::string::npos) continue;
    const std::string k = kv.substr(0, eq);
    if (!env_allowed(k) || k == "MB200_LOCAL_INDEX") continue;
    req += (first ? "" : ", ") + quote(k) + ": " + quote(kv.substr(eq + 1));
    first = false;
  }
  req += std::string(first ? "" : ", ") + "\"MB200_LOCAL_INDEX\": " +
         quote(std::to_string(rank % per_host));
  req += "}, \"token\": " + quote(env_or("MB200_ALLOCATOR_TOKEN", "")) + "}";
  send_line(req);

  std::atomic<bool> done{false};
  std::thread([&sigs] {
    while (true) {
      int sig = 0;
      if (sigwait(&sigs, &sig) != 0) return;
      send_line("{\"signal\": " + std::to_string(sig) + "}");
    }
  }).detach();
  std::thread([&done, hb] {
    while (!done.load()) {
      for (int i = 0; i < (int)(hb * 10) && !done.load(); ++i)
        std::this_thread::sleep_for(std::chrono::milliseconds(100));
      if (!done.load()) send_line("{\"hb\": 1}");
    }
  }).detach();

  int code = 1;
  std::string carry;
  char buf[65536];
  bool finished = false;
  while (!finished) {
    ssize_t n = ::recv(g_fd, buf, sizeof buf, 0);
    if (n <= 0) break;
    carry.append(buf, (size_t)n);
    size_t nl;
    while ((nl = carry.find('\n')) != std::string::npos) {
      const std::string line = carry.substr(0, nl);
      carry.erase(0, nl + 1);
      Parser p(line);
      Json msg = p.value();
      if (!p.ok || msg.kind != Json::Obj) continue;
      if (const Json* o = msg.get("out")) {
        if (o->kind == Json::Str) write_all(1, o->str);
      } else if (const Json* e = msg.get("err")) {
        if (e->kind == Json::Str) write_all(2, e->str);
      } else if (const Json* x = msg.get("exit")) {
        code = x->kind == Json::Num ? (int)x->num : 1;
        if (const Json* er = msg.get("error"))
          if (er->kind == Json::Str) write_all(2, "remote_exec: " + er->str + "\n");
        finished = true;
        break;
      }
    }
  }
  done = true;
  ::close(g_fd);
  ::_exit(code >= 0 ? code : 128 - code);   // the helper threads are still around: no unwinding
}
