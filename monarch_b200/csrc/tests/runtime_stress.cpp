// Concurrency stress of the native runtime, meant to run under ThreadSanitizer and
// AddressSanitizer (host only): channels with many concurrent posters (caller-side send fast
// path racing the writer thread), an in-process proc mesh with casts from several threads
// (comm actors routing on the delivering threads), accumulating ports, the write-ahead log and
// the preemptible reader/writer lock.  Exits 0 when every count adds up; the sanitizer reports
// decide the rest.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>

#include <unistd.h>

#include "actor/durable.h"
#include "actor/runtime.h"
#include "channel/channel.h"
#include "mesh/mesh.h"
#include "ndslice/ndslice.h"

using namespace mb;

#define CHECK(cond)                                                        \
  do {                                                                     \
    if (!(cond)) {                                                         \
      std::fprintf(stderr, "CHECK failed at %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      std::exit(1);                                                        \
    }                                                                      \
  } while (0)

static void channel_many_posters() {
  char path[128];
  std::snprintf(path, sizeof(path), "unix:/tmp/mb200_stress_%d.sock", (int)getpid());
  ChannelAddr addr = ChannelAddr::parse(path);
  auto rx = serve(addr);
  auto tx = dial(rx->addr());
  constexpr int kThreads = 6, kPer = 400;
  std::atomic<int> failed{0};
  std::vector<std::thread> posters;
  for (int t = 0; t < kThreads; ++t)
    posters.emplace_back([&, t] {
      for (int i = 0; i < kPer; ++i) {
        Frame f;
        f.head = std::to_string(t) + ":" + std::to_string(i);
        // mix of small frames (caller-side send) and large ones (writer thread)
        if (i % 7 == 0) f.parts.emplace_back(std::string(40000 + 13 * i, (char)('a' + t)));
        tx->post(std::move(f), [&](Frame&&) { failed++; });
      }
    });
  std::vector<int> next(kThreads, 0);
  for (int got = 0; got < kThreads * kPer; ++got) {
    auto f = rx->recv(20000);
    CHECK(f.has_value());
    int t = std::atoi(f->head.c_str());
    int i = std::atoi(f->head.c_str() + f->head.find(':') + 1);
    CHECK(t >= 0 && t < kThreads);
    CHECK(i == next[t]);  // per-poster order survives the two send paths
    next[t]++;
    if (i % 7 == 0) {
      CHECK(f->parts.size() == 1 && f->parts[0].size() == (size_t)(40000 + 13 * i));
      CHECK(f->parts[0][100] == (char)('a' + t));
    }
  }
  for (auto& th : posters) th.join();
  CHECK(failed == 0);
  tx->close();
  std::puts("channel_many_posters ok");
}

// Connections cut while several threads post: everything still arrives, once, in order per
// poster (resend of the unacknowledged tail after reconnect, duplicates dropped by sequence).
static void channel_reconnect_under_load() {
  auto rx = serve(ChannelAddr::parse("tcp:127.0.0.1:0"));
  ChannelAddr addr = rx->addr();
  auto tx = dial(addr);
  constexpr int kThreads = 3, kPer = 300;
  std::atomic<int> failed{0};
  std::atomic<bool> done{false};
  std::thread cutter([&] {
    while (!done) {
      usleep(3000);
      debug_drop_connections(addr);
    }
  });
  std::vector<std::thread> posters;
  for (int t = 0; t < kThreads; ++t)
    posters.emplace_back([&, t] {
      for (int i = 0; i < kPer; ++i) {
        Frame f;
        f.head = std::to_string(t) + ":" + std::to_string(i);
        tx->post(std::move(f), [&](Frame&&) { failed++; });
        if (i % 16 == 0) usleep(500);
      }
    });
  std::vector<int> next(kThreads, 0);
  for (int got = 0; got < kThreads * kPer; ++got) {
    auto f = rx->recv(30000);
    CHECK(f.has_value());
    int t = std::atoi(f->head.c_str());
    int i = std::atoi(f->head.c_str() + f->head.find(':') + 1);
    CHECK(i == next[t]);
    next[t]++;
  }
  for (auto& th : posters) th.join();
  done = true;
  cutter.join();
  CHECK(failed == 0);
  CHECK(!rx->recv(200).has_value());  // nothing delivered twice
  tx->close();
  std::puts("channel_reconnect_under_load ok");
}

static std::atomic<long> g_handled{0};
static std::atomic<long> g_bytes{0};

static void mesh_concurrent_casts() {
  register_actor_type("counter", [](const std::shared_ptr<Proc>&, const std::string&,
                                    const std::string&) {
    ActorHooks h;
    h.on_message = [](Instance&, Envelope& env) {
      g_handled++;
      g_bytes += (long)env.data.size();
      for (auto& p : env.parts) g_bytes += (long)p.size();
    };
    return h;
  });
  auto router = std::make_shared<Router>();
  auto client = Proc::create(ProcId{"stress_client", 0}, router);
  router->bind_local(client);
  router->set_home(client);
  constexpr size_t kProcs = 24;
  auto pm = ProcMesh::allocate(make_local_alloc("stressmesh", kProcs, router), router, client, 20000);
  auto res = pm->spawn("counters", "counter", "", 20000);
  CHECK(res.size() == kProcs);
  for (auto& r : res) CHECK(r.ok);
  Slice all = Slice::row_major({kProcs});
  constexpr int kThreads = 4, kPer = 60;
  std::vector<std::thread> casters;
  long expect_bytes = 0;
  for (int t = 0; t < kThreads; ++t)
    for (int i = 0; i < kPer; ++i) expect_bytes += (long)kProcs * (i % 5 == 0 ? 10000 : 10);
  for (int t = 0; t < kThreads; ++t)
    casters.emplace_back([&, t] {
      ActorId sender{ProcId{"stress_client", 0}, "caster" + std::to_string(t), 0};
      for (int i = 0; i < kPer; ++i) {
        // small bodies ride in the routing header, large ones as an envelope part
        std::string body(i % 5 == 0 ? 10000 : 10, 'x');
        pm->cast("counters", all, Selection::all(Selection::t()), sender, std::move(body), {}, {}, all);
      }
    });
  for (auto& th : casters) th.join();
  const long want = (long)kProcs * kThreads * kPer;
  for (int spin = 0; spin < 2000 && g_handled.load() < want; ++spin) usleep(5000);
  CHECK(g_handled.load() == want);
  CHECK(g_bytes.load() == expect_bytes);
  auto led = pm->ledger(5000);
  CHECK(led.size() == kProcs);
  pm->stop_actor("counters", 5000);
  pm->stop();
  std::puts("mesh_concurrent_casts ok");
}

static void durable_and_lock() {
  char path[128];
  std::snprintf(path, sizeof(path), "/tmp/mb200_stress_%d.wal", (int)getpid());
  ::unlink(path);
  {
    auto log = std::make_shared<MessageLog>(path);
    std::vector<std::thread> ws;
    for (int t = 0; t < 4; ++t)
      ws.emplace_back([&, t] {
        for (int i = 0; i < 50; ++i) {
          Envelope e;
          e.sender = ActorId{ProcId{"w", t}, "a", 0};
          e.dest = PortId{ActorId{ProcId{"w", 0}, "b", 0}, 0};
          e.data = std::string(100 + i, 'd');
          log->append(e);
          if (i % 10 == 0) log->flush();
        }
      });
    for (auto& th : ws) th.join();
    log->flush();
    CHECK(log->next_seq() == 200);
    CHECK(log->read(150).size() == 50);
  }
  ::unlink(path);

  PreemptibleRwLock lock;
  std::atomic<int> inside_w{0}, inside_r{0}, bad{0};
  std::vector<std::thread> th;
  for (int t = 0; t < 4; ++t)
    th.emplace_back([&] {
      for (int i = 0; i < 300; ++i) {
        auto g = lock.read();
        inside_r++;
        if (inside_w.load()) bad++;
        for (int k = 0; k < 50 && !g.preempted(); ++k) std::this_thread::yield();
        inside_r--;
      }
    });
  th.emplace_back([&] {
    for (int i = 0; i < 100; ++i) {
      auto g = lock.write();
      inside_w++;
      if (inside_r.load()) bad++;
      inside_w--;
    }
  });
  for (auto& t : th) t.join();
  CHECK(bad == 0);
  std::puts("durable_and_lock ok");
}

int main() {
  channel_many_posters();
  channel_reconnect_under_load();
  mesh_concurrent_casts();
  durable_and_lock();
  std::puts("runtime_stress: all ok");
  return 0;
}
