// Content manifest of a directory tree for workspace synchronisation: every regular file
// under a root with a 128-bit content hash, computed by a few threads without the GIL.
//
// Parity: hyperactor_mesh/src/code_sync (the reference delegates the diff to an rsync
// daemon; here the client and every proc compare manifests and only changed files travel).
#include "mesh/tree_manifest.h"

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <filesystem>
#include <thread>

namespace mb {

namespace {

inline uint64_t rotl(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
inline uint64_t mix(uint64_t k) {
  k ^= k >> 33;
  k *= 0xff51afd7ed558ccdULL;
  k ^= k >> 33;
  k *= 0xc4ceb9fe1a85ec53ULL;
  k ^= k >> 33;
  return k;
}

// A streaming 128-bit hash: two lanes over 16-byte blocks with cross-lane feedback and a
// length-dependent finaliser.  Not cryptographic; it only has to make an unnoticed change of
// a source file improbable (two files are compared by size and by these 128 bits).
struct Hash128 {
  uint64_t h1 = 0x9e3779b97f4a7c15ULL, h2 = 0xc2b2ae3d27d4eb4fULL, len = 0;
  unsigned char tail[16];
  size_t ntail = 0;
  void block(const unsigned char* p) {
    uint64_t k1, k2;
    std::memcpy(&k1, p, 8);
    std::memcpy(&k2, p + 8, 8);
    k1 *= 0x87c37b91114253d5ULL; k1 = rotl(k1, 31); k1 *= 0x4cf5ad432745937fULL; h1 ^= k1;
    h1 = rotl(h1, 27); h1 += h2; h1 = h1 * 5 + 0x52dce729;
    k2 *= 0x4cf5ad432745937fULL; k2 = rotl(k2, 33); k2 *= 0x87c37b91114253d5ULL; h2 ^= k2;
    h2 = rotl(h2, 31); h2 += h1; h2 = h2 * 5 + 0x38495ab5;
  }
  void update(const unsigned char* p, size_t n) {
    len += n;
    if (ntail) {
      const size_t take = std::min(n, 16 - ntail);
      std::memcpy(tail + ntail, p, take);
      ntail += take; p += take; n -= take;
      if (ntail < 16) return;
      block(tail);
      ntail = 0;
    }
    while (n >= 16) { block(p); p += 16; n -= 16; }
    if (n) { std::memcpy(tail, p, n); ntail = n; }
  }
  std::string hex() {
    if (ntail) {
      std::memset(tail + ntail, 0, 16 - ntail);
      block(tail);
    }
    h1 ^= len; h2 ^= len;
    h1 += h2; h2 += h1;
    h1 = mix(h1); h2 = mix(h2);
    h1 += h2; h2 += h1;
    char buf[40];
    std::snprintf(buf, sizeof buf, "%016llx%016llx", (unsigned long long)h1, (unsigned long long)h2);
    return buf;
  }
};

bool ends_with(const std::string& s, const std::string& suf) {
  return s.size() >= suf.size() && s.compare(s.size() - suf.size(), suf.size(), suf) == 0;
}

}  // namespace

std::string hash_file_128(const std::string& path, bool* ok) {
  *ok = false;
  int fd = ::open(path.c_str(), O_RDONLY | O_CLOEXEC);
  if (fd < 0) return "";
  Hash128 h;
  std::vector<unsigned char> buf(1 << 20);
  while (true) {
    ssize_t n = ::read(fd, buf.data(), buf.size());
    if (n < 0) {
      if (errno == EINTR) continue;
      ::close(fd);
      return "";
    }
    if (n == 0) break;
    h.update(buf.data(), (size_t)n);
  }
  ::close(fd);
  *ok = true;
  return h.hex();
}

std::vector<ManifestEntry> tree_manifest(const std::string& root,
                                         const std::vector<std::string>& skip_dirs,
                                         const std::vector<std::string>& skip_suffixes,
                                         uint64_t max_file_bytes, int threads) {
  namespace fs = std::filesystem;
  std::vector<ManifestEntry> out;
  std::error_code ec;
  const fs::path base(root);
  if (!fs::is_directory(base, ec)) return out;
  for (auto it = fs::recursive_directory_iterator(
           base, fs::directory_options::skip_permission_denied, ec);
       !ec && it != fs::recursive_directory_iterator(); it.increment(ec)) {
    const fs::directory_entry& e = *it;
    const std::string name = e.path().filename().string();
    if (e.is_directory(ec)) {
      if (e.is_symlink(ec) ||
          std::find(skip_dirs.begin(), skip_dirs.end(), name) != skip_dirs.end())
        it.disable_recursion_pending();
      continue;
    }
    if (!e.is_regular_file(ec)) continue;
    bool skip = false;
    for (const auto& suf : skip_suffixes)
      if (ends_with(name, suf)) { skip = true; break; }
    if (skip) continue;
    const uint64_t size = (uint64_t)e.file_size(ec);
    if (ec || size > max_file_bytes) { ec.clear(); continue; }
    ManifestEntry m;
    m.rel = fs::relative(e.path(), base, ec).string();
    if (ec) { ec.clear(); continue; }
    m.size = size;
    out.push_back(std::move(m));
  }
  std::sort(out.begin(), out.end(),
            [](const ManifestEntry& a, const ManifestEntry& b) { return a.rel < b.rel; });
  // hash in parallel: threads take files from a shared counter
  int n_thr = std::max(1, std::min(threads, (int)out.size()));
  std::atomic<size_t> next{0};
  auto work = [&]() {
    while (true) {
      const size_t i = next.fetch_add(1);
      if (i >= out.size()) return;
      bool ok = false;
      out[i].hash = hash_file_128((base / out[i].rel).string(), &ok);
      out[i].ok = ok;
    }
  };
  std::vector<std::thread> pool;
  for (int t = 1; t < n_thr; ++t) pool.emplace_back(work);
  work();
  for (auto& t : pool) t.join();
  out.erase(std::remove_if(out.begin(), out.end(), [](const ManifestEntry& m) { return !m.ok; }),
            out.end());
  return out;
}

}  // namespace mb
