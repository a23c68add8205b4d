// Content manifest of a directory tree (workspace synchronisation).
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace mb {

struct ManifestEntry {
  std::string rel;    // path relative to the root
  uint64_t size = 0;
  std::string hash;   // 32 hex digits
  bool ok = false;
};

// 128-bit content hash of one file (hex); *ok is false when it cannot be read.
std::string hash_file_128(const std::string& path, bool* ok);

// Every regular file under `root` (not following directory symlinks), except directories
// named in `skip_dirs`, files ending in one of `skip_suffixes` and files larger than
// `max_file_bytes`; sorted by path; hashed by up to `threads` threads.
std::vector<ManifestEntry> tree_manifest(const std::string& root,
                                         const std::vector<std::string>& skip_dirs,
                                         const std::vector<std::string>& skip_suffixes,
                                         uint64_t max_file_bytes, int threads);

}  // namespace mb
