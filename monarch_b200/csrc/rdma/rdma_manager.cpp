#include "rdma/rdma_manager.h"

#include <errno.h>
#include <string.h>
#include <sys/prctl.h>
#include <sys/uio.h>
#include <unistd.h>

#include <stdexcept>

namespace mb {

std::string RdmaBufferInfo::encode() const {
  Writer w;
  w.u64(id);
  w.u64(addr);
  w.u64(nbytes);
  w.u8(cuda ? 1 : 0);
  w.i64(device);
  w.i64(pid);
  w.str(host);
  w.str(ipc_handle);
  w.i64(ipc_offset);
  w.u64(valid_addr);
  return std::move(w.buf);
}

RdmaBufferInfo RdmaBufferInfo::decode(const std::string& bytes) {
  Reader r(bytes);
  RdmaBufferInfo b;
  b.id = r.u64();
  b.addr = r.u64();
  b.nbytes = r.u64();
  b.cuda = r.u8() != 0;
  b.device = (int32_t)r.i64();
  b.pid = r.i64();
  b.host = r.str();
  b.ipc_handle = r.str();
  b.ipc_offset = r.i64();
  b.valid_addr = r.u64();
  return b;
}

uint64_t RdmaRegistry::add(RdmaBufferInfo info) {
  std::lock_guard<std::mutex> g(mu_);
  info.id = next_++;
  uint64_t id = info.id;
  valid_.push_back(id);
  info.valid_addr = reinterpret_cast<uint64_t>(&valid_.back());
  bufs_[id] = std::move(info);
  return id;
}
bool RdmaRegistry::drop(uint64_t id) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = bufs_.find(id);
  if (it == bufs_.end()) return false;
  if (it->second.valid_addr)
    __atomic_store_n(reinterpret_cast<uint64_t*>(it->second.valid_addr), 0, __ATOMIC_RELEASE);
  bufs_.erase(it);
  return true;
}
std::optional<RdmaBufferInfo> RdmaRegistry::get(uint64_t id) const {
  std::lock_guard<std::mutex> g(mu_);
  auto it = bufs_.find(id);
  if (it == bufs_.end()) return std::nullopt;
  return it->second;
}
size_t RdmaRegistry::size() const {
  std::lock_guard<std::mutex> g(mu_);
  return bufs_.size();
}

namespace {
uint64_t header_u64(const Envelope& env, const char* key, uint64_t dflt = 0) {
  auto it = env.headers.find(key);
  if (it == env.headers.end() || it->second.empty()) return dflt;
  return std::stoull(it->second);
}
}  // namespace

ActorHooks make_rdma_manager(std::shared_ptr<RdmaRegistry> reg, RdmaCudaFallback cuda_fallback) {
  ActorHooks h;
  h.on_message = [reg, cuda_fallback](Instance& self, Envelope& env) {
    auto rp = env.headers.find(kRdmaReply);
    if (rp == env.headers.end()) return;  // nobody to answer
    PortId reply = PortId::parse(rp->second);
    std::map<std::string, std::string> out_headers{{kHdrKind, "rdma_reply"}, {"no_return", "1"}};
    std::string data;
    std::vector<std::string> parts;
    try {
      const std::string op = env.headers.count(kRdmaOp) ? env.headers.at(kRdmaOp) : "";
      const uint64_t id = header_u64(env, kRdmaId);
      if (op == "drop") {
        reg->drop(id);
      } else {
        auto info = reg->get(id);
        if (!info)
          throw std::runtime_error("buffer " + std::to_string(id) + " is not registered on " +
                                   self.id().to_string() + " (dropped?)");
        if (op == "info") {
          data = info->encode();
        } else if (op == "read" || op == "write") {
          const uint64_t off = header_u64(env, kRdmaOffset);
          const uint64_t len = op == "read" ? header_u64(env, kRdmaLen)
                                            : (env.parts.empty() ? 0 : env.parts[0].size());
          if (off > info->nbytes || len > info->nbytes - off)
            throw std::runtime_error("range [" + std::to_string(off) + ", " +
                                     std::to_string(off + len) + ") outside a buffer of " +
                                     std::to_string(info->nbytes) + " bytes");
          if (info->cuda) {
            if (!cuda_fallback)
              throw std::runtime_error("GPU buffers are reached through their IPC mapping; this "
                                       "manager serves no GPU bytes over messages");
            std::string got = cuda_fallback(*info, op, off, len,
                                            op == "write" && !env.parts.empty() ? &env.parts[0]
                                                                                 : nullptr);
            if (op == "read") parts.push_back(std::move(got));
          } else if (op == "read") {
            // the owner keeps the tensor alive while it is registered: the address is valid
            parts.emplace_back(reinterpret_cast<const char*>(info->addr + off), (size_t)len);
          } else {
            if (len) memcpy(reinterpret_cast<void*>(info->addr + off), env.parts[0].data(), len);
          }
        } else {
          throw std::runtime_error("unknown rdma op '" + op + "'");
        }
      }
      out_headers[kRdmaStatus] = "ok";
    } catch (const std::exception& ex) {
      out_headers[kRdmaStatus] = "err";
      data = ex.what();
      parts.clear();
    }
    self.send(reply, std::move(data), std::move(out_headers), std::move(parts));
  };
  h.on_undeliverable = [](Instance&, Envelope&, const std::string&) { return true; };
  return h;
}

void rdma_allow_peer_access() {
#ifdef PR_SET_PTRACER
  ::prctl(PR_SET_PTRACER, PR_SET_PTRACER_ANY, 0, 0, 0);
#endif
}

namespace {
int check_valid(int64_t pid, uint64_t valid_addr, uint64_t id) {
  if (!valid_addr) return 0;
  uint64_t word = 0;
  struct iovec l{&word, sizeof(word)};
  struct iovec r{reinterpret_cast<void*>(valid_addr), sizeof(word)};
  ssize_t k = ::process_vm_readv((pid_t)pid, &l, 1, &r, 1, 0);
  if (k != (ssize_t)sizeof(word)) return errno ? errno : EIO;
  return word == id ? 0 : kRdmaStale;
}
}  // namespace

int rdma_host_read(int64_t pid, uint64_t remote_addr, void* local, uint64_t n,
                   uint64_t valid_addr, uint64_t id) {
  if (int rc = check_valid(pid, valid_addr, id)) return rc;
  uint64_t done = 0;
  while (done < n) {
    struct iovec l{static_cast<char*>(local) + done, (size_t)(n - done)};
    struct iovec r{reinterpret_cast<void*>(remote_addr + done), (size_t)(n - done)};
    ssize_t k = ::process_vm_readv((pid_t)pid, &l, 1, &r, 1, 0);
    if (k < 0) return errno ? errno : EIO;
    if (k == 0) return EIO;
    done += (uint64_t)k;
  }
  return 0;
}

int rdma_host_write(int64_t pid, uint64_t remote_addr, const void* local, uint64_t n,
                    uint64_t valid_addr, uint64_t id) {
  if (int rc = check_valid(pid, valid_addr, id)) return rc;
  uint64_t done = 0;
  while (done < n) {
    struct iovec l{const_cast<char*>(static_cast<const char*>(local)) + done, (size_t)(n - done)};
    struct iovec r{reinterpret_cast<void*>(remote_addr + done), (size_t)(n - done)};
    ssize_t k = ::process_vm_writev((pid_t)pid, &l, 1, &r, 1, 0);
    if (k < 0) return errno ? errno : EIO;
    if (k == 0) return EIO;
    done += (uint64_t)k;
  }
  return 0;
}

}  // namespace mb
