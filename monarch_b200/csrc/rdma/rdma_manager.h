// Per-proc RDMA manager: a native actor that owns the registry of buffers exported by the
// actors of its proc and answers the requests of remote RDMABuffer handles.
//
//   info   -> where the buffer lives (process, address, size, device, CUDA IPC handle)
//   read   -> the requested byte range of a host buffer, as an out-of-band frame part
//   write  -> copies the request's frame part into a host buffer
//   drop   -> forget the buffer
//
// GPU buffers are never served through the actor: the requester maps the owner's CUDA IPC
// handle and moves the bytes with a copy kernel over NVLink.  Host buffers of another process
// on the same box are read and written in place with process_vm_readv / process_vm_writev
// (one copy, no serialisation); the message path (read / write above) is the fallback when
// the kernel refuses that, and the path between boxes.
//
// Parity: monarch_rdma/src/rdma_manager_actor.rs:58-126 (RdmaManagerActor: request_buffer,
// release_buffer, request_queue_pair); the queue pairs and memory regions of the reference
// (ibverbs) correspond to the IPC handle and the process address here.
#pragma once
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <string>

#include "actor/runtime.h"

namespace mb {

struct RdmaBufferInfo {
  uint64_t id = 0;
  uint64_t addr = 0;        // address in the owner's process (host) or on its device (cuda)
  uint64_t nbytes = 0;
  bool cuda = false;
  int32_t device = -1;
  int64_t pid = 0;
  std::string host;
  std::string ipc_handle;   // 64 bytes for cuda buffers, empty for host buffers
  int64_t ipc_offset = 0;
  // Address (in the owner's process) of a word that holds `id` while the buffer is
  // registered and 0 after it was dropped: a one-sided reader checks it in the same system
  // call that moves the data, so a stale handle is refused without a round trip.
  uint64_t valid_addr = 0;

  std::string encode() const;
  static RdmaBufferInfo decode(const std::string& bytes);
};

class RdmaRegistry {
 public:
  uint64_t add(RdmaBufferInfo info);
  bool drop(uint64_t id);
  std::optional<RdmaBufferInfo> get(uint64_t id) const;
  size_t size() const;

 private:
  mutable std::mutex mu_;
  std::map<uint64_t, RdmaBufferInfo> bufs_;
  std::deque<uint64_t> valid_;   // one word per buffer ever registered; addresses are stable
  uint64_t next_ = 1;
};

// Header keys of the manager's protocol.
constexpr const char* kRdmaOp = "rdma_op";          // info | read | write | drop
constexpr const char* kRdmaId = "rdma_id";
constexpr const char* kRdmaOffset = "rdma_offset";
constexpr const char* kRdmaLen = "rdma_len";
constexpr const char* kRdmaReply = "rdma_reply";    // port of the requester
constexpr const char* kRdmaStatus = "rdma_status";  // ok | err (on replies)

// The manager actor's hooks.  `cuda_fallback` (may be empty) is asked to serve read / write
// of CUDA buffers over messages: it gets the request envelope and the buffer and returns the
// bytes read (read) or consumes env.parts[0] (write); an exception text is sent back as error.
using RdmaCudaFallback =
    std::function<std::string(const RdmaBufferInfo&, const std::string& op, uint64_t offset,
                              uint64_t len, const std::string* payload)>;
ActorHooks make_rdma_manager(std::shared_ptr<RdmaRegistry> reg, RdmaCudaFallback cuda_fallback);

// Let other processes of this user read and write this process's memory with
// process_vm_readv / process_vm_writev (PR_SET_PTRACER_ANY).  Idempotent.
void rdma_allow_peer_access();
// One-copy transfers between this process and `pid`.  When valid_addr != 0 the word there
// must equal `id` (checked in the owner's memory alongside the transfer).  0 on success,
// kRdmaStale when the buffer is no longer registered, else errno.
constexpr int kRdmaStale = -2;
int rdma_host_read(int64_t pid, uint64_t remote_addr, void* local, uint64_t n,
                   uint64_t valid_addr = 0, uint64_t id = 0);
int rdma_host_write(int64_t pid, uint64_t remote_addr, const void* local, uint64_t n,
                    uint64_t valid_addr = 0, uint64_t id = 0);

}  // namespace mb
