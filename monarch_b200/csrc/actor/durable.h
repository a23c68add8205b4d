// Write-ahead logging of messages, and a reader/writer lock whose readers can see that a
// writer is waiting.
//
// Parity: hyperactor/src/mailbox/durable_mailbox_sender.rs (DurableMailboxSender: append +
// flush to a MessageLog before the inner sender sees the message; replay after a crash),
// hyperactor/src/checkpoint.rs (Checkpointable: save/load of actor state),
// preempt_rwlock/src/lib.rs (PreemptibleRwLock used by SharedCell).
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <functional>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "actor/runtime.h"

namespace mb {

// Append-only log of envelopes.  Record = u64 sequence number, u32 length, payload (the
// envelope's contiguous encoding), u32 checksum of the payload.  A torn tail (a crash in the
// middle of an append) is detected by length/checksum and ignored by the reader.
class MessageLog {
 public:
  // Opens (creating if needed) and scans the file: next_seq() continues after the last
  // complete record.
  explicit MessageLog(const std::string& path);
  ~MessageLog();
  MessageLog(const MessageLog&) = delete;
  MessageLog& operator=(const MessageLog&) = delete;

  uint64_t append(const Envelope& env);  // returns the record's sequence number
  void flush();                          // fflush + fsync
  uint64_t next_seq() const { return next_seq_; }
  // Complete records with seq >= from, in order.
  std::vector<std::pair<uint64_t, Envelope>> read(uint64_t from = 0) const;
  const std::string& path() const { return path_; }

 private:
  std::string path_;
  std::FILE* f_ = nullptr;
  uint64_t next_seq_ = 0;
  mutable std::mutex mu_;
};

// Posts go to the log first; only a message that was appended and flushed is forwarded.  A
// message that could not be logged is handed to on_failed (the caller's undeliverable path).
class DurableMailboxSender : public MailboxSender {
 public:
  DurableMailboxSender(std::shared_ptr<MessageLog> log, std::shared_ptr<MailboxSender> inner,
                       std::function<void(Envelope, const std::string&)> on_failed = nullptr)
      : log_(std::move(log)), inner_(std::move(inner)), on_failed_(std::move(on_failed)) {}
  void post(Envelope env) override;
  // Re-post every logged message with seq >= from (recovery after the receiver restarted).
  size_t replay(uint64_t from = 0);

 private:
  std::shared_ptr<MessageLog> log_;
  std::shared_ptr<MailboxSender> inner_;
  std::function<void(Envelope, const std::string&)> on_failed_;
  std::mutex mu_;  // keeps log order == forwarding order
};

// Actor state that can be saved and restored (the reference's Checkpointable trait).
class Checkpointable {
 public:
  virtual ~Checkpointable() = default;
  virtual std::string save() const = 0;
  virtual void load(const std::string& blob) = 0;
};
// Atomic write (temp file + rename) / read of a checkpoint blob.
void write_checkpoint(const std::string& path, const std::string& blob);
bool read_checkpoint(const std::string& path, std::string* blob);

// Readers hold the lock for long stretches (e.g. while using a shared handle); a writer that
// arrives raises `preempted` so that cooperative readers let go at their next check.  Writers
// take precedence over new readers.
class PreemptibleRwLock {
 public:
  class ReadGuard {
   public:
    ReadGuard(ReadGuard&& o) noexcept : l_(o.l_) { o.l_ = nullptr; }
    ReadGuard(const ReadGuard&) = delete;
    ~ReadGuard() { release(); }
    bool preempted() const { return l_ && l_->writers_waiting_ > 0; }
    void release();

   private:
    friend class PreemptibleRwLock;
    explicit ReadGuard(PreemptibleRwLock* l) : l_(l) {}
    PreemptibleRwLock* l_;
  };
  class WriteGuard {
   public:
    WriteGuard(WriteGuard&& o) noexcept : l_(o.l_) { o.l_ = nullptr; }
    WriteGuard(const WriteGuard&) = delete;
    ~WriteGuard() { release(); }
    void release();

   private:
    friend class PreemptibleRwLock;
    explicit WriteGuard(PreemptibleRwLock* l) : l_(l) {}
    PreemptibleRwLock* l_;
  };
  ReadGuard read();
  // timeout_ms < 0 waits forever; returns false (and no lock) on timeout.
  bool try_read_for(int64_t timeout_ms, std::unique_ptr<ReadGuard>* out);
  WriteGuard write();
  int readers() const;
  int writers_waiting() const;

 private:
  mutable std::mutex mu_;
  std::condition_variable cv_;
  int readers_ = 0;
  bool writer_ = false;
  std::atomic<int> writers_waiting_{0};  // read without the mutex by ReadGuard::preempted
};

}  // namespace mb
