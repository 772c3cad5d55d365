// Distributed queues of tensors (moodist.Queue).
//
// A queue lives on its location rank(s); any rank of the group may put into it or get from it.
// Semantics follow the reference (core/queue.cc, core/queue.h:36-58):
//   * local get pops directly; a remote get registers the caller as a waiter at the owner (Start),
//     the owner forwards the next item to it, and a timed-out getter withdraws with Stop / StopAck
//     (core/queue.cc:469-557, 999-1065);
//   * puts from one source are delivered in order: every arriving put reserves its slot before its
//     payload is complete, large payloads are pulled with a one-sided read and acknowledged with
//     QueueReadFinished, small ones travel inline in the 4 KiB message (core/cputhread.cc:4745-4866);
//   * transactions buffer puts per (source, key) at the owner and insert them atomically on commit
//     (core/queue.cc:721-762, 1067-1103);
//   * multicast queues (several locations): the first location fans every item out to the others
//     (core/queue.cc:876-890); each location serves gets from its own copy;
//   * named queues are created lazily on the owner by CreateQueueNamed (core/queue.cc:198-262).
// Queues are addressed on the wire by a 64-bit id handed out by the owner (the reference sends the raw
// address of its QueueStorage; an id keeps the message layout and cannot be dereferenced by mistake).
#pragma once

#include <cstdint>
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include "host_group.h"

namespace moodist {

struct QueueItem {
  Bytes data;
  int32_t dtype = 0;
  std::vector<int64_t> shape;
};

class QueueWork {
 public:
  virtual ~QueueWork() = default;
  // Blocks until the put's payload has left the caller's memory.
  virtual void wait() = 0;
};

class Queue {
 public:
  virtual ~Queue() = default;
  // `keep` pins the source memory until the payload has been sent / read.
  virtual std::unique_ptr<QueueWork> put(const void* data, size_t bytes, int32_t dtype,
                                         const std::vector<int64_t>& shape, uint32_t transaction,
                                         std::shared_ptr<void> keep) = 0;
  // nullopt when nothing arrived (non-blocking, or the timeout ran out). timeout_s < 0: forever.
  virtual std::optional<QueueItem> get(bool block, double timeout_s, size_t* queue_size) = 0;
  virtual size_t qsize() = 0;
  virtual bool wait(double timeout_s) = 0;
  virtual uint32_t transaction_begin() = 0;
  virtual void transaction_commit(uint32_t id) = 0;
  virtual void transaction_cancel(uint32_t id) = 0;
  virtual const std::string& name() const = 0;
};

class QueueManager {
 public:
  static std::unique_ptr<QueueManager> create(HostGroup& group);
  virtual ~QueueManager() = default;
  // Unnamed queues must be created in the same order on every rank (they get a sequential name).
  virtual std::shared_ptr<Queue> make_queue(const std::vector<int>& locations, bool streaming,
                                            const std::optional<std::string>& name) = 0;
};

}  // namespace moodist
