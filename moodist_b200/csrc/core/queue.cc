#include "queue.h"

#include <condition_variable>
#include <cstring>
#include <deque>
#include <list>
#include <map>
#include <mutex>

#include "log.h"
#include "tcp_transport.h"

namespace moodist {
namespace {

constexpr size_t kInlineLimit = 3500;              // payloads up to this size ride inside the 4 KiB message
constexpr uint32_t kFanoutMarker = 0xffffffffu;    // transactionKey of a copy sent by the first location

enum GetOp : uint8_t { kGetStart = 0, kGetStop = 1, kGetStopAck = 2, kGetSize = 3, kGetSizeReply = 4 };
enum TxOp : uint8_t { kTxCommit = 0, kTxCancel = 1 };

uint64_t name_id(const std::string& name) {  // FNV-1a, never 0
  uint64_t h = 1469598103934665603ull;
  for (unsigned char c : name) h = (h ^ c) * 1099511628211ull;
  return h ? h : 1;
}

struct Sync {
  std::mutex mu;
  std::condition_variable cv;
  bool done = false;
  std::atomic<bool> done_hint{false};  // set with `done`; polled briefly before a waiter goes to sleep
  std::string error;
  void finish(std::string err = {}) {
    std::lock_guard<std::mutex> lk(mu);
    done = true;
    error = std::move(err);
    done_hint.store(true, std::memory_order_release);
    cv.notify_all();
  }
  // false on timeout
  // `interruptible`: between slices pending signal handlers get to run, and what they raise (Ctrl-C) comes out of
  // here; for waits that may last as long as the caller likes, not for the short round trips to the engine thread
  bool wait(double timeout_s, bool interruptible = false) {
    spin_until(done_hint, spin_microseconds());
    const double deadline = timeout_s < 0 ? -1 : now_seconds() + timeout_s;
    std::unique_lock<std::mutex> lk(mu);
    while (!done) {
      double slice = 0.2;
      if (deadline >= 0) {
        double left = deadline - now_seconds();
        if (left <= 0) return false;
        slice = std::min(slice, left);
      }
      cv.wait_for(lk, std::chrono::duration<double>(slice), [&] { return done; });
      if (done) break;
      if (interruptible) {
        lk.unlock();
        check_interrupt();
        lk.lock();
      }
    }
    return true;
  }
};

struct Slot {
  bool ready = false;
  QueueItem item;
};

struct GetWait : Sync {
  std::optional<QueueItem> item;
  size_t size_after = 0;
  bool cancelled = false;
};

struct RemoteGetter {
  int rank;
  uint64_t proxy;
  uint32_t key;
};

struct Waiter {
  std::shared_ptr<GetWait> local;  // or
  std::optional<RemoteGetter> remote;
};

struct Storage {
  uint64_t id = 0;
  std::string name;
  std::vector<int> locations;
  std::deque<std::shared_ptr<Slot>> items;
  std::list<Waiter> waiters;
  std::list<std::shared_ptr<Sync>> nonempty_waiters;
  std::map<std::pair<int, uint32_t>, std::vector<std::shared_ptr<Slot>>> transactions;
  size_t ready_count() const {
    size_t n = 0;
    for (auto& s : items) {
      if (!s->ready) break;
      ++n;
    }
    return n;
  }
};

struct Outgoing {
  std::shared_ptr<void> keep;
  std::shared_ptr<Slot> slot;
  uint32_t rkey = 0;
  std::shared_ptr<Sync> done;
};

class ManagerImpl;

class WorkImpl final : public QueueWork {
 public:
  explicit WorkImpl(std::shared_ptr<Sync> s) : sync_(std::move(s)) {}
  void wait() override {
    sync_->wait(-1);
    if (!sync_->error.empty()) fail("moodist.Queue: put failed: " + sync_->error);
  }

 private:
  std::shared_ptr<Sync> sync_;
};

class ManagerImpl final : public QueueManager {
 public:
  explicit ManagerImpl(HostGroup& g) : g_(g) {
    // in one call: what peers sent before this rank made its first queue is replayed in arrival order over all types
    std::vector<std::pair<uint32_t, HostGroup::Handler>> handlers;
    handlers.emplace_back(kOpCreateQueueNamed, [this](int src, Reader& r) { on_create(src, r); });
    handlers.emplace_back(kOpCreateQueueNamedResult, [](int, Reader&) {});
    handlers.emplace_back(kOpQueuePut, [this](int src, Reader& r) { on_put(src, r); });
    handlers.emplace_back(kOpQueueReadFinished, [this](int src, Reader& r) { on_read_finished(src, r); });
    handlers.emplace_back(kOpQueueGet, [this](int src, Reader& r) { on_get(src, r); });
    handlers.emplace_back(kOpQueueTransaction, [this](int src, Reader& r) { on_transaction(src, r); });
    g_.set_handlers(std::move(handlers));
  }

  std::shared_ptr<Queue> make_queue(const std::vector<int>& locations, bool streaming,
                                    const std::optional<std::string>& name) override;

  // ---- engine-thread helpers used by QueueImpl ----
  HostGroup& g_;
  std::map<uint64_t, Storage> storages_;                 // queues located on this rank
  std::map<uint64_t, std::deque<QueueItem>> inbox_;      // items forwarded to this rank's remote gets, by queue id
  std::map<uint64_t, std::shared_ptr<GetWait>> getting_; // outstanding remote get per queue id
  std::map<uint32_t, std::shared_ptr<Sync>> stop_acks_;  // by get key
  std::map<uint32_t, std::pair<std::shared_ptr<Sync>, size_t*>> size_replies_;
  std::map<uint32_t, Outgoing> outgoing_;                // puts whose payload is still to be read, by putKey
  uint32_t next_put_key_ = 1, next_get_key_ = 1, next_tx_key_ = 1;
  uint32_t unnamed_counter_ = 0;

  Storage& storage(uint64_t id, const std::string& name, const std::vector<int>& locations) {
    auto it = storages_.find(id);
    if (it == storages_.end()) {
      Storage s;
      s.id = id;
      s.name = name;
      s.locations = locations;
      it = storages_.emplace(id, std::move(s)).first;
    } else if (it->second.locations.empty()) {
      it->second.locations = locations;
      it->second.name = name;
    }
    return it->second;
  }

  void on_create(int src, Reader& r) {
    uint32_t key, location;
    std::string name;
    bool streaming;
    std::vector<int> locations;
    r(key, name, location, streaming, locations);
    if (streaming) log_error("moodist.Queue: streaming queues are not supported; '%s' behaves as a normal queue", name.c_str());
    Storage& s = storage(name_id(name), name, locations);
    g_.send_message(src, kOpCreateQueueNamedResult, encode(key, (uint64_t)s.id, location, streaming));
  }

  // Build a QueuePut message (reference layout, core/cputhread.cc:4745-4768).
  Bytes put_message(uint64_t queue, uint64_t addr, uint64_t bytes, uint32_t put_key, uint32_t get_key, uint32_t tx_key,
                    uint64_t qsize, uint32_t rkey, const QueueItem* meta, int32_t dtype,
                    const std::vector<int64_t>& shape, const void* inline_data) {
    Writer w;
    uint32_t rkeys[4] = {rkey, 0, 0, 0};
    w(queue, addr, bytes, put_key, get_key, tx_key, qsize);
    w.raw(rkeys, sizeof(rkeys));
    w(dtype, (uint8_t)shape.size());
    for (int64_t d : shape) w(d);
    w((bool)(inline_data != nullptr || bytes == 0));
    if (inline_data && bytes) w.raw(inline_data, bytes);
    (void)meta;
    return std::move(w.out);
  }

  // Send one item to `dst` addressed to queue id `queue` there.
  void send_item(int dst, uint64_t queue, std::shared_ptr<Slot> slot, uint32_t get_key, uint32_t tx_key, uint64_t qsize) {
    const QueueItem& it = slot->item;
    uint32_t put_key = next_put_key_++;
    if (it.data.size() <= kInlineLimit) {
      g_.send_message(dst, kOpQueuePut,
                      put_message(queue, 0, it.data.size(), put_key, get_key, tx_key, qsize, 0, &it, it.dtype, it.shape,
                                  it.data.empty() ? nullptr : it.data.data()));
      return;
    }
    Outgoing o;
    o.slot = slot;
    o.rkey = MrTable::instance().add((void*)it.data.data(), it.data.size());
    outgoing_[put_key] = o;
    g_.send_message(dst, kOpQueuePut,
                    put_message(queue, (uint64_t)(uintptr_t)it.data.data(), it.data.size(), put_key, get_key, tx_key, qsize,
                                o.rkey, &it, it.dtype, it.shape, nullptr));
  }

  // Hand ready items at the head of the queue to whoever is waiting, in arrival order.
  void serve(Storage& s) {
    while (!s.items.empty() && s.items.front()->ready && !s.waiters.empty()) {
      Waiter w = std::move(s.waiters.front());
      s.waiters.pop_front();
      if (w.local) {
        if (w.local->cancelled) continue;
        std::shared_ptr<Slot> slot = s.items.front();
        s.items.pop_front();
        w.local->item = std::move(slot->item);
        w.local->size_after = s.ready_count();
        w.local->finish();
      } else {
        std::shared_ptr<Slot> slot = s.items.front();
        s.items.pop_front();
        send_item(w.remote->rank, s.id, slot, w.remote->key, 0, s.ready_count());
      }
    }
    if (!s.items.empty() && s.items.front()->ready) {
      for (auto& w : s.nonempty_waiters) w->finish();
      s.nonempty_waiters.clear();
    }
  }

  // A slot of a queue located here became ready (or was appended ready).
  void slot_ready(Storage& s, const std::shared_ptr<Slot>& slot, bool fan_out) {
    if (fan_out && s.locations.size() > 1 && s.locations[0] == g_.rank()) {
      for (size_t i = 1; i < s.locations.size(); ++i) {
        auto copy = std::make_shared<Slot>(*slot);
        send_item(s.locations[i], s.id, copy, 0, kFanoutMarker, 0);
      }
    }
    serve(s);
  }

  void on_put(int src, Reader& r) {
    uint64_t queue, addr, bytes, qsize;
    uint32_t put_key, get_key, tx_key, rkeys[4];
    int32_t dtype;
    uint8_t ndim;
    r(queue, addr, bytes, put_key, get_key, tx_key, qsize);
    r.raw(rkeys, sizeof(rkeys));
    r(dtype, ndim);
    std::vector<int64_t> shape(ndim);
    for (auto& d : shape) r(d);
    bool inlined = r.read<bool>();
    auto slot = std::make_shared<Slot>();
    slot->item.dtype = dtype;
    slot->item.shape = std::move(shape);

    // where the item goes once complete
    std::function<void()> deliver;
    if (get_key != 0) {
      // the owner's answer to this rank's remote get
      deliver = [this, queue, slot, qsize] {
        auto it = getting_.find(queue);
        if (it != getting_.end() && !it->second->cancelled) {
          it->second->item = std::move(slot->item);
          it->second->size_after = qsize;
          it->second->finish();
          getting_.erase(it);
        } else {
          inbox_[queue].push_back(std::move(slot->item));  // the getter gave up meanwhile: keep it for the next get
        }
      };
    } else {
      Storage& s = storage(queue, "", {});
      bool fan_out = tx_key != kFanoutMarker;
      if (tx_key != 0 && tx_key != kFanoutMarker) {
        s.transactions[{src, tx_key}].push_back(slot);
        deliver = [this, queue] { serve(storages_[queue]); };
      } else {
        s.items.push_back(slot);
        deliver = [this, queue, slot, fan_out] { slot_ready(storages_[queue], slot, fan_out); };
      }
    }

    if (inlined) {
      const uint8_t* b = r.take(bytes);
      slot->item.data.assign(b, b + bytes);
      slot->ready = true;
      deliver();
      return;
    }
    slot->item.data.resize(bytes);
    g_.post_read(src, slot->item.data.data(), bytes, rkeys[0], addr, [this, src, put_key, slot, deliver](bool ok) {
      if (!ok) log_error("moodist.Queue: reading a put payload from rank %d failed", src);
      g_.send_message(src, kOpQueueReadFinished, encode(put_key));
      slot->ready = true;
      deliver();
    });
  }

  void on_read_finished(int, Reader& r) {
    uint32_t put_key = r.read<uint32_t>();
    auto it = outgoing_.find(put_key);
    if (it == outgoing_.end()) return;
    MrTable::instance().remove(it->second.rkey);
    if (it->second.done) it->second.done->finish();
    outgoing_.erase(it);
  }

  void on_get(int src, Reader& r) {
    uint8_t op;
    uint64_t remote, local;
    uint32_t key;
    r(op, remote, local, key);
    switch (op) {
      case kGetStart: {
        Storage& s = storage(remote, "", {});
        Waiter w;
        w.remote = RemoteGetter{src, local, key};
        s.waiters.push_back(std::move(w));
        serve(s);
        break;
      }
      case kGetStop: {
        Storage& s = storage(remote, "", {});
        for (auto it = s.waiters.begin(); it != s.waiters.end(); ++it) {
          if (it->remote && it->remote->rank == src && it->remote->key == key) {
            s.waiters.erase(it);
            break;
          }
        }
        g_.send_message(src, kOpQueueGet, encode((uint8_t)kGetStopAck, remote, local, key));
        break;
      }
      case kGetStopAck: {
        auto it = stop_acks_.find(key);
        if (it != stop_acks_.end()) {
          it->second->finish();
          stop_acks_.erase(it);
        }
        break;
      }
      case kGetSize: {
        Storage& s = storage(remote, "", {});
        g_.send_message(src, kOpQueueGet, encode((uint8_t)kGetSizeReply, remote, (uint64_t)s.ready_count(), key));
        break;
      }
      case kGetSizeReply: {
        auto it = size_replies_.find(key);
        if (it != size_replies_.end()) {
          *it->second.second = (size_t)local;
          it->second.first->finish();
          size_replies_.erase(it);
        }
        break;
      }
    }
  }

  void on_transaction(int src, Reader& r) {
    uint64_t queue;
    uint8_t op;
    uint32_t key;
    r(queue, op, key);
    apply_transaction(storage(queue, "", {}), src, op, key);
  }

  void apply_transaction(Storage& s, int src, uint8_t op, uint32_t key) {
    auto it = s.transactions.find({src, key});
    if (it == s.transactions.end()) return;
    auto slots = std::move(it->second);
    s.transactions.erase(it);
    if (op == kTxCancel) return;
    for (auto& slot : slots) s.items.push_back(slot);
    // fan-out happens per slot once it is ready; slots already ready are handled here
    for (auto& slot : slots)
      if (slot->ready && s.locations.size() > 1 && s.locations[0] == g_.rank())
        for (size_t i = 1; i < s.locations.size(); ++i) send_item(s.locations[i], s.id, std::make_shared<Slot>(*slot), 0, kFanoutMarker, 0);
    serve(s);
  }
};

class QueueImpl final : public Queue {
 public:
  QueueImpl(ManagerImpl& m, std::string name, std::vector<int> locations)
      : m_(m), name_(std::move(name)), locations_(std::move(locations)), id_(name_id(name_)) {
    int me = m_.g_.rank();
    local_ = false;
    for (int l : locations_) local_ |= l == me;
    // puts go to the first location (it fans out); gets are served by the local copy when there is one
    put_target_ = locations_[0];
    get_target_ = local_ ? me : locations_[0];
  }

  const std::string& name() const override { return name_; }

  std::unique_ptr<QueueWork> put(const void* data, size_t bytes, int32_t dtype, const std::vector<int64_t>& shape,
                                 uint32_t transaction, std::shared_ptr<void> keep) override {
    check();
    auto done = std::make_shared<Sync>();
    int me = m_.g_.rank();
    if (put_target_ == me) {
      auto slot = std::make_shared<Slot>();
      slot->item.dtype = dtype;
      slot->item.shape = shape;
      slot->item.data.assign((const uint8_t*)data, (const uint8_t*)data + bytes);
      slot->ready = true;
      m_.g_.run_on_engine([this, slot, transaction, me] {
        Storage& s = m_.storage(id_, name_, locations_);
        if (transaction != 0) {
          s.transactions[{me, transaction}].push_back(slot);
        } else {
          s.items.push_back(slot);
          m_.slot_ready(s, slot, true);
        }
      });
      done->finish();
      return std::make_unique<WorkImpl>(done);
    }
    if (bytes <= kInlineLimit) {
      Bytes copy((const uint8_t*)data, (const uint8_t*)data + bytes);
      m_.g_.run_on_engine([this, copy = std::move(copy), dtype, shape, transaction]() mutable {
        uint32_t put_key = m_.next_put_key_++;
        m_.g_.send_message(put_target_, kOpQueuePut,
                           m_.put_message(id_, 0, copy.size(), put_key, 0, transaction, 0, 0, nullptr, dtype, shape,
                                          copy.empty() ? nullptr : copy.data()));
      });
      done->finish();
      return std::make_unique<WorkImpl>(done);
    }
    m_.g_.run_on_engine([this, data, bytes, dtype, shape, transaction, keep, done] {
      uint32_t put_key = m_.next_put_key_++;
      Outgoing o;
      o.keep = keep;
      o.done = done;
      o.rkey = MrTable::instance().add(const_cast<void*>(data), bytes);
      m_.outgoing_[put_key] = o;
      m_.g_.send_message(put_target_, kOpQueuePut,
                         m_.put_message(id_, (uint64_t)(uintptr_t)data, bytes, put_key, 0, transaction, 0, o.rkey, nullptr,
                                        dtype, shape, nullptr));
    });
    return std::make_unique<WorkImpl>(done);
  }

  std::optional<QueueItem> get(bool block, double timeout_s, size_t* queue_size) override {
    check();
    auto gw = std::make_shared<GetWait>();
    int me = m_.g_.rank();
    if (get_target_ == me) {
      m_.g_.run_on_engine([this, gw, block] {
        Storage& s = m_.storage(id_, name_, locations_);
        if (!s.items.empty() && s.items.front()->ready && s.waiters.empty()) {
          gw->item = std::move(s.items.front()->item);
          s.items.pop_front();
          gw->size_after = s.ready_count();
          gw->finish();
        } else if (!block) {
          gw->finish();
        } else {
          Waiter w;
          w.local = gw;
          s.waiters.push_back(std::move(w));
          m_.serve(s);
        }
      });
      std::exception_ptr interrupted;
      if (!wait_or_note(*gw, block ? timeout_s : -1, interrupted)) {
        // timed out (or interrupted by a signal): withdraw on the engine thread, then look once more (the item may
        // have just arrived)
        auto fin = std::make_shared<Sync>();
        m_.g_.run_on_engine([gw, fin] {
          gw->cancelled = true;
          fin->finish();
        });
        fin->wait(-1);
        if (interrupted) {
          give_back(gw);
          std::rethrow_exception(interrupted);
        }
        std::lock_guard<std::mutex> lk(gw->mu);
        if (!gw->done) return std::nullopt;
      }
      check_error();
      if (queue_size) *queue_size = gw->size_after;
      return std::move(gw->item);
    }
    // remote queue
    uint32_t key = 0;
    auto started = std::make_shared<Sync>();
    m_.g_.run_on_engine([this, gw, block, &key, started] {
      auto& box = m_.inbox_[id_];
      if (!box.empty()) {
        gw->item = std::move(box.front());
        box.pop_front();
        gw->finish();
      } else {
        key = m_.next_get_key_++;
        m_.getting_[id_] = gw;
        m_.g_.send_message(get_target_, kOpQueueGet, encode((uint8_t)kGetStart, id_, id_, key));
      }
      (void)block;
      started->finish();
    });
    started->wait(-1);
    // A non-blocking remote get still has to ask the owner; give the round trip a short moment.
    double limit = block ? timeout_s : 0.05;
    std::exception_ptr interrupted;
    if (!wait_or_note(*gw, limit, interrupted)) {
      auto ack = std::make_shared<Sync>();
      m_.g_.run_on_engine([this, key, ack] {
        m_.stop_acks_[key] = ack;
        m_.g_.send_message(get_target_, kOpQueueGet, encode((uint8_t)kGetStop, id_, id_, key));
      });
      ack->wait(10.0);  // anything forwarded before the owner saw Stop has arrived by now
      auto fin = std::make_shared<Sync>();
      m_.g_.run_on_engine([this, gw, fin] {
        if (!gw->done) {
          gw->cancelled = true;
          m_.getting_.erase(id_);
        }
        fin->finish();
      });
      fin->wait(-1);
      if (interrupted) {
        give_back(gw);
        std::rethrow_exception(interrupted);
      }
      std::lock_guard<std::mutex> lk(gw->mu);
      if (!gw->done) return std::nullopt;
    }
    check_error();
    if (queue_size) *queue_size = gw->size_after;
    return std::move(gw->item);
  }

  // The long wait of a get: false on timeout, and also when a signal handler raised in the meantime (the exception
  // is kept for the caller to rethrow once the request has been withdrawn).
  static bool wait_or_note(Sync& s, double timeout_s, std::exception_ptr& interrupted) {
    try {
      return s.wait(timeout_s, true);
    } catch (...) {
      interrupted = std::current_exception();
      return false;
    }
  }

  // An item that arrived for a get which is being abandoned goes back to the head of the line.
  void give_back(const std::shared_ptr<GetWait>& gw) {
    std::shared_ptr<QueueItem> item;
    {
      std::lock_guard<std::mutex> lk(gw->mu);
      if (!gw->done || !gw->item) return;
      item = std::make_shared<QueueItem>(std::move(*gw->item));
      gw->item.reset();
    }
    bool local = get_target_ == m_.g_.rank();
    m_.g_.run_on_engine([this, item, local] {
      if (local) {
        Storage& st = m_.storage(id_, name_, locations_);
        auto slot = std::make_shared<Slot>();
        slot->item = std::move(*item);
        slot->ready = true;
        st.items.push_front(slot);
        m_.serve(st);
      } else {
        m_.inbox_[id_].push_front(std::move(*item));
      }
    });
  }

  size_t qsize() override {
    check();
    int me = m_.g_.rank();
    auto s = std::make_shared<Sync>();
    auto out = std::make_shared<size_t>(0);
    if (get_target_ == me) {
      m_.g_.run_on_engine([this, s, out] {
        *out = m_.storage(id_, name_, locations_).ready_count();
        s->finish();
      });
    } else {
      m_.g_.run_on_engine([this, s, out] {
        uint32_t key = m_.next_get_key_++;
        m_.size_replies_[key] = {s, out.get()};
        *out = m_.inbox_[id_].size();
        m_.g_.send_message(get_target_, kOpQueueGet, encode((uint8_t)kGetSize, id_, id_, key));
      });
    }
    if (!s->wait(30.0)) fail("moodist.Queue: qsize timed out");
    return *out + (get_target_ == me ? 0 : pending_inbox());
  }

  bool wait(double timeout_s) override {
    check();
    int me = m_.g_.rank();
    if (get_target_ == me) {
      auto s = std::make_shared<Sync>();
      m_.g_.run_on_engine([this, s] {
        Storage& st = m_.storage(id_, name_, locations_);
        if (!st.items.empty() && st.items.front()->ready)
          s->finish();
        else
          st.nonempty_waiters.push_back(s);
      });
      return s->wait(timeout_s, true);
    }
    double deadline = now_seconds() + (timeout_s < 0 ? 1e18 : timeout_s);
    for (;;) {
      if (qsize() > 0) return true;
      if (now_seconds() >= deadline) return false;
      check_interrupt();
      std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
  }

  uint32_t transaction_begin() override {
    auto s = std::make_shared<Sync>();
    auto out = std::make_shared<uint32_t>(0);
    m_.g_.run_on_engine([this, s, out] {
      *out = m_.next_tx_key_++;
      if (*out == 0 || *out == kFanoutMarker) *out = m_.next_tx_key_ = 1;
      s->finish();
    });
    s->wait(-1);
    return *out;
  }
  void transaction_commit(uint32_t id) override { transaction_end(id, kTxCommit); }
  void transaction_cancel(uint32_t id) override { transaction_end(id, kTxCancel); }

 private:
  void transaction_end(uint32_t id, uint8_t op) {
    int me = m_.g_.rank();
    m_.g_.run_on_engine([this, id, op, me] {
      if (put_target_ == me)
        m_.apply_transaction(m_.storage(id_, name_, locations_), me, op, id);
      else
        m_.g_.send_message(put_target_, kOpQueueTransaction, encode(id_, op, id));
    });
  }
  size_t pending_inbox() { return 0; }
  void check() {
    if (m_.g_.in_error()) fail("moodist.Queue: process group is in an error state: " + m_.g_.error_text());
  }
  void check_error() {}

  ManagerImpl& m_;
  std::string name_;
  std::vector<int> locations_;
  uint64_t id_;
  bool local_ = false;
  int put_target_ = 0, get_target_ = 0;
};

std::shared_ptr<Queue> ManagerImpl::make_queue(const std::vector<int>& locations, bool streaming,
                                               const std::optional<std::string>& name) {
  if (locations.empty()) fail("moodist.Queue: location list is empty");
  for (int l : locations)
    if (l < 0 || l >= g_.world()) fail(strf("moodist.Queue: location %d is not a rank of this group", l));
  if (streaming) fail("moodist.Queue: streaming queues are not supported");
  std::string n = name ? *name : strf("%s.unnamed.%u", g_.name().c_str(), unnamed_counter_++);
  auto q = std::make_shared<QueueImpl>(*this, n, locations);
  // make sure every location knows the queue (name, locations) before the first put or get reaches it
  int me = g_.rank();
  g_.run_on_engine([this, n, locations, me] {
    for (int l : locations) {
      if (l == me)
        storage(name_id(n), n, locations);
      else
        g_.send_message(l, kOpCreateQueueNamed, encode((uint32_t)0, n, (uint32_t)l, false, locations));
    }
  });
  return q;
}

}  // namespace

std::unique_ptr<QueueManager> QueueManager::create(HostGroup& group) { return std::make_unique<ManagerImpl>(group); }

}  // namespace moodist
