#include "host_group.h"

#include <pthread.h>
#include <sys/prctl.h>
#include <unistd.h>

#include <atomic>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <fstream>
#include <list>
#include <map>
#include <mutex>
#include <random>
#include <thread>

#include "cpu_reduce.h"
#include "log.h"
#include "net.h"
#include "tcp_transport.h"

namespace moodist {
namespace {

// A blocked API call. The engine thread completes it; the caller sleeps in 1 s slices so that an engine
// error (dead peer, heartbeat loss) can end the wait (reference: futex waits in 1 s / 10 s slices).
struct Waiter {
  std::mutex mu;
  std::condition_variable cv;
  bool done = false;
  std::atomic<bool> done_hint{false};  // set with `done`; what a waiter polls before it goes to sleep
  std::string error;
  std::atomic<int> source{-1};  // receives: the rank the message came from
  void finish(std::string err = {}) {
    std::lock_guard<std::mutex> lk(mu);
    done = true;
    error = std::move(err);
    done_hint.store(true, std::memory_order_release);
    cv.notify_all();
  }
};

// Uninitialised bytes that only ever receive data: growing one neither copies the old contents nor fills
// the new ones, which for a gigabyte costs more than the transfer it is for.
struct Scratch {
  uint8_t* mem = nullptr;
  size_t capacity = 0;
  Scratch() = default;
  Scratch(const Scratch&) = delete;
  Scratch& operator=(const Scratch&) = delete;
  ~Scratch() { free(mem); }
  void reserve(size_t bytes) {
    if (bytes <= capacity) return;
    free(mem);
    mem = static_cast<uint8_t*>(malloc(bytes));
    capacity = mem ? bytes : 0;
    if (!mem) fail("moodist: out of memory for a receive buffer of " + std::to_string(bytes) + " bytes");
  }
  uint8_t* data() { return mem; }
};
struct ScratchPool {
  std::mutex mu;
  std::vector<std::unique_ptr<Scratch>> free;
};

struct Announce {
  uint64_t addr = 0;
  uint32_t key = 0;
  uint64_t size = 0;
  uint64_t base_off = 0;  // where the receiver wants this particular sender's data to start
};

struct OutWrite {
  int peer;
  const void* src;
  size_t bytes;
  uint64_t remote_off;
  bool posted = false;
};

// One collective in flight: a generic "everyone registers a receive buffer, announces it, and writes
// into the others' buffers" exchange, the shape shared by every CPU collective here.
struct Work {
  uint32_t op = 0;
  uint32_t step = 0;
  void* recv_base = nullptr;
  size_t recv_size = 0;
  uint64_t expect_in = 0;
  std::vector<uint64_t> base_off_for;  // per source rank (all_to_all), empty = 0
  std::vector<OutWrite> outs;
  bool need_all_announces = false;     // barrier semantics even with no data
  std::function<void()> finish;        // runs on the engine thread when the exchange is complete
  std::shared_ptr<Waiter> waiter;
  std::string label;
  // state
  bool started = false;
  uint32_t key = 0;
  bool registered = false;
  int acks_pending = 0;
  bool failed = false;
  double t0 = 0;
};

struct Mail {
  uint32_t tag;
  Bytes data;
  // a large payload that waits in the sender's memory to be fetched
  bool offer = false;
  uint64_t bytes = 0, addr = 0;
  uint32_t key = 0, id = 0;
};

struct Offer {
  std::shared_ptr<Waiter> waiter;
  uint32_t key = 0;
  std::shared_ptr<void> keep;
};

class HostGroupImpl final : public HostGroup {
 public:
  HostGroupImpl(KVStore& store, std::string key, int rank, int world)
      : name_(std::move(key)), rank_(rank), world_(world), transport_(poller_, name_, rank, world) {
    last_heard_.assign(world, now_seconds());
    peer_shutdown_.assign(world, 0);
    heartbeat_s_ = (double)env_long("MOODIST_HEARTBEAT_MS", 30000) / 1000.0;
    heartbeat_on_ = !env_flag("MOODIST_DISABLE_HEARTBEAT");
    debug_cpu_ = env_flag("MOODIST_DEBUG_CPU");
    transport_.on_recv([this](int src, Bytes payload) { on_message(src, std::move(payload)); });
    transport_.on_error([this](int peer, const std::string& why) { on_peer_error(peer, why); });

    // ---- bootstrap through the store: publish where this rank listens, learn the others
    //      (keys as in the reference, core/processgroup.cc:977-1050) ----
    std::vector<std::string> mine = transport_.listen();
    const std::string pfx = "moodist/" + name_ + "/";
    store.set_str(pfx + "moodist_pg_rank" + std::to_string(rank) + "_address", to_hex(encode(mine)));
    std::vector<std::vector<std::string>> addrs(world);
    for (int r = 0; r < world; ++r) {
      if (r == rank) {
        addrs[r] = mine;
        continue;
      }
      Bytes b = from_hex(store.get_str(pfx + "moodist_pg_rank" + std::to_string(r) + "_address"));
      decode_exact(b, addrs[r]);
    }
    transport_.connect_all(addrs);
    thread_ = std::thread([this] { run(); });
    // wait until the mesh is up (60 s like the reference's rank-info exchange, core/cputhread.cc:896-911)
    double deadline = now_seconds() + (double)env_long("MOODIST_INIT_TIMEOUT_S", 60);
    while (!mesh_ready_.load()) {
      if (now_seconds() > deadline || in_error()) {
        std::string why = in_error() ? error_text() : "timed out connecting to peers";
        stop_thread();
        fail("moodist: host engine start-up failed: " + why);
      }
      usleep(1000);
    }
    // Ranks on this machine move payloads with one process_vm_readv copy instead of a loopback socket
    // (reference: core/cputhread.cc:3369-3379, 3589-3603). Every rank publishes its pid and a probe word;
    // whoever manages to read a peer's probe word uses the direct path towards that peer, everybody else
    // stays on TCP (another machine, another PID namespace, a kernel that forbids it).
    // MOODIST_DIRECT_CPU=0 switches it off.
    if (world > 1 && env_long("MOODIST_DIRECT_CPU", 1)) {
      prctl(PR_SET_PTRACER, PR_SET_PTRACER_ANY, 0, 0, 0);  // same-user peers may read us under Yama scope 1
      std::random_device rd;
      probe_word_ = ((uint64_t)rd() << 32) ^ rd() ^ 0x6d6f6f64u;
      transport_.set_direct_min_bytes((size_t)env_long("MOODIST_DIRECT_CPU_MIN_BYTES", 8192));
      store.set(pfx + "proc/" + std::to_string(rank),
                encode(boot_id(), (int64_t)getpid(), (uint64_t)(uintptr_t)&probe_word_, probe_word_));
      for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        std::string boot;
        int64_t pid = 0;
        uint64_t addr = 0, value = 0;
        decode_exact(store.get(pfx + "proc/" + std::to_string(r)), boot, pid, addr, value);
        if (boot != boot_id()) continue;
        run_on_engine([this, r, pid, addr, value] {
          if (transport_.probe_direct(r, pid, (uintptr_t)addr, value)) ++direct_peers_;
        });
      }
    }
    store.barrier(pfx + "moodist_ready", rank, world);
  }

  ~HostGroupImpl() override {
    try {
      shutdown();
    } catch (...) {
    }
    stop_thread();
  }

  int rank() const override { return rank_; }
  int world() const override { return world_; }
  const std::string& name() const override { return name_; }

  // ---------------------------------------------------------------------------------------------
  // collectives (caller threads)
  // ---------------------------------------------------------------------------------------------
  void all_gather(const void* in, void* out, size_t bytes) override {
    auto w = new_work(kOpAllGatherCpu, "all_gather");
    uint8_t* o = static_cast<uint8_t*>(out);
    if (o + (size_t)rank_ * bytes != in && bytes) memcpy(o + (size_t)rank_ * bytes, in, bytes);
    w->recv_base = out;
    w->recv_size = bytes * world_;
    w->expect_in = (uint64_t)bytes * (world_ - 1);
    for (int p = 0; p < world_; ++p)
      if (p != rank_) w->outs.push_back({p, in, bytes, (uint64_t)rank_ * bytes});
    submit_and_wait(w);
  }

  // Receive / intermediate buffers of the collectives: reused across calls (a fresh multi-megabyte vector per
  // call costs its zero-fill and a page fault per 4 KiB). The buffer goes back to the pool when the last
  // reference (the call, or a completion still running on the engine thread) lets go of it.
  std::shared_ptr<Scratch> scratch(size_t bytes) {
    std::unique_ptr<Scratch> buf;
    std::shared_ptr<ScratchPool> pool = scratch_pool_;  // the deleter keeps the pool alive, not the group
    {
      std::lock_guard<std::mutex> lk(pool->mu);
      auto& free = pool->free;
      size_t best = free.size();
      for (size_t i = 0; i < free.size(); ++i)  // smallest buffer that is large enough
        if (free[i]->capacity >= bytes && (best == free.size() || free[i]->capacity < free[best]->capacity)) best = i;
      if (best != free.size()) {
        buf = std::move(free[best]);
        free.erase(free.begin() + best);
      } else if (!free.empty()) {  // all too small: replace one of them instead of keeping both
        buf = std::move(free.back());
        free.pop_back();
      }
    }
    if (!buf) buf = std::make_unique<Scratch>();
    buf->reserve(bytes);
    Scratch* raw = buf.release();
    return std::shared_ptr<Scratch>(raw, [pool](Scratch* b) {
      std::lock_guard<std::mutex> lk(pool->mu);
      if (pool->free.size() < 4)
        pool->free.emplace_back(b);
      else
        delete b;
    });
  }

  void reduce_scatter(const void* in, void* out, size_t count, int dtype, int op, double premul) override {
    size_t esz = cpu_dtype_size(dtype);
    if (!esz) fail("moodist: reduce_scatter: unsupported dtype for CPU tensors");
    check_op(op, dtype);
    size_t chunk = count * esz;
    const uint8_t* x = static_cast<const uint8_t*>(in);
    auto tmp = scratch(chunk * world_);
    auto w = new_work(kOpReduceScatterCpu, "reduce_scatter");
    w->recv_base = tmp->data();
    w->recv_size = chunk * world_;
    w->expect_in = (uint64_t)chunk * (world_ - 1);
    for (int p = 0; p < world_; ++p)
      if (p != rank_) w->outs.push_back({p, x + (size_t)p * chunk, chunk, (uint64_t)rank_ * chunk});
    int world = world_, rank = rank_;
    w->finish = [=] {
      std::vector<const void*> srcs(world);
      for (int r = 0; r < world; ++r) srcs[r] = r == rank ? (const void*)(x + (size_t)rank * chunk) : tmp->data() + (size_t)r * chunk;
      double scale = op == kRedAvg ? 1.0 / world : premul;
      bool use_scale = op == kRedAvg || op == kRedPremulSum;
      cpu_reduce(out, srcs.data(), world, count, dtype, op, scale, use_scale);
    };
    submit_and_wait(w);
  }

  void all_reduce(const void* in, void* out, size_t count, int dtype, int op, double premul) override {
    // reduce_scatter + all_gather over a [world, chunk] view, padded when count % world != 0
    // (same decomposition as the reference, core/processgroup.cc:1674-1722)
    size_t esz = cpu_dtype_size(dtype);
    if (!esz) fail("moodist: all_reduce: unsupported dtype for CPU tensors");
    if (count == 0) return;
    if (world_ == 1) {
      const void* srcs[1] = {in};
      check_op(op, dtype);
      cpu_reduce(out, srcs, 1, count, dtype, op, premul, op == kRedPremulSum);
      return;
    }
    // Whole multiples of the world size run in place: each rank reduces its slice straight into the output and
    // the slices are then gathered where they lie. (A peer reads slice p of this rank's input only during the
    // reduce-scatter, which ends when those reads are acknowledged, and slice p is overwritten only by what that
    // same peer sends afterwards, so input and output may be one buffer.) The few elements left over of a large
    // tensor take a padded round of their own.
    const uint8_t* x = static_cast<const uint8_t*>(in);
    uint8_t* o = static_cast<uint8_t*>(out);
    size_t chunk = count / world_;
    size_t body = chunk * world_;
    if (body != count && count * esz <= (1u << 20)) {
      // small and not divisible: one padded round costs less than a second round for the remainder
      size_t per = chunk + 1;
      Bytes pin(per * world_ * esz, 0), pout(per * world_ * esz), mine(per * esz);
      memcpy(pin.data(), x, count * esz);
      reduce_scatter(pin.data(), mine.data(), per, dtype, op, premul);
      all_gather(mine.data(), pout.data(), per * esz);
      memcpy(o, pout.data(), count * esz);
      return;
    }
    if (chunk) {
      uint8_t* mine = o + (size_t)rank_ * chunk * esz;
      reduce_scatter(x, mine, chunk, dtype, op, premul);
      all_gather(mine, o, chunk * esz);
    }
    size_t tail = count - body;
    if (tail) {
      // one element per rank, the first `tail` of them real; what the padding reduces to is never read
      Bytes pin((size_t)world_ * esz, 0), pout((size_t)world_ * esz), one(esz);
      memcpy(pin.data(), x + body * esz, tail * esz);
      reduce_scatter(pin.data(), one.data(), 1, dtype, op, premul);
      all_gather(one.data(), pout.data(), esz);
      memcpy(o + body * esz, pout.data(), tail * esz);
    }
  }

  void broadcast(void* data, size_t bytes, int root) override {
    auto w = new_work(kOpBroadcastRingCpu, "broadcast");
    if (rank_ == root) {
      for (int p = 0; p < world_; ++p)
        if (p != rank_) w->outs.push_back({p, data, bytes, 0});
    } else {
      w->recv_base = data;
      w->recv_size = bytes;
      w->expect_in = bytes;
    }
    submit_and_wait(w);
  }

  void gather(const void* in, void* out, size_t bytes, int root) override {
    auto w = new_work(kOpGatherCpu, "gather");
    if (rank_ == root) {
      uint8_t* o = static_cast<uint8_t*>(out);
      if (bytes) memcpy(o + (size_t)rank_ * bytes, in, bytes);
      w->recv_base = out;
      w->recv_size = bytes * world_;
      w->expect_in = (uint64_t)bytes * (world_ - 1);
    } else {
      w->outs.push_back({root, in, bytes, (uint64_t)rank_ * bytes});
    }
    submit_and_wait(w);
  }

  void scatter(const void* in, void* out, size_t bytes, int root) override {
    auto w = new_work(kOpScatterCpu, "scatter");
    if (rank_ == root) {
      const uint8_t* x = static_cast<const uint8_t*>(in);
      if (bytes) memcpy(out, x + (size_t)rank_ * bytes, bytes);
      for (int p = 0; p < world_; ++p)
        if (p != rank_) w->outs.push_back({p, x + (size_t)p * bytes, bytes, 0});
    } else {
      w->recv_base = out;
      w->recv_size = bytes;
      w->expect_in = bytes;
    }
    submit_and_wait(w);
  }

  void all_to_all(const void* in, void* out, const uint64_t* send_off, const uint64_t* send_bytes,
                  const uint64_t* recv_off, const uint64_t* recv_bytes) override {
    auto w = new_work(kOpAllToAllCpu, "all_to_all");
    const uint8_t* x = static_cast<const uint8_t*>(in);
    uint8_t* o = static_cast<uint8_t*>(out);
    size_t extent = 0;
    w->base_off_for.assign(world_, 0);
    for (int p = 0; p < world_; ++p) {
      extent = std::max<size_t>(extent, recv_off[p] + recv_bytes[p]);
      w->base_off_for[p] = recv_off[p];
      if (p != rank_) {
        w->expect_in += recv_bytes[p];
        w->outs.push_back({p, x + send_off[p], (size_t)send_bytes[p], 0});
      }
    }
    if (send_bytes[rank_]) memcpy(o + recv_off[rank_], x + send_off[rank_], send_bytes[rank_]);
    w->recv_base = out;
    w->recv_size = extent;
    submit_and_wait(w);
  }

  void barrier() override {
    auto w = new_work(kOpBarrier, "barrier");
    w->need_all_announces = true;
    submit_and_wait(w);
  }

  void send(const void* data, size_t bytes, int dst, uint32_t tag) override { send_wait(send_post(data, bytes, dst, tag, nullptr)); }

  std::shared_ptr<void> send_post(const void* data, size_t bytes, int dst, uint32_t tag, std::shared_ptr<void> keep) override {
    auto waiter = std::make_shared<Waiter>();
    if (bytes <= kEagerSendBytes) {
      // small: inside the message, buffered at the receiver until a receive asks for it
      Writer wr;
      wr(tag, (uint64_t)bytes);
      wr.raw(data, bytes);
      send_message(dst, kOpSendRecv, std::move(wr.out));
      waiter->finish();
      return waiter;
    }
    run_on_engine([=, this] {
      uint32_t id = ++next_offer_;
      Offer o;
      o.waiter = waiter;
      o.key = MrTable::instance().add(const_cast<void*>(data), bytes);
      o.keep = keep;
      offers_[id] = std::move(o);
      send_message(dst, kOpSendOffer, encode(tag, (uint64_t)bytes, (uint64_t)(uintptr_t)data, offers_[id].key, id));
    });
    return waiter;
  }

  void send_wait(const std::shared_ptr<void>& posted) override { wait(*std::static_pointer_cast<Waiter>(posted), "send"); }

  bool send_done(const std::shared_ptr<void>& posted) override {
    return std::static_pointer_cast<Waiter>(posted)->done_hint.load(std::memory_order_acquire);
  }

  void recv(void* data, size_t bytes, int src, uint32_t tag) override { recv_wait(recv_post(data, bytes, src, tag, nullptr)); }

  std::shared_ptr<void> recv_post(void* data, size_t bytes, int src, uint32_t tag, std::shared_ptr<void> keep) override {
    auto waiter = std::make_shared<Waiter>();
    run_on_engine([=, this] {
      pending_recvs_.push_back(PendingRecv{src, tag, data, bytes, waiter, keep});
      match_recvs();
    });
    return waiter;
  }

  void recv_wait(const std::shared_ptr<void>& posted) override { wait(*std::static_pointer_cast<Waiter>(posted), "recv"); }

  bool recv_done(const std::shared_ptr<void>& posted) override {
    return std::static_pointer_cast<Waiter>(posted)->done_hint.load(std::memory_order_acquire);
  }
  int recv_source(const std::shared_ptr<void>& posted) override { return std::static_pointer_cast<Waiter>(posted)->source.load(); }

  // ---------------------------------------------------------------------------------------------
  // messages
  // ---------------------------------------------------------------------------------------------
  void set_handler(uint32_t op, Handler h) override {
    std::vector<std::pair<uint32_t, Handler>> one;
    one.emplace_back(op, std::move(h));
    set_handlers(std::move(one));
  }

  // Messages may arrive before their subsystem registers (a peer may be a step ahead). They wait in `unhandled_`,
  // in arrival order over all message types, and are replayed on the engine thread once handlers exist. Until that
  // replay has run, new arrivals join the waiting ones instead of overtaking them, and a subsystem registers all
  // of its handlers in one call, so that messages of different types keep their order too (a queue's put,
  // then the commit of its transaction, then the next put).
  void set_handlers(std::vector<std::pair<uint32_t, Handler>> list) override {
    bool replay = false;
    {
      std::lock_guard<std::mutex> lk(handlers_mu_);
      for (auto& [op, h] : list) {
        replay |= (bool)h;
        handlers_[op] = std::move(h);
      }
      if (replay) ++pending_replays_;
    }
    if (!replay) return;
    run_on_engine([this] {
      std::deque<Parked> keep;
      while (!unhandled_.empty()) {
        Parked m = std::move(unhandled_.front());
        unhandled_.pop_front();
        Handler h;
        {
          std::lock_guard<std::mutex> lk(handlers_mu_);
          auto it = handlers_.find(m.op);
          if (it != handlers_.end()) h = it->second;
        }
        if (!h) {
          keep.push_back(std::move(m));
          continue;
        }
        try {
          Reader r(m.body);
          h(m.src, r);
        } catch (const std::exception& e) {
          set_error(strf("bad message from rank %d: %s", m.src, e.what()));
        }
      }
      unhandled_ = std::move(keep);
      std::lock_guard<std::mutex> lk(handlers_mu_);
      --pending_replays_;
    });
  }

  void send_message(int dst, uint32_t op, Bytes body) override {
    // header: u32 opType | u32 sourceRank | u32 seqid (reference: core/cputhread.cc:579-590)
    auto send = [this, dst, op, body = std::move(body)]() mutable {
      Writer w;
      w(op, (uint32_t)rank_, next_seq_to_[dst]++);
      w.raw(body.data(), body.size());
      transport_.post_send(dst, std::move(w.out));
    };
    if (std::this_thread::get_id() == thread_.get_id())
      send();
    else
      run_on_engine(std::move(send));
  }

  void run_on_engine(std::function<void()> fn) override {
    {
      std::lock_guard<std::mutex> lk(queue_mu_);
      queue_.push_back(std::move(fn));
    }
    poller_.wake();
  }

  bool on_engine_thread() const override { return std::this_thread::get_id() == thread_.get_id(); }
  std::shared_ptr<void>& extension(const std::string& key) override {
    std::lock_guard<std::mutex> lk(extensions_mu_);
    return extensions_[key];
  }
  void post_read(int src, void* local, size_t bytes, uint32_t rkey, uint64_t raddr,
                 std::function<void(bool ok)> done) override {
    transport_.post_read(src, local, bytes, rkey, (uintptr_t)raddr, std::move(done));
  }
  void post_read_strided(int src, void* local, uint64_t rows, size_t row_bytes, size_t dst_pitch, uint32_t rkey,
                         uint64_t raddr, size_t src_pitch, std::function<void(bool ok)> done) override {
    transport_.post_read_strided(src, local, rows, row_bytes, dst_pitch, rkey, (uintptr_t)raddr, src_pitch, std::move(done));
  }

  std::vector<uint64_t> transport_counters() override {
    // read on the engine thread, where the counters are written
    auto out = std::make_shared<std::vector<uint64_t>>();
    auto waiter = std::make_shared<Waiter>();
    run_on_engine([this, out, waiter] {
      *out = {transport_.bytes_sent(), transport_.bytes_received(), transport_.bytes_direct(), (uint64_t)direct_peers_,
              (uint64_t)transport_.unix_peers()};
      waiter->finish();
    });
    std::unique_lock<std::mutex> lk(waiter->mu);
    waiter->cv.wait_for(lk, std::chrono::seconds(5), [&] { return waiter->done; });
    return *out;
  }

  void inject_faults(int drop_every, int duplicate_every, int delay_ms) override {
    run_on_engine([this, drop_every, duplicate_every, delay_ms] {
      if (drop_every <= 0 && duplicate_every <= 0 && delay_ms <= 0) {
        transport_.fault_hook = nullptr;
        return;
      }
      auto count = std::make_shared<uint64_t>(0);
      transport_.fault_hook = [=](int, const Bytes&) {
        uint64_t n = ++*count;
        if (delay_ms > 0) usleep((useconds_t)delay_ms * 1000);
        if (drop_every > 0 && n % (uint64_t)drop_every == 0) return 1;
        if (duplicate_every > 0 && n % (uint64_t)duplicate_every == 0) return 2;
        return 0;
      };
    });
  }

  bool in_error() const override { return error_state_.load(); }
  std::string error_text() const override {
    std::lock_guard<std::mutex> lk(error_mu_);
    return error_text_;
  }

  void shutdown() override {
    if (shutdown_started_.exchange(true)) return;
    if (!thread_.joinable()) return;
    auto waiter = std::make_shared<Waiter>();
    run_on_engine([this, waiter] {
      shutting_down_ = true;
      shutdown_waiter_ = waiter;
      shutdown_deadline_ = now_seconds() + (double)env_long("MOODIST_SHUTDOWN_TIMEOUT_MS", 8000) / 1000.0;
      for (int p = 0; p < world_; ++p)
        if (p != rank_) send_message(p, kOpMessageShutdown, encode(true));
      check_shutdown();
    });
    std::unique_lock<std::mutex> lk(waiter->mu);
    waiter->cv.wait_for(lk, std::chrono::seconds(10), [&] { return waiter->done; });
  }

  void set_profiling(bool on) override {
    auto waiter = std::make_shared<Waiter>();
    run_on_engine([this, on, waiter] {
      if (profiling_ && !on) flush_trace();
      profiling_ = on;
      waiter->finish();
    });
    std::unique_lock<std::mutex> lk(waiter->mu);
    waiter->cv.wait_for(lk, std::chrono::seconds(10), [&] { return waiter->done; });
  }
  bool profiling() const override { return profiling_; }
  std::string last_trace_path() const override {
    std::lock_guard<std::mutex> lk(error_mu_);
    return trace_path_;
  }

 private:
  struct PendingRecv {
    int src;
    uint32_t tag;
    void* data;
    size_t bytes;
    std::shared_ptr<Waiter> waiter;
    std::shared_ptr<void> keep;  // whatever owns `data`
  };

  void check_op(int op, int dtype) {
    if (!cpu_reduce_op_supported(op, dtype))
      fail("moodist: unsupported reduce op for this dtype (CPU tensors: SUM, AVG, PRODUCT, MIN, MAX, PREMUL_SUM, and "
           "BAND / BOR / BXOR on integer types)");
  }

  std::shared_ptr<Work> new_work(uint32_t op, const char* label) {
    auto w = std::make_shared<Work>();
    w->op = op;
    w->label = label;
    w->waiter = std::make_shared<Waiter>();
    return w;
  }

  void submit_and_wait(std::shared_ptr<Work> w) {
    if (in_error()) fail("moodist: process group is in an error state: " + error_text());
    // Collectives of one group must be issued by one thread at a time, in the same order on all ranks
    // (the reference throws from a ThreadUnsafe guard, core/processgroup.cc:172-183).
    if (busy_.exchange(true)) fail("moodist: concurrent collectives on one process group are not supported");
    struct Unbusy {
      std::atomic<bool>& b;
      ~Unbusy() { b = false; }
    } unbusy{busy_};
    step_ += 0x1000;  // same stride as the reference's step values
    w->step = step_;
    run_on_engine([this, w] { works_.push_back(w); });
    wait(*w->waiter, w->label.c_str());
  }

  void wait(Waiter& wt, const char* what) {
    // A sleeping thread costs tens of microseconds to wake; most operations of the engine finish sooner than
    // that, so look at the flag for a short while first.
    spin_until(wt.done_hint, spin_us_);
    std::unique_lock<std::mutex> lk(wt.mu);
    while (!wt.done) {
      wt.cv.wait_for(lk, std::chrono::milliseconds(200));
      if (wt.done) break;
      lk.unlock();
      if (in_error()) fail(std::string("moodist: ") + what + " failed: " + error_text());
      try {
        check_interrupt();
      } catch (...) {
        // The caller is about to unwind and may free the buffers this operation still refers to: nothing of this
        // group may touch them any more, and the peers should learn that this rank is not coming.
        set_error(std::string("interrupted by a signal while waiting for ") + what);
        throw;
      }
      lk.lock();
    }
    if (!wt.error.empty()) fail(std::string("moodist: ") + what + " failed: " + wt.error);
  }

  void set_error(const std::string& why) {
    {
      std::lock_guard<std::mutex> lk(error_mu_);
      if (error_text_.empty()) error_text_ = why;
    }
    if (!error_state_.exchange(true)) {
      log_error("process group %s rank %d: %s", name_.c_str(), rank_, why.c_str());
      // tell the others: their collectives with this rank can no longer complete, and without this notice
      // they would only find out through the heartbeat
      std::string text = strf("rank %d reported: %s", rank_, why.c_str());
      run_on_engine([this, text] {
        for (int p = 0; p < world_; ++p)
          if (p != rank_ && !peer_shutdown_[p]) send_message(p, kOpErrorNotice, encode(text));
      });
    }
  }

  void on_peer_error(int peer, const std::string& why) {
    if (peer_shutdown_[peer] || shutting_down_) return;  // orderly exit of that peer
    set_error(strf("connection to rank %d lost: %s", peer, why.c_str()));
  }

  void stop_thread() {
    stop_ = true;
    poller_.wake();
    if (thread_.joinable()) thread_.join();
  }

  // ---------------------------------------------------------------------------------------------
  // engine thread
  // ---------------------------------------------------------------------------------------------
  void run() {
    pthread_setname_np(pthread_self(), "moodist-cputhrd");
    double last_beat = now_seconds();
    double last_iter = last_beat;
    double last_active = last_beat;
    while (!stop_) {
      bool busy = !works_.empty();
      // After any activity the loop keeps polling without blocking for a short while: a caller that issues
      // operations back to back (queue gets, small collectives, store-like request / reply traffic) then never
      // pays the wake-up of a sleeping thread.
      bool spin = busy || (spin_us_ > 0 && now_seconds() - last_active < spin_us_ * 1e-6);
      int events = 0;
      try {
        events = poller_.poll(spin ? 0 : 50);
      } catch (const std::exception& e) {
        // nothing a peer (or a stranger on one of the listening ports) sends may end this thread
        set_error(strf("engine thread: %s", e.what()));
      }
      double now = now_seconds();
      if (debug_cpu_ && now - last_iter > 0.001 && busy) log_info("engine: lost %.1f ms between iterations", (now - last_iter) * 1e3);
      last_iter = now;
      if (!mesh_ready_.load() && transport_.all_connected()) mesh_ready_ = true;
      // closures from other threads
      std::deque<std::function<void()>> q;
      {
        std::lock_guard<std::mutex> lk(queue_mu_);
        q.swap(queue_);
      }
      try {
        if (q.size() > 1) {
          // a burst of requests (queue puts, messages): their records leave in one write per connection
          transport_.hold_sends();
          for (auto& f : q) f();
          transport_.release_sends();
        } else {
          for (auto& f : q) f();
        }
      } catch (const std::exception& e) {
        transport_.release_sends();
        set_error(strf("engine thread: %s", e.what()));
      }
      if (events > 0 || !q.empty() || busy) last_active = now;
      // progress
      for (auto it = works_.begin(); it != works_.end();) {
        if (step_work(**it))
          it = works_.erase(it);
        else
          ++it;
      }
      if (heartbeat_on_ && mesh_ready_.load() && now - last_beat >= heartbeat_s_) {
        last_beat = now;
        heartbeat(now);
      }
      if (shutting_down_) check_shutdown();
      if (shutdown_release_ && now >= shutdown_release_at_) {
        shutdown_release_->finish();
        shutdown_release_ = nullptr;
      }
    }
    poller_.close_all();
  }

  void trace(const std::string& name, double t0, double t1, int tid) {
    if (profiling_) trace_.push_back(TraceEvent{name, tid, t0 * 1e6, (t1 - t0) * 1e6});
  }

  void flush_trace() {
    std::string path = "moodist-trace-cpu-" + name_ + "-" + std::to_string(rank_) + ".json";
    std::ofstream f(path);
    f << "{\"traceEvents\":[";
    bool first = true;
    for (auto& e : trace_) {
      if (!first) f << ",";
      first = false;
      f << strf("{\"ph\":\"X\",\"name\":\"%s\",\"ts\":%.3f,\"dur\":%.3f,\"pid\":%d,\"tid\":%d}", e.name.c_str(), e.ts_us,
                e.dur_us, rank_, e.tid);
    }
    f << "]}\n";
    trace_.clear();
    std::lock_guard<std::mutex> lk(error_mu_);
    trace_path_ = path;
  }

  bool step_work(Work& w) {
    if (error_state_) {
      if (w.registered) MrTable::instance().remove(w.key);
      w.waiter->finish(error_text());
      return true;
    }
    if (!w.started) {
      w.started = true;
      w.t0 = now_seconds();
      if (w.recv_size) {
        w.key = MrTable::instance().add(w.recv_base, w.recv_size);
        w.registered = true;
      }
      for (int p = 0; p < world_; ++p) {
        if (p == rank_) continue;
        uint64_t base_off = w.base_off_for.empty() ? 0 : w.base_off_for[p];
        send_message(p, w.op, encode(w.step, (uint64_t)(uintptr_t)w.recv_base, w.key, (uint64_t)w.recv_size, base_off));
      }
    }
    bool all_posted = true;
    for (OutWrite& o : w.outs) {
      if (o.posted) continue;
      auto it = announces_.find(ann_key(w.step, o.peer));
      if (it == announces_.end()) {
        all_posted = false;
        continue;
      }
      o.posted = true;
      if (o.bytes == 0) continue;
      const Announce& a = it->second;
      if (a.base_off + o.remote_off + o.bytes > a.size) {
        // the peer would refuse the write: say what is wrong instead of "rejected"
        set_error(strf("%s: the ranks disagree on sizes (rank %d made room for %llu bytes, this rank sends %zu bytes to offset "
                       "%llu): every rank must pass tensors of the same size and dtype",
                       w.label.c_str(), o.peer, (unsigned long long)a.size, o.bytes,
                       (unsigned long long)(a.base_off + o.remote_off)));
        w.failed = true;
        continue;
      }
      ++w.acks_pending;
      Work* wp = &w;
      transport_.post_write(o.peer, o.src, o.bytes, a.key, (uintptr_t)(a.addr + a.base_off + o.remote_off),
                            [this, wp](bool ok) {
                              --wp->acks_pending;
                              if (!ok) {
                                wp->failed = true;
                                set_error("a remote write was rejected (out of bounds or peer gone)");
                              }
                            });
    }
    if (!all_posted || w.acks_pending > 0) return false;
    if (w.registered && MrTable::instance().landed(w.key) < w.expect_in) return false;
    if (w.need_all_announces) {
      for (int p = 0; p < world_; ++p)
        if (p != rank_ && !announces_.count(ann_key(w.step, p))) return false;
    }
    // complete
    if (w.registered) MrTable::instance().remove(w.key);
    for (int p = 0; p < world_; ++p) announces_.erase(ann_key(w.step, p));
    if (w.finish) w.finish();
    trace(w.label, w.t0, now_seconds(), 0);
    w.waiter->finish();
    return true;
  }

  static uint64_t ann_key(uint32_t step, int peer) { return ((uint64_t)step << 16) | (uint32_t)peer; }

  void on_message(int src, Bytes payload) {
    try {
      Reader r(payload);
      uint32_t op, source, seq;
      r(op, source, seq);
      if ((int)source != src) {
        set_error(strf("message from rank %d claims to be from rank %u", src, source));
        return;
      }
      // TCP keeps order per connection; a gap or repeat means a lost / duplicated message
      uint32_t& expect = next_seq_from_[src];
      if (seq != expect) {
        if ((int32_t)(seq - expect) < 0) return;  // duplicate: drop
        set_error(strf("lost a message from rank %d (got sequence %u, expected %u)", src, seq, expect));
        return;
      }
      ++expect;
      last_heard_[src] = now_seconds();
      switch (op) {
        case kOpHeartbeat: return;
        case kOpErrorNotice: {
          set_error(r.read<std::string>());
          return;
        }
        case kOpMessageShutdown: {
          bool begin = r.read<bool>();
          peer_shutdown_[src] = begin ? 1 : 2;
          if (shutting_down_) check_shutdown();
          return;
        }
        case kOpSendRecv: {
          uint32_t tag;
          uint64_t bytes;
          r(tag, bytes);
          Mail m;
          m.tag = tag;
          const uint8_t* b = r.take(bytes);
          m.data.assign(b, b + bytes);
          mailbox_[src].push_back(std::move(m));
          match_recvs();
          return;
        }
        case kOpSendOffer: {
          Mail m;
          m.offer = true;
          r(m.tag, m.bytes, m.addr, m.key, m.id);
          mailbox_[src].push_back(std::move(m));
          match_recvs();
          return;
        }
        case kOpSendTaken: {
          uint32_t id;
          bool ok;
          std::string text;
          r(id, ok, text);
          auto it = offers_.find(id);
          if (it == offers_.end()) return;
          MrTable::instance().remove(it->second.key);
          it->second.waiter->finish(ok ? std::string() : text);
          offers_.erase(it);
          return;
        }
        case kOpBarrier:
        case kOpAllGatherCpu:
        case kOpReduceScatterCpu:
        case kOpBroadcastRingCpu:
        case kOpGatherCpu:
        case kOpScatterCpu:
        case kOpAllToAllCpu: {
          uint32_t step;
          Announce a;
          r(step, a.addr, a.key, a.size, a.base_off);
          // Mismatched collectives across ranks show up here as an announce whose op differs from the
          // local work with the same step (reference: "Mismatched collectives detected", cputhread.h:100-112)
          for (auto& w : works_) {
            if (w->step == step && w->op != op) {
              set_error(strf("mismatched collectives: rank %d runs op %u at step 0x%x, this rank runs %s (op %u)", src,
                             op, step, w->label.c_str(), w->op));
              return;
            }
          }
          announces_[ann_key(step, src)] = a;
          return;
        }
        default: break;
      }
      Handler h;
      bool replay_pending;
      {
        std::lock_guard<std::mutex> lk(handlers_mu_);
        auto it = handlers_.find(op);
        if (it != handlers_.end()) h = it->second;
        replay_pending = pending_replays_ > 0;
      }
      if (h && !(replay_pending && !unhandled_.empty())) {
        h(src, r);
      } else if (unhandled_.size() < 65536) {
        unhandled_.push_back(Parked{op, src, Bytes(r.p, r.end)});  // see set_handlers()
      } else {
        log_error("engine: dropping message type %u from rank %d: nobody handles it", op, src);
      }
    } catch (const std::exception& e) {
      set_error(strf("bad message from rank %d: %s", src, e.what()));
    }
  }

  void match_recvs() {
    for (auto it = pending_recvs_.begin(); it != pending_recvs_.end();) {
      if (serve_recv(*it))
        it = pending_recvs_.erase(it);
      else
        ++it;
    }
  }

  // Hands the oldest message with the request's tag to it: from its source, or (source -1: anybody) from the first
  // rank that has one. False when nothing matches yet.
  bool serve_recv(PendingRecv& want) {
    const int first = want.src < 0 ? 0 : want.src, last = want.src < 0 ? world_ - 1 : want.src;
    for (int from = first; from <= last; ++from) {
      auto box_it = mailbox_.find(from);
      if (box_it == mailbox_.end()) continue;
      auto& box = box_it->second;
      for (auto m = box.begin(); m != box.end(); ++m) {
        if (m->tag != want.tag) continue;
        want.waiter->source.store(from);
        size_t have = m->offer ? (size_t)m->bytes : m->data.size();
        if (have != want.bytes) {
          std::string text = strf("recv size mismatch: expected %zu bytes, message has %zu", want.bytes, have);
          if (m->offer) send_message(from, kOpSendTaken, encode(m->id, false, "the receiver's " + text));
          want.waiter->finish(text);
        } else if (m->offer) {
          // fetch the payload out of the sender's memory into the caller's; both ends learn how it went
          uint32_t id = m->id;
          auto waiter = want.waiter;
          auto keep = want.keep;
          post_read(from, want.data, want.bytes, m->key, m->addr, [this, from, id, waiter, keep](bool ok) {
            send_message(from, kOpSendTaken, encode(id, ok, std::string(ok ? "" : "the receiver could not read the payload")));
            waiter->finish(ok ? std::string() : "reading the sender's payload failed");
          });
        } else {
          if (want.bytes) memcpy(want.data, m->data.data(), want.bytes);
          want.waiter->finish();
        }
        box.erase(m);
        return true;
      }
    }
    return false;
  }

  // Liveness: ping up to 16 neighbours on each side; silence for 3 intervals is logged, for 6 it puts
  // the group into the error state (reference: core/cputhread.cc:5936-6016).
  void heartbeat(double now) {
    int reach = std::min(16, world_ - 1);
    for (int d = 1; d <= reach; ++d) {
      int a = (rank_ + d) % world_, b = (rank_ - d % world_ + world_) % world_;
      send_message(a, kOpHeartbeat, {});
      if (b != a) send_message(b, kOpHeartbeat, {});
    }
    for (int p = 0; p < world_; ++p) {
      if (p == rank_ || peer_shutdown_[p]) continue;
      int dist = std::min((p - rank_ + world_) % world_, (rank_ - p + world_) % world_);
      if (dist > 16) continue;
      double silent = now - last_heard_[p];
      if (silent > 6 * heartbeat_s_) {
        set_error(strf("no heartbeat from rank %d for %.1f s", p, silent));
      } else if (silent > 3 * heartbeat_s_) {
        log_error("process group %s rank %d: rank %d has been silent for %.1f s", name_.c_str(), rank_, p, silent);
      }
    }
  }

  // Coordinated shutdown: tell everyone, wait (bounded) until everyone said the same, then say "exited"
  // (reference: core/cputhread.cc:5474-5580).
  void check_shutdown() {
    if (!shutdown_waiter_) return;
    bool all = true;
    for (int p = 0; p < world_; ++p)
      if (p != rank_ && !peer_shutdown_[p]) all = false;
    if (all || now_seconds() > shutdown_deadline_ || error_state_) {
      for (int p = 0; p < world_; ++p)
        if (p != rank_) send_message(p, kOpMessageShutdown, encode(false));
      // the caller is released by the run loop a little later, so the final messages can leave the
      // socket buffers (never poll from inside a handler: it would re-enter the connection being read)
      shutdown_release_ = shutdown_waiter_;
      shutdown_waiter_ = nullptr;
      shutdown_release_at_ = now_seconds() + 0.02;
    }
  }

  std::string name_;
  int rank_, world_;
  Poller poller_;
  TcpTransport transport_;
  uint64_t probe_word_ = 0;  // same-machine peers read this word to find out whether they may read this process
  int direct_peers_ = 0;     // peers whose memory this rank reads directly (engine thread)
  std::shared_ptr<ScratchPool> scratch_pool_ = std::make_shared<ScratchPool>();
  std::thread thread_;
  std::atomic<bool> stop_{false}, mesh_ready_{false}, error_state_{false}, busy_{false}, shutdown_started_{false};
  mutable std::mutex error_mu_;
  std::string error_text_, trace_path_;

  std::mutex queue_mu_;
  std::deque<std::function<void()>> queue_;
  std::mutex handlers_mu_;
  std::map<uint32_t, Handler> handlers_;

  // engine-thread state
  std::list<std::shared_ptr<Work>> works_;
  std::map<uint64_t, Announce> announces_;
  std::map<int, uint32_t> next_seq_to_, next_seq_from_;
  std::mutex extensions_mu_;
  std::map<std::string, std::shared_ptr<void>> extensions_;  // per-group state of layered subsystems
  std::map<int, std::deque<Mail>> mailbox_;
  // payloads up to this size travel inside their message; larger ones are fetched by the receiver
  static constexpr size_t kEagerSendBytes = 64 << 10;
  std::map<uint32_t, Offer> offers_;  // large sends waiting to be fetched (engine thread)
  uint32_t next_offer_ = 0;
  struct Parked {
    uint32_t op;
    int src;
    Bytes body;
  };
  std::deque<Parked> unhandled_;  // engine thread only
  int pending_replays_ = 0;       // guarded by handlers_mu_
  std::list<PendingRecv> pending_recvs_;
  std::vector<double> last_heard_;
  std::vector<int> peer_shutdown_;
  bool shutting_down_ = false;
  std::shared_ptr<Waiter> shutdown_waiter_, shutdown_release_;
  double shutdown_deadline_ = 0, shutdown_release_at_ = 0;
  double heartbeat_s_ = 30;
  bool heartbeat_on_ = true, debug_cpu_ = false;
  double spin_us_ = spin_microseconds();
  bool profiling_ = false;
  std::vector<TraceEvent> trace_;

  uint32_t step_ = 0;  // caller side, guarded by busy_
};

}  // namespace

std::unique_ptr<HostGroup> HostGroup::create(KVStore& store, const std::string& key, int rank, int world) {
  return std::make_unique<HostGroupImpl>(store, key, rank, world);
}

}  // namespace moodist
