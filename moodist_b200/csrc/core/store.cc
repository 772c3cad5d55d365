#include "store.h"

#include <pthread.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <queue>
#include <random>
#include <set>
#include <thread>
#include <unordered_map>

#include "log.h"
#include "net.h"
#include "wire.h"

namespace moodist {

// same function as the reference (core/store.cc:1733-1743): r = 524287; r = r*42643801 + c; r % 2147483647
uint32_t store_string_hash(const std::string& s) {
  uint64_t r = 524287;
  for (unsigned char c : s) r = r * 42643801ull + c;
  return (uint32_t)(r % 2147483647ull);
}

std::vector<std::vector<int>> store_mesh(int world, uint32_t seed) {
  std::vector<std::set<int>> adj(world);
  auto link = [&](int a, int b) {
    if (a == b) return false;
    if (adj[a].count(b)) return false;
    if (adj[a].size() >= 4 || adj[b].size() >= 4) return false;
    adj[a].insert(b);
    adj[b].insert(a);
    return true;
  };
  for (int r = 0; r < world; ++r)
    if (world > 1) link(r, (r + 1) % world);
  if (world > 4) {
    // one chord per rank, drawn from a generator every rank seeds identically
    std::mt19937 rng(64 + seed);
    for (int r = 0; r < world; ++r) {
      for (int attempt = 0; attempt < 8; ++attempt) {
        int o = (int)(rng() % (uint32_t)world);
        int d = std::min((o - r + world) % world, (r - o + world) % world);
        if (d < 2) continue;  // not a neighbour: chords should shorten routes
        if (link(r, o)) break;
      }
    }
  }
  std::vector<std::vector<int>> out(world);
  for (int r = 0; r < world; ++r) out[r].assign(adj[r].begin(), adj[r].end());
  return out;
}

std::vector<int> store_first_hops(const std::vector<std::vector<int>>& mesh, int rank) {
  int world = (int)mesh.size();
  std::vector<int> hop(world, -1);
  std::queue<int> q;
  hop[rank] = rank;
  for (int n : mesh[rank]) {
    hop[n] = n;
    q.push(n);
  }
  while (!q.empty()) {
    int u = q.front();
    q.pop();
    for (int v : mesh[u]) {
      if (hop[v] != -1) continue;
      hop[v] = hop[u];
      q.push(v);
    }
  }
  return hop;
}

namespace {

// frame signatures (core/store.cc:19-29)
constexpr uint64_t kSigConnect = 0x120a63c0941561a4ull;
constexpr uint64_t kSigConnectAck = 0x120a63c0941561a5ull;
constexpr uint64_t kSigAddresses = 0x10f963c0941561a6ull;
constexpr uint64_t kSigMessage = 0x220a74d1a52672b8ull;
constexpr uint64_t kSigMessageAck = 0x220a74d1a52672b9ull;
constexpr uint64_t kSigKeepalive = 0x220a74d1a53772baull;
constexpr uint64_t kSigKeepaliveAck = 0x220a74d1a53772bbull;

enum MsgType : uint8_t {
  kDone = 3,
  kSet = 4,
  kGet = 5,
  kCheck = 6,
  kWait = 7,
  kShutdown = 8,
  kExit = 9,
  kExitAck = 0xa,
  kDiagnosticSource = 0xb,
  // extensions (the reference throws for these operations)
  kAdd = 0xc,
  kCompareSet = 0xd,
  kDelete = 0xe,
  kNumKeys = 0xf,
  // diagnostics of a request that timed out: a probe follows the route of the request; every rank it passes
  // (and the owner) reports back to the origin what it sees (the reference gathers the same reports from the
  // intermediate hops over a UDP side channel, core/store.cc:707-794, 1799-1907)
  kDiagnosticProbe = 0x10,
  kDiagnosticInfo = 0x11,
};

// In-memory image is what travels (28 bytes, little-endian), as in the reference (core/store.cc:49-63).
struct MessageHeader {
  uint32_t ttl;
  uint32_t seq;
  uint32_t destinationRank;
  uint32_t id;
  uint32_t sourceRank;
  uint32_t diagnosticSource;
  uint8_t messageType;
  bool broadcast;
};
static_assert(sizeof(MessageHeader) == 28, "MessageHeader must be 28 bytes on the wire");
constexpr size_t kSeqOffset = 8 + offsetof(MessageHeader, seq);  // inside the frame body

struct ConnectMessage {  // rendezvous with rank 0 and mesh greeting (reference: UdpConnectMessage / TcpConnectMessage)
  std::string key;
  uint32_t sourceRank = 0;
  std::string uid;
  std::string networkKey;
  std::vector<std::pair<uint32_t, std::string>> addresses;  // (port, address)
  template <class Ar>
  void wire(Ar& ar) {
    ar(key, sourceRank, uid, networkKey, addresses);
  }
};

struct AddressesMessage {
  std::string key;
  uint32_t sourceRank = 0;
  std::string sourceId;
  std::string networkKey;
  std::vector<std::pair<uint32_t, std::string>> addresses;
  template <class Ar>
  void wire(Ar& ar) {
    ar(key, sourceRank, sourceId, networkKey, addresses);
  }
};

struct WaitObj {
  std::mutex mu;
  std::condition_variable cv;
  bool done = false;
  std::atomic<bool> done_hint{false};  // set with `done`; polled briefly before the caller sleeps
  std::string error;
  Bytes result;
  void finish(Bytes r, std::string err = {}) {
    std::lock_guard<std::mutex> lk(mu);
    if (done) return;
    done = true;
    result = std::move(r);
    error = std::move(err);
    done_hint.store(true, std::memory_order_release);
    cv.notify_all();
  }
};

struct Edge {
  int peer = -1;
  std::shared_ptr<Conn> conn;
  bool connected = false;
  bool dialing = false;
  uint32_t out_seq = 0, in_seq = 0;
  std::deque<std::pair<uint32_t, Bytes>> unacked;  // frame bodies, oldest first
  std::vector<std::pair<uint32_t, std::string>> addresses;
  size_t next_addr = 0;
  double last_recv = 0, last_send = 0, next_dial = 0, down_since = 0;
  bool peer_exited = false;
};

struct PendingAtOwner {
  uint32_t requester;
  uint32_t id;
  uint8_t type;
};

class TcpStoreImpl final : public TcpStore, public std::enable_shared_from_this<TcpStoreImpl> {
 public:
  TcpStoreImpl(std::string hostname, int port, const std::string& key, int world, int rank,
               std::chrono::milliseconds timeout)
      : hostname_(std::move(hostname)), port_(port), world_(world), rank_(rank), timeout_(timeout) {
    if (world < 1 || rank < 0 || rank >= world) fail("TcpStore: bad rank/world_size");
    store_key_ = strf("%s-%d-%d-%s", hostname_.c_str(), port, world, key.substr(0, 80).c_str());
    std::random_device rd;
    uid_ = strf("%d-%08x%08x", (int)getpid(), (unsigned)rd(), (unsigned)rd());
    mesh_ = store_mesh(world, store_string_hash(store_key_));
    first_hop_ = store_first_hops(mesh_, rank);
    for (int p : mesh_[rank]) {
      edges_[p].peer = p;
      edges_[p].last_recv = now_seconds();
    }
    exit_seen_.assign(world, false);
    shutdown_seen_.assign(world, false);
    keepalive_s_ = (double)env_long("MOODIST_STORE_KEEPALIVE_MS", 20000) / 1000.0;
    fault_break_every_ = (int)env_long("MOODIST_STORE_FAULT_BREAK_EVERY", 0);
    thread_ = std::thread([this] { run(); });
    // the constructor returns once the mesh edges of this rank are up (or the timeout expires)
    double deadline = now_seconds() + std::max(1.0, (double)timeout.count() / 1000.0);
    while (!ready_.load()) {
      if (failed_.load() || now_seconds() > deadline) {
        std::string why = failed_.load() ? fatal_text() : "timed out connecting (is rank 0 reachable at " + hostname_ + ":" + std::to_string(port) + "?)";
        stop_thread();
        fail("TcpStore: " + why);
      }
      usleep(500);
    }
  }

  ~TcpStoreImpl() override {
    try {
      shutdown();
    } catch (...) {
    }
    stop_thread();
  }

  int rank() const override { return rank_; }
  int world() const override { return world_; }
  std::chrono::milliseconds timeout() const override { return timeout_; }
  void set_timeout(std::chrono::milliseconds t) override { timeout_ = t; }
  std::vector<int> edges() const override { return mesh_[rank_]; }
  void inject_faults(int break_every) override {
    post([this, break_every] { fault_break_every_ = break_every; });
  }
  uint64_t injected_breaks() override {
    auto w = std::make_shared<WaitObj>();
    post([this, w] { w->finish(encode(fault_breaks_)); });
    std::unique_lock<std::mutex> lk(w->mu);
    if (!w->cv.wait_for(lk, std::chrono::seconds(2), [&] { return w->done; })) return 0;
    uint64_t n = 0;
    decode_exact(w->result, n);
    return n;
  }

  // ---------------------------------------------------------------------------------------------
  // operations (caller threads)
  // ---------------------------------------------------------------------------------------------
  void set(const std::string& key, const Bytes& value) override { request(kSet, owner_of(key), encode(key, value), key, timeout_); }
  Bytes get(const std::string& key) override { return request(kGet, owner_of(key), encode(key), key, timeout_); }
  bool check(const std::vector<std::string>& keys) override {
    for (const auto& k : keys) {
      Bytes r = request(kCheck, owner_of(k), encode(k), k, timeout_);
      if (r.empty() || r[0] == 0) return false;
    }
    return true;
  }
  void wait(const std::vector<std::string>& keys) override { wait_for(keys, timeout_); }
  void wait_for(const std::vector<std::string>& keys, std::chrono::milliseconds timeout) override {
    double deadline = now_seconds() + (double)timeout.count() / 1000.0;
    for (const auto& k : keys) {
      double left = std::max(0.0, deadline - now_seconds());
      request(kWait, owner_of(k), encode(k), k, std::chrono::milliseconds((int64_t)(left * 1000)));
    }
  }
  int64_t add(const std::string& key, int64_t delta) override {
    Bytes r = request(kAdd, owner_of(key), encode(key, delta), key, timeout_);
    int64_t v = 0;
    decode_exact(r, v);
    return v;
  }
  Bytes compare_set(const std::string& key, const Bytes& expected, const Bytes& desired) override {
    return request(kCompareSet, owner_of(key), encode(key, expected, desired), key, timeout_);
  }
  bool delete_key(const std::string& key) override {
    Bytes r = request(kDelete, owner_of(key), encode(key), key, timeout_);
    return !r.empty() && r[0] != 0;
  }
  int64_t num_keys() override {
    int64_t total = 0;
    for (int r = 0; r < world_; ++r) {
      Bytes b = request(kNumKeys, r, {}, "<num_keys>", timeout_);
      int64_t v = 0;
      decode_exact(b, v);
      total += v;
    }
    return total;
  }

  void shutdown() override {
    if (shutdown_called_.exchange(true)) return;
    if (!thread_.joinable()) return;
    auto w = std::make_shared<WaitObj>();
    post([this, w] { begin_shutdown(w); });
    std::unique_lock<std::mutex> lk(w->mu);
    w->cv.wait_for(lk, std::chrono::seconds(5), [&] { return w->done; });
  }

  std::string describe() const override {
    return strf("TcpStore(%s, rank %d/%d, edges=%zu)", store_key_.c_str(), rank_, world_, mesh_[rank_].size());
  }

 private:
  int owner_of(const std::string& key) const { return (int)(store_string_hash(key) % (uint32_t)world_); }

  std::string fatal_text() const {
    std::lock_guard<std::mutex> lk(fatal_mu_);
    return fatal_;
  }

  void post(std::function<void()> fn) {
    {
      std::lock_guard<std::mutex> lk(queue_mu_);
      queue_.push_back(std::move(fn));
    }
    poller_.wake();
  }

  Bytes request(uint8_t type, int dest, Bytes payload, const std::string& what, std::chrono::milliseconds timeout) {
    if (shutdown_called_.load()) fail("TcpStore: the store has been shut down");
    auto w = std::make_shared<WaitObj>();
    auto idp = std::make_shared<uint32_t>(0);
    post([this, type, dest, payload = std::move(payload), w, idp]() mutable {
      if (!error_.empty()) return w->finish({}, error_);
      uint32_t id = next_id_++;
      *idp = id;
      pending_[id] = w;
      send_to(dest, type, id, std::move(payload));
    });
    double start = now_seconds();
    double limit = (double)timeout.count() / 1000.0;
    spin_until(w->done_hint, spin_microseconds());  // most requests are answered sooner than a thread wakes up
    std::unique_lock<std::mutex> lk(w->mu);
    while (!w->done) {
      w->cv.wait_for(lk, std::chrono::milliseconds(250));  // sliced so signals and shutdown are noticed
      if (!w->done) {
        lk.unlock();
        try {
          check_interrupt();
        } catch (...) {
          post([this, idp] { pending_.erase(*idp); });
          throw;
        }
        lk.lock();
      }
      if (!w->done && now_seconds() - start > limit) {
        lk.unlock();
        std::string diag = diagnose(dest, what);
        post([this, idp] { pending_.erase(*idp); });
        fail(strf("TcpStore(%s): timed out after %.1f s on key '%s' (owner rank %d). %s", store_key_.c_str(),
                  now_seconds() - start, what.c_str(), dest, diag.c_str()));
      }
    }
    if (!w->error.empty()) fail("TcpStore: " + w->error);
    return std::move(w->result);
  }

  // Which hop of the route to `dest` looks unhealthy: this rank's own view of its first hop, plus what every
  // rank further along the route (and the owner of the key) answers to a probe within about a second.
  std::string diagnose(int dest, const std::string& key) {
    auto w = std::make_shared<WaitObj>();
    auto idp = std::make_shared<uint32_t>(0);
    post([this, dest, key, w, idp] {
      std::string s;
      if (dest == rank_) {
        s = "The key lives on this rank and was never set.";
      } else {
        int hop = first_hop_[dest];
        auto it = edges_.find(hop);
        if (it == edges_.end()) {
          s = "No route to that rank.";
        } else {
          const Edge& e = it->second;
          s = strf("Route: rank %d -> rank %d%s. Edge to rank %d: %s, %zu unacknowledged messages, last heard %.1f s ago.",
                   rank_, hop, hop == dest ? "" : " -> ...", hop, e.connected ? "connected" : "NOT connected",
                   e.unacked.size(), now_seconds() - e.last_recv);
          uint32_t id = next_id_++;
          *idp = id;
          diag_reports_[id];
          send_to(dest, kDiagnosticProbe, id, encode(key));
        }
      }
      w->finish(Bytes(s.begin(), s.end()));
    });
    std::string text;
    {
      std::unique_lock<std::mutex> lk(w->mu);
      if (!w->cv.wait_for(lk, std::chrono::seconds(1), [&] { return w->done; })) return "";
      text.assign(w->result.begin(), w->result.end());
    }
    if (*idp == 0) return text;
    // reports trickle in while the probe travels; the owner's report ends the wait early
    auto done = std::make_shared<WaitObj>();
    double deadline = now_seconds() + (double)env_long("MOODIST_STORE_DIAGNOSE_MS", 1000) / 1000.0;
    std::vector<std::string> reports;
    bool reached = false;
    while (now_seconds() < deadline && !reached) {
      usleep(20000);
      auto got = std::make_shared<WaitObj>();
      post([this, idp, got] {
        std::string all;
        for (const std::string& r : diag_reports_[*idp]) all += r + "\n";
        got->finish(Bytes(all.begin(), all.end()));
      });
      std::unique_lock<std::mutex> lk(got->mu);
      if (!got->cv.wait_for(lk, std::chrono::milliseconds(500), [&] { return got->done; })) break;
      std::string all(got->result.begin(), got->result.end());
      reports.clear();
      size_t pos = 0;
      while (pos < all.size()) {
        size_t e = all.find('\n', pos);
        reports.push_back(all.substr(pos, e - pos));
        pos = e + 1;
      }
      for (const std::string& r : reports) reached = reached || r.find("owner") != std::string::npos;
    }
    post([this, idp] { diag_reports_.erase(*idp); });
    for (const std::string& r : reports) text += " " + r;
    if (!reached) text += " The probe did not reach the owner within the diagnosis window.";
    return text;
  }

  // a rank that forwards (or owns the target of) a diagnostic probe tells the origin what it sees
  void report_probe(const MessageHeader& h, int next_hop, const std::string& key) {
    std::string s;
    if (next_hop < 0) {
      auto wit = waiters_.find(key);
      s = strf("Rank %d (owner): the probe arrived; key '%s' %s, %zu request(s) wait for it.", rank_, key.c_str(),
               kv_.count(key) ? "IS set" : "has not been set", wit == waiters_.end() ? (size_t)0 : wit->second.size());
    } else {
      auto it = edges_.find(next_hop);
      if (it == edges_.end()) {
        s = strf("Rank %d: no edge towards rank %d.", rank_, next_hop);
      } else {
        const Edge& e = it->second;
        s = strf("Rank %d: forwards to rank %d over an edge that is %s, %zu unacknowledged messages, last heard %.1f s ago.",
                 rank_, next_hop, e.connected ? "connected" : "NOT connected", e.unacked.size(), now_seconds() - e.last_recv);
      }
    }
    send_to((int)h.sourceRank, kDiagnosticInfo, h.id, encode(s));
  }

  void stop_thread() {
    stop_ = true;
    poller_.wake();
    if (thread_.joinable()) thread_.join();
  }

  // ---------------------------------------------------------------------------------------------
  // I/O thread
  // ---------------------------------------------------------------------------------------------
  void run() {
    pthread_setname_np(pthread_self(), "moodist-store");
    try {
      bootstrap();
    } catch (const std::exception& e) {
      set_fatal(e.what());
    }
    double last_tick = now_seconds();
    double last_active = last_tick;
    const double spin_s = spin_microseconds() * 1e-6;
    while (!stop_) {
      // keep polling for a moment after any activity: request / reply sequences then skip the thread wake-ups
      int events = 0;
      std::deque<std::function<void()>> q;
      try {
        events = poller_.poll(now_seconds() - last_active < spin_s ? 0 : 20);
        {
          std::lock_guard<std::mutex> lk(queue_mu_);
          q.swap(queue_);
        }
        for (auto& f : q) f();
      } catch (const std::exception& e) {
        // nothing a peer (or a stranger on the rendezvous port) sends may end this thread
        log_error("TcpStore rank %d: %s", rank_, e.what());
      }
      double now = now_seconds();
      if (events > 0 || !q.empty()) last_active = now;
      if (now - last_tick > 0.05) {
        last_tick = now;
        tick(now);
      }
    }
    poller_.close_all();
  }

  void set_fatal(const std::string& why) {
    {
      std::lock_guard<std::mutex> lk(fatal_mu_);
      if (fatal_.empty()) fatal_ = why;
    }
    failed_ = true;
  }

  void bootstrap() {
    auto accept = [this](std::shared_ptr<Conn> c) { on_accept(std::move(c)); };
    int p4 = poller_.listen("0.0.0.0", 0, accept);
    int p6 = poller_.listen("::", 0, accept);
    for (const std::string& a : local_addresses()) {
      bool v6 = a.find(':') != std::string::npos;
      int port = v6 ? p6 : p4;
      if (port > 0) my_addresses_.emplace_back((uint32_t)port, a);
    }
    if (my_addresses_.empty()) fail("cannot open a listening socket");
    if (world_ == 1) {
      ready_ = true;
      return;
    }
    if (rank_ == 0) {
      // rendezvous listener on the user's port
      errno = 0;
      int a = poller_.listen("0.0.0.0", port_, [this](std::shared_ptr<Conn> c) { on_rendezvous_accept(std::move(c)); });
      int err4 = a <= 0 ? errno : 0;
      errno = 0;
      int b = poller_.listen("::", port_, [this](std::shared_ptr<Conn> c) { on_rendezvous_accept(std::move(c)); });
      int err6 = b <= 0 ? errno : 0;
      // A port that somebody else holds for one address family is not ours, even if the other family could be bound:
      // the other ranks would reach that somebody. (A family this host does not have is no reason to fail.)
      if (err4 == EADDRINUSE || err6 == EADDRINUSE || (a <= 0 && b <= 0))
        fail(strf("rank 0 cannot listen on port %d: %s", port_,
                  strerror(err4 == EADDRINUSE || err6 == EADDRINUSE ? EADDRINUSE : (err4 ? err4 : err6))));
      directory_[0] = my_addresses_;
      directory_uid_[0] = uid_;
      maybe_publish_directory();
    } else {
      dial_rendezvous();
    }
  }

  // ---- rendezvous with rank 0 ----
  void dial_rendezvous() {
    poller_.connect(hostname_, port_, [this](std::shared_ptr<Conn> c) {
      if (stop_ || ready_) {
        if (c) c->close("not needed");
        return;
      }
      if (!c) {
        rendezvous_retry_at_ = now_seconds() + 0.05;
        return;
      }
      rendezvous_ = c;
      ConnectMessage m;
      m.key = store_key_;
      m.sourceRank = (uint32_t)rank_;
      m.uid = uid_;
      m.addresses = my_addresses_;
      c->send_frame(encode(kSigConnect, m));
      auto reader = std::make_shared<FrameReader>([this](Reader& r, bool) {
        uint64_t sig = r.read<uint64_t>();
        if (sig != kSigAddresses) return;
        AddressesMessage am;
        r(am);
        if (am.key != store_key_) return;
        auto it = edges_.find((int)am.sourceRank);
        if (it != edges_.end()) {
          it->second.addresses = am.addresses;
          it->second.next_dial = 0;
        }
      });
      c->on_data([reader](const uint8_t* d, size_t n) { return (*reader)(d, n); });
      c->on_close([this](const std::string&) {
        rendezvous_ = nullptr;
        if (!ready_ && !stop_) rendezvous_retry_at_ = now_seconds() + 0.05;
      });
    });
  }

  void on_rendezvous_accept(std::shared_ptr<Conn> c) {
    std::weak_ptr<Conn> weak = c;
    auto reader = std::make_shared<FrameReader>([this, weak](Reader& r, bool) {
      auto c = weak.lock();
      if (!c) return;
      uint64_t sig = r.read<uint64_t>();
      if (sig != kSigConnect) return c->close("bad rendezvous greeting");
      ConnectMessage m;
      r(m);
      if (m.key != store_key_ || m.sourceRank >= (uint32_t)world_) {
        log_error("TcpStore rank 0: rejected a rendezvous from another store (%s)", m.key.c_str());
        return c->close("wrong store");
      }
      directory_[(int)m.sourceRank] = m.addresses;
      directory_uid_[(int)m.sourceRank] = m.uid;
      rendezvous_conns_[(int)m.sourceRank] = c;
      maybe_publish_directory();
    });
    c->on_data([reader](const uint8_t* d, size_t n) { return (*reader)(d, n); });
  }

  // once every rank has checked in, tell each rank the addresses of its mesh neighbours
  void maybe_publish_directory() {
    if ((int)directory_.size() < world_) return;
    for (int r = 0; r < world_; ++r) {
      for (int n : mesh_[r]) {
        AddressesMessage am;
        am.key = store_key_;
        am.sourceRank = (uint32_t)n;
        am.sourceId = directory_uid_[n];
        am.addresses = directory_[n];
        if (r == 0) {
          edges_[n].addresses = am.addresses;
        } else {
          auto it = rendezvous_conns_.find(r);
          if (it != rendezvous_conns_.end() && it->second->open()) it->second->send_frame(encode(kSigAddresses, am));
        }
      }
    }
  }

  // ---- mesh edges ----
  void on_accept(std::shared_ptr<Conn> c) {
    std::weak_ptr<Conn> weak = c;
    auto reader = std::make_shared<FrameReader>([this, weak](Reader& r, bool) {
      auto c = weak.lock();
      if (!c) return;
      uint64_t sig = r.read<uint64_t>();
      if (sig != kSigConnect) return c->close("bad mesh greeting");
      ConnectMessage m;
      r(m);
      auto it = edges_.find((int)m.sourceRank);
      if (m.key != store_key_ || it == edges_.end()) return c->close("not a neighbour of this store");
      Edge& e = it->second;
      if (e.conn && e.conn->open()) {
        e.conn->on_close(nullptr);
        e.conn->close("replaced by a new connection");
      }
      c->send_frame(encode(kSigConnectAck, (uint32_t)rank_));
      attach(e, c);
    });
    c->on_data([reader](const uint8_t* d, size_t n) { return (*reader)(d, n); });
  }

  void dial(Edge& e) {
    if (e.addresses.empty() || e.dialing) return;
    e.dialing = true;
    auto addr = e.addresses[e.next_addr++ % e.addresses.size()];
    int peer = e.peer;
    poller_.connect(addr.second, (int)addr.first, [this, peer](std::shared_ptr<Conn> c) {
      Edge& e = edges_[peer];
      e.dialing = false;
      if (!c || e.connected || stop_) {
        if (c) c->close("not needed");
        e.next_dial = now_seconds() + 0.05;
        return;
      }
      ConnectMessage m;
      m.key = store_key_;
      m.sourceRank = (uint32_t)rank_;
      m.uid = uid_;
      c->send_frame(encode(kSigConnect, m));
      std::weak_ptr<Conn> weak = c;
      auto acked = std::make_shared<bool>(false);
      auto reader = std::make_shared<FrameReader>([this, peer, weak, acked](Reader& r, bool) {
        auto c = weak.lock();
        if (!c) return;
        uint64_t sig = r.read<uint64_t>();
        uint32_t who = r.read<uint32_t>();
        if (sig != kSigConnectAck || (int)who != peer) return c->close("bad mesh greeting reply");
        *acked = true;
        attach(edges_[peer], c);
      });
      c->on_data([reader](const uint8_t* d, size_t n) { return (*reader)(d, n); });
      c->on_close([this, peer, acked](const std::string&) {
        if (!*acked) edges_[peer].next_dial = now_seconds() + 0.05;
      });
    });
  }

  void attach(Edge& e, std::shared_ptr<Conn> c) {
    e.conn = c;
    e.connected = true;
    e.last_recv = e.last_send = now_seconds();
    int peer = e.peer;
    auto reader = std::make_shared<FrameReader>([this, peer](Reader& r, bool) { on_frame(peer, r); });
    c->on_data([reader](const uint8_t* d, size_t n) { return (*reader)(d, n); });
    c->on_close([this, peer](const std::string& why) {
      Edge& e = edges_[peer];
      e.connected = false;
      e.conn = nullptr;
      e.down_since = now_seconds();
      e.next_dial = now_seconds() + 0.05;
      if (!e.peer_exited && !shutting_down_) log_verbose("TcpStore rank %d: edge to rank %d closed (%s)", rank_, peer, why.c_str());
    });
    // anything not acknowledged before the connection broke goes out again, in order
    for (auto& [seq, body] : e.unacked) c->send_frame(body);
    check_ready();
  }

  void check_ready() {
    if (ready_) return;
    for (auto& [p, e] : edges_)
      if (!e.connected) return;
    ready_ = true;
  }

  void tick(double now) {
    if (!ready_ && rank_ != 0 && !rendezvous_ && rendezvous_retry_at_ > 0 && now >= rendezvous_retry_at_) {
      rendezvous_retry_at_ = 0;
      dial_rendezvous();
    }
    for (auto& [p, e] : edges_) {
      if (!e.connected) {
        // the lower rank of an edge dials
        if (rank_ < p && !e.peer_exited && !e.addresses.empty() && now >= e.next_dial) dial(e);
        continue;
      }
      // keepalive: ping after 20 s of silence, drop after 40 s (reference: core/store.cc:1563-1615)
      if (now - e.last_recv > 2 * keepalive_s_) {
        e.conn->close("no traffic for twice the keepalive interval");
      } else if (now - e.last_recv > keepalive_s_ && now - e.last_send > keepalive_s_ / 4) {
        e.conn->send_frame(encode(kSigKeepalive));
        e.last_send = now;
      }
    }
    if (shutting_down_) progress_shutdown(now);
  }

  // ---- messages ----
  void send_to(int dest, uint8_t type, uint32_t id, Bytes payload) {
    MessageHeader h{};
    h.ttl = (uint32_t)world_ + 4;
    h.destinationRank = (uint32_t)dest;
    h.id = id;
    h.sourceRank = (uint32_t)rank_;
    h.diagnosticSource = (uint32_t)rank_;
    h.messageType = type;
    h.broadcast = false;
    if (dest == rank_) return handle(h, Reader(payload.data(), payload.size()));
    route(h, payload.data(), payload.size(), -1);
  }

  void broadcast(uint8_t type, Bytes payload) {
    MessageHeader h{};
    h.ttl = (uint32_t)world_ + 4;
    h.destinationRank = ~0u;
    h.id = next_id_++;
    h.sourceRank = (uint32_t)rank_;
    h.messageType = type;
    h.broadcast = true;
    seen_broadcast_.insert(((uint64_t)h.sourceRank << 32) | h.id);
    for (auto& [p, e] : edges_) send_on_edge(e, h, payload.data(), payload.size());
  }

  void route(const MessageHeader& h, const uint8_t* payload, size_t n, int from) {
    int hop = first_hop_[h.destinationRank];
    auto it = edges_.find(hop);
    if (it == edges_.end()) {
      log_error("TcpStore rank %d: no route to rank %u", rank_, h.destinationRank);
      return;
    }
    (void)from;
    send_on_edge(it->second, h, payload, n);
  }

  void send_on_edge(Edge& e, MessageHeader h, const uint8_t* payload, size_t n) {
    if (e.peer_exited) return;
    h.seq = e.out_seq++;
    Writer w;
    w(kSigMessage);
    w.raw(&h, sizeof(h));
    w.raw(payload, n);
    e.unacked.emplace_back(h.seq, w.out);
    if (e.connected && e.conn && e.conn->open()) {
      if (fault_break_every_ > 0 && ++fault_count_ % (uint64_t)fault_break_every_ == 0) {
        // injected fault: the message is lost with its connection; the redial retransmits it (and anything else
        // the peer has not acknowledged) in order, and the peer drops what it had seen already
        ++fault_breaks_;
        e.conn->close("injected fault");
        return;
      }
      e.conn->send_frame(w.out);
      e.last_send = now_seconds();
    }
  }

  void on_frame(int peer, Reader& r) {
    Edge& e = edges_[peer];
    e.last_recv = now_seconds();
    uint64_t sig = r.read<uint64_t>();
    if (sig == kSigKeepalive) {
      if (e.conn) e.conn->send_frame(encode(kSigKeepaliveAck));
      return;
    }
    if (sig == kSigKeepaliveAck) return;
    if (sig == kSigMessageAck) {
      uint32_t seq = r.read<uint32_t>();
      while (!e.unacked.empty() && (int32_t)(e.unacked.front().first - seq) <= 0) e.unacked.pop_front();
      return;
    }
    if (sig != kSigMessage) return;
    MessageHeader h;
    r.raw(&h, sizeof(h));
    if (e.conn) e.conn->send_frame(encode(kSigMessageAck, h.seq));
    if ((int32_t)(h.seq - e.in_seq) < 0) return;  // retransmission of something already handled
    e.in_seq = h.seq + 1;
    if (h.broadcast) {
      uint64_t key = ((uint64_t)h.sourceRank << 32) | h.id;
      if (!seen_broadcast_.insert(key).second) return;
      if (h.ttl > 1) {
        MessageHeader f = h;
        f.ttl = h.ttl - 1;
        for (auto& [p, other] : edges_)
          if (p != peer) send_on_edge(other, f, r.p, r.remaining());
      }
      handle(h, r);
      return;
    }
    if ((int)h.destinationRank != rank_) {
      if (h.ttl <= 1) {
        log_error("TcpStore rank %d: dropping a message for rank %u whose TTL ran out", rank_, h.destinationRank);
        return;
      }
      if (h.messageType == kDiagnosticProbe) {
        Reader rr(r.p, r.remaining());
        report_probe(h, first_hop_[h.destinationRank], rr.read<std::string>());
      }
      MessageHeader f = h;
      f.ttl = h.ttl - 1;
      route(f, r.p, r.remaining(), peer);
      return;
    }
    handle(h, r);
  }

  void reply(const MessageHeader& req, Bytes payload) { send_to((int)req.sourceRank, kDone, req.id, std::move(payload)); }

  void wake_waiters(const std::string& key) {
    auto it = waiters_.find(key);
    if (it == waiters_.end()) return;
    auto list = std::move(it->second);
    waiters_.erase(it);
    const Bytes& v = kv_[key];
    for (const PendingAtOwner& p : list) {
      MessageHeader h{};
      h.sourceRank = p.requester;
      h.id = p.id;
      reply(h, p.type == kGet ? v : Bytes{});
    }
  }

  void handle(const MessageHeader& h, Reader r) {
    switch (h.messageType) {
      case kDone: {
        auto it = pending_.find(h.id);
        if (it == pending_.end()) return;
        auto w = it->second;
        pending_.erase(it);
        w->finish(Bytes(r.p, r.end));
        return;
      }
      case kSet: {
        std::string key;
        Bytes value;
        r(key, value);
        kv_[key] = std::move(value);
        wake_waiters(key);
        reply(h, {});
        return;
      }
      case kGet:
      case kWait: {
        std::string key = r.read<std::string>();
        auto it = kv_.find(key);
        if (it != kv_.end())
          reply(h, h.messageType == kGet ? it->second : Bytes{});
        else
          waiters_[key].push_back(PendingAtOwner{h.sourceRank, h.id, h.messageType});
        return;
      }
      case kCheck: {
        std::string key = r.read<std::string>();
        reply(h, Bytes{(uint8_t)(kv_.count(key) ? 1 : 0)});
        return;
      }
      case kAdd: {
        std::string key;
        int64_t delta;
        r(key, delta);
        int64_t cur = 0;
        auto it = kv_.find(key);
        if (it != kv_.end()) cur = strtoll(std::string(it->second.begin(), it->second.end()).c_str(), nullptr, 10);
        cur += delta;
        std::string s = std::to_string(cur);
        kv_[key] = Bytes(s.begin(), s.end());
        wake_waiters(key);
        reply(h, encode(cur));
        return;
      }
      case kCompareSet: {
        std::string key;
        Bytes expected, desired;
        r(key, expected, desired);
        auto it = kv_.find(key);
        if (it == kv_.end()) {
          if (expected.empty()) {
            kv_[key] = desired;
            wake_waiters(key);
            reply(h, desired);
          } else {
            reply(h, expected);  // c10d semantics: missing key with non-empty expectation returns the expectation
          }
        } else {
          if (it->second == expected) it->second = desired;
          reply(h, it->second);
        }
        return;
      }
      case kDelete: {
        std::string key = r.read<std::string>();
        reply(h, Bytes{(uint8_t)(kv_.erase(key) ? 1 : 0)});
        return;
      }
      case kNumKeys: reply(h, encode((int64_t)kv_.size())); return;
      case kDiagnosticProbe: report_probe(h, -1, r.read<std::string>()); return;
      case kDiagnosticInfo: {
        auto it = diag_reports_.find(h.id);
        if (it != diag_reports_.end()) it->second.push_back(r.read<std::string>());
        return;
      }
      case kShutdown: shutdown_seen_[h.sourceRank] = true; return;
      case kExit: {
        exit_seen_[h.sourceRank] = true;
        auto it = edges_.find((int)h.sourceRank);
        if (it != edges_.end()) it->second.peer_exited = true;
        if (!shutting_down_ && error_.empty()) {
          // a peer left while this rank still wants the store: everything pending and later fails
          error_ = strf("store was shut down on rank %u", h.sourceRank);
          auto pend = std::move(pending_);
          pending_.clear();
          for (auto& [id, w] : pend) w->finish({}, error_);
        }
        return;
      }
      case kExitAck: return;
      default: return;
    }
  }

  // ---- three-phase shutdown ----
  void begin_shutdown(std::shared_ptr<WaitObj> w) {
    shutting_down_ = true;
    shutdown_waiter_ = std::move(w);
    shutdown_phase_ = 1;
    shutdown_seen_[rank_] = true;
    phase_deadline_ = now_seconds() + 2.0;
    auto pend = std::move(pending_);
    pending_.clear();
    for (auto& [id, pw] : pend) pw->finish({}, "store was shut down on this rank");
    if (world_ == 1 || !ready_) {
      shutdown_phase_ = 4;
      if (shutdown_waiter_) shutdown_waiter_->finish({});
      return;
    }
    broadcast(kShutdown, {});
  }

  void progress_shutdown(double now) {
    auto all = [&](const std::vector<bool>& v) {
      for (int r = 0; r < world_; ++r)
        if (r != rank_ && !v[r] && !exit_seen_[r]) return false;
      return true;
    };
    if (shutdown_phase_ == 1 && (all(shutdown_seen_) || now > phase_deadline_)) {
      shutdown_phase_ = 2;
      phase_deadline_ = now + 1.0;
      exit_seen_[rank_] = true;
      broadcast(kExit, {});
    } else if (shutdown_phase_ == 2 && (all(exit_seen_) || now > phase_deadline_)) {
      shutdown_phase_ = 3;
      phase_deadline_ = now + 0.05;
      broadcast(kExitAck, {});
    } else if (shutdown_phase_ == 3 && now > phase_deadline_) {
      shutdown_phase_ = 4;
      if (shutdown_waiter_) shutdown_waiter_->finish({});
    }
  }

  std::string hostname_;
  int port_, world_, rank_;
  std::chrono::milliseconds timeout_;
  std::string store_key_, uid_;
  std::vector<std::vector<int>> mesh_;
  std::vector<int> first_hop_;

  Poller poller_;
  std::thread thread_;
  std::atomic<bool> stop_{false}, ready_{false}, failed_{false}, shutdown_called_{false};
  mutable std::mutex fatal_mu_;
  std::string fatal_;
  std::mutex queue_mu_;
  std::deque<std::function<void()>> queue_;

  // I/O-thread state
  std::vector<std::pair<uint32_t, std::string>> my_addresses_;
  std::map<int, Edge> edges_;
  std::shared_ptr<Conn> rendezvous_;
  double rendezvous_retry_at_ = 0;
  std::map<int, std::vector<std::pair<uint32_t, std::string>>> directory_;
  std::map<int, std::string> directory_uid_;
  std::map<int, std::shared_ptr<Conn>> rendezvous_conns_;
  std::unordered_map<std::string, Bytes> kv_;
  std::unordered_map<std::string, std::vector<PendingAtOwner>> waiters_;
  std::unordered_map<uint32_t, std::shared_ptr<WaitObj>> pending_;
  std::unordered_map<uint32_t, std::vector<std::string>> diag_reports_;  // probe id -> reports received so far
  int fault_break_every_ = 0;   // test hook: every Nth message, the edge's connection is cut instead of used
  uint64_t fault_count_ = 0, fault_breaks_ = 0;
  double keepalive_s_ = 20;     // ping after this much silence, drop the connection after twice as much
  std::set<uint64_t> seen_broadcast_;
  uint32_t next_id_ = 1;
  std::string error_;
  bool shutting_down_ = false;
  int shutdown_phase_ = 0;
  double phase_deadline_ = 0;
  std::shared_ptr<WaitObj> shutdown_waiter_;
  std::vector<bool> shutdown_seen_, exit_seen_;
};

}  // namespace

namespace {
std::mutex g_live_mu;
std::vector<std::weak_ptr<TcpStore>>& live_stores() {
  static auto* v = new std::vector<std::weak_ptr<TcpStore>>();  // never destroyed: used while the process exits
  return *v;
}
}  // namespace

std::shared_ptr<TcpStore> TcpStore::create(const std::string& hostname, int port, const std::string& key, int world,
                                           int rank, std::chrono::milliseconds timeout) {
  auto store = std::make_shared<TcpStoreImpl>(hostname, port, key, world, rank, timeout);
  std::lock_guard<std::mutex> lk(g_live_mu);
  auto& live = live_stores();
  live.erase(std::remove_if(live.begin(), live.end(), [](const std::weak_ptr<TcpStore>& w) { return w.expired(); }), live.end());
  live.push_back(store);
  return store;
}

void TcpStore::shutdown_all() {
  std::vector<std::shared_ptr<TcpStore>> alive;
  {
    std::lock_guard<std::mutex> lk(g_live_mu);
    for (auto& w : live_stores())
      if (auto s = w.lock()) alive.push_back(std::move(s));
  }
  for (auto& s : alive) {
    try {
      s->shutdown();
    } catch (...) {
    }
  }
}

}  // namespace moodist
