#include "tcp_transport.h"

#include <sys/socket.h>
#include <sys/uio.h>
#include <unistd.h>

#include <algorithm>
#include <cerrno>
#include <cstring>
#include <deque>
#include <functional>
#include <mutex>
#include <random>

#include "log.h"

namespace moodist {

// ------------------------------------------------------------------------------------------------
// registered memory
// ------------------------------------------------------------------------------------------------
namespace {
struct Region {
  uintptr_t base = 0;
  size_t size = 0;
  uint64_t landed = 0;
  bool live = false;
};
struct MrState {
  std::mutex mu;
  std::vector<Region> regions;
  std::vector<uint32_t> free_keys;
};
MrState& mr_state() {
  static MrState* s = new MrState();
  return *s;
}
}  // namespace

MrTable& MrTable::instance() {
  static MrTable t;
  return t;
}
uint32_t MrTable::add(void* base, size_t size) {
  MrState& s = mr_state();
  std::lock_guard<std::mutex> lk(s.mu);
  uint32_t key;
  if (!s.free_keys.empty()) {
    key = s.free_keys.back();
    s.free_keys.pop_back();
  } else {
    key = (uint32_t)s.regions.size();
    s.regions.emplace_back();
  }
  s.regions[key] = Region{(uintptr_t)base, size, 0, true};
  return key;
}
void MrTable::remove(uint32_t key) {
  MrState& s = mr_state();
  std::lock_guard<std::mutex> lk(s.mu);
  if (key < s.regions.size() && s.regions[key].live) {
    s.regions[key].live = false;
    s.free_keys.push_back(key);
  }
}
void* MrTable::check(uint32_t key, uintptr_t addr, size_t bytes) {
  MrState& s = mr_state();
  std::lock_guard<std::mutex> lk(s.mu);
  if (key >= s.regions.size()) return nullptr;
  const Region& r = s.regions[key];
  if (!r.live || addr < r.base || bytes > r.size || addr - r.base > r.size - bytes) return nullptr;
  return (void*)addr;
}
uint64_t MrTable::landed(uint32_t key) {
  MrState& s = mr_state();
  std::lock_guard<std::mutex> lk(s.mu);
  return key < s.regions.size() ? s.regions[key].landed : 0;
}
void MrTable::add_landed(uint32_t key, uint64_t n) {
  MrState& s = mr_state();
  std::lock_guard<std::mutex> lk(s.mu);
  if (key < s.regions.size()) s.regions[key].landed += n;
}

// ------------------------------------------------------------------------------------------------
// copies between address spaces of one machine
// ------------------------------------------------------------------------------------------------
bool vm_read(int64_t pid, void* local, uintptr_t remote, size_t bytes) {
  uint8_t* l = (uint8_t*)local;
  while (bytes) {
    iovec li{l, bytes}, ri{(void*)remote, bytes};
    ssize_t n = process_vm_readv((pid_t)pid, &li, 1, &ri, 1, 0);
    if (n <= 0) return false;
    l += n;
    remote += (size_t)n;
    bytes -= (size_t)n;
  }
  return true;
}

bool vm_read_strided(int64_t pid, void* local, size_t dst_pitch, uintptr_t remote, size_t src_pitch, uint64_t rows,
                     size_t row_bytes) {
  constexpr int kBatch = 512;  // well under IOV_MAX
  iovec li[kBatch], ri[kBatch];
  for (uint64_t r0 = 0; r0 < rows; r0 += kBatch) {
    int n = (int)std::min<uint64_t>(kBatch, rows - r0);
    for (int i = 0; i < n; ++i) {
      li[i] = iovec{(uint8_t*)local + (r0 + i) * dst_pitch, row_bytes};
      ri[i] = iovec{(void*)(remote + (r0 + i) * src_pitch), row_bytes};
    }
    ssize_t got = process_vm_readv((pid_t)pid, li, n, ri, n, 0);
    if (got != (ssize_t)((size_t)n * row_bytes)) {
      // a short transfer stops at an iovec boundary or inside one: finish row by row
      for (int i = 0; i < n; ++i)
        if (!vm_read(pid, li[i].iov_base, (uintptr_t)ri[i].iov_base, row_bytes)) return false;
    }
  }
  return true;
}

// ------------------------------------------------------------------------------------------------
// transport
// ------------------------------------------------------------------------------------------------
struct TcpTransport::Peer {
  std::shared_ptr<Conn> conn;
  bool ready = false;
  int64_t pid = 0;             // > 0: this rank may read that process's memory
  bool reads_me = false;       // the peer has told us it may read ours
  int64_t reader_pid = 0;
  std::vector<std::pair<std::string, int>> candidates;
  size_t next_candidate = 0;
  int attempts = 0;
  struct Queued {
    Bytes header;
    const void* payload;
    size_t n;
    std::shared_ptr<void> keep;
  };
  std::deque<Queued> backlog;  // records issued before the connection was ready
  std::function<void()> dial;  // tries the next advertised address of this peer (dialing side only)
};

TcpTransport::TcpTransport(Poller& poller, std::string group, int rank, int world)
    : poller_(poller), group_(std::move(group)), rank_(rank), world_(world) {
  peers_.resize(world);
  for (auto& p : peers_) p = std::make_unique<Peer>();
  sink_.resize(1 << 16);
}

TcpTransport::~TcpTransport() {
  for (auto& p : peers_)
    if (p->conn) {
      p->conn->on_close(nullptr);
      p->conn->on_data(nullptr);
      p->conn->close("transport destroyed");
    }
}

std::vector<std::string> TcpTransport::listen() {
  auto accept = [this](std::shared_ptr<Conn> c) {
    // the dialer speaks first; until its greeting arrives the connection has no owner
    std::weak_ptr<Conn> weak = c;
    auto reader = std::make_shared<FrameReader>([this, weak](Reader& r, bool) {
      auto c = weak.lock();
      if (!c) return;
      uint64_t sig = 0;
      std::string group;
      uint32_t peer = ~0u;
      try {
        r(sig, group, peer);
      } catch (const WireError&) {
        sig = 0;
      }
      if (sig != kTcpDevSig || group != group_ || peer >= (uint32_t)world_ || (int)peer == rank_) {
        c->close("bad greeting");
        return;
      }
      if (peers_[peer]->conn && peers_[peer]->conn->open()) {
        c->close("duplicate connection");
        return;
      }
      c->send_frame(encode(kTcpDevSig, group_, (uint32_t)rank_));
      attach((int)peer, c);
      peers_[peer]->ready = true;
    });
    c->on_data([reader](const uint8_t* d, size_t n) { return (*reader)(d, n); });
  };
  int p4 = poller_.listen("0.0.0.0", 0, accept);
  int p6 = poller_.listen("::", 0, accept);
  std::vector<std::string> out;
  // Ranks of one machine (and one network namespace) talk over a unix-domain socket, which costs a fraction of
  // loopback TCP per message; it is advertised first, and a rank elsewhere finds nobody behind the name and goes
  // on to the TCP addresses. The name lives in the abstract namespace: nothing to unlink.
  if (!env_flag("MOODIST_DISABLE_UNIX_SOCKETS")) {
    std::string name = strf("unix:moodist-%016llx-%d-%d-%08x", (unsigned long long)std::hash<std::string>{}(group_), rank_,
                            (int)getpid(), (unsigned)std::random_device{}());
    try {
      poller_.listen(name, 0, accept);
      out.push_back(name + " 0");
    } catch (const std::exception& e) {
      log_info("tcp transport: no unix-domain listener (%s), TCP only", e.what());
    }
  }
  for (const std::string& a : local_addresses()) {
    bool v6 = a.find(':') != std::string::npos;
    int port = v6 ? p6 : p4;
    if (port > 0) out.push_back(a + " " + std::to_string(port));
  }
  if (out.empty()) fail("tcp transport: could not open a listening socket");
  return out;
}

void TcpTransport::connect_all(const std::vector<std::vector<std::string>>& addrs) {
  for (int r = rank_ + 1; r < world_; ++r) {
    Peer& p = *peers_[r];
    for (const std::string& s : addrs[r]) {
      auto sp = s.rfind(' ');
      if (sp == std::string::npos) continue;
      p.candidates.emplace_back(s.substr(0, sp), atoi(s.c_str() + sp + 1));
    }
    // Same host is the common case here: loopback works even when no other interface is shared.
    // the closure lives in the peer record and refers to itself through it (a shared_ptr to itself would
    // never be released)
    p.dial = [this, r]() {
      Peer& p = *peers_[r];
      if (p.ready) return;
      if (p.candidates.empty()) {
        if (error_) error_(r, "peer advertised no address");
        return;
      }
      if (p.attempts > 20 * (int)p.candidates.size()) {
        if (error_) error_(r, "could not connect to any advertised address");
        return;
      }
      auto cand = p.candidates[p.next_candidate % p.candidates.size()];
      ++p.next_candidate;
      ++p.attempts;
      poller_.connect(cand.first, cand.second, [this, r](std::shared_ptr<Conn> c) {
        Peer& p = *peers_[r];
        if (p.ready) {
          if (c) c->close("not needed");
          return;
        }
        if (!c) {
          p.dial();
          return;
        }
        c->send_frame(encode(kTcpDevSig, group_, (uint32_t)rank_));
        std::weak_ptr<Conn> weak = c;
        auto greeted = std::make_shared<bool>(false);
        auto reader = std::make_shared<FrameReader>([this, r, weak, greeted](Reader& rd, bool) {
          auto c = weak.lock();
          if (!c) return;
          uint64_t sig = 0;
          std::string group;
          uint32_t peer = ~0u;
          try {
            rd(sig, group, peer);
          } catch (const WireError&) {
            sig = 0;
          }
          if (sig != kTcpDevSig || group != group_ || (int)peer != r) {
            c->close("bad greeting reply");
            return;
          }
          *greeted = true;
          attach(r, c);
          Peer& p = *peers_[r];
          p.ready = true;
          while (!p.backlog.empty()) {
            auto q = std::move(p.backlog.front());
            p.backlog.pop_front();
            send_record(r, std::move(q.header), q.payload, q.n, std::move(q.keep));
          }
        });
        c->on_data([reader](const uint8_t* d, size_t n) { return (*reader)(d, n); });
        c->on_close([this, r, greeted](const std::string&) {
          if (!*greeted) peers_[r]->dial();  // wrong process behind that address: try the next one
        });
      });
    };
    p.dial();
  }
}

bool TcpTransport::all_connected() const { return connected_count() == world_ - 1; }
int TcpTransport::unix_peers() const {
  int n = 0;
  for (int r = 0; r < world_; ++r) {
    if (r == rank_ || !peers_[r]->ready || !peers_[r]->conn || peers_[r]->conn->fd() < 0) continue;
    sockaddr_storage ss;
    socklen_t len = sizeof(ss);
    if (getsockname(peers_[r]->conn->fd(), (sockaddr*)&ss, &len) == 0 && ss.ss_family == AF_UNIX) ++n;
  }
  return n;
}
void TcpTransport::hold_sends() {
  for (int r = 0; r < world_; ++r)
    if (r != rank_ && peers_[r]->conn) peers_[r]->conn->cork();
}
void TcpTransport::release_sends() {
  for (int r = 0; r < world_; ++r)
    if (r != rank_ && peers_[r]->conn) peers_[r]->conn->uncork();
}
int TcpTransport::connected_count() const {
  int n = 0;
  for (int r = 0; r < world_; ++r)
    if (r != rank_ && peers_[r]->ready) ++n;
  return n;
}

void TcpTransport::attach(int peer, std::shared_ptr<Conn> c) {
  Peer& p = *peers_[peer];
  p.conn = c;
  c->peer_name = "rank " + std::to_string(peer);
  auto reader = std::make_shared<FrameReader>([this, peer](Reader& r, bool) { handle_record(peer, r); });
  c->on_data([reader](const uint8_t* d, size_t n) { return (*reader)(d, n); });
  c->on_close([this, peer](const std::string& why) {
    peers_[peer]->ready = false;
    // every operation still waiting on this peer fails
    if (error_) error_(peer, why);
  });
  // acceptor side: flush what was queued while waiting for the dialer
  if (peer < rank_) {
    p.ready = true;
    while (!p.backlog.empty()) {
      auto q = std::move(p.backlog.front());
      p.backlog.pop_front();
      send_record(peer, std::move(q.header), q.payload, q.n, std::move(q.keep));
    }
  }
}

void TcpTransport::send_record(int peer, Bytes header, const void* payload, size_t n, std::shared_ptr<void> keep) {
  Peer& p = *peers_[peer];
  if (!p.ready || !p.conn || !p.conn->open()) {
    p.backlog.push_back(Peer::Queued{std::move(header), payload, n, std::move(keep)});
    return;
  }
  p.conn->cork();  // header and payload leave in one writev
  p.conn->send_frame(header);
  if (n) p.conn->send_ref(payload, n, std::move(keep));
  p.conn->uncork();
  bytes_sent_ += header.size() + 8 + n;
}

void TcpTransport::post_write(int dst, const void* src, size_t bytes, uint32_t rkey, uintptr_t raddr, Done done,
                              std::shared_ptr<void> keep) {
  if (dst == rank_) {
    void* d = MrTable::instance().check(rkey, raddr, bytes);
    if (d && bytes) memcpy(d, src, bytes);
    if (d) MrTable::instance().add_landed(rkey, bytes);
    if (done) done(d != nullptr);
    return;
  }
  uint64_t index = next_index_++;
  if (peers_[dst]->reads_me && bytes >= direct_min_) {
    // the receiver checks the destination against its table and then fetches the bytes itself
    Pending pend{std::move(done), nullptr, bytes};
    pend.keep = std::move(keep);
    pending_[index] = std::move(pend);
    send_record(dst, encode((uint8_t)kMsgWriteDirect, index, rkey, (uint64_t)raddr, (uint64_t)bytes, (uint64_t)(uintptr_t)src),
                nullptr, 0, nullptr);
    return;
  }
  pending_[index] = Pending{std::move(done), nullptr, bytes};
  send_record(dst, encode((uint8_t)kMsgWrite, index, rkey, (uint64_t)raddr, (uint64_t)bytes), src, bytes,
              std::move(keep));
}

bool TcpTransport::probe_direct(int peer, int64_t pid, uintptr_t probe_addr, uint64_t probe_value) {
  if (peer == rank_ || pid <= 0) return false;
  uint64_t v = 0;
  if (!vm_read(pid, &v, probe_addr, sizeof(v)) || v != probe_value) return false;
  peers_[peer]->pid = pid;
  send_record(peer, encode((uint8_t)kMsgDirectOk, (int64_t)getpid()), nullptr, 0, nullptr);
  return true;
}

void TcpTransport::post_read(int dst, void* local, size_t bytes, uint32_t rkey, uintptr_t raddr, Done done) {
  if (dst == rank_) {
    void* s = MrTable::instance().check(rkey, raddr, bytes);
    if (s && bytes) memcpy(local, s, bytes);
    if (done) done(s != nullptr);
    return;
  }
  uint64_t index = next_index_++;
  if (peers_[dst]->pid > 0 && bytes >= direct_min_) {
    Pending pend{std::move(done), local, bytes};
    pend.raddr = raddr;
    pend.peer = dst;
    pending_[index] = std::move(pend);
    send_record(dst, encode((uint8_t)kMsgReadCheck, index, rkey, (uint64_t)raddr, (uint64_t)bytes), nullptr, 0, nullptr);
    return;
  }
  pending_[index] = Pending{std::move(done), local, bytes};
  send_record(dst, encode((uint8_t)kMsgRead, index, rkey, (uint64_t)raddr, (uint64_t)bytes), nullptr, 0, nullptr);
}

void TcpTransport::post_read_strided(int dst, void* local, uint64_t rows, size_t row_bytes, size_t dst_pitch, uint32_t rkey,
                                     uintptr_t raddr, size_t src_pitch, Done done) {
  if (rows <= 1 || (src_pitch == row_bytes && dst_pitch == row_bytes)) {
    post_read(dst, local, (size_t)rows * row_bytes, rkey, raddr, std::move(done));
    return;
  }
  if (dst == rank_) {
    uint64_t span = (rows - 1) * (uint64_t)src_pitch + row_bytes;
    uint8_t* s = (uint8_t*)MrTable::instance().check(rkey, raddr, span);
    if (s)
      for (uint64_t r = 0; r < rows; ++r) memcpy((uint8_t*)local + r * dst_pitch, s + r * src_pitch, row_bytes);
    if (done) done(s != nullptr);
    return;
  }
  uint64_t index = next_index_++;
  Pending pend{std::move(done), local, (size_t)rows * row_bytes};
  pend.rows = rows;
  pend.row_bytes = row_bytes;
  pend.dst_pitch = dst_pitch;
  if (peers_[dst]->pid > 0 && (size_t)rows * row_bytes >= direct_min_) {
    pend.raddr = raddr;
    pend.src_pitch = src_pitch;
    pend.peer = dst;
    pending_[index] = std::move(pend);
    uint64_t span = (rows - 1) * (uint64_t)src_pitch + row_bytes;
    send_record(dst, encode((uint8_t)kMsgReadCheck, index, rkey, (uint64_t)raddr, span), nullptr, 0, nullptr);
    return;
  }
  pending_[index] = std::move(pend);
  send_record(dst, encode((uint8_t)kMsgReadStrided, index, rkey, (uint64_t)raddr, rows, (uint64_t)row_bytes, (uint64_t)src_pitch),
              nullptr, 0, nullptr);
}

void TcpTransport::post_send(int dst, Bytes payload) {
  int copies = 1;
  if (fault_hook) {
    int f = fault_hook(dst, payload);
    if (f == 1) return;
    if (f == 2) copies = 2;
  }
  for (int i = 0; i < copies; ++i) {
    if (dst == rank_) {
      if (recv_) recv_(rank_, payload);
      continue;
    }
    uint64_t index = next_index_++;
    auto keep = std::make_shared<Bytes>(i + 1 == copies ? std::move(payload) : payload);
    send_record(dst, encode((uint8_t)kMsgSend, index, (uint64_t)keep->size()), keep->data(), keep->size(), keep);
  }
}

void TcpTransport::handle_record(int peer, Reader& r) {
  Peer& p = *peers_[peer];
  uint8_t type = r.read<uint8_t>();
  bytes_recv_ += r.remaining() + 9;
  switch (type) {
    case kMsgWrite: {
      uint64_t index, raddr, bytes;
      uint32_t rkey;
      r(index, rkey, raddr, bytes);
      void* dst = MrTable::instance().check(rkey, (uintptr_t)raddr, bytes);
      auto conn = p.conn;
      if (!dst) {
        // out-of-bounds or unknown region: swallow the payload, report the error to the writer
        log_error("tcp transport: rank %d wrote outside registered memory (key %u, %llu bytes)", peer, rkey,
                  (unsigned long long)bytes);
        auto sink = std::make_shared<Bytes>(bytes);
        conn->read_into(sink->data(), bytes, [this, peer, index, sink] {
          send_record(peer, encode((uint8_t)kMsgCompletionError, index), nullptr, 0, nullptr);
        });
        if (bytes == 0) send_record(peer, encode((uint8_t)kMsgCompletionError, index), nullptr, 0, nullptr);
        break;
      }
      auto finish = [this, peer, index, rkey, bytes] {
        bytes_recv_ += bytes;
        MrTable::instance().add_landed(rkey, bytes);
        send_record(peer, encode((uint8_t)kMsgCompletionSuccess, index), nullptr, 0, nullptr);
      };
      if (bytes == 0)
        finish();
      else
        conn->read_into(dst, bytes, finish);
      break;
    }
    case kMsgCompletionSuccess:
    case kMsgCompletionError: {
      uint64_t index = r.read<uint64_t>();
      auto it = pending_.find(index);
      if (it == pending_.end()) break;
      Done done = std::move(it->second.done);
      pending_.erase(it);
      if (done) done(type == kMsgCompletionSuccess);
      break;
    }
    case kMsgSend: {
      uint64_t index, bytes;
      r(index, bytes);
      auto buf = std::make_shared<Bytes>(bytes);
      auto deliver = [this, peer, buf, bytes] {
        bytes_recv_ += bytes;
        if (recv_) recv_(peer, std::move(*buf));
      };
      if (bytes == 0)
        deliver();
      else
        p.conn->read_into(buf->data(), bytes, deliver);
      break;
    }
    case kMsgRead: {
      uint64_t index, raddr, bytes;
      uint32_t rkey;
      r(index, rkey, raddr, bytes);
      void* src = MrTable::instance().check(rkey, (uintptr_t)raddr, bytes);
      if (!src) {
        log_error("tcp transport: rank %d read outside registered memory (key %u)", peer, rkey);
        send_record(peer, encode((uint8_t)kMsgCompletionError, index), nullptr, 0, nullptr);
        break;
      }
      send_record(peer, encode((uint8_t)kMsgReadSuccess, index, (uint64_t)bytes), src, bytes, nullptr);
      break;
    }
    case kMsgReadStrided: {
      uint64_t index, raddr, rows, row_bytes, src_pitch;
      uint32_t rkey;
      r(index, rkey, raddr, rows, row_bytes, src_pitch);
      // the span the request touches, with overflow checks: (rows - 1) * src_pitch + row_bytes
      uint64_t span = 0, total = 0;
      bool bad = rows == 0 || row_bytes == 0 || __builtin_mul_overflow(rows - 1, src_pitch, &span) ||
                 __builtin_add_overflow(span, row_bytes, &span) || __builtin_mul_overflow(rows, row_bytes, &total);
      uint8_t* src = bad ? nullptr : (uint8_t*)MrTable::instance().check(rkey, (uintptr_t)raddr, span);
      if (!src) {
        log_error("tcp transport: rank %d strided read outside registered memory (key %u)", peer, rkey);
        send_record(peer, encode((uint8_t)kMsgCompletionError, index), nullptr, 0, nullptr);
        break;
      }
      Peer& q = *peers_[peer];
      if (!q.ready || !q.conn || !q.conn->open()) break;  // the requester is gone
      q.conn->cork();  // header and every run leave in as few writev calls as possible
      q.conn->send_frame(encode((uint8_t)kMsgReadSuccess, index, total));
      for (uint64_t k = 0; k < rows; ++k) q.conn->send_ref(src + k * src_pitch, (size_t)row_bytes, nullptr);
      q.conn->uncork();
      bytes_sent_ += total;
      break;
    }
    case kMsgReadSuccess: {
      uint64_t index, bytes;
      r(index, bytes);
      auto it = pending_.find(index);
      if (it == pending_.end() || it->second.bytes != bytes) {
        p.conn->close("unexpected read reply");
        break;
      }
      Pending pend = std::move(it->second);
      pending_.erase(it);
      auto finish = [this, pend, bytes] {
        bytes_recv_ += bytes;
        if (pend.done) pend.done(true);
      };
      if (bytes == 0) {
        finish();
      } else if (pend.rows <= 1) {
        p.conn->read_into(pend.local, bytes, finish);
      } else {
        // scatter the reply: one run at a time, each completion arms the next
        struct Scatter {
          std::shared_ptr<Conn> conn;
          uint8_t* base;
          uint64_t rows, k = 0;
          size_t row_bytes, pitch;
          std::function<void()> finish;
          std::function<void()> step;
        };
        auto sc = std::make_shared<Scatter>();
        sc->conn = p.conn;
        sc->base = (uint8_t*)pend.local;
        sc->rows = pend.rows;
        sc->row_bytes = pend.row_bytes;
        sc->pitch = pend.dst_pitch;
        sc->finish = finish;
        std::weak_ptr<Scatter> weak = sc;
        sc->step = [weak] {
          auto s = weak.lock();
          if (!s) return;
          if (++s->k == s->rows) {
            auto fin = std::move(s->finish);
            fin();
            return;
          }
          auto keep = s;
          s->conn->read_into(s->base + s->k * s->pitch, s->row_bytes, [keep] { keep->step(); });
        };
        auto keep = sc;
        p.conn->read_into(sc->base, sc->row_bytes, [keep] { keep->step(); });
      }
      break;
    }
    case kMsgDirectOk: {
      int64_t pid = r.read<int64_t>();
      p.reads_me = pid > 0;
      p.reader_pid = pid;
      break;
    }
    case kMsgWriteDirect: {
      uint64_t index, raddr, bytes, src;
      uint32_t rkey;
      r(index, rkey, raddr, bytes, src);
      void* dst = MrTable::instance().check(rkey, (uintptr_t)raddr, bytes);
      bool ok = dst != nullptr && p.pid > 0;
      if (!ok) {
        log_error("tcp transport: rank %d asked for a direct write outside registered memory (key %u, %llu bytes)", peer,
                  rkey, (unsigned long long)bytes);
      } else if (!vm_read(p.pid, dst, (uintptr_t)src, bytes)) {
        log_error("tcp transport: reading %llu bytes from rank %d's memory failed: %s", (unsigned long long)bytes, peer,
                  strerror(errno));
        ok = false;
      }
      if (ok) {
        bytes_direct_ += bytes;
        MrTable::instance().add_landed(rkey, bytes);
      }
      send_record(peer, encode((uint8_t)(ok ? kMsgCompletionSuccess : kMsgCompletionError), index), nullptr, 0, nullptr);
      break;
    }
    case kMsgReadCheck: {
      uint64_t index, raddr, span;
      uint32_t rkey;
      r(index, rkey, raddr, span);
      bool ok = MrTable::instance().check(rkey, (uintptr_t)raddr, span) != nullptr;
      if (!ok) log_error("tcp transport: rank %d read outside registered memory (key %u)", peer, rkey);
      send_record(peer, encode((uint8_t)(ok ? kMsgReadGranted : kMsgCompletionError), index), nullptr, 0, nullptr);
      break;
    }
    case kMsgReadGranted: {
      uint64_t index = r.read<uint64_t>();
      auto it = pending_.find(index);
      if (it == pending_.end()) break;
      Pending pend = std::move(it->second);
      pending_.erase(it);
      bool ok = pend.rows <= 1 ? vm_read(p.pid, pend.local, pend.raddr, pend.bytes)
                               : vm_read_strided(p.pid, pend.local, pend.dst_pitch, pend.raddr, pend.src_pitch, pend.rows,
                                                 pend.row_bytes);
      if (ok)
        bytes_direct_ += pend.bytes;
      else
        log_error("tcp transport: reading from rank %d's memory failed: %s", peer, strerror(errno));
      if (pend.done) pend.done(ok);
      break;
    }
    default:
      p.conn->close("unknown record type");
  }
}

}  // namespace moodist
