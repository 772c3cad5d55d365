#include "setup_comms.h"

#include <deque>
#include <map>
#include <random>

#include "log.h"
#include "net.h"

namespace moodist {
namespace {

class SetupCommsImpl final : public SetupComms {
 public:
  SetupCommsImpl(KVStore& store, const std::string& key, int rank, int world, double timeout_s)
      : key_(key), rank_(rank), world_(world), timeout_(timeout_s) {
    std::random_device rd;
    sender_id_ = ((uint64_t)rd() << 32) ^ rd();
    if (world == 1) return;
    // listen, publish, dial the next rank; the previous rank dials us
    auto accept = [this](std::shared_ptr<Conn> c) { on_accept(std::move(c)); };
    int p4 = poller_.listen("0.0.0.0", 0, accept);
    int p6 = poller_.listen("::", 0, accept);
    std::vector<std::string> mine;
    for (const std::string& a : local_addresses()) {
      int port = a.find(':') != std::string::npos ? p6 : p4;
      if (port > 0) mine.push_back(a + " " + std::to_string(port));
    }
    if (mine.empty()) fail("setup comms: cannot listen");
    const std::string pfx = "moodist/setup/" + key + "/";
    store.set_str(pfx + std::to_string(rank), to_hex(encode(mine)));
    int next = (rank + 1) % world;
    std::vector<std::string> theirs;
    decode_exact(from_hex(store.get_str(pfx + std::to_string(next))), theirs);
    for (const std::string& s : theirs) {
      auto sp = s.rfind(' ');
      if (sp != std::string::npos) candidates_.emplace_back(s.substr(0, sp), atoi(s.c_str() + sp + 1));
    }
    dial();
    double deadline = now_seconds() + timeout_;
    while (!(next_ && next_ready_ && prev_)) {
      if (now_seconds() > deadline) fail("setup comms: timed out building the ring");
      poller_.poll(10);
    }
  }

  std::vector<Bytes> allgather_bytes(const Bytes& mine) override {
    std::vector<Bytes> all(world_);
    all[rank_] = mine;
    if (world_ == 1) return all;
    // classic ring: in step s every rank forwards the blob that originated s ranks behind it
    uint32_t round = ++ag_round_;
    Bytes cur = mine;
    int origin = rank_;
    for (int s = 0; s < world_ - 1; ++s) {
      send_frame(kSetupSigAllGather, (uint32_t)origin, (uint32_t)round, 1, cur);
      Pending m = wait_for([&](const Pending& p) { return p.sig == kSetupSigAllGather && p.dst == round; });
      origin = (int)m.src;
      cur = std::move(m.payload);
      all[origin] = cur;
    }
    return all;
  }

  void send_bytes(int dst, const Bytes& payload) override {
    if (dst == rank_) {
      inbox_.push_back(Pending{kSetupSigMessage, (uint32_t)rank_, (uint32_t)rank_, 0, payload});
      return;
    }
    send_frame(kSetupSigMessage, (uint32_t)rank_, (uint32_t)dst, (uint32_t)world_, payload);
  }

  Bytes recv_bytes(int src) override {
    Pending m = wait_for([&](const Pending& p) { return p.sig == kSetupSigMessage && (int)p.src == src; });
    return std::move(m.payload);
  }

 private:
  struct Pending {
    uint64_t sig;
    uint32_t src, dst, ttl;
    Bytes payload;
  };

  void dial() {
    if (candidates_.empty()) fail("setup comms: the next rank published no address");
    auto cand = candidates_[attempt_++ % candidates_.size()];
    poller_.connect(cand.first, cand.second, [this](std::shared_ptr<Conn> c) {
      if (!c) {
        if (attempt_ < 200) dial();
        return;
      }
      next_ = c;
      // first frame: dst = ~0, payload "connect" + group key
      Writer w;
      w(kSetupSigMessage, sender_id_, (uint32_t)rank_, ~0u, 1u);
      std::string hello = "connect" + key_;
      w.raw(hello.data(), hello.size());
      c->send_frame(w.out);
      next_ready_ = true;
      c->on_close([this](const std::string&) { next_ = nullptr; });
    });
  }

  void on_accept(std::shared_ptr<Conn> c) {
    std::weak_ptr<Conn> weak = c;
    auto reader = std::make_shared<FrameReader>([this, weak](Reader& r, bool) {
      auto c = weak.lock();
      if (!c) return;
      uint64_t sig, sender;
      uint32_t src, dst, ttl;
      r(sig, sender, src, dst, ttl);
      if (dst == ~0u) {
        std::string hello((const char*)r.p, r.remaining());
        if (sig != kSetupSigMessage || hello != "connect" + key_ || (int)src != (rank_ - 1 + world_) % world_) {
          c->close("not the previous rank of this ring");
          return;
        }
        prev_ = c;
        return;
      }
      if (c != prev_) return;
      Pending m{sig, src, dst, ttl, Bytes(r.p, r.end)};
      if (sig == kSetupSigMessage && (int)dst != rank_) {
        if (ttl > 1) send_frame(sig, src, dst, ttl - 1, m.payload);  // not for us: pass it on
        return;
      }
      inbox_.push_back(std::move(m));
    });
    c->on_data([reader](const uint8_t* d, size_t n) { return (*reader)(d, n); });
  }

  void send_frame(uint64_t sig, uint32_t src, uint32_t dst, uint32_t ttl, const Bytes& payload) {
    if (!next_) fail("setup comms: the connection to the next rank is gone");
    Writer w;
    w(sig, sender_id_, src, dst, ttl);
    w.raw(payload.data(), payload.size());
    next_->send_frame(w.out);
  }

  template <class Pred>
  Pending wait_for(Pred pred) {
    double deadline = now_seconds() + timeout_;
    for (;;) {
      for (auto it = inbox_.begin(); it != inbox_.end(); ++it) {
        if (pred(*it)) {
          Pending m = std::move(*it);
          inbox_.erase(it);
          return m;
        }
      }
      if (now_seconds() > deadline) fail("setup comms: timed out waiting for a message");
      poller_.poll(10);
    }
  }

  std::string key_;
  int rank_, world_;
  double timeout_;
  uint64_t sender_id_ = 0;
  Poller poller_;
  std::vector<std::pair<std::string, int>> candidates_;
  int attempt_ = 0;
  std::shared_ptr<Conn> next_, prev_;
  bool next_ready_ = false;
  std::deque<Pending> inbox_;
  uint32_t ag_round_ = 0;
};

}  // namespace

std::unique_ptr<SetupComms> SetupComms::create(KVStore& store, const std::string& group_key, int rank, int world,
                                               double timeout_s) {
  return std::make_unique<SetupCommsImpl>(store, group_key, rank, world, timeout_s);
}

}  // namespace moodist
