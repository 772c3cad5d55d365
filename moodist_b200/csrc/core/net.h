// Non-blocking sockets on one epoll loop: listeners, outgoing connections with retry across several
// candidate addresses, a per-connection write queue, Unix-domain fd passing, and the framed stream
//     u32 0x40ea69f4 | u32 bodyBytes | body            (0xf555d4e4 when a file descriptor rides along)
// that all control-plane TCP traffic uses. Reference: core/socket.cc:107-363, 447-1250 (epoll sockets,
// write queue, sendFd/recvFd) and core/connection.cc:33-34, 51-224 (framing).
//
// Unlike the reference (global socket threads + a thread pool), every Poller is driven by exactly one
// thread — the owner's progress thread — so handlers never race with the owner's other work.
#pragma once

#include <sys/socket.h>

#include <cstdint>
#include <deque>
#include <functional>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include "wire.h"

namespace moodist {

constexpr uint32_t kFrameSig = 0x40ea69f4u;
constexpr uint32_t kFrameSigFd = 0xf555d4e4u;

class Poller;

// A connected stream socket (TCP or Unix). Not thread safe: use from the poller thread only.
class Conn : public std::enable_shared_from_this<Conn> {
 public:
  // Called with newly arrived bytes; return how many were consumed (the rest is kept and offered again
  // together with later bytes). Returning SIZE_MAX closes the connection (protocol error).
  using DataFn = std::function<size_t(const uint8_t* data, size_t n)>;
  using CloseFn = std::function<void(const std::string& why)>;

  ~Conn();
  int fd() const { return fd_; }
  bool open() const { return fd_ >= 0 && !closed_; }

  void on_data(DataFn f) { on_data_ = f ? std::make_shared<DataFn>(std::move(f)) : nullptr; }
  void on_close(CloseFn f) { on_close_ = std::move(f); }

  // "Direct" receive: the next `n` incoming bytes are written straight into `dst` (no staging copy),
  // then `done` runs. Only valid from inside the data callback or `done` itself.
  void read_into(void* dst, size_t n, std::function<void()> done);

  // Queue bytes for sending. `keep` (optional) is held until the bytes are on the wire — used to send
  // user memory without copying it (the reference's zero-copy iovec path, core/tcpdev.cc:264-274).
  void send(Bytes data);
  void send_ref(const void* p, size_t n, std::shared_ptr<void> keep = nullptr, std::function<void()> sent = nullptr);
  // One framed message: signature, length, body.
  void send_frame(const Bytes& body);
  // Framed message plus one file descriptor (Unix sockets only).
  void send_frame_fd(const Bytes& body, int fd);
  size_t queued_bytes() const { return queued_; }

  void close(const std::string& why = "closed locally");

  std::string peer_name;  // for diagnostics

 private:
  friend class Poller;
  Conn(Poller* p, int fd) : poller_(p), fd_(fd) {}
  void handle_readable();
  void handle_writable();
  void flush();
  void update_interest();

  struct Out {
    Bytes owned;
    const uint8_t* ptr = nullptr;
    size_t len = 0, off = 0;
    std::shared_ptr<void> keep;
    std::function<void()> sent;
    int pass_fd = -1;
  };

  Poller* poller_;
  int fd_ = -1;
  bool closed_ = false, want_write_ = false, connecting_ = false;
  std::deque<Out> out_;
  size_t queued_ = 0;
  // receive buffer: raw storage (never zero-filled on growth) with `in_len_` valid bytes at its start
  std::unique_ptr<uint8_t[]> in_mem_;
  size_t in_cap_ = 0, in_len_ = 0;
  int cork_ = 0;  // while > 0, send*() only queue; uncork() flushes (one writev for a header and its payload)
  uint8_t* direct_dst_ = nullptr;
  size_t direct_left_ = 0;
  std::function<void()> direct_done_;
  std::shared_ptr<DataFn> on_data_;  // shared: a handler may replace itself while it runs
  CloseFn on_close_;
  std::function<void(bool)> on_connect_;
  std::deque<int> received_fds_;

 public:
  // Between cork() and the matching uncork() nothing is written to the socket; uncork() sends everything queued
  // with as few system calls as possible. Calls nest.
  void cork() { ++cork_; }
  void uncork() {
    if (cork_ > 0 && --cork_ == 0 && !connecting_ && !closed_) flush();
  }
  // fds received with SCM_RIGHTS, in arrival order
  int take_fd() {
    if (received_fds_.empty()) return -1;
    int f = received_fds_.front();
    received_fds_.pop_front();
    return f;
  }
};

// Helper that splits a Conn's byte stream into frames.
class FrameReader {
 public:
  using FrameFn = std::function<void(Reader& body, bool has_fd)>;
  explicit FrameReader(FrameFn f) : fn_(std::move(f)) {}
  size_t operator()(const uint8_t* data, size_t n);

 private:
  FrameFn fn_;
};

class Poller {
 public:
  Poller();
  ~Poller();

  // Listen on an address ("0.0.0.0", "::", "127.0.0.1", or "unix:<abstract name>"), port 0 = any.
  // Returns the bound port (0 for Unix). `accept` receives each new connection.
  int listen(const std::string& addr, int port, std::function<void(std::shared_ptr<Conn>)> accept);
  // Start a non-blocking connect. `done(conn)` gets nullptr on failure.
  void connect(const std::string& addr, int port, std::function<void(std::shared_ptr<Conn>)> done);

  // Run handlers for whatever is ready; waits at most timeout_ms.
  int poll(int timeout_ms);  // returns how many descriptors had events
  // Wake a poll() in progress from another thread.
  void wake();

  void close_all();

 private:
  friend class Conn;
  struct Listener {
    int fd;
    std::function<void(std::shared_ptr<Conn>)> accept;
  };
  void add(int fd, uint32_t events);
  void mod(int fd, uint32_t events);
  void del(int fd);

  int ep_ = -1, wake_fd_ = -1;
  std::unordered_map<int, Listener> listeners_;
  std::unordered_map<int, std::shared_ptr<Conn>> conns_;
};

// Local addresses a peer could reach this host on (IPv4 + IPv6, loopback last).
std::vector<std::string> local_addresses();
// The kernel's boot id: equal on two processes <=> same host (reference: core/group.cc:178-199).
std::string boot_id();

}  // namespace moodist
