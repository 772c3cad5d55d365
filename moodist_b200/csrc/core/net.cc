#include "net.h"

#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/uio.h>
#include <sys/un.h>
#include <unistd.h>

#include <cstring>
#include <fstream>

#include "log.h"

namespace moodist {
namespace {

void set_nonblock(int fd) {
  int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, fl | O_NONBLOCK);
  fcntl(fd, F_SETFD, FD_CLOEXEC);
}

void tune_tcp(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  // Socket buffer sizes are left to the kernel's auto-tuning: with explicit 4 MiB buffers a burst of a few
  // thousand 4-8 KiB one-sided reads stalled for 200 ms at a time on loopback (the persist timer after a
  // closed window), 231 ms per strided reshard against 27 ms without. MOODIST_SOCKET_BUFFER_BYTES > 0 sets them.
  static const long buf_env = env_long("MOODIST_SOCKET_BUFFER_BYTES", 0);
  if (buf_env > 0) {
    int buf = (int)buf_env;
    setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
    setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
  }
}

bool is_unix(const std::string& addr) { return addr.rfind("unix:", 0) == 0; }

socklen_t fill_unix(const std::string& addr, sockaddr_un& a) {
  std::string name = addr.substr(5);
  memset(&a, 0, sizeof(a));
  a.sun_family = AF_UNIX;
  size_t n = std::min(name.size(), sizeof(a.sun_path) - 2);
  memcpy(a.sun_path + 1, name.data(), n);  // abstract namespace: leading NUL
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
}

bool fill_inet(const std::string& addr, int port, sockaddr_storage& ss, socklen_t& len) {
  memset(&ss, 0, sizeof(ss));
  auto* a4 = reinterpret_cast<sockaddr_in*>(&ss);
  auto* a6 = reinterpret_cast<sockaddr_in6*>(&ss);
  std::string host = addr;
  unsigned scope = 0;
  auto pct = host.find('%');
  if (pct != std::string::npos) {
    scope = if_nametoindex(host.substr(pct + 1).c_str());
    host = host.substr(0, pct);
  }
  if (inet_pton(AF_INET, host.c_str(), &a4->sin_addr) == 1) {
    a4->sin_family = AF_INET;
    a4->sin_port = htons((uint16_t)port);
    len = sizeof(sockaddr_in);
    return true;
  }
  if (inet_pton(AF_INET6, host.c_str(), &a6->sin6_addr) == 1) {
    a6->sin6_family = AF_INET6;
    a6->sin6_port = htons((uint16_t)port);
    a6->sin6_scope_id = scope;
    len = sizeof(sockaddr_in6);
    return true;
  }
  // host name: blocking resolve (bootstrap only)
  addrinfo hints{}, *res = nullptr;
  hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(host.c_str(), nullptr, &hints, &res) != 0 || !res) return false;
  memcpy(&ss, res->ai_addr, res->ai_addrlen);
  len = res->ai_addrlen;
  if (ss.ss_family == AF_INET) a4->sin_port = htons((uint16_t)port);
  if (ss.ss_family == AF_INET6) a6->sin6_port = htons((uint16_t)port);
  freeaddrinfo(res);
  return true;
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// Conn
// ------------------------------------------------------------------------------------------------

Conn::~Conn() {
  if (fd_ >= 0) ::close(fd_);
  for (int f : received_fds_) ::close(f);
  for (auto& o : out_)
    if (o.pass_fd >= 0) ::close(o.pass_fd);
}

void Conn::close(const std::string& why) {
  if (closed_) return;
  closed_ = true;
  auto self = shared_from_this();
  if (fd_ >= 0) {
    poller_->del(fd_);
    poller_->conns_.erase(fd_);
    ::close(fd_);
    fd_ = -1;
  }
  if (on_connect_) {
    auto f = std::move(on_connect_);
    on_connect_ = nullptr;
    f(false);
  }
  if (on_close_) {
    auto f = on_close_;
    f(why);
  }
}

void Conn::update_interest() {
  if (fd_ < 0) return;
  bool need = !out_.empty() || connecting_;
  if (need != want_write_) {
    want_write_ = need;
    poller_->mod(fd_, EPOLLIN | EPOLLRDHUP | (need ? EPOLLOUT : 0));
  }
}

void Conn::send(Bytes data) {
  if (closed_ || data.empty()) return;
  Out o;
  o.owned = std::move(data);
  o.ptr = o.owned.data();
  o.len = o.owned.size();
  queued_ += o.len;
  out_.push_back(std::move(o));
  out_.back().ptr = out_.back().owned.data();
  if (!connecting_ && cork_ == 0) flush();
}

void Conn::send_ref(const void* p, size_t n, std::shared_ptr<void> keep, std::function<void()> sent) {
  if (closed_) return;
  if (n == 0) {
    if (out_.empty()) {
      if (sent) sent();
      return;
    }
  }
  Out o;
  o.ptr = static_cast<const uint8_t*>(p);
  o.len = n;
  o.keep = std::move(keep);
  o.sent = std::move(sent);
  queued_ += n;
  out_.push_back(std::move(o));
  if (!connecting_ && cork_ == 0) flush();
}

void Conn::send_frame(const Bytes& body) {
  if (body.size() > 0xffffff00ull) fail("net: a frame carries at most 4 GiB, not " + std::to_string(body.size()) + " bytes");
  Bytes f(8 + body.size());
  uint32_t sig = kFrameSig, n = (uint32_t)body.size();
  memcpy(f.data(), &sig, 4);
  memcpy(f.data() + 4, &n, 4);
  if (!body.empty()) memcpy(f.data() + 8, body.data(), body.size());
  send(std::move(f));
}

void Conn::send_frame_fd(const Bytes& body, int fd) {
  if (closed_) return;
  Bytes f(8 + body.size());
  uint32_t sig = kFrameSigFd, n = (uint32_t)body.size();
  memcpy(f.data(), &sig, 4);
  memcpy(f.data() + 4, &n, 4);
  if (!body.empty()) memcpy(f.data() + 8, body.data(), body.size());
  Out o;
  o.owned = std::move(f);
  o.len = o.owned.size();
  o.pass_fd = dup(fd);
  queued_ += o.len;
  out_.push_back(std::move(o));
  out_.back().ptr = out_.back().owned.data();
  if (!connecting_ && cork_ == 0) flush();
}

void Conn::flush() {
  while (!out_.empty() && !closed_) {
    Out& o = out_.front();
    if (o.off == o.len) {
      auto sent = std::move(o.sent);
      out_.pop_front();
      if (sent) sent();
      continue;
    }
    ssize_t r;
    if (o.pass_fd >= 0 && o.off == 0) {
      iovec iov{const_cast<uint8_t*>(o.ptr), o.len};
      alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
      msghdr mh{};
      mh.msg_iov = &iov;
      mh.msg_iovlen = 1;
      mh.msg_control = ctrl;
      mh.msg_controllen = sizeof(ctrl);
      cmsghdr* c = CMSG_FIRSTHDR(&mh);
      c->cmsg_level = SOL_SOCKET;
      c->cmsg_type = SCM_RIGHTS;
      c->cmsg_len = CMSG_LEN(sizeof(int));
      memcpy(CMSG_DATA(c), &o.pass_fd, sizeof(int));
      r = sendmsg(fd_, &mh, MSG_NOSIGNAL);
      if (r > 0) {
        ::close(o.pass_fd);
        o.pass_fd = -1;
      }
    } else {
      // gather up to 64 queued buffers into one writev
      iovec iov[64];
      int cnt = 0;
      for (auto it = out_.begin(); it != out_.end() && cnt < 64; ++it) {
        if (it->pass_fd >= 0 && it != out_.begin()) break;
        if (it->len == it->off) {
          if (it == out_.begin()) break;
          continue;
        }
        iov[cnt].iov_base = const_cast<uint8_t*>(it->ptr + it->off);
        iov[cnt].iov_len = it->len - it->off;
        ++cnt;
      }
      msghdr mh{};
      mh.msg_iov = iov;
      mh.msg_iovlen = cnt;
      r = sendmsg(fd_, &mh, MSG_NOSIGNAL);
    }
    if (r < 0) {
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) break;
      close(std::string("send failed: ") + strerror(errno));
      return;
    }
    size_t n = (size_t)r;
    queued_ -= n;
    while (n > 0 && !out_.empty()) {
      Out& f = out_.front();
      size_t take = std::min(n, f.len - f.off);
      f.off += take;
      n -= take;
      if (f.off == f.len) {
        auto sent = std::move(f.sent);
        out_.pop_front();
        if (sent) sent();
      } else {
        break;
      }
    }
  }
  update_interest();
}

void Conn::handle_writable() {
  if (connecting_) {
    int err = 0;
    socklen_t len = sizeof(err);
    getsockopt(fd_, SOL_SOCKET, SO_ERROR, &err, &len);
    connecting_ = false;
    if (err != 0) {
      close(std::string("connect failed: ") + strerror(err));
      return;
    }
    if (on_connect_) {
      auto f = std::move(on_connect_);
      on_connect_ = nullptr;
      f(true);
    }
  }
  flush();
}

void Conn::read_into(void* dst, size_t n, std::function<void()> done) {
  direct_dst_ = static_cast<uint8_t*>(dst);
  direct_left_ = n;
  direct_done_ = std::move(done);
}

void Conn::handle_readable() {
  auto self = shared_from_this();
  for (int rounds = 0; rounds < 64 && !closed_; ++rounds) {
    if (direct_left_ > 0 && in_len_ == 0) {
      // payload mode: straight into the destination buffer
      ssize_t r = ::recv(fd_, direct_dst_, direct_left_, 0);
      if (r < 0) {
        if (errno == EINTR) continue;
        if (errno == EAGAIN || errno == EWOULDBLOCK) return;
        close(std::string("recv failed: ") + strerror(errno));
        return;
      }
      if (r == 0) {
        close("peer closed the connection");
        return;
      }
      direct_dst_ += r;
      direct_left_ -= r;
      if (direct_left_ == 0 && direct_done_) {
        auto f = std::move(direct_done_);
        direct_done_ = nullptr;
        f();
      }
      continue;
    }
    size_t old = in_len_;
    constexpr size_t kChunk = 256 * 1024;
    if (old + kChunk > in_cap_) {
      size_t cap = std::max(in_cap_ * 2, old + kChunk);
      std::unique_ptr<uint8_t[]> grown(new uint8_t[cap]);
      if (old) memcpy(grown.get(), in_mem_.get(), old);
      in_mem_ = std::move(grown);
      in_cap_ = cap;
    }
    iovec iov{in_mem_.get() + old, kChunk};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int) * 4)] = {};
    msghdr mh{};
    mh.msg_iov = &iov;
    mh.msg_iovlen = 1;
    mh.msg_control = ctrl;
    mh.msg_controllen = sizeof(ctrl);
    ssize_t r = recvmsg(fd_, &mh, MSG_CMSG_CLOEXEC);
    if (r < 0) {
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) return;
      close(std::string("recv failed: ") + strerror(errno));
      return;
    }
    if (r == 0) {
      close("peer closed the connection");
      return;
    }
    for (cmsghdr* c = CMSG_FIRSTHDR(&mh); c; c = CMSG_NXTHDR(&mh, c)) {
      if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
        size_t nfd = (c->cmsg_len - CMSG_LEN(0)) / sizeof(int);
        for (size_t i = 0; i < nfd; ++i) {
          int f;
          memcpy(&f, CMSG_DATA(c) + i * sizeof(int), sizeof(int));
          received_fds_.push_back(f);
        }
      }
    }
    in_len_ = old + r;
    // hand the buffered bytes to the consumer
    size_t pos = 0;
    while (pos < in_len_ && !closed_) {
      if (direct_left_ > 0) {
        size_t take = std::min(direct_left_, in_len_ - pos);
        memcpy(direct_dst_, in_mem_.get() + pos, take);
        direct_dst_ += take;
        direct_left_ -= take;
        pos += take;
        if (direct_left_ == 0 && direct_done_) {
          auto f = std::move(direct_done_);
          direct_done_ = nullptr;
          f();
        }
        continue;
      }
      if (!on_data_) break;
      std::shared_ptr<DataFn> fn = on_data_;
      size_t used;
      try {
        used = (*fn)(in_mem_.get() + pos, in_len_ - pos);
      } catch (const std::exception& e) {
        // Bytes that do not decode (a stranger on this port, a damaged stream) end this connection, not the thread
        // that serves all of them.
        close(std::string("undecodable data: ") + e.what());
        return;
      }
      if (used == SIZE_MAX) {
        close("protocol error");
        return;
      }
      if (used == 0) break;
      pos += used;
    }
    if (closed_) return;
    if (pos > 0) {
      if (pos < in_len_) memmove(in_mem_.get(), in_mem_.get() + pos, in_len_ - pos);
      in_len_ -= pos;
    }
    if ((size_t)r < kChunk) return;  // drained the socket
  }
}

size_t FrameReader::operator()(const uint8_t* data, size_t n) {
  if (n < 8) return 0;
  uint32_t sig, len;
  memcpy(&sig, data, 4);
  memcpy(&len, data + 4, 4);
  if (sig != kFrameSig && sig != kFrameSigFd) return SIZE_MAX;
  if (n < 8 + (size_t)len) return 0;
  Reader r(data + 8, len);
  fn_(r, sig == kFrameSigFd);
  return 8 + (size_t)len;
}

// ------------------------------------------------------------------------------------------------
// Poller
// ------------------------------------------------------------------------------------------------

Poller::Poller() {
  ep_ = epoll_create1(EPOLL_CLOEXEC);
  wake_fd_ = eventfd(0, EFD_CLOEXEC | EFD_NONBLOCK);
  if (ep_ < 0 || wake_fd_ < 0) fail("net: cannot create epoll instance");
  add(wake_fd_, EPOLLIN);
}

Poller::~Poller() {
  close_all();
  if (wake_fd_ >= 0) ::close(wake_fd_);
  if (ep_ >= 0) ::close(ep_);
}

void Poller::close_all() {
  for (auto& [fd, l] : listeners_) {
    del(fd);
    ::close(fd);
  }
  listeners_.clear();
  auto copy = conns_;
  for (auto& [fd, c] : copy) {
    c->on_close_ = nullptr;
    c->close("poller shut down");
  }
  conns_.clear();
}

void Poller::add(int fd, uint32_t events) {
  epoll_event ev{};
  ev.events = events;
  ev.data.fd = fd;
  epoll_ctl(ep_, EPOLL_CTL_ADD, fd, &ev);
}
void Poller::mod(int fd, uint32_t events) {
  epoll_event ev{};
  ev.events = events;
  ev.data.fd = fd;
  epoll_ctl(ep_, EPOLL_CTL_MOD, fd, &ev);
}
void Poller::del(int fd) { epoll_ctl(ep_, EPOLL_CTL_DEL, fd, nullptr); }

void Poller::wake() {
  uint64_t one = 1;
  (void)!write(wake_fd_, &one, 8);
}

int Poller::listen(const std::string& addr, int port, std::function<void(std::shared_ptr<Conn>)> accept) {
  int fd;
  int bound = 0;
  if (is_unix(addr)) {
    fd = socket(AF_UNIX, SOCK_STREAM, 0);
    if (fd < 0) fail("net: socket(AF_UNIX) failed");
    sockaddr_un a;
    socklen_t len = fill_unix(addr, a);
    if (bind(fd, (sockaddr*)&a, len) != 0) {
      ::close(fd);
      fail("net: cannot bind " + addr + ": " + strerror(errno));
    }
  } else {
    sockaddr_storage ss;
    socklen_t len;
    if (!fill_inet(addr, port, ss, len)) fail("net: bad listen address " + addr);
    fd = socket(ss.ss_family, SOCK_STREAM, 0);
    if (fd < 0) return -1;
    int one = 1;
    setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    if (ss.ss_family == AF_INET6) setsockopt(fd, IPPROTO_IPV6, IPV6_V6ONLY, &one, sizeof(one));
    if (bind(fd, (sockaddr*)&ss, len) != 0) {
      ::close(fd);
      return -1;
    }
    sockaddr_storage got;
    socklen_t gl = sizeof(got);
    getsockname(fd, (sockaddr*)&got, &gl);
    bound = ntohs(got.ss_family == AF_INET ? ((sockaddr_in*)&got)->sin_port : ((sockaddr_in6*)&got)->sin6_port);
  }
  set_nonblock(fd);
  if (::listen(fd, 512) != 0) {
    ::close(fd);
    return -1;
  }
  listeners_[fd] = Listener{fd, std::move(accept)};
  add(fd, EPOLLIN);
  return bound;
}

void Poller::connect(const std::string& addr, int port, std::function<void(std::shared_ptr<Conn>)> done) {
  int fd;
  int rc;
  if (is_unix(addr)) {
    fd = socket(AF_UNIX, SOCK_STREAM, 0);
    if (fd < 0) return done(nullptr);
    set_nonblock(fd);
    sockaddr_un a;
    socklen_t len = fill_unix(addr, a);
    rc = ::connect(fd, (sockaddr*)&a, len);
  } else {
    sockaddr_storage ss;
    socklen_t len;
    if (!fill_inet(addr, port, ss, len)) return done(nullptr);
    fd = socket(ss.ss_family, SOCK_STREAM, 0);
    if (fd < 0) return done(nullptr);
    set_nonblock(fd);
    tune_tcp(fd);
    rc = ::connect(fd, (sockaddr*)&ss, len);
  }
  if (rc != 0 && errno != EINPROGRESS) {
    ::close(fd);
    return done(nullptr);
  }
  std::shared_ptr<Conn> c(new Conn(this, fd));
  c->peer_name = addr + ":" + std::to_string(port);
  conns_[fd] = c;
  c->connecting_ = true;
  c->want_write_ = true;
  std::weak_ptr<Conn> weak = c;
  c->on_connect_ = [weak, done](bool ok) {
    auto s = weak.lock();
    done(ok ? s : nullptr);
  };
  add(fd, EPOLLIN | EPOLLRDHUP | EPOLLOUT);
}

int Poller::poll(int timeout_ms) {
  epoll_event evs[64];
  int n = epoll_wait(ep_, evs, 64, timeout_ms);
  for (int i = 0; i < n; ++i) {
    int fd = evs[i].data.fd;
    if (fd == wake_fd_) {
      uint64_t v;
      (void)!read(wake_fd_, &v, 8);
      continue;
    }
    auto li = listeners_.find(fd);
    if (li != listeners_.end()) {
      for (;;) {
        int cfd = accept4(fd, nullptr, nullptr, SOCK_NONBLOCK | SOCK_CLOEXEC);
        if (cfd < 0) break;
        sockaddr_storage ss;
        socklen_t sl = sizeof(ss);
        if (getsockname(cfd, (sockaddr*)&ss, &sl) == 0 && ss.ss_family != AF_UNIX) tune_tcp(cfd);
        std::shared_ptr<Conn> c(new Conn(this, cfd));
        conns_[cfd] = c;
        add(cfd, EPOLLIN | EPOLLRDHUP);
        auto acc = li->second.accept;
        acc(c);
        li = listeners_.find(fd);
        if (li == listeners_.end()) break;
      }
      continue;
    }
    auto ci = conns_.find(fd);
    if (ci == conns_.end()) continue;
    std::shared_ptr<Conn> c = ci->second;
    if (evs[i].events & EPOLLOUT) c->handle_writable();
    if (c->open() && (evs[i].events & (EPOLLIN | EPOLLHUP | EPOLLRDHUP | EPOLLERR))) c->handle_readable();
  }
  return n > 0 ? n : 0;
}

// ------------------------------------------------------------------------------------------------
// host information
// ------------------------------------------------------------------------------------------------

std::vector<std::string> local_addresses() {
  std::vector<std::string> routable, loop;
  ifaddrs* ifa = nullptr;
  if (getifaddrs(&ifa) == 0) {
    for (ifaddrs* i = ifa; i; i = i->ifa_next) {
      if (!i->ifa_addr || !(i->ifa_flags & IFF_UP)) continue;
      char buf[INET6_ADDRSTRLEN + IF_NAMESIZE + 2];
      if (i->ifa_addr->sa_family == AF_INET) {
        auto* a = (sockaddr_in*)i->ifa_addr;
        inet_ntop(AF_INET, &a->sin_addr, buf, sizeof(buf));
        ((i->ifa_flags & IFF_LOOPBACK) ? loop : routable).push_back(buf);
      } else if (i->ifa_addr->sa_family == AF_INET6) {
        auto* a = (sockaddr_in6*)i->ifa_addr;
        if (IN6_IS_ADDR_LINKLOCAL(&a->sin6_addr)) continue;
        inet_ntop(AF_INET6, &a->sin6_addr, buf, sizeof(buf));
        ((i->ifa_flags & IFF_LOOPBACK) ? loop : routable).push_back(buf);
      }
    }
    freeifaddrs(ifa);
  }
  if (loop.empty()) loop.push_back("127.0.0.1");
  routable.insert(routable.end(), loop.begin(), loop.end());
  return routable;
}

std::string boot_id() {
  std::ifstream f("/proc/sys/kernel/random/boot_id");
  std::string s;
  if (f) std::getline(f, s);
  if (s.empty()) {
    char host[256] = {};
    gethostname(host, sizeof(host) - 1);
    s = host;
  }
  return s;
}

}  // namespace moodist
