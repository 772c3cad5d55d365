#include "symm_heap.h"

#include <fcntl.h>
#include <poll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <cstring>
#include <map>
#include <mutex>
#include <random>
#include <thread>
#include <unordered_map>

#include "cuda_loader.h"
#include "log.h"
#include "wire.h"

namespace moodist {
namespace {

constexpr uint64_t kMagic = 0x4d42484541503031ull;  // "MBHEAP01"
constexpr size_t kFlagRegion = 2u << 20;            // flag page + status word + small tables
constexpr size_t kStatusOffset = 64 * 1024;

enum MsgKind : uint32_t { kMapChunk = 1, kMcHandle = 2 };

struct Msg {
  uint64_t magic;
  uint32_t kind;
  uint32_t reserved;
  char src_uid[64];
  char key[128];
  uint64_t offset;
  uint64_t size;
};

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

sockaddr_un abstract_addr(const std::string& name, socklen_t& len) {
  sockaddr_un a{};
  a.sun_family = AF_UNIX;
  size_t n = std::min(name.size(), sizeof(a.sun_path) - 2);
  a.sun_path[0] = 0;
  memcpy(a.sun_path + 1, name.data(), n);
  len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + n);
  return a;
}

bool send_all(int fd, const void* p, size_t n) {
  const char* b = (const char*)p;
  while (n) {
    ssize_t r = ::send(fd, b, n, MSG_NOSIGNAL);
    if (r <= 0) {
      if (r < 0 && errno == EINTR) continue;
      return false;
    }
    b += r;
    n -= r;
  }
  return true;
}
bool recv_all(int fd, void* p, size_t n) {
  char* b = (char*)p;
  while (n) {
    ssize_t r = ::recv(fd, b, n, 0);
    if (r <= 0) {
      if (r < 0 && errno == EINTR) continue;
      return false;
    }
    b += r;
    n -= r;
  }
  return true;
}

// receives exactly one Msg; the fd (if any) arrives with the first byte
bool recv_msg_with_fd(int sock, Msg& m, int& fd) {
  fd = -1;
  size_t got = 0;
  while (got < sizeof(m)) {
    iovec iov{(char*)&m + got, sizeof(m) - got};
    alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
    msghdr mh{};
    mh.msg_iov = &iov;
    mh.msg_iovlen = 1;
    mh.msg_control = ctrl;
    mh.msg_controllen = sizeof(ctrl);
    ssize_t r = recvmsg(sock, &mh, MSG_CMSG_CLOEXEC);
    if (r <= 0) {
      if (r < 0 && errno == EINTR) continue;
      return false;
    }
    for (cmsghdr* c = CMSG_FIRSTHDR(&mh); c; c = CMSG_NXTHDR(&mh, c)) {
      if (c->cmsg_level == SOL_SOCKET && c->cmsg_type == SCM_RIGHTS) {
        int f;
        memcpy(&f, CMSG_DATA(c), sizeof(int));
        if (fd >= 0) close(fd);
        fd = f;
      }
    }
    got += r;
  }
  return true;
}

struct Chunk {
  size_t offset = 0;
  size_t size = 0;
  CUmemGenericAllocationHandle handle = 0;
  bool dedicated = false;
};

struct Mirror {
  CUdeviceptr base = 0;
  std::map<size_t, Chunk> chunks;  // by offset
};

struct PeerInfo {
  std::string uid;
  std::string sock;
  std::map<size_t, bool> sent;  // chunk offsets already delivered
  int groups = 0;               // attached groups that include this peer; the entry goes with the last one
};

struct GroupState {
  Chunk chunk;
  std::vector<std::string> peer_uids;
  CUmemGenericAllocationHandle mc_handle = 0;
  CUdeviceptr mc_va = 0;
  size_t mc_size = 0;
  bool bound = false;
};

class SymmHeapImpl final : public SymmHeap {
 public:
  explicit SymmHeapImpl(int device) : device_(device) {
    const CudaApi& cu = cuda_required();
    CU_CHECK(cu.cuDeviceGet(&cudev_, device));
    CU_CHECK(cu.cuDevicePrimaryCtxRetain(&ctx_, cudev_));
    CU_CHECK(cu.cuCtxSetCurrent(ctx_));
    prop_ = CUmemAllocationProp{};
    prop_.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop_.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop_.location.id = device;
    prop_.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CU_CHECK(cu.cuMemGetAllocationGranularity(&gran_, &prop_, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    if (gran_ < (2u << 20)) gran_ = 2u << 20;
    reserved_ = (size_t)env_long("MOODIST_HEAP_VA_GB", 256) << 30;
    grow_ = (size_t)env_long("MOODIST_HEAP_GROW_MB", 1024) << 20;
    CU_CHECK(cu.cuMemAddressReserve(&base_, reserved_, gran_, 0, 0));
    std::random_device rd;
    uint64_t rnd = ((uint64_t)rd() << 32) ^ rd();
    uid_ = strf("%d-%d-%016llx", (int)getpid(), device, (unsigned long long)rnd);
    sock_name_ = "moodist-heap-" + uid_;
    start_server();
    log_verbose("symm heap: device %d base %p reserved %zu GiB uid %s", device, (void*)base_, reserved_ >> 30,
                uid_.c_str());
  }

  ~SymmHeapImpl() override {
    stop_ = true;
    if (wake_fd_ >= 0) {
      uint64_t one = 1;
      (void)!write(wake_fd_, &one, 8);
    }
    if (server_.joinable()) server_.join();
    if (listen_fd_ >= 0) close(listen_fd_);
    if (wake_fd_ >= 0) close(wake_fd_);
    // Device memory is reclaimed by the driver at process exit; explicit teardown of mappings that peers
    // may still be reading is deliberately not attempted here.
  }

  int device() const override { return device_; }
  void* base() const override { return (void*)base_; }
  size_t reserved_bytes() const override { return reserved_; }
  size_t mapped_bytes() const override { return mapped_end_; }
  size_t allocated_bytes() const override { return allocated_; }

  void* alloc(size_t bytes) override {
    if (bytes == 0) bytes = 1;
    bytes = round_up(bytes, 512);
    std::lock_guard<std::mutex> lk(mu_);
    set_ctx();
    for (int attempt = 0; attempt < 2; ++attempt) {
      // best fit
      auto best = free_.end();
      for (auto it = free_.begin(); it != free_.end(); ++it)
        if (it->second >= bytes && (best == free_.end() || it->second < best->second)) best = it;
      if (best != free_.end()) {
        size_t off = best->first, sz = best->second;
        free_.erase(best);
        if (sz > bytes) free_[off + bytes] = sz - bytes;
        live_[off] = bytes;
        allocated_ += bytes;
        return (void*)(base_ + off);
      }
      if (attempt == 0) {
        size_t want = std::max(round_up(bytes, gran_), grow_);
        if (!grow_locked(want, false, nullptr)) {
          // memory is tight: try the exact size
          if (!grow_locked(round_up(bytes, gran_), false, nullptr)) return nullptr;
        }
      }
    }
    return nullptr;
  }

  void free(void* p) override {
    if (!p) return;
    std::lock_guard<std::mutex> lk(mu_);
    size_t off = (CUdeviceptr)p - base_;
    auto it = live_.find(off);
    if (it == live_.end()) {
      log_error("symm heap: free of unknown pointer %p", p);
      return;
    }
    size_t sz = it->second;
    live_.erase(it);
    allocated_ -= sz;
    // coalesce with neighbours
    auto next = free_.lower_bound(off);
    if (next != free_.end() && next->first == off + sz) {
      sz += next->second;
      next = free_.erase(next);
    }
    if (next != free_.begin()) {
      auto prev = std::prev(next);
      if (prev->first + prev->second == off) {
        prev->second += sz;
        return;
      }
    }
    free_[off] = sz;
  }

  int64_t offset_of(const void* p, size_t bytes) const override {
    CUdeviceptr a = (CUdeviceptr)p;
    if (a < base_ || a + bytes > base_ + mapped_end_) return -1;
    return (int64_t)(a - base_);
  }

  GroupMemory attach_group(KVStore& store, const std::string& key, int rank, int world, size_t staging_bytes,
                           bool want_nvls) override {
    const CudaApi& cu = cuda_required();
    set_ctx();
    const std::string pfx = "moodist/heap/" + key + "/";
    // 1. who is in the group
    store.set(pfx + "peer/" + std::to_string(rank), encode(uid_, sock_name_));
    std::vector<std::string> uids(world), socks(world);
    for (int r = 0; r < world; ++r) decode_exact(store.get(pfx + "peer/" + std::to_string(r)), uids[r], socks[r]);

    // 2. multicast granularity decides the chunk alignment
    int mc_supported = 0;
    cu.cuDeviceGetAttribute(&mc_supported, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cudev_);
    bool nvls = want_nvls && mc_supported && world > 1 && !env_flag("MOODIST_DISABLE_NVLS");
    size_t chunk_bytes = round_up(kFlagRegion + staging_bytes, gran_);
    CUmulticastObjectProp mp{};
    size_t mc_gran = gran_;
    if (nvls) {
      mp.numDevices = (unsigned)world;
      mp.size = chunk_bytes;
      mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      if (cu.cuMulticastGetGranularity(&mc_gran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) nvls = false;
      if (nvls) {
        chunk_bytes = round_up(chunk_bytes, mc_gran);
        mp.size = chunk_bytes;
      }
    }

    GroupState gs;
    {
      std::lock_guard<std::mutex> lk(mu_);
      // 3. make every member a known peer and bring it up to date with the existing chunks
      for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        PeerInfo& pi = peers_[uids[r]];
        pi.uid = uids[r];
        pi.sock = socks[r];
        pi.groups++;
        gs.peer_uids.push_back(uids[r]);
        {
          std::lock_guard<std::mutex> lk2(mirror_mu_);
          ensure_mirror_locked(uids[r]);
        }
        for (auto& [off, ch] : chunks_)
          if (!deliver_locked(pi, ch, kAttachConnectSeconds))
            fail("symm heap: peer " + pi.uid + " did not map a chunk (is the process alive?)");
      }
      // 4. this rank's flag page + staging chunk (delivered to all known peers by grow_locked)
      if (!grow_locked(chunk_bytes, true, &gs.chunk)) fail("symm heap: cannot allocate group staging memory");
    }
    CU_CHECK(cu.cuMemsetD8(base_ + gs.chunk.offset, 0, kFlagRegion));
    CU_CHECK(cu.cuStreamSynchronize(nullptr));
    store.set(pfx + "chunk/" + std::to_string(rank), encode((uint64_t)gs.chunk.offset, (uint64_t)gs.chunk.size));
    std::vector<uint64_t> offs(world), sizes(world);
    for (int r = 0; r < world; ++r) decode_exact(store.get(pfx + "chunk/" + std::to_string(r)), offs[r], sizes[r]);
    // every rank has created its chunk and received the acks of all its peers
    store.barrier(pfx + "mapped", rank, world);

    GroupMemory gm;
    gm.staging_bytes = staging_bytes;
    gm.heap_base.resize(world);
    gm.stage.resize(world);
    gm.flags.resize(world);
    {
      std::lock_guard<std::mutex> lk(mirror_mu_);
      for (int r = 0; r < world; ++r) {
        CUdeviceptr hb = r == rank ? base_ : mirrors_.at(uids[r]).base;
        if (r != rank && !mirrors_.at(uids[r]).chunks.count(offs[r]))
          fail(strf("symm heap: rank %d's group chunk was not mapped here", r));
        gm.heap_base[r] = (void*)hb;
        gm.flags[r] = (uint32_t*)(hb + offs[r]);
        gm.stage[r] = (void*)(hb + offs[r] + kFlagRegion);
      }
    }
    gm.status = (uint32_t*)(base_ + gs.chunk.offset + kStatusOffset);

    // 5. NVLS alias. Every step is agreed on through the store so all ranks end in the same mode.
    if (nvls) {
      bool ok = true;
      if (rank == 0) {
        try {
          CU_CHECK(cu.cuMulticastCreate(&gs.mc_handle, &mp));
          int fd = -1;
          CU_CHECK(cu.cuMemExportToShareableHandle(&fd, gs.mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
          for (int r = 1; r < world; ++r) {
            Msg m{};
            m.magic = kMagic;
            m.kind = kMcHandle;
            snprintf(m.src_uid, sizeof(m.src_uid), "%s", uid_.c_str());
            snprintf(m.key, sizeof(m.key), "%s", key.c_str());
            m.size = chunk_bytes;
            if (!request(socks[r], m, fd)) ok = false;
          }
          close(fd);
        } catch (const std::exception& e) {
          log_info("NVLS setup failed on rank 0: %s", e.what());
          ok = false;
        }
        store.set_str(pfx + "mc_created", ok ? "1" : "0");
      } else {
        ok = store.get_str(pfx + "mc_created") == "1";
        if (ok) {
          int fd = take_pending_fd(key);
          if (fd < 0) {
            ok = false;
          } else {
            CUresult r = cu.cuMemImportFromShareableHandle(&gs.mc_handle, (void*)(uintptr_t)fd,
                                                           CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            close(fd);
            ok = r == CUDA_SUCCESS;
          }
        }
      }
      if (ok) ok = cu.cuMulticastAddDevice(gs.mc_handle, cudev_) == CUDA_SUCCESS;
      ok = agree(store, pfx + "mc_added", rank, world, ok);
      if (ok) {
        ok = cu.cuMulticastBindMem(gs.mc_handle, 0, gs.chunk.handle, 0, chunk_bytes, 0) == CUDA_SUCCESS;
        gs.bound = ok;
      }
      ok = agree(store, pfx + "mc_bound", rank, world, ok);
      if (ok) {
        CUresult r = cu.cuMemAddressReserve(&gs.mc_va, chunk_bytes, mc_gran, 0, 0);
        if (r == CUDA_SUCCESS) r = cu.cuMemMap(gs.mc_va, chunk_bytes, 0, gs.mc_handle, 0);
        if (r == CUDA_SUCCESS) {
          CUmemAccessDesc ad{};
          ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
          ad.location.id = device_;
          ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
          r = cu.cuMemSetAccess(gs.mc_va, chunk_bytes, &ad, 1);
        }
        ok = r == CUDA_SUCCESS;
      }
      ok = agree(store, pfx + "mc_mapped", rank, world, ok);
      if (ok) {
        gs.mc_size = chunk_bytes;
        gm.mc_flags = (uint32_t*)gs.mc_va;
        gm.mc_stage = (void*)(gs.mc_va + kFlagRegion);
        log_verbose("NVLS multicast alias ready for group %s (%zu MiB)", key.c_str(), chunk_bytes >> 20);
      } else {
        log_info("NVLS unavailable for group %s; using P2P kernels", key.c_str());
      }
    }
    {
      std::lock_guard<std::mutex> lk(mu_);
      groups_[key] = gs;
    }
    return gm;
  }

  void detach_group(const std::string& key) override {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = groups_.find(key);
    if (it == groups_.end()) return;
    const CudaApi& cu = cuda();
    GroupState& gs = it->second;
    set_ctx();
    if (gs.mc_va) {
      cu.cuMemUnmap(gs.mc_va, gs.mc_size);
      cu.cuMemAddressFree(gs.mc_va, gs.mc_size);
    }
    if (gs.bound) cu.cuMulticastUnbind(gs.mc_handle, cudev_, 0, gs.mc_size);
    if (gs.mc_handle) cu.cuMemRelease(gs.mc_handle);
    // The chunk itself stays mapped: peers may hold its mapping and the range is never reused.
    // A peer that no attached group includes any more is forgotten: later heap growth must not try to reach
    // a process that may have exited (it would sit in connect() while holding the heap's mutex).
    for (const std::string& uid : gs.peer_uids) {
      auto pit = peers_.find(uid);
      if (pit != peers_.end() && --pit->second.groups <= 0) peers_.erase(pit);
    }
    groups_.erase(it);
  }

  std::string describe() const override {
    return strf("SymmHeap(device=%d, base=%p, mapped=%zu MiB, allocated=%zu MiB, chunks=%zu, peers=%zu)", device_,
                (void*)base_, mapped_end_ >> 20, allocated_ >> 20, chunks_.size(), peers_.size());
  }

 private:
  void set_ctx() {
    CUcontext cur = nullptr;
    const CudaApi& cu = cuda();
    cu.cuCtxGetCurrent(&cur);
    if (cur != ctx_) cu.cuCtxSetCurrent(ctx_);
  }

  // all ranks publish ok/fail; result is the AND
  static bool agree(KVStore& store, const std::string& tag, int rank, int world, bool ok) {
    store.set_str(tag + "/" + std::to_string(rank), ok ? "1" : "0");
    bool all = true;
    for (int r = 0; r < world; ++r) all = (store.get_str(tag + "/" + std::to_string(r)) == "1") && all;
    return all;
  }

  // Create + map a chunk at the end of the mapped range; deliver it to every known peer.
  bool grow_locked(size_t size, bool dedicated, Chunk* out) {
    const CudaApi& cu = cuda();
    if (mapped_end_ + size > reserved_) return false;
    Chunk ch;
    ch.offset = mapped_end_;
    ch.size = size;
    ch.dedicated = dedicated;
    CUresult r = cu.cuMemCreate(&ch.handle, size, &prop_, 0);
    if (r != CUDA_SUCCESS) {
      log_verbose("symm heap: cuMemCreate(%zu) failed: %s", size, cu_error_string(r).c_str());
      return false;
    }
    r = cu.cuMemMap(base_ + ch.offset, size, 0, ch.handle, 0);
    if (r == CUDA_SUCCESS) {
      CUmemAccessDesc ad{};
      ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      ad.location.id = device_;
      ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      r = cu.cuMemSetAccess(base_ + ch.offset, size, &ad, 1);
    }
    if (r != CUDA_SUCCESS) {
      cu.cuMemRelease(ch.handle);
      log_error("symm heap: mapping a new chunk failed: %s", cu_error_string(r).c_str());
      return false;
    }
    mapped_end_ += size;
    chunks_[ch.offset] = ch;
    if (!dedicated) {
      // merge with a free block that ends exactly where this chunk starts
      size_t off = ch.offset, sz = size;
      if (!free_.empty()) {
        auto last = std::prev(free_.end());
        if (last->first + last->second == off) {
          off = last->first;
          sz += last->second;
          free_.erase(last);
        }
      }
      free_[off] = sz;
    }
    // A peer that cannot be reached any more (its process is gone) is dropped with an error in the log: the
    // chunk is mapped and usable here, and the groups that included that peer fail at their next collective
    // on their own. Growing the heap is called from the allocator, where throwing would leak the chunk.
    for (auto it = peers_.begin(); it != peers_.end();) {
      if (deliver_locked(it->second, ch, kGrowConnectSeconds)) {
        ++it;
      } else {
        log_error("symm heap: peer %s did not map a new chunk (process gone?); it is dropped from this heap",
                  it->first.c_str());
        it = peers_.erase(it);
      }
    }
    if (out) *out = ch;
    return true;
  }

  // While a group forms, a peer's server may still be starting: wait long. Later the peer either answers at
  // once or is gone.
  static constexpr double kAttachConnectSeconds = 60, kGrowConnectSeconds = 3;

  bool deliver_locked(PeerInfo& pi, const Chunk& ch, double connect_seconds) {
    if (pi.sent.count(ch.offset)) return true;
    const CudaApi& cu = cuda();
    int fd = -1;
    CU_CHECK(cu.cuMemExportToShareableHandle(&fd, ch.handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    Msg m{};
    m.magic = kMagic;
    m.kind = kMapChunk;
    snprintf(m.src_uid, sizeof(m.src_uid), "%s", uid_.c_str());
    m.offset = ch.offset;
    m.size = ch.size;
    bool ok = heap_request(pi.sock, &m, sizeof(m), fd, connect_seconds);
    close(fd);
    if (ok) pi.sent[ch.offset] = true;
    return ok;
  }

  bool request(const std::string& sock, const Msg& m, int fd) {
    return heap_request(sock, &m, sizeof(m), fd, kAttachConnectSeconds);
  }

  Mirror& ensure_mirror_locked(const std::string& uid) {
    auto it = mirrors_.find(uid);
    if (it != mirrors_.end()) return it->second;
    Mirror m;
    CU_CHECK(cuda().cuMemAddressReserve(&m.base, reserved_, gran_, 0, 0));
    return mirrors_[uid] = m;
  }

  int take_pending_fd(const std::string& key) {
    double deadline = now_seconds() + 60;
    while (now_seconds() < deadline) {
      {
        std::lock_guard<std::mutex> lk(mirror_mu_);
        auto it = pending_mc_.find(key);
        if (it != pending_mc_.end()) {
          int fd = it->second;
          pending_mc_.erase(it);
          return fd;
        }
      }
      usleep(1000);
    }
    return -1;
  }

  void start_server() {
    listen_fd_ = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC | SOCK_NONBLOCK, 0);
    if (listen_fd_ < 0) fail("symm heap: cannot create unix socket");
    socklen_t len;
    sockaddr_un a = abstract_addr(sock_name_, len);
    if (bind(listen_fd_, (sockaddr*)&a, len) != 0 || listen(listen_fd_, 64) != 0)
      fail(std::string("symm heap: cannot listen on abstract socket: ") + strerror(errno));
    wake_fd_ = eventfd(0, EFD_CLOEXEC | EFD_NONBLOCK);
    server_ = std::thread([this] { serve(); });
  }

  void serve() {
    pthread_setname_np(pthread_self(), "moodist-heap");
    cuda().cuCtxSetCurrent(ctx_);
    while (!stop_) {
      pollfd pf[2] = {{listen_fd_, POLLIN, 0}, {wake_fd_, POLLIN, 0}};
      int n = poll(pf, 2, 1000);
      if (n <= 0) continue;
      if (!(pf[0].revents & POLLIN)) continue;
      int c = accept4(listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
      if (c < 0) continue;
      timeval tv{30, 0};
      setsockopt(c, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
      Msg m{};
      int fd = -1;
      int32_t status = -1;
      if (recv_msg_with_fd(c, m, fd) && m.magic == kMagic) {
        m.src_uid[sizeof(m.src_uid) - 1] = 0;
        m.key[sizeof(m.key) - 1] = 0;
        try {
          status = handle(m, fd);
        } catch (const std::exception& e) {
          log_error("symm heap server: %s", e.what());
          status = -2;
        }
      }
      send_all(c, &status, 4);
      close(c);
    }
  }

  int32_t handle(const Msg& m, int& fd) {
    const CudaApi& cu = cuda();
    if (m.kind == kMapChunk) {
      if (fd < 0) return -3;
      CUmemGenericAllocationHandle h;
      CUresult r = cu.cuMemImportFromShareableHandle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      close(fd);
      fd = -1;
      if (r != CUDA_SUCCESS) {
        log_error("symm heap: import of a peer chunk failed: %s", cu_error_string(r).c_str());
        return -4;
      }
      std::lock_guard<std::mutex> lk(mirror_mu_);
      Mirror& mir = ensure_mirror_locked(m.src_uid);
      if (m.offset + m.size > reserved_) return -5;
      if (mir.chunks.count(m.offset)) {
        cu.cuMemRelease(h);
        return 0;
      }
      r = cu.cuMemMap(mir.base + m.offset, m.size, 0, h, 0);
      if (r == CUDA_SUCCESS) {
        CUmemAccessDesc ad{};
        ad.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        ad.location.id = device_;
        ad.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        r = cu.cuMemSetAccess(mir.base + m.offset, m.size, &ad, 1);
      }
      if (r != CUDA_SUCCESS) {
        log_error("symm heap: mapping a peer chunk failed: %s", cu_error_string(r).c_str());
        cu.cuMemRelease(h);
        return -6;
      }
      Chunk ch;
      ch.offset = m.offset;
      ch.size = m.size;
      ch.handle = h;
      mir.chunks[m.offset] = ch;
      return 0;
    }
    if (m.kind == kMcHandle) {
      if (fd < 0) return -3;
      std::lock_guard<std::mutex> lk(mirror_mu_);
      pending_mc_[m.key] = fd;
      fd = -1;
      return 0;
    }
    return -7;
  }

  int device_;
  CUdevice cudev_{};
  CUcontext ctx_{};
  CUmemAllocationProp prop_{};
  size_t gran_ = 0, reserved_ = 0, grow_ = 0;
  CUdeviceptr base_ = 0;
  std::string uid_, sock_name_;

  // mu_ guards the heap and peers_ and may be held while waiting for a peer's acknowledgement;
  // mirror_mu_ guards what the server thread touches and is never held across a request, so two
  // processes delivering chunks to each other cannot deadlock.
  mutable std::mutex mu_;
  std::mutex mirror_mu_;
  size_t mapped_end_ = 0, allocated_ = 0;
  std::map<size_t, Chunk> chunks_;
  std::map<size_t, size_t> free_;  // offset -> size
  std::map<size_t, size_t> live_;  // offset -> size
  std::unordered_map<std::string, PeerInfo> peers_;
  std::unordered_map<std::string, Mirror> mirrors_;
  std::unordered_map<std::string, int> pending_mc_;
  std::unordered_map<std::string, GroupState> groups_;

  int listen_fd_ = -1, wake_fd_ = -1;
  std::thread server_;
  std::atomic<bool> stop_{false};
};

std::mutex g_heaps_mu;
std::map<int, std::unique_ptr<SymmHeapImpl>>& heaps() {
  static auto* m = new std::map<int, std::unique_ptr<SymmHeapImpl>>();  // intentionally leaked at exit
  return *m;
}

}  // namespace

bool heap_request(const std::string& sock, const void* msg, size_t bytes, int fd, double connect_seconds) {
  int s = socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (s < 0) return false;
  socklen_t len;
  sockaddr_un a = abstract_addr(sock, len);
  double deadline = now_seconds() + connect_seconds;
  while (connect(s, (sockaddr*)&a, len) != 0) {
    if (now_seconds() > deadline) {
      close(s);
      return false;
    }
    usleep(2000);
  }
  iovec iov{const_cast<void*>(msg), bytes};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))] = {};
  msghdr mh{};
  mh.msg_iov = &iov;
  mh.msg_iovlen = 1;
  if (fd >= 0) {
    mh.msg_control = ctrl;
    mh.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&mh);
    c->cmsg_level = SOL_SOCKET;
    c->cmsg_type = SCM_RIGHTS;
    c->cmsg_len = CMSG_LEN(sizeof(int));
    memcpy(CMSG_DATA(c), &fd, sizeof(int));
  }
  ssize_t r;
  do {
    r = sendmsg(s, &mh, MSG_NOSIGNAL);
  } while (r < 0 && errno == EINTR);
  bool ok = r == (ssize_t)bytes;
  int32_t status = -1;
  ok = ok && recv_all(s, &status, 4) && status == 0;
  close(s);
  return ok;
}

SymmHeap& SymmHeap::instance(int device) {
  std::lock_guard<std::mutex> lk(g_heaps_mu);
  auto& m = heaps();
  auto it = m.find(device);
  if (it == m.end()) it = m.emplace(device, std::make_unique<SymmHeapImpl>(device)).first;
  return *it->second;
}

bool SymmHeap::exists(int device) {
  std::lock_guard<std::mutex> lk(g_heaps_mu);
  return heaps().count(device) != 0;
}

}  // namespace moodist
