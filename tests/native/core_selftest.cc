// Stand-alone checks of the torch-free core: wire format golden bytes, the registered-memory table,
// the bootstrap ring (ranks as threads), the store mesh, and the CPU reduce loops.
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <cstddef>
#include <cmath>
#include <cstring>
#include <condition_variable>
#include <cstdio>
#include <map>
#include <mutex>
#include <optional>
#include <thread>
#include <variant>

#include "core/cpu_allocator.h"
#include "core/compile_plan.h"
#include "core/cpu_reduce.h"
#include "core/host_group.h"
#include "core/log.h"
#include "core/numa.h"
#include "core/queue.h"
#include "core/topology.h"
#include "core/setup_comms.h"
#include "core/store.h"
#include "core/symm_heap.h"
#include "core/tcp_transport.h"
#include "core/wire.h"

using namespace moodist;

static int failures = 0;
#define CHECK(cond)                                              \
  do {                                                           \
    if (!(cond)) {                                               \
      fprintf(stderr, "FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond); \
      ++failures;                                                \
    }                                                            \
  } while (0)

struct MemStore : KVStore {
  std::mutex mu;
  std::condition_variable cv;
  std::map<std::string, std::vector<uint8_t>> kv;
  void set(const std::string& k, const std::vector<uint8_t>& v) override {
    std::lock_guard<std::mutex> lk(mu);
    kv[k] = v;
    cv.notify_all();
  }
  std::vector<uint8_t> get(const std::string& k) override {
    std::unique_lock<std::mutex> lk(mu);
    cv.wait(lk, [&] { return kv.count(k) != 0; });
    return kv[k];
  }
  bool check(const std::vector<std::string>& keys) override {
    std::lock_guard<std::mutex> lk(mu);
    for (auto& k : keys)
      if (!kv.count(k)) return false;
    return true;
  }
  void wait(const std::vector<std::string>& keys) override {
    for (auto& k : keys) get(k);
  }
};

struct Sample {
  uint32_t a = 0;
  std::string s;
  std::vector<uint16_t> v;
  template <class Ar>
  void wire(Ar& ar) {
    ar(a, s, v);
  }
};

static void test_wire() {
  // scalars raw, strings / vectors with u64 lengths, bool and optional flag as one byte, variant index u64
  Bytes b = encode((uint32_t)0x01020304, std::string("ab"), std::vector<uint16_t>{1, 2}, true, std::optional<uint8_t>(7),
                   std::optional<uint8_t>(), std::variant<int32_t, std::string>(std::string("z")),
                   std::pair<uint8_t, uint8_t>(5, 6));
  CHECK(to_hex(b) ==
        "04030201"
        "0200000000000000" "6162"
        "0200000000000000" "01000200"
        "01"
        "01" "07"
        "00"
        "0100000000000000" "0100000000000000" "7a"
        "0506");
  uint32_t a;
  std::string s;
  std::vector<uint16_t> v;
  bool flag;
  std::optional<uint8_t> o1, o2;
  std::variant<int32_t, std::string> var;
  std::pair<uint8_t, uint8_t> pr;
  decode_exact(b, a, s, v, flag, o1, o2, var, pr);
  CHECK(a == 0x01020304 && s == "ab" && v.size() == 2 && v[1] == 2 && flag && o1 && *o1 == 7 && !o2);
  CHECK(var.index() == 1 && std::get<1>(var) == "z" && pr.second == 6);
  Sample in{9, "hello", {3, 4, 5}}, out;
  decode_exact(encode(in), out);
  CHECK(out.a == 9 && out.s == "hello" && out.v.size() == 3);
  std::map<std::string, int32_t> m{{"k", -1}}, m2;
  decode_exact(encode(m), m2);
  CHECK(m2["k"] == -1);
  bool threw = false;
  try {
    Bytes extra = encode((uint8_t)1, (uint8_t)2);
    uint8_t x;
    decode_exact(extra, x);
  } catch (const WireError&) {
    threw = true;
  }
  CHECK(threw);  // trailing bytes are an error
  threw = false;
  try {
    Bytes shortb = {5, 0, 0, 0, 0, 0, 0, 0, 'a'};
    std::string t;
    decode_exact(shortb, t);
  } catch (const WireError&) {
    threw = true;
  }
  CHECK(threw);  // length beyond the buffer
  CHECK(from_hex(to_hex(b)) == b);
}

// Decoding bytes nobody encoded: damaged copies of a valid message, cut copies, and noise. Every attempt either
// succeeds or throws WireError; under the address sanitizer a read past the buffer or a huge allocation driven by a
// length field would show.
static void test_wire_fuzz() {
  Bytes good = encode((uint32_t)7, std::string("hello world"), std::vector<uint16_t>{1, 2, 3, 4}, true, std::optional<uint8_t>(7),
                      std::variant<int32_t, std::string>(std::string("z")), std::map<std::string, int32_t>{{"k", -1}, {"l", 2}},
                      std::vector<std::string>{"a", "bb"});
  uint64_t state = 12345;
  auto rnd = [&] {
    state = state * 6364136223846793005ull + 1442695040888963407ull;
    return (uint32_t)(state >> 33);
  };
  int decoded = 0, refused = 0;
  for (int round = 0; round < 20000; ++round) {
    Bytes b = good;
    int mode = round % 3;
    if (mode == 0) {
      for (int k = 0; k < 1 + (int)(rnd() % 3); ++k) b[rnd() % b.size()] = (uint8_t)rnd();
    } else if (mode == 1) {
      b.resize(rnd() % (b.size() + 1));
    } else {
      b.resize(rnd() % 64);
      for (auto& x : b) x = (uint8_t)rnd();
    }
    try {
      uint32_t a;
      std::string s;
      std::vector<uint16_t> v;
      bool flag;
      std::optional<uint8_t> o;
      std::variant<int32_t, std::string> var;
      std::map<std::string, int32_t> m;
      std::vector<std::string> vs;
      decode_exact(b, a, s, v, flag, o, var, m, vs);
      ++decoded;
    } catch (const WireError&) {
      ++refused;
    }
  }
  CHECK(decoded + refused == 20000 && refused > 10000);
}

static void test_mr_table() {
  std::vector<uint8_t> buf(1000);
  uint32_t k = MrTable::instance().add(buf.data(), buf.size());
  uintptr_t base = (uintptr_t)buf.data();
  CHECK(MrTable::instance().check(k, base, 1000) != nullptr);
  CHECK(MrTable::instance().check(k, base + 999, 1) != nullptr);
  CHECK(MrTable::instance().check(k, base + 999, 2) == nullptr);   // runs past the end
  CHECK(MrTable::instance().check(k, base - 1, 1) == nullptr);     // starts before
  CHECK(MrTable::instance().check(k, base, (size_t)-1) == nullptr);  // overflow
  CHECK(MrTable::instance().check(k + 1000, base, 1) == nullptr);  // unknown key
  MrTable::instance().remove(k);
  CHECK(MrTable::instance().check(k, base, 1) == nullptr);
}

static void test_setup_comms(int world) {
  MemStore store;
  std::vector<std::thread> th;
  std::vector<int> ok(world, 0);
  for (int r = 0; r < world; ++r) {
    th.emplace_back([&, r] {
      try {
        auto sc = SetupComms::create(store, "ringtest" + std::to_string(world), r, world, 20.0);
        auto all = sc->allgather(std::string("rank") + std::to_string(r));
        bool good = (int)all.size() == world;
        for (int i = 0; i < world && good; ++i) good = all[i] == "rank" + std::to_string(i);
        auto nums = sc->allgather((uint64_t)(r * 7));
        for (int i = 0; i < world; ++i) good = good && nums[i] == (uint64_t)(i * 7);
        // routed point-to-point: everyone sends to the rank two ahead (forwarded through one hop)
        int dst = (r + 2) % world, src = (r - 2 + 2 * world) % world;
        sc->send_to(dst, std::vector<int32_t>{r, r + 1});
        auto got = sc->recv_from<std::vector<int32_t>>(src);
        good = good && got.size() == 2 && got[0] == src;
        bool threw = false;
        sc->send_to((r + 1) % world, (uint32_t)5);
        try {
          sc->recv_from<std::string>((r - 1 + world) % world);  // wrong type must not be misread
        } catch (const WireError&) {
          threw = true;
        }
        good = good && threw;
        sc->allgather((uint8_t)0);  // keep everyone alive until all messages were delivered
        ok[r] = good;
      } catch (const std::exception& e) {
        fprintf(stderr, "setup comms rank %d: %s\n", r, e.what());
      }
    });
  }
  for (auto& t : th) t.join();
  for (int r = 0; r < world; ++r) CHECK(ok[r]);
}

static void test_reduce() {
  float a[5] = {1, 2, 3, 4, 5}, b[5] = {5, 4, 3, 2, 1}, o[5];
  const void* srcs[2] = {a, b};
  cpu_reduce(o, srcs, 2, 5, kDtF32, kRedAvg, 0.5, true);
  CHECK(o[0] == 3.f && o[4] == 3.f);
  cpu_reduce(o, srcs, 2, 5, kDtF32, kRedMax, 1, false);
  CHECK(o[0] == 5.f && o[2] == 3.f);
  uint16_t x[2] = {float_to_bf16(1.5f), float_to_bf16(-2.f)}, y[2] = {float_to_bf16(0.25f), float_to_bf16(8.f)}, z[2];
  const void* s2[2] = {x, y};
  cpu_reduce(z, s2, 2, 2, kDtBF16, kRedSum, 1, false);
  CHECK(bf16_to_float(z[0]) == 1.75f && bf16_to_float(z[1]) == 6.f);
  for (float f : {0.f, 1.f, -1.f, 65504.f, 1e-5f, 0.333f}) CHECK(std::fabs(f16_to_float(float_to_f16(f)) - f) <= std::fabs(f) * 1e-3f + 1e-7f);
  int64_t i1[2] = {1LL << 40, -5}, i2[2] = {3, -7}, io[2];
  const void* s3[2] = {i1, i2};
  cpu_reduce(io, s3, 2, 2, kDtI64, kRedMin, 1, false);
  CHECK(io[0] == 3 && io[1] == -7);
}

static void test_mesh_and_alloc() {
  for (int world : {1, 2, 4, 5, 8, 33}) {
    auto mesh = store_mesh(world, 99);
    auto hops = store_first_hops(mesh, 0);
    for (int d = 0; d < world; ++d) CHECK(hops[d] >= 0);
    for (auto& adj : mesh) CHECK(adj.size() <= 4);
  }
  void* p = cpu_alloc(1000);
  CHECK(p && cpu_allocator_owns(p) && ((uintptr_t)p & 63) == 0);
  void* base;
  size_t size;
  CHECK(cpu_allocator_region(p, &base, &size) && size >= 1000);
  cpu_free(p);
  int onstack;
  CHECK(!cpu_allocator_owns(&onstack));
}

// A recorded machine instead of NVML: `n` GPUs; with `nvswitch` every GPU has 18 links that end in a switch,
// otherwise GPUs 0-1 and 2-3 are joined by direct links and the rest only by PCIe; `no_p2p` breaks one pair.
struct FakeProbe : TopologyProbe {
  int n;
  bool nvswitch;
  int broken_a = -1, broken_b = -1;
  FakeProbe(int n_, bool sw) : n(n_), nvswitch(sw) {}
  int device_count() override { return n; }
  bool pci_bus_id(int d, std::string* out) override {
    char buf[32];
    snprintf(buf, sizeof(buf), "00000000:%02X:00.0", 0x1b + d * 0x10);
    *out = buf;
    return true;
  }
  int numa_node(int d) override { return d < n / 2 ? 0 : 1; }
  bool link_up(int d, int l) override { return nvswitch ? l < 18 : (d < 4 && l < 4); }
  bool link_remote(int d, int l, std::string* pci) override {
    if (nvswitch) {
      *pci = "00000000:05:00.0";  // a switch, not in the GPU table
      return true;
    }
    (void)l;
    return pci_bus_id(d ^ 1, pci);
  }
  int p2p_ok(int a, int b) override {
    return !((a == broken_a && b == broken_b) || (a == broken_b && b == broken_a));
  }
};

static void test_topology() {
  FakeProbe sw(8, true);
  NodeTopology t = discover_topology(sw);
  CHECK(t.gpus.size() == 8 && t.nvswitch && t.all_p2p);
  CHECK(t.gpus[3].nvlinks_up == 18 && t.gpus[3].nvlinks_to_switch == 18 && t.gpus[5].numa_node == 1);
  CHECK(t.gpus[1].pci_bus_id == "00000000:2b:00.0");
  CHECK(t.link[0][7] == LinkKind::NvLink && t.link[2][2] == LinkKind::Self);
  NodeTopology back = NodeTopology::decode(t.encode());
  CHECK(back.describe() == t.describe());

  FakeProbe pcie(6, false);
  NodeTopology p = discover_topology(pcie);
  CHECK(!p.nvswitch && p.all_p2p);
  CHECK(p.link[0][1] == LinkKind::NvLink && p.link[2][3] == LinkKind::NvLink);
  CHECK(p.link[0][2] == LinkKind::Pcie && p.link[4][5] == LinkKind::Pcie);
  CHECK(p.gpus[0].nvlinks_up == 4 && p.gpus[0].nvlinks_to_switch == 0 && p.gpus[5].nvlinks_up == 0);

  FakeProbe broken(4, true);
  broken.broken_a = 1;
  broken.broken_b = 2;
  NodeTopology b = discover_topology(broken);
  CHECK(!b.all_p2p && !b.nvswitch && b.link[1][2] == LinkKind::None && b.link[0][3] == LinkKind::NvLink);

  // groups
  std::vector<std::string> one(4, t.node_id);
  GroupTopology g = make_group_topology(2, one, {0, 1, 2, 3}, t);
  CHECK(g.single_node && g.kernels_usable && g.local_ranks.size() == 4);
  g = make_group_topology(0, one, {0, 1, 1, 3}, t);
  CHECK(!g.kernels_usable && g.why_not.find("share GPU 1") != std::string::npos);
  g = make_group_topology(0, one, {0, 1, 2, 3}, b);
  CHECK(!g.kernels_usable && g.why_not.find("cannot address") != std::string::npos);
  std::vector<std::string> two = {t.node_id, t.node_id, "other-machine", "other-machine"};
  g = make_group_topology(1, two, {0, 1, -1, -1}, t);
  CHECK(!g.single_node && g.num_nodes == 2 && !g.kernels_usable && g.local_ranks.size() == 2);

  // NUMA text parsing and the (possibly trivial) layout of this host
  auto cpus = parse_cpu_list("0-3,8,10-11\n");
  CHECK(cpus.size() == 7 && cpus[4] == 8 && cpus[6] == 11);
  CHECK(parse_cpu_list("").empty() && parse_cpu_list("x").empty());
  CHECK(numa_node_count() >= 1);
  CHECK(!read_boot_id().empty());
  CHECK(numa_node_of_pci("ffff:ff:1f.7") == -1);
  CHECK(!bind_thread_to_numa_node(100000));
}

// Random N-d redistributions: the global tensor is cut into input boxes one way and output boxes another way
// (random cuts per dimension, boxes dealt to ranks at random, some inputs replicated); executing every rank's
// pieces on byte buffers must reproduce the global tensor in every output box, each element written once.
static void test_planner_random() {
  uint64_t seed = 12345;
  auto rnd = [&](uint64_t n) {
    seed = seed * 6364136223846793005ull + 1442695040888963407ull;
    return (seed >> 33) % n;
  };
  auto cuts = [&](int64_t extent) {
    std::vector<int64_t> c{0};
    int parts = 1 + (int)rnd(3);
    for (int i = 1; i < parts; ++i) c.push_back(1 + (int64_t)rnd((uint64_t)extent - 1 > 0 ? extent - 1 : 1));
    c.push_back(extent);
    std::sort(c.begin(), c.end());
    c.erase(std::unique(c.begin(), c.end()), c.end());
    return c;
  };
  for (int iter = 0; iter < 200; ++iter) {
    const int nd = 1 + (int)rnd(4), world = 1 + (int)rnd(4);
    const size_t esz = (size_t[]){1, 2, 4, 8}[rnd(4)];
    std::vector<int64_t> shape(nd);
    int64_t total = 1;
    for (auto& d : shape) {
      d = 1 + (int64_t)rnd(9);
      total *= d;
    }
    auto boxes_of = [&](bool replicate) {
      std::vector<std::vector<int64_t>> c;
      for (int d = 0; d < nd; ++d) c.push_back(cuts(shape[d]));
      std::vector<BoxSpec> out;
      std::vector<size_t> idx(nd, 0);
      while (true) {
        BoxSpec b;
        b.rank = (int)rnd(world);
        for (int d = 0; d < nd; ++d) {
          b.offset.push_back(c[d][idx[d]]);
          b.shape.push_back(c[d][idx[d] + 1] - c[d][idx[d]]);
        }
        out.push_back(b);
        if (replicate && rnd(4) == 0) {  // the same data also lives on another rank
          BoxSpec r = b;
          r.rank = (int)rnd(world);
          out.push_back(r);
        }
        int d = nd - 1;
        while (d >= 0 && ++idx[d] + 1 >= c[d].size()) idx[d--] = 0;
        if (d < 0) break;
      }
      return out;
    };
    std::vector<BoxSpec> ins = boxes_of(true), outs = boxes_of(false);
    // global tensor: element i holds bytes derived from i
    std::vector<uint8_t> global((size_t)total * esz);
    for (size_t i = 0; i < global.size(); ++i) global[i] = (uint8_t)(i * 131 + 7);
    auto strides = [&](const std::vector<int64_t>& sh) {
      std::vector<int64_t> st(sh.size(), 1);
      for (int d = (int)sh.size() - 2; d >= 0; --d) st[d] = st[d + 1] * sh[d + 1];
      return st;
    };
    auto fill_box = [&](const BoxSpec& b) {  // the box's contents as a contiguous local tensor
      std::vector<uint8_t> buf((size_t)b.numel() * esz);
      auto gst = strides(shape), lst = strides(b.shape);
      for (int64_t e = 0; e < b.numel(); ++e) {
        int64_t rem = e, g = 0;
        for (int d = 0; d < nd; ++d) {
          int64_t i = rem / lst[d];
          rem -= i * lst[d];
          g += (b.offset[d] + i) * gst[d];
        }
        memcpy(&buf[(size_t)e * esz], &global[(size_t)g * esz], esz);
      }
      return buf;
    };
    // per rank: its input tensors in plan order
    std::vector<std::vector<std::vector<uint8_t>>> in_bufs(world);
    for (auto& b : ins) in_bufs[b.rank].push_back(fill_box(b));
    for (int r = 0; r < world; ++r) {
      RedistributionPlan plan = plan_redistribution(shape, esz, ins, outs, r, world);
      std::vector<std::vector<uint8_t>> out_bufs;
      std::vector<std::vector<uint8_t>> written;
      for (auto& b : plan.outputs[r]) {
        out_bufs.emplace_back((size_t)b.numel() * esz, 0xEE);
        written.emplace_back((size_t)b.numel() * esz, 0);
      }
      for (auto& pc : plan.pieces) {
        CHECK(pc.src_rank >= 0 && pc.src_rank < world && pc.src_input < (int)in_bufs[pc.src_rank].size());
        const auto& src = in_bufs[pc.src_rank][pc.src_input];
        auto& dst = out_bufs[pc.dst_output];
        for (uint64_t row = 0; row < pc.rows; ++row) {
          uint64_t so = pc.src_offset + row * pc.src_pitch, dof = pc.dst_offset + row * pc.dst_pitch;
          CHECK(so + pc.row_bytes <= src.size() && dof + pc.row_bytes <= dst.size());
          if (so + pc.row_bytes > src.size() || dof + pc.row_bytes > dst.size()) return;
          memcpy(&dst[dof], &src[so], pc.row_bytes);
          for (uint64_t k = 0; k < pc.row_bytes; ++k) ++written[pc.dst_output][dof + k];
        }
      }
      for (size_t j = 0; j < plan.outputs[r].size(); ++j) {
        CHECK(out_bufs[j] == fill_box(plan.outputs[r][j]));
        bool once = true;
        for (uint8_t w : written[j]) once = once && w == 1;
        CHECK(once);  // every byte written exactly once, replicated inputs included
      }
    }
  }
  // an output element nobody holds is an error
  bool threw = false;
  try {
    BoxSpec in{0, {0}, {4}}, out{0, {0}, {8}};
    plan_redistribution({8}, 4, {in}, {out}, 0, 1);
  } catch (const std::exception&) {
    threw = true;
  }
  CHECK(threw);
}

// The symmetric heap's request channel against peers that are gone or refuse: a socket nobody listens on
// gives up after the connect window (heap growth uses a short one so that an exited peer cannot stall the
// allocator), and a peer that answers non-zero is a failure too.
static void test_heap_request() {
  char msg[64] = {1, 2, 3};
  double t0 = now_seconds();
  CHECK(!heap_request("moodist-selftest-no-such-socket-" + std::to_string(getpid()), msg, sizeof(msg), -1, 0.3));
  double dt = now_seconds() - t0;
  CHECK(dt >= 0.25 && dt < 3.0);
  // a live peer: answers 0 the first time, 7 the second
  std::string name = "moodist-selftest-heap-" + std::to_string(getpid());
  int ls = socket(AF_UNIX, SOCK_STREAM, 0);
  sockaddr_un a{};
  a.sun_family = AF_UNIX;
  memcpy(a.sun_path + 1, name.data(), name.size());
  socklen_t len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + name.size());
  CHECK(bind(ls, (sockaddr*)&a, len) == 0 && listen(ls, 4) == 0);
  std::thread server([&] {
    for (int32_t status : {0, 7}) {
      int c = accept(ls, nullptr, nullptr);
      char buf[64];
      size_t got = 0;
      while (got < sizeof(buf)) {
        ssize_t r = recv(c, buf + got, sizeof(buf) - got, 0);
        if (r <= 0) break;
        got += (size_t)r;
      }
      (void)!write(c, &status, 4);
      close(c);
    }
  });
  CHECK(heap_request(name, msg, sizeof(msg), -1, 1.0));
  CHECK(!heap_request(name, msg, sizeof(msg), -1, 1.0));
  server.join();
  close(ls);
}

// The host engine with its ranks as threads of this process: every collective against what the ranks can work out
// themselves, receives posted before the sends of a ring, and a queue fed by every rank. (Run under the thread
// sanitizer this is where the engine thread, the callers and the completion flags meet.)
static void test_host_group(int world) {
  MemStore store;
  std::vector<std::thread> ranks;
  for (int r = 0; r < world; ++r) {
    ranks.emplace_back([&, r] {
      try {
        auto g = HostGroup::create(store, "selftest-host-group-" + std::to_string(world), r, world);
        auto queues = QueueManager::create(*g);
        // all_reduce: divisible, small with a remainder (padded round), large with a remainder (in place + tail)
        for (size_t n : {(size_t)world * 64, (size_t)1000 + 1, (size_t)(300 << 10) + (size_t)world - 1}) {
          std::vector<float> x(n);
          for (size_t i = 0; i < n; ++i) x[i] = (float)((i % 13) + r);
          g->all_reduce(x.data(), x.data(), n, kDtF32, kRedSum, 1.0);
          bool ok = true;
          for (size_t i = 0; i < n; ++i) ok = ok && x[i] == (float)(world * (i % 13) + world * (world - 1) / 2);
          CHECK(ok);
        }
        // all_gather / reduce_scatter (average) / broadcast
        std::vector<int32_t> mine(257, r), all((size_t)257 * world, -1);
        g->all_gather(mine.data(), all.data(), mine.size() * 4);
        for (int p = 0; p < world; ++p) CHECK(all[(size_t)p * 257] == p && all[(size_t)p * 257 + 256] == p);
        std::vector<double> in((size_t)world * 5), out(5);
        for (size_t i = 0; i < in.size(); ++i) in[i] = (double)(r + 1) * (double)(i / 5 + 1);
        g->reduce_scatter(in.data(), out.data(), 5, kDtF64, kRedAvg, 1.0);
        CHECK(std::fabs(out[0] - (double)(r + 1) * (world + 1) / 2.0) < 1e-9);
        std::vector<uint8_t> b(3000, (uint8_t)r);
        g->broadcast(b.data(), b.size(), world - 1);
        CHECK(b[0] == world - 1 && b[2999] == world - 1);
        // uneven all_to_all: rank s sends (s + d + 1) bytes to rank d
        std::vector<uint64_t> so(world), sb(world), ro(world), rb(world);
        uint64_t soff = 0, roff = 0;
        for (int d = 0; d < world; ++d) {
          so[d] = soff, sb[d] = (uint64_t)(r + d + 1), soff += sb[d];
          ro[d] = roff, rb[d] = (uint64_t)(d + r + 1), roff += rb[d];
        }
        std::vector<uint8_t> sendbuf(soff), recvbuf(roff, 0xee);
        for (int d = 0; d < world; ++d) std::fill(sendbuf.begin() + so[d], sendbuf.begin() + so[d] + sb[d], (uint8_t)(16 * r + d));
        g->all_to_all(sendbuf.data(), recvbuf.data(), so.data(), sb.data(), ro.data(), rb.data());
        for (int s2 = 0; s2 < world; ++s2) CHECK(recvbuf[ro[s2]] == (uint8_t)(16 * s2 + r) && recvbuf[ro[s2] + rb[s2] - 1] == (uint8_t)(16 * s2 + r));
        // a ring whose receives are posted first
        if (world > 1) {
          int nxt = (r + 1) % world, prv = (r + world - 1) % world;
          std::vector<int64_t> got(100, -1), give(100, r);
          auto posted = g->recv_post(got.data(), got.size() * 8, prv, 7, nullptr);
          g->send(give.data(), give.size() * 8, nxt, 7);
          g->recv_wait(posted);
          CHECK(g->recv_done(posted) && got[0] == prv && got[99] == prv);
          // the same with payloads that are not copied into a message but fetched by the receiver, the send
          // posted first this time
          std::vector<int64_t> big_got(100000, -1), big_give(100000, r + 1000);
          auto sent = g->send_post(big_give.data(), big_give.size() * 8, nxt, 8, nullptr);
          g->recv(big_got.data(), big_got.size() * 8, prv, 8);
          g->send_wait(sent);
          CHECK(g->send_done(sent) && big_got[0] == prv + 1000 && big_got[99999] == prv + 1000);
        }
        // everybody puts into a queue that lives on rank 0
        auto q = queues->make_queue({0}, false, std::string("selftest"));
        int64_t item[4] = {r, r, r, r};
        q->put(item, sizeof(item), 4, {4}, 0, nullptr)->wait();
        if (r == 0) {
          int64_t sum = 0;
          for (int i = 0; i < world; ++i) {
            auto it = q->get(true, 30.0, nullptr);
            CHECK(it.has_value() && it->data.size() == sizeof(item));
            if (it) {
              int64_t v;
              memcpy(&v, it->data.data(), 8);
              sum += v;
            }
          }
          CHECK(sum == (int64_t)world * (world - 1) / 2);
        }
        g->barrier();
        q.reset();
        queues.reset();
        g->shutdown();
      } catch (const std::exception& e) {
        fprintf(stderr, "host group rank %d of %d: %s\n", r, world, e.what());
        ++failures;
      }
    });
  }
  for (auto& t : ranks) t.join();
}

int main() {
  test_host_group(1);
  test_host_group(2);
  test_host_group(4);
  test_heap_request();
  test_wire();
  test_wire_fuzz();
  test_planner_random();
  test_topology();
  test_mr_table();
  test_reduce();
  test_mesh_and_alloc();
  test_setup_comms(1);
  test_setup_comms(2);
  test_setup_comms(5);
  printf("%s\n", failures ? "CORE SELFTEST FAILED" : "CORE SELFTEST OK");
  return failures ? 1 : 0;
}
