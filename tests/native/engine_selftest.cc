// Stand-alone check of the host engine: N ranks as threads of one process over loopback TCP with an
// in-memory store. Exits 0 when all_gather / reduce_scatter / all_reduce / broadcast / barrier match.
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "core/host_group.h"
#include "core/log.h"

using namespace moodist;

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

int main(int argc, char** argv) {
  int world = argc > 1 ? atoi(argv[1]) : 2;
  size_t n = argc > 2 ? atol(argv[2]) : 100000;
  MemStore store;
  std::vector<std::thread> th;
  std::vector<int> ok(world, 0);
  for (int r = 0; r < world; ++r) {
    th.emplace_back([&, r] {
      try {
        auto g = HostGroup::create(store, "selftest", r, world);
        std::vector<float> in(n), out(n * world);
        for (size_t i = 0; i < n; ++i) in[i] = (float)(r * 1000 + (i % 997));
        g->all_gather(in.data(), out.data(), n * 4);
        bool good = true;
        for (int p = 0; p < world; ++p)
          for (size_t i = 0; i < n; i += 13) good &= out[p * n + i] == (float)(p * 1000 + (i % 997));
        std::vector<float> rin(n * world), rout(n);
        for (size_t i = 0; i < n * world; ++i) rin[i] = (float)((i % 31) + r);
        g->reduce_scatter(rin.data(), rout.data(), n, 6, 1 /*avg*/, 1.0);
        for (size_t i = 0; i < n; i += 7) {
          float e = 0;
          for (int p = 0; p < world; ++p) e += (float)(((r * n + i) % 31) + p);
          good &= std::fabs(rout[i] - e / world) < 1e-4;
        }
        std::vector<double> ar(1001);
        for (size_t i = 0; i < ar.size(); ++i) ar[i] = r + (double)i;
        g->all_reduce(ar.data(), ar.data(), ar.size(), 7 /*f64*/, 0, 1.0);
        for (size_t i = 0; i < ar.size(); ++i) good &= ar[i] == world * (double)i + world * (world - 1) / 2.0;
        std::vector<int> b(50, r == 1 % world ? 42 : 0);
        g->broadcast(b.data(), b.size() * 4, 1 % world);
        good &= b[49] == 42;
        g->barrier();
        ok[r] = good;
        g->shutdown();
      } catch (const std::exception& e) {
        fprintf(stderr, "rank %d: %s\n", r, e.what());
      }
    });
  }
  for (auto& t : th) t.join();
  int all = 1;
  for (int r = 0; r < world; ++r) all &= ok[r];
  printf("%s\n", all ? "ENGINE SELFTEST OK" : "ENGINE SELFTEST FAILED");
  return all ? 0 : 1;
}
