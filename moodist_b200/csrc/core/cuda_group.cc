#include "cuda_group.h"

#include <cuda_runtime_api.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>

#include "kernels/kernels_api.h"
#include "log.h"
#include "symm_heap.h"
#include "topology.h"
#include "wire.h"

namespace moodist {
namespace {

void rt_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) fail(std::string(what) + " failed: " + cudaGetErrorString(e));
}
#define RT_CHECK(x) rt_check((x), #x)

const char* rc_name(int rc) {
  switch (rc) {
    case MB_ERR_ARG: return "unsupported argument combination";
    case MB_ERR_ALIGN: return "misaligned pointer or pitch";
    case MB_ERR_DRIVER: return "driver entry point unavailable";
    case MB_ERR_LAUNCH: return "kernel launch failed";
    case MB_ERR_TOO_BIG: return "message larger than the staging area";
    default: return "unknown error";
  }
}

std::string status_text(uint32_t st) {
  uint32_t code = st & 0xffff, peer = st >> 16;
  const char* what = "device-side failure";
  switch (code) {
    case 0x201: what = "timed out at entry waiting for a peer to finish the previous collective"; break;
    case 0x202: what = "timed out waiting for a peer's data"; break;
    case 0x203: what = "timed out waiting for a peer's address announcement"; break;
    case 0x204: what = "timed out at exit waiting for a peer"; break;
    case 0x205: what = "timed out waiting for the sender of a point-to-point CUDA tensor (Queue item or recv)"; break;
    case 0x101: what = "GEMM producer timed out"; break;
    case 0x102: what = "GEMM MMA issuer timed out"; break;
    case 0x103: what = "GEMM epilogue timed out"; break;
    case 0x104: what = "fused all-gather GEMM timed out waiting for a shard"; break;
    case 0x105: what = "GEMM drain timed out"; break;
  }
  return strf("moodist: collective failed on the device: %s (code 0x%x, peer rank %u)", what, code, peer);
}

}  // namespace

// MOODIST_VARIANT_TABLE names a JSON file {"<world size>": {"MOODIST_...": <integer>, ...}, ...} written by
// `python -m moodist_b200.utils.tuning sweep.jsonl --table FILE` from a sweep on the machine at hand. Only this
// shape is understood: one object of objects of integers.
std::map<std::string, long> load_variant_table(const std::string& path, int world) {
  std::map<std::string, long> out;
  std::ifstream f(path);
  if (!f) {
    log_error("MOODIST_VARIANT_TABLE: cannot read %s; built-in thresholds stay", path.c_str());
    return out;
  }
  std::stringstream ss;
  ss << f.rdbuf();
  const std::string t = ss.str();
  size_t i = 0;
  auto skip = [&] { while (i < t.size() && (isspace((unsigned char)t[i]) || t[i] == ',')) ++i; };
  auto str = [&](std::string& v) {
    skip();
    if (i >= t.size() || t[i] != '"') return false;
    size_t e = t.find('"', i + 1);
    if (e == std::string::npos) return false;
    v = t.substr(i + 1, e - i - 1);
    i = e + 1;
    return true;
  };
  auto expect = [&](char ch) {
    skip();
    if (i < t.size() && t[i] == ch) {
      ++i;
      return true;
    }
    return false;
  };
  bool ok = expect('{');
  const std::string want = std::to_string(world);
  while (ok) {
    std::string key;
    if (!str(key)) break;
    ok = expect(':') && expect('{');
    while (ok) {
      std::string name;
      if (!str(name)) break;
      if (!expect(':')) {
        ok = false;
        break;
      }
      skip();
      char* end = nullptr;
      long v = strtol(t.c_str() + i, &end, 10);
      if (end == t.c_str() + i) {
        ok = false;
        break;
      }
      i = (size_t)(end - t.c_str());
      if (key == want) out[name] = v;
    }
    ok = ok && expect('}');
  }
  if (!ok) {
    log_error("MOODIST_VARIANT_TABLE: %s is not {\"world\": {\"NAME\": integer}}; built-in thresholds stay",
              path.c_str());
    out.clear();
  }
  return out;
}

namespace {

class CudaGroupImpl final : public CudaGroup {
 public:
  CudaGroupImpl(KVStore& store, const std::string& key, int rank, int world, int device)
      : key_(key), rank_(rank), world_(world), device_(device) {
    if (world > MB_MAX_RANKS) fail(strf("moodist: CUDA groups support at most %d ranks per node", MB_MAX_RANKS));
    RT_CHECK(cudaSetDevice(device));
    RT_CHECK(cudaFree(nullptr));  // make sure the primary context exists
    memset(&comm_, 0, sizeof(comm_));
    comm_.rank = rank;
    comm_.world = world;
    comm_.wait_ns = (uint64_t)env_long("MOODIST_DEVICE_TIMEOUT_MS", 30000) * 1000000ull;
    comm_.max_ctas = (int)env_long("MOODIST_MAX_CTAS", 0);
    comm_.tuning = env_long("MOODIST_AG_STAGGER", 1) ? MB_TUNE_STAGGER : 0;
    if (const char* tp = getenv("MOODIST_VARIANT_TABLE"); tp && *tp) table_ = load_variant_table(tp, world);
    stats_every_ = (int)env_long("MOODIST_STATS_SAMPLE", 64);
    nvtx_ = env_flag("MOODIST_NVTX");
    push_bytes_ = (size_t)threshold("MOODIST_AG_PUSH_BYTES", 1 << 20);
    // Pushing large shards (two pipelined halves per CTA) beat the pull on 2 GPUs from 32 MiB up (447 vs 421 GB/s)
    // but lost on 8 (456-499 vs 557-597 GB/s: seven incoming write streams per GPU plus the copy out of
    // staging), so it stays off unless asked for.
    push_large_ = threshold("MOODIST_AG_PUSH_LARGE_BYTES", -1);
    // Copy-engine variant (DMA copies between one-warp flag kernels): taken from this many bytes per rank up
    // when the group prefers kernel-less transfers, always when it is forced, and on its own from
    // MOODIST_CE_AUTO_BYTES up (-1: never on its own).
    ce_min_ = threshold("MOODIST_CE_MIN_BYTES", 1 << 20);
    // measured on 8 GPUs: the DMA all-gather reaches 612-683 GB/s from 64 MiB per rank up (pull kernel 557-597,
    // NCCL 600-664); the DMA reduce-scatter (544 GB/s) stays behind the kernel (605-637), so only the all-gather
    // switches on its own
    ce_auto_ = threshold("MOODIST_CE_AUTO_BYTES", 48 << 20);
    ce_auto_rs_ = threshold("MOODIST_CE_AUTO_RS_BYTES", -1);
    ar_compose_ = threshold("MOODIST_AR_COMPOSE_BYTES", -1);
    // smallest message (bytes) for which the NVLS variant is picked automatically; -1 = never
    nvls_ar_min_ = threshold("MOODIST_NVLS_AR_MIN_BYTES", 2 << 20);
    nvls_rs_min_ = threshold("MOODIST_NVLS_RS_MIN_BYTES", -1);
    // measured on 8 GPUs: the multimem.st all-gather wins between 32 KiB and ~2 MiB per rank, the P2P pull above
    nvls_ag_min_ = threshold("MOODIST_NVLS_AG_MIN_BYTES", 32 << 10);
    nvls_ag_max_ = threshold("MOODIST_NVLS_AG_MAX_BYTES", 3 << 20);
    ar_oneshot_ = threshold("MOODIST_AR_ONESHOT_BYTES", 2 << 20);
    RT_CHECK(cudaHostAlloc((void**)&status_host_, 64, cudaHostAllocMapped));
    memset((void*)status_host_, 0, 64);
    void* dptr = nullptr;
    RT_CHECK(cudaHostGetDevicePointer(&dptr, (void*)status_host_, 0));
    comm_.status = (uint32_t*)dptr;
    // MOODIST_FORCE_STAGING=1 gives a one-rank group its staging area too, so the fused kernels can be run
    // (and profiled) on a single GPU
    if (world > 1) check_topology(store, key, rank, world, device);
    if (world > 1 || env_flag("MOODIST_FORCE_STAGING")) {
      size_t staging = (size_t)env_long("MOODIST_STAGING_MB", 1024) << 20;
      heap_ = &SymmHeap::instance(device);
      mem_ = heap_->attach_group(store, key, rank, world, staging, true);
      attached_ = true;
      for (int r = 0; r < world; ++r) {
        comm_.peer[r] = mem_.heap_base[r];
        comm_.stage[r] = mem_.stage[r];
        comm_.flags[r] = mem_.flags[r];
      }
      comm_.staging_bytes = mem_.staging_bytes;
      comm_.mc_stage = mem_.mc_stage;
      comm_.mc_flags = mem_.mc_flags;
    }
    RT_CHECK(cudaEventCreateWithFlags(&order_, cudaEventDisableTiming));
    log_verbose("cuda group %s rank %d/%d on device %d ready (nvls=%d)", key.c_str(), rank, world, device,
                comm_.mc_stage != nullptr);
  }

  ~CudaGroupImpl() override {
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
    for (auto& [name, st] : stats_)
      for (auto& pr : st.pending) {
        cudaEventDestroy(pr.first);
        cudaEventDestroy(pr.second);
      }
    if (attached_) heap_->detach_group(key_);
    if (order_) cudaEventDestroy(order_);
    if (scratch_) cudaFree(scratch_);
    if (status_host_) cudaFreeHost((void*)status_host_);
  }

  // Every rank publishes which machine and which physical GPU it runs on; a group whose ranks cannot address
  // each other's memory (several machines, two ranks on one GPU, a pair without peer access) is refused here
  // with the reason, before any memory is exchanged.
  void check_topology(KVStore& store, const std::string& key, int rank, int world, int device) {
    char pci[32] = {0};
    if (cudaDeviceGetPCIBusId(pci, sizeof(pci), device) != cudaSuccess) pci[0] = 0;
    const NodeTopology& local = local_topology();
    store.set(key + "/topo/" + std::to_string(rank), encode(local.node_id, std::string(pci)));
    std::vector<std::string> nodes(world), pcis(world);
    for (int r = 0; r < world; ++r) {
      std::vector<uint8_t> v = store.get(key + "/topo/" + std::to_string(r));
      decode_exact(v, nodes[r], pcis[r]);
    }
    // physical index of each rank's GPU in this machine's table (ranks elsewhere: -1)
    std::vector<int> devs(world, -1);
    for (int r = 0; r < world; ++r) {
      if (nodes[r] != nodes[rank]) continue;
      std::string want = pcis[r];
      for (auto& ch : want) ch = (char)tolower((unsigned char)ch);
      bool found = false;
      for (auto& g : local.gpus) {
        // CUDA prints a 4-digit PCI domain, NVML an 8-digit one
        if (!want.empty() && g.pci_bus_id.size() >= want.size() &&
            g.pci_bus_id.compare(g.pci_bus_id.size() - want.size(), want.size(), want) == 0) {
          devs[r] = g.index;
          found = true;
        }
      }
      if (!found) {
        // no NVML table: still tell two ranks on one GPU apart by bus id
        for (int q = 0; q < r; ++q)
          if (nodes[q] == nodes[r] && pcis[q] == pcis[r] && !pcis[r].empty())
            fail(strf("moodist: ranks %d and %d both use the GPU at %s; every rank of a CUDA group needs its own GPU",
                      q, r, pcis[r].c_str()));
        devs[r] = 1000 + r;  // distinct placeholder outside the table
      }
    }
    GroupTopology g = make_group_topology(rank, nodes, devs, local);
    if (!g.kernels_usable) fail("moodist: CUDA group cannot be formed: " + g.why_not);
    numa_node_ = -1;
    for (auto& gi : local.gpus)
      if (gi.index == devs[rank]) numa_node_ = gi.numa_node;
    if (numa_node_ < 0 && pci[0]) numa_node_ = numa_node_of_pci(pci);
  }

  int rank() const override { return rank_; }
  int world() const override { return world_; }
  int device() const override { return device_; }
  int numa_node() const override { return numa_node_; }
  bool has_nvls() const override { return comm_.mc_stage != nullptr; }
  GroupOptions& options() override { return opts_; }
  const void* comm_struct() const override { return &comm_; }
  uint64_t launches() const override { return launches_; }

  // Ordering between collectives costs nothing while the caller stays on one stream: only when the
  // stream changes is an event recorded at the tail of the previous stream and waited on by the new one.
  uint32_t next_seq(CUstream_st* s) override {
    check_status();
    if (have_last_ && last_stream_ != s) {
      RT_CHECK(cudaEventRecord(order_, last_stream_));
      RT_CHECK(cudaStreamWaitEvent(s, order_, 0));
    }
    return ++seq_;
  }
  void finish_op(CUstream_st* s) override {
    last_stream_ = s;
    have_last_ = true;
    ++launches_;
  }

  void* scratch(size_t bytes) override {
    if (bytes > scratch_bytes_) {
      if (scratch_) {
        cudaDeviceSynchronize();
        cudaFree(scratch_);
      }
      scratch_bytes_ = std::max<size_t>(bytes, 1 << 20);
      RT_CHECK(cudaMalloc(&scratch_, scratch_bytes_));
    }
    return scratch_;
  }

  void check_status() override {
    uint32_t st = *status_host_;
    if (st != 0) {
      *status_host_ = 0;
      fail(status_text(st));
    }
  }

  // A threshold comes from the environment when the variable is set, else from the measured table loaded at
  // group creation (MOODIST_VARIANT_TABLE), else from the built-in value.
  long threshold(const char* name, long dflt) const {
    if (getenv(name)) return env_long(name, dflt);
    auto it = table_.find(name);
    return it == table_.end() ? dflt : it->second;
  }

  // ---- per-op counters: calls, bytes, kernel family chosen, and device time of every k-th call ----
  struct Stat {
    uint64_t calls = 0, bytes = 0, timed = 0;
    double us = 0;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> pending;
  };
  class OpScope {
   public:
    OpScope(CudaGroupImpl* g, const char* op, const char* variant, size_t bytes, CUstream_st* s) : g_(g), s_(s) {
      if (g->nvtx_) {
        // a range per collective on the host timeline of profilers that follow NVTX (MOODIST_NVTX=1)
        nvtxRangePushA((std::string("moodist ") + op + "/" + variant).c_str());
        ranged_ = true;
      }
      st_ = &g->stats_[std::string(op) + "/" + variant];
      st_->calls++;
      st_->bytes += bytes;
      if (g->stats_every_ > 0 && st_->calls % (uint64_t)g->stats_every_ == 1 && st_->pending.size() < 64) {
        if (cudaEventCreate(&a_) == cudaSuccess && cudaEventCreate(&b_) == cudaSuccess) {
          timed_ = true;
          // the ordering wait that next_seq may add belongs to the op's cost as its caller sees it
          cudaEventRecord(a_, (cudaStream_t)s);
        }
      }
    }
    ~OpScope() {
      if (ranged_) nvtxRangePop();
      if (timed_) {
        cudaEventRecord(b_, (cudaStream_t)s_);
        st_->pending.emplace_back(a_, b_);
      }
    }

   private:
    CudaGroupImpl* g_;
    Stat* st_;
    CUstream_st* s_;
    cudaEvent_t a_ = nullptr, b_ = nullptr;
    bool timed_ = false, ranged_ = false;
  };
  void drain(Stat& st, bool wait) {
    auto it = st.pending.begin();
    while (it != st.pending.end()) {
      if (wait) cudaEventSynchronize(it->second);
      float ms = 0;
      if (cudaEventQuery(it->second) == cudaSuccess && cudaEventElapsedTime(&ms, it->first, it->second) == cudaSuccess) {
        st.us += ms * 1e3;
        st.timed++;
        cudaEventDestroy(it->first);
        cudaEventDestroy(it->second);
        it = st.pending.erase(it);
      } else {
        ++it;
      }
    }
  }
  std::vector<OpStat> stats(bool wait) override {
    std::lock_guard<std::mutex> lk(mu_);
    std::vector<OpStat> out;
    for (auto& [name, st] : stats_) {
      drain(st, wait);
      out.push_back(OpStat{name, st.calls, st.bytes, st.timed, st.us});
    }
    return out;
  }
  void note_op(const char* op, const char* variant, size_t bytes) override {
    std::lock_guard<std::mutex> lk(mu_);
    Stat& st = stats_[std::string(op) + "/" + variant];
    st.calls++;
    st.bytes += bytes;
  }

  void note(const char* op, const char* variant, size_t bytes) {  // mu_ held
    Stat& st = stats_[std::string(op) + "/" + variant];
    st.calls++;
    st.bytes += bytes;
  }

  int64_t heap_off(const void* p, size_t bytes) const {
    if (!heap_ || opts_.force_kernel_less == 2) return -1;
    return heap_->offset_of(p, bytes);
  }

  // method option: 0 forces the P2P kernels, 1 the NVLS kernels; otherwise the size threshold decides
  bool want_nvls(long min_bytes, size_t bytes) const {
    if (!mb_nvls_available(&comm_) || opts_.method == 0) return false;
    if (opts_.method == 1) return true;
    return min_bytes >= 0 && bytes >= (size_t)min_bytes;
  }

  void run(int rc, const char* what) {
    if (rc != MB_OK) fail(strf("moodist: %s: %s", what, rc_name(rc)));
  }

  bool want_ce(size_t bytes, long auto_min) const {
    if (world_ == 1 || !attached_ || opts_.method == 0 || opts_.method == 1) return false;
    if (opts_.force_kernel_less == 1 || opts_.method == 2) return true;
    if (opts_.prefer_kernel_less && bytes >= (size_t)ce_min_) return true;
    return auto_min >= 0 && bytes >= (size_t)auto_min;
  }
  uint8_t* stage_half(int r, uint32_t seq) const {
    return (uint8_t*)comm_.stage[r] + (uint64_t)(seq & 1) * (comm_.staging_bytes / 2);
  }

  // All-gather with DMA copies: stage the shard, exchange "ready", pull every peer's staged shard straight into
  // place. At step i every rank reads from rank+i, so each source serves one reader at a time.
  void all_gather_ce(const uint8_t* in, uint8_t* out, size_t count, size_t esz, CUstream_st* s) {
    const size_t half = comm_.staging_bytes / 2;
    const size_t piece = std::min(count, (half / esz) & ~(size_t)63);
    cudaStream_t cs = (cudaStream_t)s;
    for (size_t done = 0; done < count; done += piece) {
      const size_t n = std::min(piece, count - done);
      uint32_t seq = next_seq(s);
      run(mb_ce_phase(&comm_, seq, 0, s), "all_gather (copy engine)");
      RT_CHECK(cudaMemcpyAsync(stage_half(rank_, seq), in + done * esz, n * esz, cudaMemcpyDeviceToDevice, cs));
      run(mb_ce_phase(&comm_, seq, 1, s), "all_gather (copy engine)");
      uint8_t* own = out + ((size_t)rank_ * count + done) * esz;
      if (own != in + done * esz)
        RT_CHECK(cudaMemcpyAsync(own, in + done * esz, n * esz, cudaMemcpyDeviceToDevice, cs));
      for (int i = 1; i < world_; ++i) {
        int p = (rank_ + i) % world_;
        RT_CHECK(cudaMemcpyAsync(out + ((size_t)p * count + done) * esz, stage_half(p, seq), n * esz,
                                 cudaMemcpyDeviceToDevice, cs));
      }
      run(mb_ce_phase(&comm_, seq, 2, s), "all_gather (copy engine)");
      finish_op(s);
      ce_copies_ += (uint64_t)world_ + 1;
    }
  }

  // Reduce-scatter with DMA copies: push this rank's slice for owner p into slot [rank] of p's staging half,
  // exchange "ready", then one local kernel reduces the world inputs (fp32 accumulate, scale, cast).
  void reduce_scatter_ce(const uint8_t* in, uint8_t* out, size_t count, int idt, int odt, int op, float premul,
                         CUstream_st* s) {
    const size_t isz = mb_dtype_size(idt), osz = mb_dtype_size(odt);
    const size_t half = comm_.staging_bytes / 2;
    const size_t piece = std::min(count, (half / (isz * (size_t)world_)) & ~(size_t)63);
    cudaStream_t cs = (cudaStream_t)s;
    for (size_t done = 0; done < count; done += piece) {
      const size_t n = std::min(piece, count - done);
      uint32_t seq = next_seq(s);
      run(mb_ce_phase(&comm_, seq, 0, s), "reduce_scatter (copy engine)");
      for (int i = 1; i < world_; ++i) {
        int p = (rank_ + i) % world_;
        RT_CHECK(cudaMemcpyAsync(stage_half(p, seq) + (size_t)rank_ * n * isz, in + ((size_t)p * count + done) * isz,
                                 n * isz, cudaMemcpyDeviceToDevice, cs));
      }
      run(mb_ce_phase(&comm_, seq, 1, s), "reduce_scatter (copy engine)");
      run(mb_reduce_local(&comm_, seq, in + ((size_t)rank_ * count + done) * isz, out + done * osz, n, idt, odt, op,
                          premul, s),
          "reduce_scatter (copy engine)");
      run(mb_ce_phase(&comm_, seq, 2, s), "reduce_scatter (copy engine)");
      finish_op(s);
      ce_copies_ += (uint64_t)world_ - 1;
    }
  }

  void all_gather(const void* in, void* out, size_t count, int idt, int odt, CUstream_st* s) override {
    std::lock_guard<std::mutex> lk(mu_);
    all_gather_locked(in, out, count, idt, odt, s);
  }
  // Which kernel family runs, and into how many pieces a call is split, depends only on values every rank
  // shares (element count, dtypes, group options, thresholds): ranks that decided differently would launch
  // kernels that wait for each other's flags in different places. Whether THIS rank's tensor lies in the
  // symmetric heap only selects a mode inside the chosen kernel, which every kernel announces to its peers.
  void all_gather_locked(const void* in, void* out, size_t count, int idt, int odt, CUstream_st* s) {
    size_t osz = mb_dtype_size(odt), isz = mb_dtype_size(idt);
    if (!osz || !isz) fail("moodist: all_gather: unsupported dtype");
    if (count == 0) return;
    if (idt == odt && want_ce(count * isz, ce_auto_)) {
      OpScope sc(this, "all_gather", "copy_engine", count * isz, s);
      all_gather_ce((const uint8_t*)in, (uint8_t*)out, count, isz, s);
      return;
    }
    if (idt == odt && world_ > 1 && want_nvls(nvls_ag_min_, count * isz) &&
        (opts_.method == 1 || nvls_ag_max_ < 0 || count * isz <= (size_t)nvls_ag_max_) &&
        (size_t)world_ * count * isz <= comm_.staging_bytes / 2) {
      OpScope sc(this, "all_gather", "nvls", count * isz, s);
      uint32_t seq = next_seq(s);
      run(mb_all_gather_nvls(&comm_, seq, in, out, count * isz, count * isz, s), "all_gather (NVLS)");
      finish_op(s);
      return;
    }
    const bool push_class = count * osz <= push_bytes_ || (push_large_ >= 0 && count * osz >= (size_t)push_large_);
    // this rank's mode inside the P2P kernel: read in place from the heap, pushed, or staged and pulled
    int64_t off = idt == odt ? heap_off(in, count * isz) : -1;
    if (off < 0 && push_class) off = -2;
    size_t half = comm_.staging_bytes / 2;
    size_t piece = count;
    if (world_ > 1 && push_class && (size_t)world_ * count * osz > half) {
      piece = (half / ((size_t)world_ * osz)) & ~(size_t)63;  // every peer's slot of a piece fits one half
    } else if (world_ > 1 && !push_class && count * osz > half) {
      piece = (half / osz) & ~(size_t)63;
    }
    OpScope sc(this, "all_gather", world_ == 1 ? "local" : (push_class ? "p2p_push" : "p2p_pull"), count * isz, s);
    for (size_t done = 0; done < count; done += piece) {
      size_t n = std::min(piece, count - done);
      uint32_t seq = next_seq(s);
      run(mb_all_gather(&comm_, seq, (const uint8_t*)in + done * isz, off < 0 ? off : off + (int64_t)(done * isz),
                        (uint8_t*)out + done * osz, n, count, idt, odt, s),
          "all_gather");
      finish_op(s);
    }
  }

  void reduce_scatter(const void* in, void* out, size_t count, int idt, int odt, int op, float premul,
                      CUstream_st* s) override {
    std::lock_guard<std::mutex> lk(mu_);
    reduce_scatter_locked(in, out, count, idt, odt, op, premul, s);
  }
  void reduce_scatter_locked(const void* in, void* out, size_t count, int idt, int odt, int op, float premul,
                             CUstream_st* s) {
    size_t osz = mb_dtype_size(odt), isz = mb_dtype_size(idt);
    if (!osz || !isz) fail("moodist: reduce_scatter: unsupported dtype");
    if (count == 0) return;
    const bool ce_types = (idt == odt && (idt == MB_F32 || idt == MB_BF16 || idt == MB_F16)) ||
                          (idt == MB_BF16 && odt == MB_F32) || (idt == MB_F32 && odt == MB_BF16);
    if (ce_types && want_ce(count * isz, ce_auto_rs_)) {
      OpScope sc(this, "reduce_scatter", "copy_engine", count * isz * world_, s);
      reduce_scatter_ce((const uint8_t*)in, (uint8_t*)out, count, idt, odt, op, premul, s);
      return;
    }
    size_t half = comm_.staging_bytes / 2;
    size_t piece = count;
    // pointer alignment is a per-rank fact: the NVLS kernel copes with any on its own (see the all-gather note)
    if (world_ > 1 && want_nvls(nvls_rs_min_, count * isz) && (size_t)world_ * count * isz <= half &&
        (idt == MB_F32 || idt == MB_BF16) && (odt == MB_F32 || odt == MB_BF16) &&
        (op == MB_SUM || op == MB_AVG || op == MB_PREMUL_SUM) && (count * isz) % 16 == 0) {
      OpScope sc(this, "reduce_scatter", "nvls", count * isz * world_, s);
      uint32_t seq = next_seq(s);
      run(mb_reduce_scatter_nvls(&comm_, seq, in, out, count, count, idt, odt, op, premul, s), "reduce_scatter (NVLS)");
      finish_op(s);
      return;
    }
    int64_t off = heap_off(in, count * isz * world_);
    if (world_ > 1 && count * isz * world_ > half) piece = (half / (isz * world_)) & ~(size_t)63;
    OpScope sc(this, "reduce_scatter", world_ == 1 ? "local" : "p2p", count * isz * world_, s);
    for (size_t done = 0; done < count; done += piece) {
      size_t n = std::min(piece, count - done);
      uint32_t seq = next_seq(s);
      run(mb_reduce_scatter(&comm_, seq, (const uint8_t*)in + done * isz, off < 0 ? -1 : off + (int64_t)(done * isz),
                            (uint8_t*)out + done * osz, n, count, idt, odt, op, premul, s),
          "reduce_scatter");
      finish_op(s);
    }
  }

  void all_reduce(const void* in, void* out, size_t count, int dt, int op, float premul, CUstream_st* s) override {
    std::lock_guard<std::mutex> lk(mu_);
    size_t sz = mb_dtype_size(dt);
    if (!sz) fail("moodist: all_reduce: unsupported dtype");
    if (count == 0) return;
    // Large buffers, opt-in (MOODIST_AR_COMPOSE_BYTES): the reduce-scatter kernel into this rank's slice of `out`,
    // then the (DMA) all-gather in place. From the 8-GPU sweep's parts (reduce-scatter 605-614 GB/s, DMA all-gather
    // 612-683 GB/s) this should give 609-638 GB/s bus bandwidth against 574-586 for the NVLS kernel; it stays
    // off until that is measured as a whole.
    if (ar_compose_ >= 0 && world_ > 1 && count * sz >= (size_t)ar_compose_ && count % (size_t)world_ == 0 &&
        ((count / world_) * sz) % 16 == 0 && (op == MB_SUM || op == MB_AVG || op == MB_PREMUL_SUM)) {
      note("all_reduce", "composed", count * sz);
      const size_t chunk = count / world_;
      uint8_t* mine = (uint8_t*)out + (size_t)rank_ * chunk * sz;
      reduce_scatter_locked(in, mine, chunk, dt, dt, op, premul, s);
      all_gather_locked(mine, out, chunk, dt, dt, s);
      return;
    }
    size_t half = comm_.staging_bytes / 2;
    size_t oneshot_max = (size_t)ar_oneshot_;
    // two-shot needs 2*world*chunk bytes of the half; keep pieces well inside
    size_t piece = count;
    if (world_ > 1 && count * sz * 2 + (size_t)world_ * 2 * 64 * sz > half)
      piece = ((half / (2 * sz)) - (size_t)world_ * 128) & ~(size_t)63;
    for (size_t done = 0; done < count; done += piece) {
      size_t n = std::min(piece, count - done);
      int variant = (n * sz <= oneshot_max) ? 0 : 1;
      bool nvls = world_ > 1 && want_nvls(nvls_ar_min_, n * sz) && (dt == MB_F32 || dt == MB_BF16) &&
                  (op == MB_SUM || op == MB_AVG || op == MB_PREMUL_SUM);
      OpScope sc(this, "all_reduce", world_ == 1 ? "local" : (nvls ? "nvls" : (variant == 0 ? "p2p_oneshot" : "p2p_twoshot")),
                 n * sz, s);
      uint32_t seq = next_seq(s);
      if (nvls)
        run(mb_all_reduce_nvls(&comm_, seq, (const uint8_t*)in + done * sz, (uint8_t*)out + done * sz, n, dt, op, premul, s),
            "all_reduce (NVLS)");
      else
        run(mb_all_reduce(&comm_, seq, (const uint8_t*)in + done * sz, (uint8_t*)out + done * sz, n, dt, op, premul,
                          variant, s),
            "all_reduce");
      finish_op(s);
    }
  }

  void broadcast(void* data, size_t bytes, int root, CUstream_st* s) override {
    std::lock_guard<std::mutex> lk(mu_);
    if (bytes == 0 || world_ == 1) return;
    size_t half = comm_.staging_bytes / 2;
    size_t piece = std::min(bytes, half & ~(size_t)1023);
    OpScope sc(this, "broadcast", "p2p_pull", bytes, s);
    for (size_t done = 0; done < bytes; done += piece) {
      size_t n = std::min(piece, bytes - done);
      uint32_t seq = next_seq(s);
      run(mb_broadcast(&comm_, seq, (uint8_t*)data + done, -1, n, root, s), "broadcast");
      finish_op(s);
    }
  }

  void all_to_all(const void* in, void* out, const uint64_t* send_off, const uint64_t* send_bytes,
                  const uint64_t* recv_off, const uint64_t* recv_bytes, CUstream_st* s) override {
    std::lock_guard<std::mutex> lk(mu_);
    mb_a2a_table_t tab;
    memset(&tab, 0, sizeof(tab));
    size_t total = 0;
    for (int r = 0; r < world_; ++r) {
      tab.send_off[r] = send_off[r];
      tab.send_bytes[r] = send_bytes[r];
      tab.recv_off[r] = recv_off[r];
      tab.recv_bytes[r] = recv_bytes[r];
      total = std::max<size_t>(total, recv_off[r] + recv_bytes[r]);
    }
    // senders write straight into the output when it lives in the symmetric heap, else into staging
    int64_t off = heap_off(out, total);
    size_t sent = 0;
    for (int r = 0; r < world_; ++r) sent += send_bytes[r];
    OpScope sc(this, "all_to_all", "p2p_push", sent, s);
    uint32_t seq = next_seq(s);
    run(mb_all_to_all(&comm_, seq, in, off, out, &tab, s), "all_to_all");
    finish_op(s);
  }

  void barrier(CUstream_st* s) override {
    std::lock_guard<std::mutex> lk(mu_);
    OpScope sc(this, "barrier", "flags", 0, s);
    uint32_t seq = next_seq(s);
    run(mb_barrier(&comm_, seq, s), "barrier");
    finish_op(s);
  }

  std::string describe() const override {
    return strf("CudaGroup(%s, rank %d/%d, device %d, nvls=%d, seq=%u)", key_.c_str(), rank_, world_, device_,
                (int)has_nvls(), seq_);
  }

 private:
  std::string key_;
  int rank_, world_, device_;
  mb_comm_t comm_;
  GroupOptions opts_;
  SymmHeap* heap_ = nullptr;
  GroupMemory mem_;
  bool attached_ = false;
  volatile uint32_t* status_host_ = nullptr;
  cudaEvent_t order_ = nullptr;
  CUstream_st* last_stream_ = nullptr;
  bool have_last_ = false;
  uint32_t seq_ = 0;
  size_t push_bytes_ = 0;
  long push_large_ = -1;
  long ce_min_ = 1 << 20, ce_auto_ = -1, ce_auto_rs_ = -1, ar_compose_ = -1;
  int numa_node_ = -1;
  uint64_t ce_copies_ = 0;
  long nvls_ar_min_ = -1, nvls_rs_min_ = -1, nvls_ag_min_ = -1, nvls_ag_max_ = -1;
  long ar_oneshot_ = 2 << 20;
  int stats_every_ = 64;
  bool nvtx_ = false;
  std::map<std::string, long> table_;
  std::map<std::string, Stat> stats_;
  uint64_t launches_ = 0;
  void* scratch_ = nullptr;
  size_t scratch_bytes_ = 0;
  std::mutex mu_;
};

}  // namespace

std::unique_ptr<CudaGroup> CudaGroup::create(KVStore& store, const std::string& key, int rank, int world,
                                             int device) {
  return std::make_unique<CudaGroupImpl>(store, key, rank, world, device);
}

}  // namespace moodist
