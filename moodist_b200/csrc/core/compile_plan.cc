#include "compile_plan.h"

#include <algorithm>
#include <condition_variable>
#include <cstring>
#include <map>
#include <mutex>

#include "log.h"
#include "tcp_transport.h"

namespace moodist {
namespace {

struct Box {
  std::vector<int64_t> lo, hi;  // half-open
  bool empty() const {
    for (size_t d = 0; d < lo.size(); ++d)
      if (hi[d] <= lo[d]) return true;
    return false;
  }
};

Box to_box(const BoxSpec& s) {
  Box b;
  b.lo = s.offset;
  b.hi.resize(s.offset.size());
  for (size_t d = 0; d < s.offset.size(); ++d) b.hi[d] = s.offset[d] + s.shape[d];
  return b;
}

Box intersect(const Box& a, const Box& b) {
  Box r;
  r.lo.resize(a.lo.size());
  r.hi.resize(a.lo.size());
  for (size_t d = 0; d < a.lo.size(); ++d) {
    r.lo[d] = std::max(a.lo[d], b.lo[d]);
    r.hi[d] = std::min(a.hi[d], b.hi[d]);
  }
  return r;
}

// a minus b (b inside a), as disjoint boxes: peel one slab per side per dimension
void subtract(const Box& a, const Box& b, std::vector<Box>& out) {
  Box rest = a;
  for (size_t d = 0; d < a.lo.size(); ++d) {
    if (rest.lo[d] < b.lo[d]) {
      Box s = rest;
      s.hi[d] = b.lo[d];
      out.push_back(s);
      rest.lo[d] = b.lo[d];
    }
    if (b.hi[d] < rest.hi[d]) {
      Box s = rest;
      s.lo[d] = b.hi[d];
      out.push_back(s);
      rest.hi[d] = b.hi[d];
    }
  }
}

void check_box(const BoxSpec& b, const std::vector<int64_t>& shape, int world, const char* what) {
  if (b.rank < 0 || b.rank >= world) fail(strf("compile_op: %s names rank %d outside the group", what, b.rank));
  if (b.offset.size() != shape.size() || b.shape.size() != shape.size())
    fail(strf("compile_op: %s must have %zu dimensions", what, shape.size()));
  for (size_t d = 0; d < shape.size(); ++d) {
    if (b.offset[d] < 0 || b.shape[d] < 0 || b.offset[d] + b.shape[d] > shape[d])
      fail(strf("compile_op: %s exceeds the global shape in dimension %zu", what, d));
  }
}

// pieces that copy box `I` from an input tensor laid out as `in` to an output tensor laid out as `out`
void emit_pieces(const Box& I, const BoxSpec& in, const BoxSpec& out, size_t esz, CopyPiece proto,
                 std::vector<CopyPiece>& pieces) {
  const int nd = (int)I.lo.size();
  if (nd == 0) {
    proto.rows = 1;
    proto.row_bytes = esz;
    pieces.push_back(proto);
    return;
  }
  std::vector<int64_t> s(nd), istr(nd), ostr(nd);
  for (int d = 0; d < nd; ++d) s[d] = I.hi[d] - I.lo[d];
  int64_t a = 1, b = 1;
  for (int d = nd - 1; d >= 0; --d) {
    istr[d] = a;
    ostr[d] = b;
    a *= in.shape[d];
    b *= out.shape[d];
  }
  // trailing dimensions that span both parents completely merge into one contiguous row
  int c = nd - 1;
  while (c > 0 && s[c] == in.shape[c] && s[c] == out.shape[c]) --c;
  int64_t row_elems = 1;
  for (int d = c; d < nd; ++d) row_elems *= s[d];
  auto base = [&](const BoxSpec& t, const std::vector<int64_t>& str) {
    int64_t off = 0;
    for (int d = 0; d < nd; ++d) off += (I.lo[d] - t.offset[d]) * str[d];
    return off;
  };
  int64_t src0 = base(in, istr), dst0 = base(out, ostr);
  if (c == 0) {
    proto.rows = 1;
    proto.row_bytes = (uint64_t)row_elems * esz;
    proto.src_offset = (uint64_t)src0 * esz;
    proto.dst_offset = (uint64_t)dst0 * esz;
    proto.src_pitch = proto.dst_pitch = proto.row_bytes;
    pieces.push_back(proto);
    return;
  }
  // rows along dimension c-1, one piece per index combination of the dimensions before it
  const int rd = c - 1;
  std::vector<int64_t> idx(rd > 0 ? rd : 0, 0);
  for (;;) {
    int64_t so = src0, dof = dst0;
    for (int d = 0; d < rd; ++d) {
      so += idx[d] * istr[d];
      dof += idx[d] * ostr[d];
    }
    CopyPiece p = proto;
    p.rows = (uint64_t)s[rd];
    p.row_bytes = (uint64_t)row_elems * esz;
    p.src_offset = (uint64_t)so * esz;
    p.dst_offset = (uint64_t)dof * esz;
    p.src_pitch = (uint64_t)istr[rd] * esz;
    p.dst_pitch = (uint64_t)ostr[rd] * esz;
    pieces.push_back(p);
    int d = rd - 1;
    while (d >= 0 && ++idx[d] == s[d]) idx[d--] = 0;
    if (d < 0) break;
  }
}

}  // namespace

RedistributionPlan plan_redistribution(const std::vector<int64_t>& shape, size_t elem_size,
                                       const std::vector<BoxSpec>& all_inputs, const std::vector<BoxSpec>& all_outputs,
                                       int rank, int world) {
  if (shape.size() > 10) fail("compile_op: at most 10 dimensions are supported");
  if (elem_size == 0) fail("compile_op: unsupported dtype");
  RedistributionPlan plan;
  plan.rank = rank;
  plan.world = world;
  plan.elem_size = elem_size;
  plan.shape = shape;
  plan.inputs.resize(world);
  plan.outputs.resize(world);
  for (const BoxSpec& b : all_inputs) {
    check_box(b, shape, world, "an input");
    plan.inputs[b.rank].push_back(b);
  }
  for (const BoxSpec& b : all_outputs) {
    check_box(b, shape, world, "an output");
    plan.outputs[b.rank].push_back(b);
  }
  plan.stage_offset.resize(world);
  plan.stage_bytes.assign(world, 0);
  for (int r = 0; r < world; ++r) {
    uint64_t off = 0;
    for (const BoxSpec& b : plan.inputs[r]) {
      plan.stage_offset[r].push_back(off);
      off += ((uint64_t)b.numel() * elem_size + 255) & ~(uint64_t)255;
    }
    plan.stage_bytes[r] = off;
  }

  // Source preference: this rank's own inputs first, then the other ranks starting after this one, so
  // that replicated data is fetched locally and remote load spreads over the ranks.
  struct Src {
    int rank, index;
  };
  std::vector<Src> order;
  for (int i = 0; i < world; ++i) {
    int r = (rank + i) % world;
    for (int k = 0; k < (int)plan.inputs[r].size(); ++k) order.push_back({r, k});
  }
  // every rank plans every rank's outputs: that tells this rank who reads its inputs
  plan.readers.assign(plan.inputs[rank].size(), {});
  for (int dst = 0; dst < world; ++dst) {
    std::vector<Src> ord;
    for (int i = 0; i < world; ++i) {
      int r = (dst + i) % world;
      for (int k = 0; k < (int)plan.inputs[r].size(); ++k) ord.push_back({r, k});
    }
    for (int j = 0; j < (int)plan.outputs[dst].size(); ++j) {
      const BoxSpec& ob = plan.outputs[dst][j];
      std::vector<Box> remaining;
      if (ob.numel() > 0) remaining.push_back(to_box(ob));
      for (const Src& s : ord) {
        if (remaining.empty()) break;
        const BoxSpec& ib = plan.inputs[s.rank][s.index];
        if (ib.numel() == 0) continue;
        Box inbox = to_box(ib);
        std::vector<Box> next;
        for (const Box& R : remaining) {
          Box I = intersect(R, inbox);
          if (I.empty()) {
            next.push_back(R);
            continue;
          }
          subtract(R, I, next);
          if (dst == rank) {
            CopyPiece proto;
            proto.src_rank = s.rank;
            proto.src_input = s.index;
            proto.dst_output = j;
            emit_pieces(I, ib, ob, elem_size, proto, plan.pieces);
            if (s.rank != rank && std::find(plan.sources.begin(), plan.sources.end(), s.rank) == plan.sources.end())
              plan.sources.push_back(s.rank);
          }
          if (s.rank == rank && dst != rank) {
            auto& rd = plan.readers[s.index];
            if (std::find(rd.begin(), rd.end(), dst) == rd.end()) rd.push_back(dst);
          }
        }
        remaining.swap(next);
      }
      if (!remaining.empty()) {
        std::string at;
        for (int64_t v : remaining[0].lo) at += std::to_string(v) + ",";
        fail(strf("compile_op: output %d of rank %d has elements that no input covers (first uncovered element at [%s])", j,
                  dst, at.c_str()));
      }
    }
  }
  return plan;
}

// ------------------------------------------------------------------------------------------------
// host executor
// ------------------------------------------------------------------------------------------------
namespace {

struct Sync {
  std::mutex mu;
  std::condition_variable cv;
  bool done = false;
  std::string error;
  void finish(std::string e = {}) {
    std::lock_guard<std::mutex> lk(mu);
    done = true;
    error = std::move(e);
    cv.notify_all();
  }
};

struct RemoteInput {
  uint64_t addr;
  uint32_t rkey;
  uint64_t bytes;
};

// Shared per group: routes kOpCustom messages to the executor of the op they name.
class CustomRouter {
 public:
  using Fn = std::function<void(int src, uint32_t call, uint8_t kind, Reader& r)>;
  // One router per group, kept by the group itself: it goes when the group goes. (A process-wide table keyed by
  // the group's address would hand a stale router, whose handler was installed on a group that no longer
  // exists, to the next group that happens to be allocated at the same address.)
  static CustomRouter& of(HostGroup& g) {
    static std::mutex mu;
    std::lock_guard<std::mutex> lk(mu);
    std::shared_ptr<void>& slot = g.extension("custom-op-router");
    if (!slot) {
      auto r = std::make_shared<CustomRouter>();
      slot = r;
      CustomRouter* p = r.get();
      g.set_handler(kOpCustom, [p](int src, Reader& rd) {
        uint32_t op, call;
        uint8_t kind;
        rd(op, call, kind);
        Fn fn;
        {
          std::lock_guard<std::mutex> lk(p->mu_);
          auto it = p->ops_.find(op);
          if (it != p->ops_.end()) fn = it->second;
        }
        if (fn)
          fn(src, call, kind, rd);
        else
          p->early_[op].emplace_back(src, call, kind, Bytes(rd.p, rd.end));
      });
    }
    return *static_cast<CustomRouter*>(slot.get());
  }
  void add(HostGroup& g, uint32_t op, Fn fn) {
    {
      std::lock_guard<std::mutex> lk(mu_);
      ops_[op] = fn;
    }
    g.run_on_engine([this, op, fn] {
      auto it = early_.find(op);
      if (it == early_.end()) return;
      auto list = std::move(it->second);
      early_.erase(it);
      for (auto& [src, call, kind, body] : list) {
        Reader r(body);
        fn(src, call, kind, r);
      }
    });
  }
  void remove(uint32_t op) {
    std::lock_guard<std::mutex> lk(mu_);
    ops_.erase(op);
  }

 private:
  std::mutex mu_;
  std::map<uint32_t, Fn> ops_;
  std::map<uint32_t, std::vector<std::tuple<int, uint32_t, uint8_t, Bytes>>> early_;  // engine thread only
};

class HostRedistributionImpl final : public HostRedistribution {
 public:
  HostRedistributionImpl(HostGroup& g, std::shared_ptr<RedistributionPlan> plan, uint32_t op_id)
      : g_(g), plan_(std::move(plan)), op_(op_id) {
    CustomRouter::of(g_).add(g_, op_, [this](int src, uint32_t call, uint8_t kind, Reader& r) { on_message(src, call, kind, r); });
  }
  ~HostRedistributionImpl() override { CustomRouter::of(g_).remove(op_); }

  void run(const std::vector<const void*>& inputs, const std::vector<void*>& outputs) override {
    const RedistributionPlan& p = *plan_;
    if (inputs.size() != p.inputs[p.rank].size() || outputs.size() != p.outputs[p.rank].size())
      fail("compile_op: wrong number of input or output tensors");
    if (g_.in_error()) fail("compile_op: process group is in an error state: " + g_.error_text());
    auto sync = std::make_shared<Sync>();
    uint32_t call = ++calls_;
    g_.run_on_engine([this, call, inputs, outputs, sync] { start(call, inputs, outputs, sync); });
    std::unique_lock<std::mutex> lk(sync->mu);
    while (!sync->done) {
      sync->cv.wait_for(lk, std::chrono::milliseconds(200));
      if (!sync->done && g_.in_error()) {
        lk.unlock();
        fail("compile_op: " + g_.error_text());
      }
    }
    if (!sync->error.empty()) fail("compile_op: " + sync->error);
  }

 private:
  struct Call {
    std::vector<const void*> inputs;
    std::vector<void*> outputs;
    std::shared_ptr<Sync> sync;
    std::vector<uint32_t> keys;                       // registration of each local input
    std::map<int, std::vector<RemoteInput>> remote;   // announcements received, by source rank
    int reads_pending = 0;
    bool reads_posted = false;
    int readers_done = 0, readers_total = 0;
    bool failed = false, sources_told = false;
  };

  void start(uint32_t call, const std::vector<const void*>& inputs, const std::vector<void*>& outputs,
             std::shared_ptr<Sync> sync) {
    const RedistributionPlan& p = *plan_;
    Call& c = calls_state_[call];
    c.inputs = inputs;
    c.outputs = outputs;
    c.sync = std::move(sync);
    // register my inputs and announce them to whoever reads them
    std::vector<int> all_readers;
    for (size_t i = 0; i < inputs.size(); ++i) {
      uint64_t bytes = (uint64_t)p.inputs[p.rank][i].numel() * p.elem_size;
      c.keys.push_back(MrTable::instance().add(const_cast<void*>(inputs[i]), bytes));
      for (int r : p.readers[i])
        if (std::find(all_readers.begin(), all_readers.end(), r) == all_readers.end()) all_readers.push_back(r);
    }
    c.readers_total = (int)all_readers.size();
    for (int r : all_readers) {
      Writer w;
      w(op_, call, (uint8_t)0, (uint32_t)inputs.size());
      for (size_t i = 0; i < inputs.size(); ++i)
        w((uint64_t)(uintptr_t)inputs[i], c.keys[i], (uint64_t)p.inputs[p.rank][i].numel() * p.elem_size);
      g_.send_message(r, kOpCustom, std::move(w.out));
    }
    // local pieces need nobody
    for (const CopyPiece& pc : p.pieces) {
      if (pc.src_rank != p.rank) continue;
      const uint8_t* s = (const uint8_t*)inputs[pc.src_input] + pc.src_offset;
      uint8_t* d = (uint8_t*)outputs[pc.dst_output] + pc.dst_offset;
      for (uint64_t r = 0; r < pc.rows; ++r) memcpy(d + r * pc.dst_pitch, s + r * pc.src_pitch, pc.row_bytes);
    }
    progress(call);
  }

  void on_message(int src, uint32_t call, uint8_t kind, Reader& r) {
    Call& c = calls_state_[call];  // may arrive before the local call started: the entry waits for it
    if (kind == 0) {
      uint32_t n = r.read<uint32_t>();
      std::vector<RemoteInput> v(n);
      for (auto& ri : v) r(ri.addr, ri.rkey, ri.bytes);
      c.remote[src] = std::move(v);
    } else {
      ++c.readers_done;
    }
    if (c.sync) progress(call);
  }

  void progress(uint32_t call) {
    auto it = calls_state_.find(call);
    if (it == calls_state_.end()) return;
    Call& c = it->second;
    const RedistributionPlan& p = *plan_;
    if (!c.reads_posted) {
      for (int s : p.sources)
        if (!c.remote.count(s)) return;  // still waiting for an announcement
      c.reads_posted = true;
      for (const CopyPiece& pc : p.pieces) {
        if (pc.src_rank == p.rank) continue;
        const RemoteInput& ri = c.remote[pc.src_rank].at(pc.src_input);
        uint8_t* d = (uint8_t*)c.outputs[pc.dst_output] + pc.dst_offset;
        // a strided piece is one request: the peer streams the runs back to back, they are scattered on arrival
        ++c.reads_pending;
        g_.post_read_strided(pc.src_rank, d, pc.rows, pc.row_bytes, pc.dst_pitch, ri.rkey, ri.addr + pc.src_offset,
                             pc.src_pitch, [this, call](bool ok) {
                               auto it = calls_state_.find(call);
                               if (it == calls_state_.end()) return;
                               if (!ok) it->second.failed = true;
                               --it->second.reads_pending;
                               progress(call);
                             });
      }
    }
    if (c.reads_pending > 0) return;
    if (!c.sources_told) {
      c.sources_told = true;
      for (int s : p.sources) g_.send_message(s, kOpCustom, encode(op_, call, (uint8_t)1));
    }
    if (c.readers_done < c.readers_total) return;
    for (uint32_t k : c.keys) MrTable::instance().remove(k);
    auto sync = c.sync;
    bool failed = c.failed;
    calls_state_.erase(it);
    sync->finish(failed ? "a remote read failed" : "");
  }

  HostGroup& g_;
  std::shared_ptr<RedistributionPlan> plan_;
  uint32_t op_;
  uint32_t calls_ = 0;
  std::map<uint32_t, Call> calls_state_;  // engine thread only
};

}  // namespace

std::unique_ptr<HostRedistribution> HostRedistribution::create(HostGroup& group, std::shared_ptr<RedistributionPlan> plan,
                                                              uint32_t op_id) {
  return std::make_unique<HostRedistributionImpl>(group, std::move(plan), op_id);
}

}  // namespace moodist
