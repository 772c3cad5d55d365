// sm_100a collective kernels over NVLink peer memory (plain P2P loads/stores; the NVLS multimem
// variants live in collectives_nvls.cu). One launch per collective: rendezvous, data movement, the
// reduction with fp32 accumulation, the premul/avg scale and any dtype cast all happen in the kernel.
//
// Reference counterparts: allgather_local (core/allgather.cc:381-390, 556-566), reduce_scatter_local
// (core/reduce_scatter.cc:180-191, 344-352), alltoall (core/alltoall.cc:30-67), the all_reduce =
// reduce_scatter + all_gather composition (core/processgroup.cc:1674-1722), and the pull-chain
// broadcast (core/processgroup.cc:1728-1910). Differences by design: peers are reached through one
// symmetric heap mapping instead of per-tensor IPC handles; tensors outside the heap go through a
// double-buffered staging area so no exit barrier is needed; waits are bounded; AVG/PREMUL_SUM are
// folded into the reduce loop (the reference runs a separate torch mul_, processgroup.cc:1664-1667);
// bf16 accumulates in fp32 (the reference accumulates in bf16, core/kernels.cc:472-481).
#include <cuda_runtime.h>

#include "coll.cuh"

namespace mb {
namespace coll {

constexpr int kThreads = 512;

struct Launch {
  int grid;
};

// dflt: CTA cap when the group sets none. Measured on 8 B200s: pulls (all-gather, all-to-all) peak with 64
// CTAs and degrade beyond, pushes (reduce-scatter) keep gaining up to 128.
static inline int pick_grid(const mb_comm_t* c, size_t bytes, int dflt = 64) {
  int maxc = c->max_ctas > 0 ? c->max_ctas : dflt;
  if (maxc > kMaxCtas) maxc = kMaxCtas;
  size_t g = (bytes + 32767) / 32768;
  if (g < 1) g = 1;
  if (g > (size_t)maxc) g = maxc;
  return (int)g;
}

// lane 0 waits for peer p's announcement, result broadcast to the warp
// `direct` tells how peer p takes part in this op: 1 = its tensor lives in its symmetric heap at `off`
// and is read in place, 0 = it goes through the staging areas. Each rank decides for itself, so a
// consumer always follows what the producer announced.
__device__ __forceinline__ bool wait_announce_warp(const mb_comm_t& c, uint32_t seq, int p, uint64_t& off,
                                                   uint32_t& direct) {
  uint32_t lo = 0, hi = 0, ok = 1, aux = 0;
  if ((threadIdx.x & 31) == 0) {
    uint64_t o;
    ok = wait_announce(c, seq, p, o, aux);
    lo = (uint32_t)o;
    hi = (uint32_t)(o >> 32);
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  lo = __shfl_sync(0xffffffffu, lo, 0);
  hi = __shfl_sync(0xffffffffu, hi, 0);
  direct = __shfl_sync(0xffffffffu, aux, 0);
  off = (uint64_t)lo | ((uint64_t)hi << 32);
  return ok != 0;
}

// ---------------------------------------------------------------------------------------------
// barrier
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(32, 1) barrier_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq) {
  int t = threadIdx.x;
  if (t < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[t] + F_DONE + c.rank, seq);
    if (!wait_geq_sys(c.flags[c.rank] + F_DONE + t, seq, c.wait_ns)) fail(c, kTimeoutExit, t);
  }
}

// ---------------------------------------------------------------------------------------------
// all-gather
// ---------------------------------------------------------------------------------------------
// kCast: 0 bytes (same dtype), else converts InT -> OutT while staging.
template <typename InT, typename OutT, bool kCast>
__global__ void MB_COLL_BOUNDS
    all_gather_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq, const void* in, int64_t in_heap_off,
                      void* out, size_t count, size_t out_stride) {
  // How this rank offers its shard (in_heap_off): >= 0 in place from its heap (mode 1), -1 staged locally and
  // pulled by the peers (mode 0), -2 pushed into every peer's staging slot (mode 2: one NVLink write latency
  // instead of an announce + read round trip, at the price of a local copy on the receiver; for small shards).
  const int b = blockIdx.x, G = gridDim.x;
  const uint32_t mode = in_heap_off >= 0 ? 1u : (in_heap_off == -2 ? 2u : 0u);
  entry_wait(c, seq);
  size_t begin, len;
  slice_of(count, G, b, begin, len);
  OutT* o = reinterpret_cast<OutT*>(out);
  const InT* src_local = reinterpret_cast<const InT*>(in);
  const size_t h0 = first_half<OutT>(len);
  if (b == 0) announce(c, seq, mode == 1 ? (uint64_t)in_heap_off : 0, mode);
  if (mode == 0) {
    OutT* st = reinterpret_cast<OutT*>(stage_ptr(c, c.rank, seq));
    if constexpr (kCast) {
      cta_cast_copy<InT, OutT>(st + begin, src_local + begin, len, 1.f, false);
    } else {
      cta_copy(st + begin, src_local + begin, len * sizeof(OutT));
    }
    signal_ready(c, seq, b, 0, -1);
  } else if (mode == 2) {
    // big slices go out in two halves, each with its own READY bank, so that the receivers copy the first
    // half out of staging while the second is still crossing NVLink
    for (int h = 0; h < 2; ++h) {
      const size_t hb = h ? begin + h0 : begin, hl = h ? len - h0 : h0;
      if (h && hl == 0) break;
      for (int i = 1; i < c.world; ++i) {
        int p = (c.rank + i) % c.world;
        OutT* st = reinterpret_cast<OutT*>(stage_ptr(c, p, seq)) + (size_t)c.rank * count;
        if constexpr (kCast) {
          cta_cast_copy<InT, OutT>(st + hb, src_local + hb, hl, 1.f, false);
        } else {
          cta_copy(st + hb, src_local + hb, hl * sizeof(OutT));
        }
      }
      signal_ready(c, seq, b, h, -1);
    }
  }
  // own shard straight into place
  if constexpr (kCast) {
    cta_cast_copy<InT, OutT>(o + (size_t)c.rank * out_stride + begin, src_local + begin, len, 1.f, false);
  } else {
    if ((const void*)(o + (size_t)c.rank * out_stride) != in)
      cta_copy(o + (size_t)c.rank * out_stride + begin, src_local + begin, len * sizeof(OutT));
  }
  const PeerInfo pi = wait_peers_warp(c, seq, b, 0);
  const int start = (c.tuning & MB_TUNE_STAGGER) ? b : 0;  // staggered: CTAs read different peers at any moment
  for (int i = 0; i < c.world - 1; ++i) {
    int p = (c.rank - 1 - (start + i) % (c.world - 1) + 2 * c.world) % c.world;  // pushes arrive from rank-1 first
    const bool ok = __shfl_sync(0xffffffffu, pi.ok, p) != 0;
    const uint32_t pmode = __shfl_sync(0xffffffffu, pi.mode, p);
    const uint64_t off = (uint64_t)__shfl_sync(0xffffffffu, pi.lo, p) | ((uint64_t)__shfl_sync(0xffffffffu, pi.hi, p) << 32);
    const OutT* src;
    if (pmode == 0) {
      src = reinterpret_cast<const OutT*>(stage_ptr(c, p, seq));
    } else if (pmode == 2) {
      src = reinterpret_cast<const OutT*>(stage_ptr(c, c.rank, seq)) + (size_t)p * count;
    } else {
      src = reinterpret_cast<const OutT*>(reinterpret_cast<const uint8_t*>(c.peer[p]) + off);
    }
    // a pushed slice is complete up to h0 so far; pulled ones (modes 0, 1) are read whole
    const size_t n = pmode == 2 ? h0 : len;
    if (ok) cta_copy(o + (size_t)p * out_stride + begin, src + begin, n * sizeof(OutT));
  }
  if (h0 < len) {
    const uint32_t ok2 = wait_bank_warp(c, seq, b, 1, pi, 2u);
    for (int i = 0; i < c.world - 1; ++i) {
      int p = (c.rank - 1 - (start + i) % (c.world - 1) + 2 * c.world) % c.world;
      const bool ok = __shfl_sync(0xffffffffu, ok2, p) != 0;
      const uint32_t pmode = __shfl_sync(0xffffffffu, pi.mode, p);
      if (pmode != 2 || !ok) continue;
      const OutT* src = reinterpret_cast<const OutT*>(stage_ptr(c, c.rank, seq)) + (size_t)p * count;
      cta_copy(o + (size_t)p * out_stride + begin + h0, src + begin + h0, (len - h0) * sizeof(OutT));
    }
  }
  exit_done(c, seq, mode == 1);
}

// ---------------------------------------------------------------------------------------------
// reduce-scatter
// ---------------------------------------------------------------------------------------------
template <typename InT, typename OutT, int kOp>
__global__ void MB_COLL_BOUNDS
    reduce_scatter_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq, const void* in, int64_t in_heap_off,
                          void* out, size_t count, size_t in_stride, float scale, int use_scale) {
  const int b = blockIdx.x, G = gridDim.x;
  const bool direct = in_heap_off >= 0;
  entry_wait(c, seq);
  size_t begin, len;
  slice_of(count, G, b, begin, len);
  const InT* x = reinterpret_cast<const InT*>(in);
  const InT* srcs[MB_MAX_RANKS];
  srcs[0] = x + (size_t)c.rank * in_stride + begin;
  const size_t h0 = first_half<InT>(len);
  if (b == 0) announce(c, seq, direct ? (uint64_t)in_heap_off : 0, direct ? 1u : 0u);
  if (!direct) {
    // push this rank's contribution for every other owner into that owner's staging slot [rank];
    // one fence + flag round for all of them (the owners need every source before they can reduce anyway)
    // two halves, two READY banks: the owners reduce the first half while the second is still arriving
    for (int h = 0; h < 2; ++h) {
      const size_t hb = h ? begin + h0 : begin, hl = h ? len - h0 : h0;
      if (h && hl == 0) break;
      for (int i = 1; i < c.world; ++i) {
        int p = (c.rank + i) % c.world;
        InT* dst = reinterpret_cast<InT*>(stage_ptr(c, p, seq)) + (size_t)c.rank * count + hb;
        cta_copy(dst, x + (size_t)p * in_stride + hb, hl * sizeof(InT));
      }
      signal_ready(c, seq, b, h, -1);
    }
  }
  const PeerInfo pi = wait_peers_warp(c, seq, b, 0);
  const bool ok = all_peers_ok(pi);
  for (int i = 1; i < c.world; ++i) {
    int p = (c.rank + i) % c.world;
    const uint32_t pdirect = __shfl_sync(0xffffffffu, pi.mode, p);
    const uint64_t off = (uint64_t)__shfl_sync(0xffffffffu, pi.lo, p) | ((uint64_t)__shfl_sync(0xffffffffu, pi.hi, p) << 32);
    if (pdirect != 1u) {
      srcs[i] = reinterpret_cast<const InT*>(stage_ptr(c, c.rank, seq)) + (size_t)p * count + begin;
    } else {
      srcs[i] = reinterpret_cast<const InT*>(reinterpret_cast<const uint8_t*>(c.peer[p]) + off) +
                (size_t)c.rank * in_stride + begin;
    }
  }
  // Peers that push (every rank that is not read in place) have delivered [0, h0) of the slice so far.
  const bool any_pushed = __any_sync(0xffffffffu, (threadIdx.x & 31) < c.world && (threadIdx.x & 31) != c.rank &&
                                                      pi.mode == 0u);
  if (h0 == len || !any_pushed) {
    if (ok) cta_reduce<InT, OutT, kOp>(reinterpret_cast<OutT*>(out) + begin, srcs, c.world, len, scale, use_scale);
  } else {
    if (ok) cta_reduce<InT, OutT, kOp>(reinterpret_cast<OutT*>(out) + begin, srcs, c.world, h0, scale, use_scale);
    const bool ok2 = __all_sync(0xffffffffu, wait_bank_warp(c, seq, b, 1, pi, 0u) != 0);
    for (int i = 0; i < c.world; ++i) srcs[i] += h0;
    if (ok2) cta_reduce<InT, OutT, kOp>(reinterpret_cast<OutT*>(out) + begin + h0, srcs, c.world, len - h0, scale,
                                         use_scale);
  }
  exit_done(c, seq, direct);
}

// ---------------------------------------------------------------------------------------------
// all-reduce
// ---------------------------------------------------------------------------------------------
// one-shot: every rank pushes its whole vector to every peer's slot [rank], then reduces world inputs.
template <typename T, int kOp>
__global__ void MB_COLL_BOUNDS
    all_reduce_oneshot_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq, const void* in, void* out,
                              size_t count, float scale, int use_scale) {
  const int b = blockIdx.x, G = gridDim.x;
  entry_wait(c, seq);
  size_t begin, len;
  slice_of(count, G, b, begin, len);
  const T* x = reinterpret_cast<const T*>(in);
  for (int i = 1; i < c.world; ++i) {
    int p = (c.rank + i) % c.world;
    T* dst = reinterpret_cast<T*>(stage_ptr(c, p, seq)) + (size_t)c.rank * count + begin;
    cta_copy(dst, x + begin, len * sizeof(T));
  }
  signal_ready(c, seq, b, 0, -1);
  const T* srcs[MB_MAX_RANKS];
  // fixed source order (rank 0, 1, ...) so every rank computes bit-identical sums
  bool ok = true;
  for (int p = 0; p < c.world; ++p) {
    if (p == c.rank) {
      srcs[p] = x + begin;
    } else {
      ok = wait_ready_warp(c, seq, p, b, 0) && ok;
      srcs[p] = reinterpret_cast<const T*>(stage_ptr(c, c.rank, seq)) + (size_t)p * count + begin;
    }
  }
  if (ok) cta_reduce<T, T, kOp>(reinterpret_cast<T*>(out) + begin, srcs, c.world, len, scale, use_scale);
  exit_done(c, seq, false);
}

// two-shot in one launch: reduce-scatter into the owner, owner pushes the reduced chunk to everyone.
template <typename T, int kOp>
__global__ void MB_COLL_BOUNDS
    all_reduce_twoshot_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq, const void* in, void* out,
                              size_t count, size_t chunk, float scale, int use_scale) {
  const int b = blockIdx.x, G = gridDim.x;
  entry_wait(c, seq);
  const T* x = reinterpret_cast<const T*>(in);
  T* y = reinterpret_cast<T*>(out);
  auto chunk_len = [&](int r) -> size_t {
    size_t s = (size_t)r * chunk;
    if (s >= count) return 0;
    return count - s < chunk ? count - s : chunk;
  };
  // phase 1: contributions to owners (region A of the staging half: [world][chunk])
  for (int i = 1; i < c.world; ++i) {
    int p = (c.rank + i) % c.world;
    size_t begin, len;
    slice_of(chunk_len(p), G, b, begin, len);
    T* dst = reinterpret_cast<T*>(stage_ptr(c, p, seq)) + (size_t)c.rank * chunk + begin;
    cta_copy(dst, x + (size_t)p * chunk + begin, len * sizeof(T));
    signal_ready(c, seq, b, 0, p);
  }
  // phase 2: reduce own chunk, write it locally and into region B ([world][chunk]) of every peer
  size_t begin, len;
  slice_of(chunk_len(c.rank), G, b, begin, len);
  const T* srcs[MB_MAX_RANKS];
  bool ok = true;
  for (int p = 0; p < c.world; ++p) {
    if (p == c.rank) {
      srcs[p] = x + (size_t)c.rank * chunk + begin;
    } else {
      ok = wait_ready_warp(c, seq, p, b, 0) && ok;
      srcs[p] = reinterpret_cast<const T*>(stage_ptr(c, c.rank, seq)) + (size_t)p * chunk + begin;
    }
  }
  T* mine = y + (size_t)c.rank * chunk + begin;
  if (ok) cta_reduce<T, T, kOp>(mine, srcs, c.world, len, scale, use_scale);
  __syncthreads();  // reduced slice visible to the whole CTA before it is pushed
  for (int i = 1; i < c.world; ++i) {
    int p = (c.rank + i) % c.world;
    T* dst = reinterpret_cast<T*>(stage_ptr(c, p, seq)) + (size_t)(c.world + c.rank) * chunk + begin;
    cta_copy(dst, mine, len * sizeof(T));
  }
  signal_ready(c, seq, b, 1, -1);
  // phase 3: collect the other owners' chunks from region B
  for (int i = 1; i < c.world; ++i) {
    int p = (c.rank + i) % c.world;
    slice_of(chunk_len(p), G, b, begin, len);
    if (wait_ready_warp(c, seq, p, b, 1)) {
      const T* src = reinterpret_cast<const T*>(stage_ptr(c, c.rank, seq)) + (size_t)(c.world + p) * chunk + begin;
      cta_copy(y + (size_t)p * chunk + begin, src, len * sizeof(T));
    }
  }
  exit_done(c, seq, false);
}

// ---------------------------------------------------------------------------------------------
// broadcast (pull from the root's staging copy, or straight from the root's heap memory)
// ---------------------------------------------------------------------------------------------
__global__ void MB_COLL_BOUNDS
    broadcast_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq, void* data, int64_t heap_off, size_t bytes,
                     int root) {
  const int b = blockIdx.x, G = gridDim.x;
  const bool direct = heap_off >= 0;
  entry_wait(c, seq);
  size_t begin, len;
  slice_of(bytes, G, b, begin, len);
  uint8_t* d = reinterpret_cast<uint8_t*>(data);
  if (c.rank == root) {
    if (b == 0) announce(c, seq, direct ? (uint64_t)heap_off : 0, direct ? 1u : 0u);
    if (!direct) {
      cta_copy(stage_ptr(c, root, seq) + begin, d + begin, len);
      signal_ready(c, seq, b, 0, -1);
    }
  } else {
    const uint8_t* src;
    uint64_t off;
    uint32_t rdirect;
    bool ok = wait_announce_warp(c, seq, root, off, rdirect);
    if (!rdirect) {
      ok = ok && wait_ready_warp(c, seq, root, b, 0);
      src = stage_ptr(c, root, seq);
    } else {
      src = reinterpret_cast<const uint8_t*>(c.peer[root]) + off;
    }
    if (ok) cta_copy(d + begin, src + begin, len);
  }
  exit_done(c, seq, direct && c.rank == root);
}

// ---------------------------------------------------------------------------------------------
// all-to-all with per-peer byte counts
// ---------------------------------------------------------------------------------------------
// Push protocol, addressed by the receiver: every rank tells each peer where that peer's segment has to land
// (inside its symmetric heap when the output tensor lives there, else inside its staging half, laid out like
// the output); senders write their segments straight from the input over NVLink (posted writes, no staging
// on the sending side) in two halves; the last CTA of a sender's grid to finish a half raises one flag per
// peer, so the two sides need not agree on a grid size; receivers copy each half out of staging while the
// next one is arriving (nothing to copy when the output is in the heap).
__device__ __forceinline__ size_t a2a_first_half(size_t bytes) {
  if (bytes < (1u << 20)) return bytes;
  return (bytes / 2) & ~(size_t)255;
}
__global__ void MB_COLL_BOUNDS
    all_to_all_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq, const void* in, int64_t out_heap_off,
                      void* out, const __grid_constant__ mb_a2a_table_t tab) {
  const int b = blockIdx.x, G = gridDim.x;
  const bool out_direct = out_heap_off >= 0;
  entry_wait(c, seq);
  const uint8_t* x = reinterpret_cast<const uint8_t*>(in);
  uint8_t* y = reinterpret_cast<uint8_t*>(out);
  size_t begin, len;
  if (b == 0) {
    int t = threadIdx.x;
    if (t < c.world && t != c.rank) {
      uint64_t off = out_direct ? (uint64_t)out_heap_off + tab.recv_off[t] : tab.recv_off[t];
      uint32_t* a = c.flags[t] + F_ANN + ((seq & 1) * MB_MAX_RANKS + c.rank) * 4;
      a[0] = (uint32_t)off;
      a[1] = (uint32_t)(off >> 32);
      a[2] = out_direct ? 1u : 0u;
      __threadfence_system();
      st_release_sys(a + 3, seq);
    }
  }
  // own segment
  slice_of(tab.recv_bytes[c.rank], G, b, begin, len);
  cta_copy(y + tab.recv_off[c.rank] + begin, x + tab.send_off[c.rank] + begin, len);
  // where each peer wants its segment
  const PeerInfo dst = [&] {
    const int lane = threadIdx.x & 31;
    PeerInfo r{1u, 0u, 0u, 0u};
    if (lane < c.world && lane != c.rank) {
      uint64_t off;
      uint32_t aux;
      r.ok = wait_announce(c, seq, lane, off, aux);
      r.lo = (uint32_t)off;
      r.hi = (uint32_t)(off >> 32);
      r.mode = aux;
    }
    __syncwarp();
    return r;
  }();
  __shared__ uint32_t s_last;
  for (int h = 0; h < 2; ++h) {
    for (int i = 1; i < c.world; ++i) {
      int p = (c.rank + i) % c.world;
      const size_t h0 = a2a_first_half(tab.send_bytes[p]);
      const size_t hb = h ? h0 : 0, hl = h ? tab.send_bytes[p] - h0 : h0;
      const bool ok = __shfl_sync(0xffffffffu, dst.ok, p) != 0;
      const uint32_t pdirect = __shfl_sync(0xffffffffu, dst.mode, p);
      const uint64_t off = (uint64_t)__shfl_sync(0xffffffffu, dst.lo, p) | ((uint64_t)__shfl_sync(0xffffffffu, dst.hi, p) << 32);
      uint8_t* d = (pdirect ? reinterpret_cast<uint8_t*>(c.peer[p]) : stage_ptr(c, p, seq)) + off;
      slice_of(hl, G, b, begin, len);
      if (ok && len) cta_copy(d + hb + begin, x + tab.send_off[p] + hb + begin, len);
    }
    // the last CTA of this grid to get here tells every peer that half h of its segment is complete
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      uint32_t* cnt = c.flags[c.rank] + F_LOCAL + 2 + h;
      uint32_t old = atom_add_acqrel_gpu(cnt, 1u);
      s_last = (old == (uint32_t)G - 1);
      if (s_last) *cnt = 0;
    }
    __syncthreads();
    if (s_last) {
      int t = threadIdx.x;
      if (t < c.world && t != c.rank) {
        __threadfence_system();
        st_release_sys(c.flags[t] + (h ? F_READY2 : F_READY) + c.rank * kMaxCtas, seq);
      }
    }
    __syncthreads();
  }
  // receive side
  for (int h = 0; h < 2; ++h) {
    uint32_t okl = 1;
    {
      const int lane = threadIdx.x & 31;
      if (lane < c.world && lane != c.rank) {
        okl = wait_geq_sys(c.flags[c.rank] + (h ? F_READY2 : F_READY) + lane * kMaxCtas, seq, c.wait_ns);
        if (!okl) fail(c, kTimeoutReady, lane);
      }
      __syncwarp();
    }
    if (out_direct) continue;  // the segments were written in place
    for (int i = 1; i < c.world; ++i) {
      int p = (c.rank - i + c.world) % c.world;
      const bool ok = __shfl_sync(0xffffffffu, okl, p) != 0;
      const size_t h0 = a2a_first_half(tab.recv_bytes[p]);
      const size_t hb = h ? h0 : 0, hl = h ? tab.recv_bytes[p] - h0 : h0;
      slice_of(hl, G, b, begin, len);
      if (ok && len)
        cta_copy(y + tab.recv_off[p] + hb + begin, stage_ptr(c, c.rank, seq) + tab.recv_off[p] + hb + begin, len);
    }
  }
  exit_done(c, seq, false);
}

// ---------------------------------------------------------------------------------------------
// compile_op lowering: 2-D pieces, sources in peers' staging areas (inputs are staged first)
// ---------------------------------------------------------------------------------------------
__global__ void MB_COLL_BOUNDS
    gather_scatter_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq, const mb_stage_copy_t* stage_in,
                          int num_stage, const mb_piece_t* pieces, int num_pieces) {
  const int b = blockIdx.x, G = gridDim.x;
  entry_wait(c, seq);
  for (int i = 0; i < num_stage; ++i) {
    size_t begin, len;
    slice_of(stage_in[i].bytes, G, b, begin, len);
    cta_copy(stage_ptr(c, c.rank, seq) + stage_in[i].dst_off + begin,
             reinterpret_cast<const uint8_t*>(stage_in[i].src) + begin, len);
  }
  signal_ready(c, seq, b, 0, -1);
  // every peer's inputs must be completely staged before pieces are read: wait for all of its CTAs
  __shared__ uint32_t s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  for (int idx = threadIdx.x; idx < c.world * G; idx += blockDim.x) {
    int p = idx / G, pb = idx % G;
    if (p != c.rank) {
      if (!wait_geq_sys(c.flags[c.rank] + F_READY + p * kMaxCtas + pb, seq, c.wait_ns)) {
        fail(c, kTimeoutReady, p);
        s_ok = 0;
      }
    }
  }
  __syncthreads();
  if (s_ok) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int i = 0; i < num_pieces; ++i) {
      mb_piece_t pc = pieces[i];
      const uint8_t* sbase = pc.src_rank == c.rank && pc.src_local
                                 ? reinterpret_cast<const uint8_t*>(pc.src_local)
                                 : stage_ptr(c, pc.src_rank, seq) + pc.src_off;
      uint8_t* dbase = reinterpret_cast<uint8_t*>(pc.dst);
      bool vec = ((pc.row_bytes | pc.src_pitch | pc.dst_pitch | (uintptr_t)sbase | (uintptr_t)dbase) & 15) == 0;
      if (pc.rows == 1 || (pc.src_pitch == pc.row_bytes && pc.dst_pitch == pc.row_bytes)) {
        size_t begin, len;
        slice_of((size_t)pc.rows * pc.row_bytes, G, b, begin, len);
        cta_copy(dbase + begin, sbase + begin, len);
      } else {
        // one warp per row, rows dealt round-robin over all warps of the grid
        for (uint32_t r = b * nwarps + warp; r < pc.rows; r += G * nwarps) {
          const uint8_t* s = sbase + (size_t)r * pc.src_pitch;
          uint8_t* d = dbase + (size_t)r * pc.dst_pitch;
          if (vec) {
            for (uint64_t j = lane * 16; j < pc.row_bytes; j += 32 * 16) st_stream16(d + j, ld_stream16(s + j));
          } else {
            for (uint64_t j = lane; j < pc.row_bytes; j += 32) d[j] = s[j];
          }
        }
      }
    }
  }
  exit_done(c, seq, false);
}

// ---------------------------------------------------------------------------------------------
// local cast / scale copy (world == 1 paths, staging helpers)
// ---------------------------------------------------------------------------------------------
template <typename InT, typename OutT>
__global__ void MB_COLL_BOUNDS
    copy_cast_kernel(const void* in, void* out, size_t count, float scale, int use_scale) {
  size_t begin, len;
  slice_of(count, gridDim.x, blockIdx.x, begin, len);
  cta_cast_copy<InT, OutT>(reinterpret_cast<OutT*>(out) + begin, reinterpret_cast<const InT*>(in) + begin, len,
                           scale, use_scale);
}
__global__ void MB_COLL_BOUNDS copy_bytes_kernel(const void* in, void* out, size_t bytes) {
  size_t begin, len;
  slice_of(bytes, gridDim.x, blockIdx.x, begin, len);
  cta_copy(reinterpret_cast<uint8_t*>(out) + begin, reinterpret_cast<const uint8_t*>(in) + begin, len);
}

static inline int check_launch() { return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH; }

static inline size_t dtype_size(int dt) {
  switch (dt) {
    case MB_U8:
    case MB_I8: return 1;
    case MB_I16:
    case MB_F16:
    case MB_BF16: return 2;
    case MB_I32:
    case MB_F32: return 4;
    case MB_I64:
    case MB_F64: return 8;
    default: return 0;
  }
}

}  // namespace coll
}  // namespace mb

using namespace mb::coll;

#define MB_STREAM(s) static_cast<cudaStream_t>(s)

extern "C" size_t mb_dtype_size(int dt) { return dtype_size(dt); }

extern "C" int mb_barrier(const mb_comm_t* c, uint32_t seq, void* stream) {
  if (c->world == 1) return MB_OK;
  barrier_kernel<<<1, 32, 0, MB_STREAM(stream)>>>(*c, seq);
  return check_launch();
}

extern "C" int mb_copy_cast(const void* in, void* out, size_t count, int in_dtype, int out_dtype, float scale,
                            int use_scale, void* stream) {
  if (count == 0) return MB_OK;
  size_t bytes = count * dtype_size(in_dtype);
  int grid = (int)((bytes + 65535) / 65536);
  if (grid < 1) grid = 1;
  if (grid > 592) grid = 592;
  cudaStream_t s = MB_STREAM(stream);
  if (in_dtype == out_dtype && !use_scale) {
    copy_bytes_kernel<<<grid, kThreads, 0, s>>>(in, out, bytes);
    return check_launch();
  }
#define CC(IDT, ODT, IT, OT)                                                             \
  if (in_dtype == IDT && out_dtype == ODT) {                                             \
    copy_cast_kernel<IT, OT><<<grid, kThreads, 0, s>>>(in, out, count, scale, use_scale); \
    return check_launch();                                                               \
  }
  CC(MB_F32, MB_F32, float, float)
  CC(MB_BF16, MB_BF16, __nv_bfloat16, __nv_bfloat16)
  CC(MB_F16, MB_F16, __half, __half)
  CC(MB_F64, MB_F64, double, double)
  CC(MB_F32, MB_BF16, float, __nv_bfloat16)
  CC(MB_BF16, MB_F32, __nv_bfloat16, float)
  CC(MB_F32, MB_F16, float, __half)
  CC(MB_F16, MB_F32, __half, float)
  CC(MB_I32, MB_I32, int32_t, int32_t)
  CC(MB_I64, MB_I64, int64_t, int64_t)
#undef CC
  return MB_ERR_ARG;
}

extern "C" int mb_all_gather(const mb_comm_t* c, uint32_t seq, const void* in, int64_t in_heap_off, void* out,
                             size_t count, size_t out_stride, int in_dtype, int out_dtype, void* stream) {
  size_t osz = dtype_size(out_dtype);
  if (!osz || !dtype_size(in_dtype)) return MB_ERR_ARG;
  if (c->world == 1) return mb_copy_cast(in, out, count, in_dtype, out_dtype, 1.f, 0, stream);
  if (in_heap_off == -2 && (size_t)c->world * count * osz > c->staging_bytes / 2) in_heap_off = -1;
  if (in_heap_off < 0 && count * osz > c->staging_bytes / 2) return MB_ERR_TOO_BIG;
  if (in_heap_off >= 0 && in_dtype != out_dtype) return MB_ERR_ARG;
  int grid = pick_grid(c, count * osz);
  cudaStream_t s = MB_STREAM(stream);
  if (in_dtype == out_dtype) {
    // byte-wise: run as uint8 elements
    all_gather_kernel<uint8_t, uint8_t, false><<<grid, kThreads, 0, s>>>(*c, seq, in, in_heap_off, out, count * osz,
                                                                         out_stride * osz);
    return check_launch();
  }
#define AG(IDT, ODT, IT, OT)                                                                             \
  if (in_dtype == IDT && out_dtype == ODT) {                                                             \
    all_gather_kernel<IT, OT, true><<<grid, kThreads, 0, s>>>(*c, seq, in, in_heap_off, out, count, out_stride); \
    return check_launch();                                                                               \
  }
  AG(MB_F32, MB_BF16, float, __nv_bfloat16)
  AG(MB_BF16, MB_F32, __nv_bfloat16, float)
  AG(MB_F32, MB_F16, float, __half)
  AG(MB_F16, MB_F32, __half, float)
#undef AG
  return MB_ERR_ARG;
}

namespace {
template <typename InT, typename OutT>
int launch_rs(const mb_comm_t* c, uint32_t seq, const void* in, int64_t off, void* out, size_t count, size_t stride,
              int op, float scale, int use_scale, int grid, cudaStream_t s) {
  switch (op) {
    case MB_MIN:
      reduce_scatter_kernel<InT, OutT, MB_MIN><<<grid, kThreads, 0, s>>>(*c, seq, in, off, out, count, stride, 1.f, 0);
      break;
    case MB_MAX:
      reduce_scatter_kernel<InT, OutT, MB_MAX><<<grid, kThreads, 0, s>>>(*c, seq, in, off, out, count, stride, 1.f, 0);
      break;
    default:
      reduce_scatter_kernel<InT, OutT, MB_SUM><<<grid, kThreads, 0, s>>>(*c, seq, in, off, out, count, stride, scale,
                                                                         use_scale);
  }
  return check_launch();
}
template <typename T>
int launch_ar(const mb_comm_t* c, uint32_t seq, const void* in, void* out, size_t count, int op, float scale,
              int use_scale, int variant, cudaStream_t s) {
  if (variant == 0) {
    int grid = pick_grid(c, count * sizeof(T));
    switch (op) {
      case MB_MIN: all_reduce_oneshot_kernel<T, MB_MIN><<<grid, kThreads, 0, s>>>(*c, seq, in, out, count, 1.f, 0); break;
      case MB_MAX: all_reduce_oneshot_kernel<T, MB_MAX><<<grid, kThreads, 0, s>>>(*c, seq, in, out, count, 1.f, 0); break;
      default: all_reduce_oneshot_kernel<T, MB_SUM><<<grid, kThreads, 0, s>>>(*c, seq, in, out, count, scale, use_scale);
    }
  } else {
    size_t chunk = (count + c->world - 1) / c->world;
    chunk = (chunk + 63) & ~(size_t)63;
    int grid = pick_grid(c, chunk * sizeof(T));
    switch (op) {
      case MB_MIN: all_reduce_twoshot_kernel<T, MB_MIN><<<grid, kThreads, 0, s>>>(*c, seq, in, out, count, chunk, 1.f, 0); break;
      case MB_MAX: all_reduce_twoshot_kernel<T, MB_MAX><<<grid, kThreads, 0, s>>>(*c, seq, in, out, count, chunk, 1.f, 0); break;
      default: all_reduce_twoshot_kernel<T, MB_SUM><<<grid, kThreads, 0, s>>>(*c, seq, in, out, count, chunk, scale, use_scale);
    }
  }
  return check_launch();
}
bool op_scale(int op, int world, float premul, float* scale, int* use_scale) {
  *scale = 1.f;
  *use_scale = 0;
  switch (op) {
    case MB_SUM: return true;
    case MB_AVG: *scale = 1.0f / (float)world; *use_scale = 1; return true;
    case MB_PREMUL_SUM: *scale = premul; *use_scale = 1; return true;
    case MB_MIN:
    case MB_MAX: return true;
    default: return false;
  }
}
}  // namespace

// ---------------------------------------------------------------------------------------------
// copy-engine ("kernel-less") variants: the bytes move with stream-ordered DMA copies issued by the host,
// these one-warp kernels only run the flag protocol around them, and the reduce-scatter adds one local
// reduction. No SM time is spent on the transfer itself, so a GEMM running next to it keeps its SMs.
// (The reference's counterpart orders cuMemcpy2DAsync copies with IPC events, core/processgroup.cc.)
// ---------------------------------------------------------------------------------------------
namespace {
__global__ void __launch_bounds__(32, 1) ce_begin_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq) {
  entry_wait(c, seq);  // every rank has finished the op two steps back: this staging half is free everywhere
}
// this rank's bytes for the op are in place (its own staging half, or its slots in the peers' halves):
// tell every peer and wait until every peer has said the same
__global__ void __launch_bounds__(32, 1) ce_ready_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq) {
  announce(c, seq, 0, 0u);
  signal_ready(c, seq, 0, 0, -1);
  (void)wait_peers_warp(c, seq, 0, 0);
}
__global__ void __launch_bounds__(32, 1) ce_end_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq) {
  exit_done(c, seq, false);
}
// out[0..count) = op over `nsrc` local buffers (this rank's own slice and the staged slices of the peers)
template <typename InT, typename OutT, int kOp>
__global__ void MB_COLL_BOUNDS
    reduce_local_kernel(const InT* s0, const InT* staged, size_t slot_stride, int rank, int world, OutT* out,
                        size_t count, float scale, int use_scale) {
  size_t begin, len;
  slice_of(count, gridDim.x, blockIdx.x, begin, len);
  const InT* srcs[MB_MAX_RANKS];
  srcs[0] = s0 + begin;
  int n = 1;
  for (int p = 0; p < world; ++p)
    if (p != rank) srcs[n++] = staged + (size_t)p * slot_stride + begin;
  cta_reduce<InT, OutT, kOp>(out + begin, srcs, world, len, scale, use_scale);
}
template <typename InT, typename OutT>
int launch_reduce_local(const void* s0, const void* staged, size_t slot_stride, int rank, int world, void* out,
                        size_t count, int op, float scale, int use_scale, int grid, cudaStream_t s) {
  auto a = reinterpret_cast<const InT*>(s0);
  auto b = reinterpret_cast<const InT*>(staged);
  auto o = reinterpret_cast<OutT*>(out);
  switch (op) {
    case MB_MIN: reduce_local_kernel<InT, OutT, MB_MIN><<<grid, kThreads, 0, s>>>(a, b, slot_stride, rank, world, o, count, 1.f, 0); break;
    case MB_MAX: reduce_local_kernel<InT, OutT, MB_MAX><<<grid, kThreads, 0, s>>>(a, b, slot_stride, rank, world, o, count, 1.f, 0); break;
    default: reduce_local_kernel<InT, OutT, MB_SUM><<<grid, kThreads, 0, s>>>(a, b, slot_stride, rank, world, o, count, scale, use_scale);
  }
  return check_launch();
}
}  // namespace

// ---------------------------------------------------------------------------------------------
// point-to-point flags: a producer's stream raises a word once its data is in place, a consumer's stream
// (on another GPU, through its mapping of the producer's memory) waits for it before it copies
// ---------------------------------------------------------------------------------------------
namespace mb {
namespace coll {
__global__ void __launch_bounds__(32, 1) flag_set_kernel(uint32_t* flag, uint32_t value) {
  if (threadIdx.x == 0) {
    __threadfence_system();  // everything this stream wrote before is visible to whoever sees the flag
    st_release_sys(flag, value);
  }
}
__global__ void __launch_bounds__(32, 1)
    flag_wait_kernel(const uint32_t* flag, uint32_t value, uint32_t* status, uint64_t wait_ns, uint32_t code) {
  if (threadIdx.x == 0) {
    if (!wait_geq_sys(flag, value, wait_ns)) {
      volatile uint32_t* s = status;
      if (*s == 0) *s = code;
    }
  }
}
}  // namespace coll
}  // namespace mb

extern "C" int mb_flag_set(uint32_t* flag, uint32_t value, void* stream) {
  flag_set_kernel<<<1, 32, 0, MB_STREAM(stream)>>>(flag, value);
  return check_launch();
}

// Bounded: when `flag` has not reached `value` after wait_ns the kernel records `code` in *status (if it is
// still 0) and ends; what follows on the stream runs all the same, so the host must check the status word.
extern "C" int mb_flag_wait(const uint32_t* flag, uint32_t value, uint32_t* status, uint64_t wait_ns, uint32_t code,
                            void* stream) {
  flag_wait_kernel<<<1, 32, 0, MB_STREAM(stream)>>>(flag, value, status, wait_ns, code);
  return check_launch();
}

extern "C" int mb_ce_phase(const mb_comm_t* c, uint32_t seq, int phase, void* stream) {
  cudaStream_t s = MB_STREAM(stream);
  switch (phase) {
    case 0: ce_begin_kernel<<<1, 32, 0, s>>>(*c, seq); break;
    case 1: ce_ready_kernel<<<1, 32, 0, s>>>(*c, seq); break;
    case 2: ce_end_kernel<<<1, 32, 0, s>>>(*c, seq); break;
    default: return MB_ERR_ARG;
  }
  return check_launch();
}

extern "C" int mb_reduce_local(const mb_comm_t* c, uint32_t seq, const void* own, void* out, size_t count,
                               int in_dtype, int out_dtype, int op, float premul, void* stream) {
  float scale;
  int use_scale;
  if (!op_scale(op, c->world, premul, &scale, &use_scale)) return MB_ERR_ARG;
  size_t isz = dtype_size(in_dtype);
  if (!isz) return MB_ERR_ARG;
  const void* staged = reinterpret_cast<const uint8_t*>(c->stage[c->rank]) + (uint64_t)(seq & 1) * (c->staging_bytes >> 1);
  int grid = pick_grid(c, count * isz, 64);
  cudaStream_t s = MB_STREAM(stream);
#define RL(IDT, ODT, IT, OT) \
  if (in_dtype == IDT && out_dtype == ODT) \
    return launch_reduce_local<IT, OT>(own, staged, count, c->rank, c->world, out, count, op, scale, use_scale, grid, s);
  RL(MB_F32, MB_F32, float, float)
  RL(MB_BF16, MB_BF16, __nv_bfloat16, __nv_bfloat16)
  RL(MB_BF16, MB_F32, __nv_bfloat16, float)
  RL(MB_F32, MB_BF16, float, __nv_bfloat16)
  RL(MB_F16, MB_F16, __half, __half)
#undef RL
  return MB_ERR_ARG;
}

extern "C" int mb_reduce_scatter(const mb_comm_t* c, uint32_t seq, const void* in, int64_t in_heap_off, void* out,
                                 size_t count, size_t in_stride, int in_dtype, int out_dtype, int op, float premul,
                                 void* stream) {
  size_t isz = dtype_size(in_dtype);
  if (!isz || !dtype_size(out_dtype)) return MB_ERR_ARG;
  float scale;
  int use_scale;
  if (!op_scale(op, c->world, premul, &scale, &use_scale)) return MB_ERR_ARG;
  if (c->world == 1) return mb_copy_cast(in, out, count, in_dtype, out_dtype, scale, use_scale, stream);
  if (in_heap_off < 0 && (size_t)c->world * count * isz > c->staging_bytes / 2) return MB_ERR_TOO_BIG;
  (void)in_stride;
  int grid = pick_grid(c, count * isz, count * isz >= (8u << 20) ? 128 : 64);
  cudaStream_t s = MB_STREAM(stream);
#define RS(IDT, ODT, IT, OT) \
  if (in_dtype == IDT && out_dtype == ODT) \
    return launch_rs<IT, OT>(c, seq, in, in_heap_off, out, count, in_stride, op, scale, use_scale, grid, s);
  RS(MB_F32, MB_F32, float, float)
  RS(MB_BF16, MB_BF16, __nv_bfloat16, __nv_bfloat16)
  RS(MB_BF16, MB_F32, __nv_bfloat16, float)
  RS(MB_F32, MB_BF16, float, __nv_bfloat16)
  RS(MB_F16, MB_F16, __half, __half)
  RS(MB_F64, MB_F64, double, double)
  RS(MB_I32, MB_I32, int32_t, int32_t)
  RS(MB_I64, MB_I64, int64_t, int64_t)
  RS(MB_U8, MB_U8, uint8_t, uint8_t)
#undef RS
  return MB_ERR_ARG;
}

extern "C" int mb_all_reduce(const mb_comm_t* c, uint32_t seq, const void* in, void* out, size_t count, int dtype,
                             int op, float premul, int variant, void* stream) {
  size_t sz = dtype_size(dtype);
  if (!sz) return MB_ERR_ARG;
  float scale;
  int use_scale;
  if (!op_scale(op, c->world, premul, &scale, &use_scale)) return MB_ERR_ARG;
  if (c->world == 1) return mb_copy_cast(in, out, count, dtype, dtype, scale, use_scale, stream);
  size_t half = c->staging_bytes / 2;
  if (variant == 0 && (size_t)c->world * count * sz > half) variant = 1;
  if (variant == 1) {
    size_t chunk = ((count + c->world - 1) / c->world + 63) & ~(size_t)63;
    if (2 * (size_t)c->world * chunk * sz > half) return MB_ERR_TOO_BIG;
  }
  cudaStream_t s = MB_STREAM(stream);
#define AR(DT, T) \
  if (dtype == DT) return launch_ar<T>(c, seq, in, out, count, op, scale, use_scale, variant, s);
  AR(MB_F32, float)
  AR(MB_BF16, __nv_bfloat16)
  AR(MB_F16, __half)
  AR(MB_F64, double)
  AR(MB_I32, int32_t)
  AR(MB_I64, int64_t)
  AR(MB_U8, uint8_t)
#undef AR
  return MB_ERR_ARG;
}

extern "C" int mb_broadcast(const mb_comm_t* c, uint32_t seq, void* data, int64_t heap_off, size_t bytes, int root,
                            void* stream) {
  if (c->world == 1 || bytes == 0) return MB_OK;
  if (heap_off < 0 && bytes > c->staging_bytes / 2) return MB_ERR_TOO_BIG;
  int grid = pick_grid(c, bytes);
  broadcast_kernel<<<grid, kThreads, 0, MB_STREAM(stream)>>>(*c, seq, data, heap_off, bytes, root);
  return check_launch();
}

extern "C" int mb_all_to_all(const mb_comm_t* c, uint32_t seq, const void* in, int64_t out_heap_off, void* out,
                             const mb_a2a_table_t* tab, void* stream) {
  size_t total = 0, biggest = 0;
  for (int r = 0; r < c->world; ++r) {
    size_t end = tab->recv_off[r] + tab->recv_bytes[r];
    if (end > total) total = end;
    if (tab->recv_bytes[r] > biggest) biggest = tab->recv_bytes[r];
    if (tab->send_bytes[r] > biggest) biggest = tab->send_bytes[r];
  }
  if (c->world == 1) {
    if (tab->send_bytes[0] == 0) return MB_OK;
    return mb_copy_cast((const uint8_t*)in + tab->send_off[0], (uint8_t*)out + tab->recv_off[0], tab->send_bytes[0],
                        MB_U8, MB_U8, 1.f, 0, stream);
  }
  // incoming segments are laid out in the staging half like in the output tensor
  if (out_heap_off < 0 && total > c->staging_bytes / 2) return MB_ERR_TOO_BIG;
  int grid = pick_grid(c, biggest);  // ranks may pick different grids: nothing in the protocol depends on it
  all_to_all_kernel<<<grid, kThreads, 0, MB_STREAM(stream)>>>(*c, seq, in, out_heap_off, out, *tab);
  return check_launch();
}

extern "C" int mb_gather_scatter(const mb_comm_t* c, uint32_t seq, const mb_stage_copy_t* stage_in, int num_stage,
                                 const mb_piece_t* pieces, int num_pieces, size_t max_bytes, void* stream) {
  int grid = pick_grid(c, max_bytes);
  gather_scatter_kernel<<<grid, kThreads, 0, MB_STREAM(stream)>>>(*c, seq, stage_in, num_stage, pieces, num_pieces);
  return check_launch();
}
