// Device-side building blocks shared by the collective kernels: the flag-page protocol (announce /
// ready / done words in every rank's peer-mapped flag page), bounded waits that record a status code
// instead of hanging, and vectorised copy / reduce loops over peer memory.
//
// Protocol, per collective with sequence number `seq` (same on every rank, +1 per collective):
//   entry   wait DONE[p] >= seq-2 for every p: the op two steps back has been fully consumed everywhere,
//           so the staging half (seq&1) may be overwritten and peers' halves may be written to.
//   ready   a producer CTA b publishes READY[rank][b] = seq in the consumer's page after its slice is
//           in place (st.release.sys after a system fence); consumers poll their own page only.
//   done    the last CTA of a rank's grid publishes DONE[rank] = seq in every page. Ops whose peers read
//           this rank's *user* memory directly additionally hold one CTA until every DONE[p] >= seq.
// The reference does the same rendezvous with step values written into peer-mapped arrays but spins
// without bound (core/kernels.cc:583-731).
#pragma once

#include "kernels_api.h"
#include "ptx.cuh"

namespace mb {
namespace coll {

// Register budget of the 512-thread collective kernels. A collective usually runs on a side stream under a
// persistent tcgen05 GEMM that holds one CTA on every SM (192 threads x 120 registers = 23,040 of the SM's
// 65,536, and nearly all of its shared memory). With 80 registers per thread a collective CTA takes 40,960
// and fits beside it; at the 84-128 the compiler picks on its own it does not, and then either kernel keeps
// the other off every SM it occupies: the GEMM runs on the SMs the collective left over and its statically
// assigned tiles on the missing SMs wait for the collective to end. ptxas reports no spills at 80 for the
// float / bf16 paths (a few hundred bytes for the 64-bit integer min / max variants).
#define MB_COLL_REGS 80
#define MB_COLL_BOUNDS __maxnreg__(MB_COLL_REGS)

constexpr int kMaxCtas = 128;  // READY has room for this many producer CTAs per rank
constexpr int F_DONE = 0;      // [8]
constexpr int F_ANN = 16;      // [2][8][4]  {off_lo, off_hi, aux, seq}, bank = seq & 1 (a fast peer may already
                               //            announce op seq+1 while this rank still reads the one for seq)
constexpr int F_LOCAL = 96;    // [8]     local-grid counters (own page only)
constexpr int F_TABLE = 128;   // [8][4]  all-to-all: {src_off_lo, src_off_hi, bytes_lo, bytes_hi}
constexpr int F_READY = 256;   // [8][kMaxCtas]
constexpr int F_READY2 = F_READY + MB_MAX_RANKS * kMaxCtas;  // second bank (two-phase ops)
constexpr int F_CHUNK = F_READY2 + MB_MAX_RANKS * kMaxCtas;  // AG->GEMM: [8][32] arrival words (value = seq)
constexpr int F_RSCNT = F_CHUNK + 256;                       // GEMM->RS: [2 banks][128] arrival counters
static_assert(F_RSCNT + 256 <= MB_FLAG_WORDS, "flag page too small");

enum Status : uint32_t {
  kTimeoutEntry = 0x201,
  kTimeoutReady = 0x202,
  kTimeoutAnnounce = 0x203,
  kTimeoutExit = 0x204,
};

// The status word may live in host-mapped memory, so no atomics: the first writer (nearly) wins.
__device__ __forceinline__ void fail(const mb_comm_t& c, uint32_t code, int peer) {
  volatile uint32_t* s = c.status;
  if (*s == 0) *s = code | ((uint32_t)peer << 16);
}

__device__ __forceinline__ uint8_t* stage_ptr(const mb_comm_t& c, int r, uint32_t seq) {
  return reinterpret_cast<uint8_t*>(c.stage[r]) + (uint64_t)(seq & 1) * (c.staging_bytes >> 1);
}

// All threads of the CTA call this. Threads 0..world-1 each wait on one peer.
__device__ __forceinline__ void entry_wait(const mb_comm_t& c, uint32_t seq) {
  int t = threadIdx.x;
  if (t < c.world && t != c.rank) {
    if (!wait_geq_sys(c.flags[c.rank] + F_DONE + t, seq - 2, c.wait_ns)) fail(c, kTimeoutEntry, t);
  }
  __syncthreads();
}

// Publish {offset, aux} of this rank's source to every peer (one CTA, threads 0..world-1).
__device__ __forceinline__ void announce(const mb_comm_t& c, uint32_t seq, uint64_t off, uint32_t aux) {
  int t = threadIdx.x;
  if (t < c.world && t != c.rank) {
    uint32_t* a = c.flags[t] + F_ANN + ((seq & 1) * MB_MAX_RANKS + c.rank) * 4;
    a[0] = (uint32_t)off;
    a[1] = (uint32_t)(off >> 32);
    a[2] = aux;
    __threadfence_system();
    st_release_sys(a + 3, seq);
  }
}
// Any thread: wait for peer p's announcement and read it.
__device__ __forceinline__ bool wait_announce(const mb_comm_t& c, uint32_t seq, int p, uint64_t& off, uint32_t& aux) {
  const uint32_t* a = c.flags[c.rank] + F_ANN + ((seq & 1) * MB_MAX_RANKS + p) * 4;
  if (!wait_geq_sys(a + 3, seq, c.wait_ns)) {
    fail(c, kTimeoutAnnounce, p);
    off = 0;
    aux = 0;
    return false;
  }
  off = (uint64_t)ld_relaxed_sys(a) | ((uint64_t)ld_relaxed_sys(a + 1) << 32);
  aux = ld_relaxed_sys(a + 2);
  return true;
}

// After the CTA's data for this op is written: tell peer(s) that slice `b` is ready.
// Called by all threads; thread t < world signals peer t (or only `only_peer` if >= 0).
__device__ __forceinline__ void signal_ready(const mb_comm_t& c, uint32_t seq, int b, int bank, int only_peer) {
  __syncthreads();
  int t = threadIdx.x;
  if (t < c.world && t != c.rank && (only_peer < 0 || t == only_peer)) {
    __threadfence_system();
    st_release_sys(c.flags[t] + (bank ? F_READY2 : F_READY) + c.rank * kMaxCtas + b, seq);
  }
}
// One thread per warp polls, then the warp proceeds. Returns false on timeout (status recorded).
__device__ __forceinline__ bool wait_ready_warp(const mb_comm_t& c, uint32_t seq, int p, int b, int bank) {
  uint32_t ok = 1;
  if ((threadIdx.x & 31) == 0) {
    ok = wait_geq_sys(c.flags[c.rank] + (bank ? F_READY2 : F_READY) + p * kMaxCtas + b, seq, c.wait_ns);
    if (!ok) fail(c, kTimeoutReady, p);
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}

// Every lane p < world of the calling warp waits for peer p at the same time: its announcement and, unless
// that peer is read in place (mode 1), the READY word of slice b. Callers read a peer's answer with
// __shfl_sync(field, p). Sequential waits cost one flag latency per peer; this costs one in total.
struct PeerInfo {
  uint32_t ok, lo, hi, mode;
};
__device__ __forceinline__ PeerInfo wait_peers_warp(const mb_comm_t& c, uint32_t seq, int b, int bank) {
  const int lane = threadIdx.x & 31;
  PeerInfo r{1u, 0u, 0u, 0u};
  if (lane < c.world && lane != c.rank) {
    uint64_t off;
    uint32_t aux;
    r.ok = wait_announce(c, seq, lane, off, aux);
    r.lo = (uint32_t)off;
    r.hi = (uint32_t)(off >> 32);
    r.mode = aux;
    if (r.ok && aux != 1u) {
      r.ok = wait_geq_sys(c.flags[c.rank] + (bank ? F_READY2 : F_READY) + lane * kMaxCtas + b, seq, c.wait_ns);
      if (!r.ok) fail(c, kTimeoutReady, lane);
    }
  }
  __syncwarp();
  return r;
}
// Second phase of a two-bank transfer: every lane p < world whose peer pushes its data (announced mode ==
// push_mode) waits for that peer's READY word of slice b in `bank`. Returns the per-lane result (the first
// phase's result for lanes that had nothing to wait for).
__device__ __forceinline__ uint32_t wait_bank_warp(const mb_comm_t& c, uint32_t seq, int b, int bank, const PeerInfo& pi,
                                                   uint32_t push_mode) {
  const int lane = threadIdx.x & 31;
  uint32_t ok = pi.ok;
  if (lane < c.world && lane != c.rank && pi.ok && pi.mode == push_mode) {
    ok = wait_geq_sys(c.flags[c.rank] + (bank ? F_READY2 : F_READY) + lane * kMaxCtas + b, seq, c.wait_ns);
    if (!ok) fail(c, kTimeoutReady, lane);
  }
  __syncwarp();
  return ok;
}
// A CTA slice of `len` elements is sent in two halves (one READY bank each) when it is big enough for the
// receiver's copy-out / reduce of the first half to hide under the arrival of the second. Same answer on
// every rank: it depends only on the element count and the grid.
constexpr size_t kTwoPhaseBytes = 64 << 10;
template <typename T>
__device__ __forceinline__ size_t first_half(size_t len) {
  if (len * sizeof(T) < kTwoPhaseBytes) return len;
  size_t h = len / 2;
  return h - h % (256 / sizeof(T));  // keep the second half 256-byte aligned relative to the slice
}
__device__ __forceinline__ bool all_peers_ok(const PeerInfo& r) {
  return __all_sync(0xffffffffu, r.ok != 0);
}

// End of op. The last CTA of the grid publishes DONE[rank] = seq everywhere; with `hold` it also waits
// until every peer is done (their reads of this rank's user memory have finished).
__device__ __forceinline__ void exit_done(const mb_comm_t& c, uint32_t seq, bool hold) {
  __shared__ uint32_t s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t* cnt = c.flags[c.rank] + F_LOCAL;
    uint32_t old = atom_add_acqrel_gpu(cnt, 1u);
    s_last = (old == gridDim.x - 1);
    if (s_last) *cnt = 0;
  }
  __syncthreads();
  if (!s_last) return;
  int t = threadIdx.x;
  if (t < c.world) {
    __threadfence_system();
    st_release_sys(c.flags[t] + F_DONE + c.rank, seq);
    if (hold && t != c.rank) {
      if (!wait_geq_sys(c.flags[c.rank] + F_DONE + t, seq, c.wait_ns)) fail(c, kTimeoutExit, t);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// data movement
// ---------------------------------------------------------------------------------------------
// CTA-cooperative byte copy. Fast path when both pointers are 16-byte aligned.
template <int kUnroll = 8>
__device__ __forceinline__ void cta_copy(void* dst, const void* src, size_t bytes) {
  uint8_t* d = reinterpret_cast<uint8_t*>(dst);
  const uint8_t* s = reinterpret_cast<const uint8_t*>(src);
  const int nt = blockDim.x, tid = threadIdx.x;
  if ((((uintptr_t)d | (uintptr_t)s) & 15) == 0) {
    size_t nvec = bytes >> 4;
    size_t step = (size_t)nt * kUnroll;
    size_t i = 0;
    for (; i + step <= nvec; i += step) {
      uint4 v[kUnroll];
#pragma unroll
      for (int k = 0; k < kUnroll; ++k) v[k] = ld_stream16(s + ((i + tid + (size_t)k * nt) << 4));
#pragma unroll
      for (int k = 0; k < kUnroll; ++k) st_stream16(d + ((i + tid + (size_t)k * nt) << 4), v[k]);
    }
    for (size_t j = i + tid; j < nvec; j += nt) st_stream16(d + (j << 4), ld_stream16(s + (j << 4)));
    for (size_t j = (nvec << 4) + tid; j < bytes; j += nt) d[j] = s[j];
  } else {
    for (size_t j = tid; j < bytes; j += nt) d[j] = s[j];
  }
}

// element <-> accumulator conversions
template <typename T>
struct Acc {
  using type = float;
};
template <>
struct Acc<double> {
  using type = double;
};
template <>
struct Acc<int32_t> {
  using type = int64_t;
};
template <>
struct Acc<int64_t> {
  using type = int64_t;
};
template <>
struct Acc<uint8_t> {
  using type = int64_t;
};
template <>
struct Acc<int8_t> {
  using type = int64_t;
};
template <>
struct Acc<int16_t> {
  using type = int64_t;
};

template <typename A, typename T>
__device__ __forceinline__ A to_acc(T v) {
  return static_cast<A>(v);
}
template <>
__device__ __forceinline__ float to_acc<float, __nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <>
__device__ __forceinline__ float to_acc<float, __half>(__half v) {
  return __half2float(v);
}
template <typename T, typename A>
__device__ __forceinline__ T from_acc(A v) {
  return static_cast<T>(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16, float>(float v) {
  return __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ __half from_acc<__half, float>(float v) {
  return __float2half_rn(v);
}

template <int kOp, typename A>
__device__ __forceinline__ A combine(A a, A b) {
  if constexpr (kOp == MB_MIN) return b < a ? b : a;
  if constexpr (kOp == MB_MAX) return b > a ? b : a;
  return a + b;
}

// a 16-byte vector of T
template <typename T>
struct Vec {
  static constexpr int N = 16 / sizeof(T);
  union {
    uint4 u;
    T e[N];
  };
};

// CTA-cooperative cast+scale copy: dst[i] = OutT(acc(src[i]) * scale). Pointers may be unaligned.
template <typename InT, typename OutT>
__device__ __forceinline__ void cta_cast_copy(OutT* dst, const InT* src, size_t n, float scale, bool use_scale) {
  using A = typename Acc<InT>::type;
  constexpr int N = Vec<InT>::N < Vec<OutT>::N ? Vec<InT>::N : Vec<OutT>::N;  // elements per step
  const int nt = blockDim.x, tid = threadIdx.x;
  bool aligned = ((uintptr_t)src % (N * sizeof(InT)) == 0) && ((uintptr_t)dst % (N * sizeof(OutT)) == 0);
  size_t nv = aligned ? n / N : 0;
  for (size_t i = tid; i < nv; i += nt) {
    InT in[N];
    OutT out[N];
    if constexpr (N * sizeof(InT) == 16)
      *reinterpret_cast<uint4*>(in) = ld_stream16(src + i * N);
    else if constexpr (N * sizeof(InT) == 8)
      *reinterpret_cast<uint2*>(in) = *reinterpret_cast<const uint2*>(src + i * N);
    else
      *reinterpret_cast<uint32_t*>(in) = *reinterpret_cast<const uint32_t*>(src + i * N);
#pragma unroll
    for (int k = 0; k < N; ++k) {
      A a = to_acc<A, InT>(in[k]);
      if (use_scale) a = static_cast<A>(a * scale);
      out[k] = from_acc<OutT, A>(a);
    }
    if constexpr (N * sizeof(OutT) == 16)
      st_stream16(dst + i * N, *reinterpret_cast<uint4*>(out));
    else if constexpr (N * sizeof(OutT) == 8)
      *reinterpret_cast<uint2*>(dst + i * N) = *reinterpret_cast<uint2*>(out);
    else
      *reinterpret_cast<uint32_t*>(dst + i * N) = *reinterpret_cast<uint32_t*>(out);
  }
  for (size_t i = nv * N + tid; i < n; i += nt) {
    A a = to_acc<A, InT>(src[i]);
    if (use_scale) a = static_cast<A>(a * scale);
    dst[i] = from_acc<OutT, A>(a);
  }
}

// CTA-cooperative N-way reduce: dst[i] = OutT(op_r(src[r][i]) * scale), accumulate in Acc<InT>.
// src pointers may be peer memory. kMaxSrc bounds the unrolled source loop.
template <typename InT, typename OutT, int kOp>
__device__ __forceinline__ void cta_reduce(OutT* dst, const InT* const* src, int nsrc, size_t n, float scale,
                                           bool use_scale) {
  using A = typename Acc<InT>::type;
  constexpr int N = Vec<InT>::N;
  const int nt = blockDim.x, tid = threadIdx.x;
  bool aligned = ((uintptr_t)dst % (N * sizeof(OutT) < 16 ? N * sizeof(OutT) : 16) == 0);
  for (int r = 0; r < nsrc; ++r) aligned = aligned && (((uintptr_t)src[r] & 15) == 0);
  size_t nv = aligned ? n / N : 0;
  for (size_t i = tid; i < nv; i += nt) {
    A acc[N];
    Vec<InT> v[MB_MAX_RANKS];
#pragma unroll
    for (int r = 0; r < MB_MAX_RANKS; ++r)
      if (r < nsrc) v[r].u = ld_stream16(src[r] + i * N);
#pragma unroll
    for (int k = 0; k < N; ++k) acc[k] = to_acc<A, InT>(v[0].e[k]);
#pragma unroll
    for (int r = 1; r < MB_MAX_RANKS; ++r)
      if (r < nsrc) {
#pragma unroll
        for (int k = 0; k < N; ++k) acc[k] = combine<kOp, A>(acc[k], to_acc<A, InT>(v[r].e[k]));
      }
    OutT out[N];
#pragma unroll
    for (int k = 0; k < N; ++k) {
      A a = acc[k];
      if (use_scale) a = static_cast<A>(a * scale);
      out[k] = from_acc<OutT, A>(a);
    }
    if constexpr (N * sizeof(OutT) == 16) {
      st_stream16(dst + i * N, *reinterpret_cast<uint4*>(out));
    } else if constexpr (N * sizeof(OutT) == 32) {
      st_stream16(dst + i * N, reinterpret_cast<uint4*>(out)[0]);
      st_stream16(dst + i * N + N / 2, reinterpret_cast<uint4*>(out)[1]);
    } else if constexpr (N * sizeof(OutT) == 8) {
      *reinterpret_cast<uint2*>(dst + i * N) = *reinterpret_cast<uint2*>(out);
    } else {
#pragma unroll
      for (int k = 0; k < N; ++k) dst[i * N + k] = out[k];
    }
  }
  for (size_t i = nv * N + tid; i < n; i += nt) {
    A a = to_acc<A, InT>(src[0][i]);
    for (int r = 1; r < nsrc; ++r) a = combine<kOp, A>(a, to_acc<A, InT>(src[r][i]));
    if (use_scale) a = static_cast<A>(a * scale);
    dst[i] = from_acc<OutT, A>(a);
  }
}

// slice b of n elements split over `parts` CTAs, boundaries on multiples of 64 elements
__device__ __forceinline__ void slice_of(size_t n, int parts, int b, size_t& begin, size_t& len) {
  size_t per = (n + parts - 1) / parts;
  per = (per + 63) & ~(size_t)63;
  begin = (size_t)b * per;
  if (begin > n) begin = n;
  size_t end = begin + per;
  if (end > n) end = n;
  len = end - begin;
}

}  // namespace coll
}  // namespace mb
