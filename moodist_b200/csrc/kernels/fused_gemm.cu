// Fused collective GEMMs: ONE kernel does the NVLink transfer and the tcgen05 tiles.
//
//   mb_ag_gemm  C = gather(A shards) · B^T   or   C = A · gather(B shards)^T
//     CTAs [0, C) are copy CTAs, CTAs [C, C+G) run the persistent GEMM of gemm_tcgen05.cuh: copy CTA j
//     pushes sub-chunk j of this rank's shard into every rank's staging area (plain 16-byte stores over
//     NVLink, own copy first) and publishes an arrival word in the receiver's flag page. The GEMM's TMA
//     producer waits on the word of the sub-chunk a tile needs, then loads it with TMA from LOCAL memory.
//     Tiles are walked own shard first, then in push-arrival order, so the transfer hides behind the math.
//
//   mb_gemm_rs  out = reduce_scatter(A · B^T) over rows
//     Every CTA runs the GEMM; the epilogue writes each bf16 tile straight into the owner rank's staging
//     slot for this source (remote stores) and bumps the owner's per-row-block counter. Tiles for other
//     owners are computed first. Afterwards the CTAs reduce this rank's row blocks as their counters fill
//     up: fp32 accumulation over the ranks' slots, optional scale, bf16 (or fp32) result.
//
// No TMA instruction touches another GPU's memory and no load uses cluster multicast: remote data moves
// with ordinary ld/st only. The reference has neither op (it has no GEMM at all).
#include "coll.cuh"
#include "gemm_pair_tcgen05.cuh"

#include <cstdlib>

namespace mb {
namespace gemm {
int make_tmap_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
int sm_count();
}  // namespace gemm

namespace fused {

using namespace mb::gemm;
using namespace mb::coll;

constexpr int kMaxSubs = 32;  // arrival words per shard (F_CHUNK holds 8 x 32)

struct GatherArgs {
  const void* shard;   // this rank's rows [shard_rows, row_bytes/2 elements], row pitch = row_bytes
  uint64_t row_bytes;  // bytes per row (K * 2)
  int shard_rows, sub_rows, subs_per_shard;
};

// ------------------------------------------------------------------------------------------------
// AG -> GEMM
// ------------------------------------------------------------------------------------------------
// Every CTA runs the tile loop on its first 192 threads; four more warps per CTA move the data: in CTA j < subs
// they push sub-chunk j of this rank's shard into every rank's staging area (own copy first) and raise the
// arrival word. All 148 SMs compute; the pushes ride on warps that would not exist otherwise.
// kPair: the tiles run on CTA pairs (cta_group::2, the grid is launched as clusters of two).
constexpr int kCopyThreads = 128;
constexpr int kAgThreads = kNumThreads + kCopyThreads;

__device__ __forceinline__ void copy_warps_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// cta_copy for a subset of the CTA: `tid` in [0, nt)
__device__ __forceinline__ void warps_copy(void* dst, const void* src, size_t bytes, int tid, int nt) {
  uint8_t* d = reinterpret_cast<uint8_t*>(dst);
  const uint8_t* s = reinterpret_cast<const uint8_t*>(src);
  constexpr int kUnroll = 8;
  size_t nvec = bytes >> 4;  // callers pass 16-byte aligned pointers and row sizes
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
}

template <bool kBMn, typename OutT, bool kPair>
__global__ void __launch_bounds__(kAgThreads, 1)
    ag_gemm_kernel(const __grid_constant__ Params p, const __grid_constant__ CUtensorMap tmap_a,
                   const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ mb_comm_t c, uint32_t seq,
                   const __grid_constant__ GatherArgs g) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  if (threadIdx.x < kNumThreads) {
    if constexpr (kPair) {
      gemm_pair_body<false, kBMn, OutT, true, false>(p, &tmap_a, &tmap_b, smem_raw);
    } else {
      gemm_body<false, kBMn, OutT, true, false>(p, &tmap_a, &tmap_b, smem_raw);
    }
  } else {
    // ---- copy warps ----
    const int tid = threadIdx.x - kNumThreads;
    const int j = blockIdx.x;
    if constexpr (kPair) cluster_sync_all();  // pairs with the cluster barrier at the start of the tile loop
    if (j < g.subs_per_shard) {
      // the staging half written below was last used two collectives ago: wait until every rank is past it
      if (tid < c.world && tid != c.rank) {
        if (!wait_geq_sys(c.flags[c.rank] + F_DONE + tid, seq - 2, c.wait_ns)) fail(c, kTimeoutEntry, tid);
      }
      copy_warps_sync();
      const int row0 = j * g.sub_rows;
      const int rows = min(g.sub_rows, g.shard_rows - row0);
      const uint8_t* src = reinterpret_cast<const uint8_t*>(g.shard) + (uint64_t)row0 * g.row_bytes;
      const uint64_t bytes = (uint64_t)rows * g.row_bytes;
      const uint64_t dst_off = ((uint64_t)c.rank * g.shard_rows + row0) * g.row_bytes;
      for (int i = 0; i < c.world; ++i) {
        const int dst = (c.rank + i) % c.world;  // own copy first: the local tiles start on it
        warps_copy(stage_ptr(c, dst, seq) + dst_off, src, bytes, tid, kCopyThreads);
        copy_warps_sync();
        if (tid == 0) {
          __threadfence_system();
          st_release_sys(c.flags[dst] + F_CHUNK + c.rank * kMaxSubs + j, seq);
        }
      }
    }
    if constexpr (kPair) cluster_sync_all();  // pairs with the one at the end of the tile loop
  }
  exit_done(c, seq, false);
}

// ------------------------------------------------------------------------------------------------
// GEMM -> RS
// ------------------------------------------------------------------------------------------------
struct ReduceArgs {
  void* out;            // [scatter_rows, N] result rows of this rank
  int64_t ldo;          // elements
  int out_fp32;
  float scale;
  int use_scale;
  int bank;             // counter bank (seq & 1)
  uint32_t expected;    // arrivals per 128-row block: 4 warps x tiles_n x world
};

template <bool kBMn, bool kPair>
__global__ void __launch_bounds__(kNumThreads, 1)
    gemm_rs_kernel(const __grid_constant__ Params p, const __grid_constant__ CUtensorMap tmap_a,
                   const __grid_constant__ CUtensorMap tmap_b, const __grid_constant__ mb_comm_t c, uint32_t seq,
                   const __grid_constant__ ReduceArgs r) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  entry_wait(c, seq);  // peers' staging halves are written by the epilogue
  if constexpr (kPair) {
    gemm_pair_body<false, kBMn, __nv_bfloat16, false, true>(p, &tmap_a, &tmap_b, smem_raw);
  } else {
    gemm_body<false, kBMn, __nv_bfloat16, false, true>(p, &tmap_a, &tmap_b, smem_raw);
  }

  // ---- reduce this rank's rows as their blocks complete ----
  const int blocks = p.scatter_rows / BM;
  const int col_chunks = (p.N + 255) / 256;
  const int units = blocks * col_chunks;
  uint32_t* counters = c.flags[c.rank] + F_RSCNT + r.bank * 128;
  const uint8_t* stage = stage_ptr(c, c.rank, seq);
  const uint64_t slot_bytes = (uint64_t)p.scatter_rows * p.ldc * 2;
  __shared__ uint32_t s_ok;
  for (int u = blockIdx.x; u < units; u += gridDim.x) {
    const int blk = u / col_chunks, cc = u - blk * col_chunks;
    if (threadIdx.x == 0) {
      s_ok = wait_geq_sys(counters + blk, r.expected, c.wait_ns);
      if (!s_ok) fail(c, kTimeoutReady, blk);
    }
    __syncthreads();
    if (s_ok) {
      const int col0 = cc * 256;
      const int ncols = min(256, p.N - col0);
      const int vec_per_row = ncols / 8;  // 8 bf16 per 16 bytes; N is a multiple of 8
      for (int i = threadIdx.x; i < BM * vec_per_row; i += blockDim.x) {
        const int row = blk * BM + i / vec_per_row;
        const int col = col0 + (i % vec_per_row) * 8;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int s = 0; s < c.world; ++s) {
          uint4 v = ld_stream16(stage + (uint64_t)s * slot_bytes + ((uint64_t)row * p.ldc + col) * 2);
          float2 f;
          f = unpack_bf16x2(v.x); acc[0] += f.x; acc[1] += f.y;
          f = unpack_bf16x2(v.y); acc[2] += f.x; acc[3] += f.y;
          f = unpack_bf16x2(v.z); acc[4] += f.x; acc[5] += f.y;
          f = unpack_bf16x2(v.w); acc[6] += f.x; acc[7] += f.y;
        }
        if (r.use_scale) {
#pragma unroll
          for (int k = 0; k < 8; ++k) acc[k] *= r.scale;
        }
        if (r.out_fp32) {
          float* o = reinterpret_cast<float*>(r.out) + (int64_t)row * r.ldo + col;
          *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
          *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
        } else {
          uint4 o;
          o.x = pack_bf16x2(acc[0], acc[1]);
          o.y = pack_bf16x2(acc[2], acc[3]);
          o.z = pack_bf16x2(acc[4], acc[5]);
          o.w = pack_bf16x2(acc[6], acc[7]);
          *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(r.out) + (int64_t)row * r.ldo + col) = o;
        }
      }
    }
    __syncthreads();
  }
  // Counters are zeroed for the launch after next (same bank) by the CTA that leaves last; nobody can
  // add to this bank again before this rank publishes DONE for this collective.
  __shared__ uint32_t s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t* cnt = c.flags[c.rank] + F_LOCAL + 1;
    uint32_t old = atom_add_acqrel_gpu(cnt, 1u);
    s_last = (old == gridDim.x - 1);
    if (s_last) *cnt = 0;
  }
  __syncthreads();
  if (s_last) {
    for (int i = threadIdx.x; i < blocks; i += blockDim.x) counters[i] = 0;
    __threadfence();
  }
  exit_done(c, seq, false);
}

static_assert(kPairSmemBytes == kSmemBytes, "both tile loops use the same shared-memory budget");

// MOODIST_FUSED_PAIR=0 keeps the fused kernels on the one-SM tile loop
bool fused_pair_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("MOODIST_FUSED_PAIR");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v != 0;
}

// launch as clusters of two CTAs (pair == true) or plainly
template <typename K, typename... Args>
int launch_maybe_clustered(K kern, bool pair, int grid, int threads, cudaStream_t s, Args... args) {
  if (!pair) {
    kern<<<grid, threads, kSmemBytes, s>>>(args...);
    return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
  }
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
  cfg.stream = s;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, args...) == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

template <typename K>
int configure(K kern) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) == cudaSuccess ? MB_OK
                                                                                                             : MB_ERR_LAUNCH;
}

}  // namespace fused
}  // namespace mb

using namespace mb::fused;

// C[M,N] = gather(A)[M,K] · B^T (gather_on_b = 0; A shard = [M/world, K]) or
// C[M,N] = A[M,K] · gather(B)[N,K]^T (gather_on_b = 1; B shard = [N/world, K]). bf16, K-major shards.
// The gathered operand lands in this rank's staging half; `gathered_out` (optional, device pointer
// to the caller's [rows, K] buffer) receives nothing here: callers that need the gathered operand again
// (backward) read it from the staging area through mb_stage_pointer while the next collective has not run.
extern "C" int mb_ag_gemm(const mb_comm_t* c, uint32_t seq, const void* shard, const void* other, void* C, int M, int N,
                          int K, int64_t ld_other, int64_t ldc, int gather_on_b, int other_mn_major, int out_fp32,
                          int epilogue, int comm_ctas, void* stream) {
  const int world = c->world;
  const int full_rows = gather_on_b ? N : M;
  // CTA pairs walk 256-row tiles of the gathered operand: every shard must be a whole number of them
  const bool pair = fused_pair_enabled() && full_rows % (world * kPairBM) == 0 && M >= kPairBM;
  const int ext = pair ? kPairBM : (gather_on_b ? BN : BM);
  if (other_mn_major && gather_on_b == 0) {
    // B may be MN-major ([K, N]); a gathered A is always K-major
  } else if (other_mn_major) {
    return MB_ERR_ARG;  // gathered B with MN-major A is not wired up
  }
  if (full_rows % (world * ext) != 0 || K % 8 != 0 || N % 8 != 0) return MB_ERR_ARG;
  const int shard_rows = full_rows / world;
  const uint64_t row_bytes = (uint64_t)K * 2;
  if ((uint64_t)full_rows * row_bytes > c->staging_bytes / 2) return MB_ERR_TOO_BIG;
  if (comm_ctas <= 0) comm_ctas = kMaxSubs;  // sub-chunks of the shard = CTAs whose copy warps push one each
  if (comm_ctas > kMaxSubs) comm_ctas = kMaxSubs;
  // rows per arrival word: as fine as the 32 words per shard allow (a tile load waits for every word its rows
  // touch), so that many CTAs' copy warps share the pushing
  int sub_rows = ((shard_rows + comm_ctas - 1) / comm_ctas + 7) / 8 * 8;
  int subs = (shard_rows + sub_rows - 1) / sub_rows;
  int gemm_ctas = sm_count();
  if (pair) gemm_ctas &= ~1;
  if (gemm_ctas < subs) return MB_ERR_ARG;  // every sub-chunk needs a CTA to push it

  const uint8_t* stage = reinterpret_cast<const uint8_t*>(c->stage[c->rank]) + (uint64_t)(seq & 1) * (c->staging_bytes >> 1);
  Params p{};
  CUtensorMap ta, tb;
  int rc;
  if (!gather_on_b) {
    rc = make_tmap_bf16(&ta, stage, M, K, K, BM);
    if (rc) return rc;
    rc = other_mn_major ? make_tmap_bf16(&tb, other, K, N, ld_other, 64)
                        : make_tmap_bf16(&tb, other, N, K, ld_other, pair ? BN / 2 : BN);
  } else {
    rc = make_tmap_bf16(&ta, other, M, K, ld_other, BM);
    if (rc) return rc;
    rc = make_tmap_bf16(&tb, stage, N, K, K, pair ? BN / 2 : BN);
  }
  if (rc) return rc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.C = C;
  p.ldc = ldc;
  p.tiles_m = pair ? (M + kPairBM - 1) / kPairBM : (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.group_m = 8;
  p.epilogue = epilogue;
  p.status = c->status;
  p.wait_ns = c->wait_ns;
  p.num_gemm_ctas = gemm_ctas;
  p.cta_base = 0;
  p.ready = c->flags[c->rank] + F_CHUNK;
  p.epoch = seq;
  p.shard_rows = shard_rows;
  p.sub_rows = sub_rows;
  p.subs_per_shard = kMaxSubs;  // flag index = shard * kMaxSubs + sub
  p.gather_on_b = gather_on_b;
  p.first_shard = c->rank;
  p.num_shards = world;
  GatherArgs g{shard, row_bytes, shard_rows, sub_rows, subs};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = gemm_ctas;  // persistent: all of them stay for the whole kernel, whatever the tile count
#define LAUNCH_AG(BMN, OT, PAIR)                                                    \
  {                                                                                \
    auto kern = ag_gemm_kernel<BMN, OT, PAIR>;                                     \
    static bool cfg = false;                                                       \
    if (!cfg) {                                                                    \
      if (configure(kern)) return MB_ERR_LAUNCH;                                   \
      cfg = true;                                                                  \
    }                                                                              \
    return launch_maybe_clustered(kern, PAIR, grid, kAgThreads, s, p, ta, tb, *c, seq, g); \
  }
#define LAUNCH_AG2(BMN, OT) \
  if (pair) LAUNCH_AG(BMN, OT, true) else LAUNCH_AG(BMN, OT, false)
  if (other_mn_major) {
    if (out_fp32) LAUNCH_AG2(true, float) else LAUNCH_AG2(true, __nv_bfloat16)
  } else {
    if (out_fp32) LAUNCH_AG2(false, float) else LAUNCH_AG2(false, __nv_bfloat16)
  }
#undef LAUNCH_AG2
#undef LAUNCH_AG
}

// Address of this rank's staging half for collective `seq` (where mb_ag_gemm left the gathered operand).
extern "C" void* mb_stage_pointer(const mb_comm_t* c, uint32_t seq) {
  return reinterpret_cast<uint8_t*>(c->stage[c->rank]) + (uint64_t)(seq & 1) * (c->staging_bytes >> 1);
}

// out[M/world, N] = scale * sum over ranks of (A · B^T)[this rank's rows]. A [M,K] and B ([N,K], or [K,N]
// with b_mn_major) are this rank's operands (K = the locally held slice of the reduction dimension).
extern "C" int mb_gemm_rs(const mb_comm_t* c, uint32_t seq, const void* A, const void* B, void* out, int M, int N, int K,
                          int64_t lda, int64_t ldb, int64_t ldo, int b_mn_major, int out_fp32, float scale,
                          int use_scale, void* stream) {
  const int world = c->world;
  if (M % (world * BM) != 0 || N % 8 != 0 || K % 8 != 0) return MB_ERR_ARG;
  const int rows = M / world;
  if (rows / BM > 128) return MB_ERR_TOO_BIG;
  // On 8 GPUs the pair loop made this kernel slower (1.16 ms against 1.04 ms for the tensor-parallel MLP shape:
  // the MMA issuer waits for the remote-store epilogues of both CTAs before it may reuse an accumulator), on 2
  // GPUs faster (3.6 against 4.2 ms); it is opt-in: MOODIST_FUSED_PAIR_RS=1.
  static const bool rs_pair = [] {
    const char* e = getenv("MOODIST_FUSED_PAIR_RS");
    return e && e[0] == '1';
  }();
  const bool pair = rs_pair && fused_pair_enabled() && rows % kPairBM == 0;
  const uint64_t slot_bytes = (uint64_t)rows * N * 2;
  if (slot_bytes * world > c->staging_bytes / 2) return MB_ERR_TOO_BIG;
  Params p{};
  CUtensorMap ta, tb;
  int rc = make_tmap_bf16(&ta, A, M, K, lda, BM);
  if (rc) return rc;
  rc = b_mn_major ? make_tmap_bf16(&tb, B, K, N, ldb, 64) : make_tmap_bf16(&tb, B, N, K, ldb, pair ? BN / 2 : BN);
  if (rc) return rc;
  p.M = M;
  p.N = N;
  p.K = K;
  p.C = nullptr;
  p.ldc = N;
  p.tiles_m = pair ? M / kPairBM : M / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.group_m = 8;
  p.status = c->status;
  p.wait_ns = c->wait_ns;
  p.first_shard = c->rank;
  p.num_shards = world;
  p.scatter_rows = rows;
  const int bank = seq & 1;
  for (int r = 0; r < world; ++r) {
    uint8_t* st = reinterpret_cast<uint8_t*>(c->stage[r]) + (uint64_t)bank * (c->staging_bytes >> 1);
    p.scatter_dst[r] = st + (uint64_t)c->rank * slot_bytes;
    p.scatter_cnt[r] = c->flags[r] + F_RSCNT + bank * 128;
  }
  int tiles = p.tiles_m * p.tiles_n;
  int grid;
  if (pair) {
    int clusters = sm_count() / 2;
    grid = 2 * (tiles < clusters ? tiles : clusters);
  } else {
    grid = tiles < sm_count() ? tiles : sm_count();
  }
  p.num_gemm_ctas = grid;
  // arrivals per 128-row block: one per epilogue warp (4) per column tile per source rank, in both tile loops
  ReduceArgs r{out, ldo, out_fp32, scale, use_scale, bank, (uint32_t)(4 * p.tiles_n * world)};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define LAUNCH_RS(BMN, PAIR)                                                   \
  {                                                                            \
    auto kern = gemm_rs_kernel<BMN, PAIR>;                                     \
    static bool cfg = false;                                                   \
    if (!cfg) {                                                                \
      if (configure(kern)) return MB_ERR_LAUNCH;                               \
      cfg = true;                                                              \
    }                                                                          \
    return launch_maybe_clustered(kern, PAIR, grid, kNumThreads, s, p, ta, tb, *c, seq, r); \
  }
  if (b_mn_major) {
    if (pair) LAUNCH_RS(true, true) else LAUNCH_RS(true, false)
  } else {
    if (pair) LAUNCH_RS(false, true) else LAUNCH_RS(false, false)
  }
#undef LAUNCH_RS
}
