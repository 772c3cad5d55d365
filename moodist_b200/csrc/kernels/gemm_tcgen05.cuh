// Persistent, warp-specialised bf16 GEMM for sm_100a built directly on tcgen05.mma / TMEM / TMA.
//
//   C[M,N] = A · B^T   with A given either K-major ([M,K] row-major) or MN-major ([K,M] row-major)
//                      and  B given either K-major ([N,K] row-major) or MN-major ([K,N] row-major)
//
// One CTA per SM walks output tiles of 128x256 (fp32 accumulators: 256 TMEM columns, double
// buffered = all 512 columns, so the epilogue of tile i overlaps the main loop of tile i+1).
//   warp 0      TMA producer   (one lane): 4-stage ring of {A 128x64, B 256x64} bf16 tiles, 128B swizzle
//   warp 1      MMA issuer     (one lane): 4 x tcgen05.mma 128x256x16 per stage, tcgen05.commit frees the stage
//   warps 2-5   epilogue       (128 thr) : tcgen05.ld 32 lanes x 32 columns, convert, 16-byte stores
//
// The kernel body is a template so the fused collectives can reuse it:
//   * kGatherWait: before loading a tile whose gathered-operand rows belong to shard `c`, the producer
//     waits (bounded) until ready[c] reaches the launch's epoch — the all-gather half of AG->GEMM, whose
//     copy CTAs run in the same grid (see ag_gemm.cu).
//   * kScatterOut: the epilogue writes the tile to the owner rank's staging buffer over NVLink and
//     bumps a per-shard counter there — the scatter half of GEMM->RS (see gemm_rs.cu).
// The reference library has no GEMM at all (its kernels are copy/reduce loops, core/kernels.cc:28-413);
// these ops exist because the benchmark models (FSDP / tensor-parallel blocks) consume all-gather and
// produce reduce-scatter around a GEMM.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include "ptx.cuh"

namespace mb {
namespace gemm {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int kStages = 4;
constexpr int UMMA_K = 16;
constexpr int kATileBytes = BM * BK * 2;  // 16 KiB
constexpr int kBTileBytes = BN * BK * 2;  // 32 KiB
constexpr int kStageBytes = kATileBytes + kBTileBytes;
constexpr int kNumThreads = 192;
constexpr int kTmemCols = 512;
constexpr int kAccCols = BN;  // fp32 columns per accumulator buffer
constexpr int kEpiRowBytes = 144;                  // 128-byte line + 16 bytes of padding: conflict-free 16-byte accesses
constexpr int kEpiPatchBytes = 32 * kEpiRowBytes;  // one patch per epilogue warp
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align slack*/ + 256 /*barriers*/ + 4 * kEpiPatchBytes;

enum Epilogue : int { kEpiNone = 0, kEpiSilu = 1 };

// status word values (first failure wins)
enum Status : uint32_t {
  kOk = 0,
  kTimeoutProducer = 0x101,
  kTimeoutMma = 0x102,
  kTimeoutEpilogue = 0x103,
  kTimeoutGather = 0x104,
  kTimeoutDrain = 0x105,
};

struct Params {
  int M, N, K;
  void* C;
  int64_t ldc;       // elements
  int tiles_m, tiles_n;
  int group_m;       // raster group height in tiles
  int epilogue;
  uint32_t* status;  // device word, 0 = ok
  uint64_t wait_ns;  // cap for every wait inside the kernel
  int num_gemm_ctas; // how many CTAs of the grid run the GEMM
  int cta_base;      // they are CTAs [cta_base, cta_base + num_gemm_ctas); lower ones belong to the fused wrapper

  // ---- AG->GEMM: arrival flags for the gathered operand ----
  const uint32_t* ready;  // flag words in local memory, one per (shard, sub-chunk)
  uint32_t epoch;         // a flag >= epoch means that sub-chunk has landed for this launch
  int shard_rows;         // rows of the gathered operand per rank (multiple of the tile extent)
  int sub_rows;           // rows per arrival flag (multiple of the tile extent)
  int subs_per_shard;
  int gather_on_b;        // 0: A rows (M) are gathered, 1: B rows (N) are gathered
  int first_shard;        // this rank: its shard is consumed first, then rank-1, rank-2, ... (arrival order)
  int num_shards;

  // ---- GEMM->RS: per-owner output ----
  void* scatter_dst[8];      // this rank's slot in each owner's staging buffer ([scatter_rows, ldc])
  uint32_t* scatter_cnt[8];  // arrival counters of each owner, one word per 128-row block of its shard
  int scatter_rows;          // output rows per owner (multiple of BM)
};

// Barrier over the 192 threads that run the tile loop (named barrier 1). In the plain GEMM kernels that is
// the whole CTA; the fused all-gather kernel has four more warps that move data and must not be waited for.
__device__ __forceinline__ void body_sync() { asm volatile("bar.sync 1, 192;" ::: "memory"); }

// The status word may be host-mapped memory, so no atomics: first writer (nearly) wins.
__device__ __forceinline__ void report(const Params& p, uint32_t code) {
  volatile uint32_t* s = p.status;
  if (s && *s == 0) *s = code;
}

// tile index -> (m, n) with a grouped raster so concurrently running CTAs share A and B panels in L2
__device__ __forceinline__ void tile_coords(const Params& p, int t, int& tm, int& tn) {
  int per_group = p.group_m * p.tiles_n;
  int g = t / per_group;
  int first_m = g * p.group_m;
  int gsz = min(p.group_m, p.tiles_m - first_m);
  int r = t - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

// Walk order of the fused variants.
//  gather : all tiles of one shard of the gathered operand are consecutive; shards are visited own first,
//           then in the order their pushes arrive (rank-1, rank-2, ...). flag = arrival word to wait on.
//  scatter: tiles owned by other ranks first (rank+1, rank+2, ...), this rank's own rows last, so remote
//           partial sums are on the wire while the local ones are still being computed.
template <bool kGatherWait, bool kScatterOut>
__device__ __forceinline__ void tile_map(const Params& p, int t, int& tm, int& tn, int& flag, int* nflags = nullptr) {
  flag = 0;
  if (nflags) *nflags = 1;
  if constexpr (kGatherWait) {
    const int ext = p.gather_on_b ? BN : BM;
    const int other = p.gather_on_b ? p.tiles_m : p.tiles_n;
    const int blocks = p.shard_rows / ext;
    const int per_shard = blocks * other;
    const int si = t / per_shard, within = t - si * per_shard;
    const int shard = (p.first_shard - si + 2 * p.num_shards) % p.num_shards;
    const int blk = within / other, o = within - blk * other;
    if (p.gather_on_b) {
      tn = shard * blocks + blk;
      tm = o;
    } else {
      tm = shard * blocks + blk;
      tn = o;
    }
    // the tile's rows of the gathered operand may span several arrival sub-chunks
    const int first = (blk * ext) / p.sub_rows, last = (blk * ext + ext - 1) / p.sub_rows;
    flag = shard * p.subs_per_shard + first;
    if (nflags) *nflags = last - first + 1;
  } else if constexpr (kScatterOut) {
    const int blocks = p.scatter_rows / BM;
    const int per_shard = blocks * p.tiles_n;
    const int si = t / per_shard, within = t - si * per_shard;
    const int shard = (p.first_shard + 1 + si) % p.num_shards;
    tm = shard * blocks + within / p.tiles_n;
    tn = within % p.tiles_n;
  } else {
    tile_coords(p, t, tm, tn);
  }
}

template <bool kAMn, bool kBMn, typename OutT, bool kGatherWait, bool kScatterOut>
__device__ __forceinline__ void gemm_body(const Params& p, const CUtensorMap* tmap_a, const CUtensorMap* tmap_b,
                                          uint8_t* smem_raw) {
  // ---- carve shared memory (tiles need 1024-byte alignment for the 128B swizzle) ----
  uint32_t raw = smem_u32(smem_raw);
  uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  uint8_t* tiles = smem_raw + pad;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + kStages * kStageBytes);
  uint64_t* full = bars;                   // [kStages]
  uint64_t* empty = bars + kStages;        // [kStages]
  uint64_t* acc_full = bars + 2 * kStages; // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;
  uint8_t* epi_patch = reinterpret_cast<uint8_t*>(bars) + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;
  const int cta = blockIdx.x - p.cta_base;
  const int stride = p.num_gemm_ctas;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(tmap_a);
    tma_prefetch_desc(tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  body_sync();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // =============================== TMA producer ===============================
    if (lane == 0) {
      uint32_t it = 0;  // k-blocks issued so far
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += stride) {
        int tm, tn, flag, nflags;
        tile_map<kGatherWait, kScatterOut>(p, t, tm, tn, flag, &nflags);
        if constexpr (kGatherWait) {
          for (int f = 0; f < nflags && ok; ++f) {
            if (!wait_geq_sys(p.ready + flag + f, p.epoch, p.wait_ns)) {  // written by peers: system scope
              report(p, kTimeoutGather);
              ok = false;
            }
          }
          if (!ok) break;
          fence_proxy_async_all();  // the landed rows were written by ordinary stores; TMA reads them next
        }
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          int s = it % kStages;
          uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, p.wait_ns)) {
            report(p, kTimeoutProducer);
            ok = false;
            break;
          }
          uint8_t* sa = tiles + s * kStageBytes;
          uint8_t* sb = sa + kATileBytes;
          mbar_arrive_expect_tx(&full[s], kStageBytes);
          if constexpr (!kAMn) {
            tma_load_2d(sa, tmap_a, &full[s], kb * BK, tm * BM);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * 8192, tmap_a, &full[s], tm * BM + c * 64, kb * BK);
          }
          if constexpr (!kBMn) {
            tma_load_2d(sb, tmap_b, &full[s], kb * BK, tn * BN);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * 8192, tmap_b, &full[s], tn * BN + c * 64, kb * BK);
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        // let the copies still in flight land before this CTA's shared memory is given up
        uint32_t lo = it > (uint32_t)kStages ? it - kStages : 0;
        for (uint32_t i = lo; i < it; ++i) {
          if (!mbar_wait(&full[i % kStages], (i / kStages) & 1, p.wait_ns)) report(p, kTimeoutDrain);
        }
      }
    }
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(true, kAMn, kBMn, BM, BN);
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += stride, ++local_tile) {
        uint32_t acc = local_tile & 1;
        uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1, p.wait_ns)) {
          report(p, kTimeoutMma);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        uint32_t d_tmem = tmem_base + acc * kAccCols;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          int s = it % kStages;
          uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&full[s], ph, p.wait_ns)) {
            report(p, kTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          uint32_t sa = smem_u32(tiles + s * kStageBytes);
          uint32_t sb = sa + kATileBytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 8-row groups are 1024 B apart, a K step of 16 elements is 32 B inside the swizzle row.
            // MN-major: 64-element column blocks are 8192 B apart (LBO), 8-row K groups 1024 B apart (SBO),
            //           a K step of 16 rows is 2048 B.
            uint64_t da = kAMn ? make_smem_desc(sa + k * 2048, 8192, 1024) : make_smem_desc(sa + k * 32, 0, 1024);
            uint64_t db = kBMn ? make_smem_desc(sb + k * 2048, 8192, 1024) : make_smem_desc(sb + k * 32, 0, 1024);
            tc_mma_f16(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          tc_commit(&empty[s]);  // stage reusable once these MMAs have read it
        }
        if (ok) tc_commit(&acc_full[acc]);
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // =============================== epilogue (warps 2..5) ===============================
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint32_t local_tile = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += stride, ++local_tile) {
      int tm, tn, flag;
      tile_map<kGatherWait, kScatterOut>(p, t, tm, tn, flag);
      uint32_t acc = local_tile & 1;
      uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_ph, p.wait_ns)) {
        if (lane == 0) report(p, kTimeoutEpilogue);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // Output rows of this warp: 32 consecutive rows starting at row0. Each lane owns one row in TMEM; to
      // write full 128-byte lines (instead of 32 scattered 16-byte pieces per instruction, which wastes DRAM
      // sectors locally and NVLink packets remotely) the row pieces go through a per-warp shared-memory
      // patch and leave as 4 rows x 128 bytes per store instruction.
      const int row0 = tm * BM + q * 32;
      OutT* cbase;
      if constexpr (kScatterOut) {
        const int owner = (tm * BM) / p.scatter_rows;  // M is a multiple of scatter_rows * num_shards here
        cbase = reinterpret_cast<OutT*>(p.scatter_dst[owner]) + (int64_t)(row0 - owner * p.scatter_rows) * p.ldc;
      } else {
        cbase = reinterpret_cast<OutT*>(p.C) + (int64_t)row0 * p.ldc;
      }
      uint8_t* patch = epi_patch + (warp - 2) * kEpiPatchBytes;
      const uint32_t taddr = tmem_base + acc * kAccCols + ((uint32_t)(q * 32) << 16);
      constexpr int kColsPerPass = 128 / (int)sizeof(OutT);  // columns that make one 128-byte line
      constexpr int kLdsPerPass = kColsPerPass / 32;
#pragma unroll 1
      for (int c = 0; c < BN / kColsPerPass; ++c) {
#pragma unroll
        for (int h = 0; h < kLdsPerPass; ++h) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * kColsPerPass + h * 32, r);
          tmem_ld_wait();
          if (p.epilogue == kEpiSilu) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float x = __uint_as_float(r[i]);
              r[i] = __float_as_uint(x / (1.0f + __expf(-x)));
            }
          }
          uint4* dst = reinterpret_cast<uint4*>(patch + lane * kEpiRowBytes + h * (32 * (int)sizeof(OutT)));
          if constexpr (sizeof(OutT) == 2) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(r[g * 8 + 0]), __uint_as_float(r[g * 8 + 1]));
              v.y = pack_bf16x2(__uint_as_float(r[g * 8 + 2]), __uint_as_float(r[g * 8 + 3]));
              v.z = pack_bf16x2(__uint_as_float(r[g * 8 + 4]), __uint_as_float(r[g * 8 + 5]));
              v.w = pack_bf16x2(__uint_as_float(r[g * 8 + 6]), __uint_as_float(r[g * 8 + 7]));
              dst[g] = v;
            }
          } else {
#pragma unroll
            for (int g = 0; g < 8; ++g) dst[g] = make_uint4(r[g * 4], r[g * 4 + 1], r[g * 4 + 2], r[g * 4 + 3]);
          }
        }
        __syncwarp();
        const int col = tn * BN + c * kColsPerPass + (lane & 7) * (16 / (int)sizeof(OutT));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = i * 4 + (lane >> 3);
          const uint4 v = *reinterpret_cast<const uint4*>(patch + rr * kEpiRowBytes + (lane & 7) * 16);
          if (row0 + rr < p.M && col < p.N) *reinterpret_cast<uint4*>(cbase + (int64_t)rr * p.ldc + col) = v;
        }
        __syncwarp();
      }
      // accumulator buffer may be overwritten by the MMA warp from here on
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if constexpr (kScatterOut) {
        // this warp's 32 rows of the tile are on their way: one arrival per warp on the owner's counter
        // of that 128-row block (the owner waits for 4 x tiles_n x ranks arrivals)
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const int owner = (tm * BM) / p.scatter_rows;
          const int blk = tm - owner * (p.scatter_rows / BM);
          red_add_release_sys(p.scatter_cnt[owner] + blk, 1u);
        }
      }
    }
    if (!ok && lane == 0) *abort_flag = 1;
  }

  tc_fence_before_sync();
  body_sync();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace gemm
}  // namespace mb
