// Two-SM variant of the persistent bf16 GEMM: a cluster of two CTAs computes one 256x256 output tile with
// tcgen05.mma.cta_group::2 (M = 256 split as 128 rows per CTA, N = 256).
//
// Why: with one CTA per 128x256 tile every SM pulls A (16 KiB) and the whole B tile (32 KiB) through L2
// per 64-wide K step; at full tensor throughput that is ~90 B/clk/SM, which is where the one-SM kernel
// stalls (tensor pipe ~80 % busy, the rest waiting on operand arrival). In a pair each CTA loads only its
// own 128 rows of A and HALF of the B tile (16 KiB): the tensor cores of both SMs read both halves of B
// from the two shared memories. L2->SM traffic per FLOP drops by a third and six stages fit instead of four.
//
// Roles per CTA (192 threads, same as the one-SM kernel):
//   warp 0  TMA producer: loads this CTA's A rows and B half into its OWN shared memory; the byte count
//           is signalled on the LEADER's `full` barrier (plain TMA loads of local memory, no multicast)
//   warp 1  leader only: issues the MMAs; tcgen05.commit arrives on `empty` / `acc_full` in both CTAs
//   warps 2-5  epilogue for this CTA's 128 rows (its own TMEM lanes), then arrive on the leader's `acc_empty`
// Every wait is bounded; a CTA that gives up raises the status word, and both CTAs always reach the final
// cluster barrier, after which each frees its TMEM.
#pragma once

#include "gemm_tcgen05.cuh"

namespace mb {
namespace gemm {

constexpr int kPairBM = 256;  // rows of a pair tile (128 per CTA)
constexpr int kPairStages = 6;
constexpr int kPairBHalfBytes = (BN / 2) * BK * 2;                  // 16 KiB: this CTA's half of the B tile
constexpr int kPairStageBytes = kATileBytes + kPairBHalfBytes;      // 32 KiB per CTA per stage
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 256 + 4 * kEpiPatchBytes;

enum PairStatus : uint32_t {
  kTimeoutPairProducer = 0x111,
  kTimeoutPairMma = 0x112,
  kTimeoutPairEpilogue = 0x113,
};

// Walk order of the fused variants over 256-row pair tiles (same idea as tile_map of the one-SM kernel).
// row_in_shard: first row of the tile inside its shard of the gathered operand (gather only).
template <bool kGatherWait, bool kScatterOut>
__device__ __forceinline__ void pair_tile_map(const Params& p, int t, int& tm, int& tn, int& shard, int& row_in_shard) {
  shard = 0;
  row_in_shard = 0;
  if constexpr (kGatherWait) {
    const int other = p.gather_on_b ? p.tiles_m : p.tiles_n;
    const int blocks = p.shard_rows / kPairBM;  // BN == kPairBM: both gathered extents are 256 rows per tile
    const int per_shard = blocks * other;
    const int si = t / per_shard, within = t - si * per_shard;
    shard = (p.first_shard - si + 2 * p.num_shards) % p.num_shards;
    const int blk = within / other, o = within - blk * other;
    if (p.gather_on_b) {
      tn = shard * blocks + blk;
      tm = o;
    } else {
      tm = shard * blocks + blk;
      tn = o;
    }
    row_in_shard = blk * kPairBM;
  } else if constexpr (kScatterOut) {
    const int blocks = p.scatter_rows / kPairBM;
    const int per_shard = blocks * p.tiles_n;
    const int si = t / per_shard, within = t - si * per_shard;
    shard = (p.first_shard + 1 + si) % p.num_shards;
    tm = shard * blocks + within / p.tiles_n;
    tn = within % p.tiles_n;
  } else {
    tile_coords(p, t, tm, tn);
  }
}

template <bool kAMn, bool kBMn, typename OutT, bool kGatherWait = false, bool kScatterOut = false>
__device__ __forceinline__ void gemm_pair_body(const Params& p, const CUtensorMap* tmap_a, const CUtensorMap* tmap_b,
                                               uint8_t* smem_raw) {
  uint32_t raw = smem_u32(smem_raw);
  uint32_t pad = (1024u - (raw & 1023u)) & 1023u;
  uint8_t* tiles = smem_raw + pad;
  uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + kPairStages * kPairStageBytes);
  uint64_t* full = bars;                        // [kPairStages]  used in the leader
  uint64_t* empty = bars + kPairStages;         // [kPairStages]  one per CTA
  uint64_t* acc_full = bars + 2 * kPairStages;  // [2]            one per CTA
  uint64_t* acc_empty = acc_full + 2;           // [2]            used in the leader
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;
  uint8_t* epi_patch = reinterpret_cast<uint8_t*>(bars) + 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta_rank = cluster_ctarank();  // 0 = leader
  const bool leader = cta_rank == 0;
  const int num_tiles = p.tiles_m * p.tiles_n;  // tiles_m counts 256-row pair tiles here
  const int kblocks = (p.K + BK - 1) / BK;
  const int pair = (blockIdx.x - p.cta_base) >> 1;
  const int stride = p.num_gemm_ctas >> 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kPairStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 8);  // 4 epilogue warps in each of the two CTAs
    }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(tmap_a);
    tma_prefetch_desc(tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_base_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  body_sync();
  cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // =============================== TMA producer (both CTAs) ===============================
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += stride) {
        int tm, tn, shard, row_in_shard;
        pair_tile_map<kGatherWait, kScatterOut>(p, t, tm, tn, shard, row_in_shard);
        const int row_a = tm * kPairBM + (int)cta_rank * BM;     // this CTA's 128 rows of A
        const int row_b = tn * BN + (int)cta_rank * (BN / 2);    // this CTA's 128 rows (N) of B
        if constexpr (kGatherWait) {
          // the 128 gathered rows this CTA loads may span several arrival sub-chunks
          const int r0 = row_in_shard + (int)cta_rank * BM;
          const int first = r0 / p.sub_rows, last = (r0 + BM - 1) / p.sub_rows;
          for (int f = first; f <= last && ok; ++f) {
            if (!wait_geq_sys(p.ready + shard * p.subs_per_shard + f, p.epoch, p.wait_ns)) {
              report(p, kTimeoutGather);
              ok = false;
            }
          }
          if (!ok) break;
          fence_proxy_async_all();  // the rows were written by ordinary stores; TMA reads them next
        }
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          int s = it % kPairStages;
          uint32_t ph = (it / kPairStages) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, p.wait_ns)) {
            report(p, kTimeoutPairProducer);
            ok = false;
            break;
          }
          uint8_t* sa = tiles + s * kPairStageBytes;
          uint8_t* sb = sa + kATileBytes;
          // both CTAs' bytes are expected on the leader's barrier
          if (leader) mbar_arrive_expect_tx(&full[s], 2 * kPairStageBytes);
          const uint32_t bar = map_to_cta(smem_u32(&full[s]), 0);
          if constexpr (!kAMn) {
            tma_load_2d_pair(sa, tmap_a, bar, kb * BK, row_a);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d_pair(sa + c * 8192, tmap_a, bar, row_a + c * 64, kb * BK);
          }
          if constexpr (!kBMn) {
            tma_load_2d_pair(sb, tmap_b, bar, kb * BK, row_b);
          } else {
#pragma unroll
            for (int c = 0; c < (BN / 2) / 64; ++c)
              tma_load_2d_pair(sb + c * 8192, tmap_b, bar, row_b + c * 64, kb * BK);
          }
        }
      }
      if (!ok) *abort_flag = 1;
    }
  } else if (warp == 1) {
    // =============================== MMA issuer (leader CTA only) ===============================
    if (lane == 0 && leader) {
      constexpr uint32_t idesc = make_idesc_f16(true, kAMn, kBMn, kPairBM, BN);
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += stride, ++local_tile) {
        uint32_t acc = local_tile & 1;
        uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait(&acc_empty[acc], acc_ph ^ 1, p.wait_ns)) {
          report(p, kTimeoutPairMma);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        uint32_t d_tmem = tmem_base + acc * kAccCols;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          int s = it % kPairStages;
          uint32_t ph = (it / kPairStages) & 1;
          if (!mbar_wait(&full[s], ph, p.wait_ns)) {
            report(p, kTimeoutPairMma);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          uint32_t sa = smem_u32(tiles + s * kPairStageBytes);
          uint32_t sb = sa + kATileBytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            uint64_t da = kAMn ? make_smem_desc(sa + k * 2048, 8192, 1024) : make_smem_desc(sa + k * 32, 0, 1024);
            uint64_t db = kBMn ? make_smem_desc(sb + k * 2048, 8192, 1024) : make_smem_desc(sb + k * 32, 0, 1024);
            tc_mma_f16_pair(d_tmem, da, db, idesc, (kb | k) != 0);
          }
          tc_commit_pair(&empty[s], 0x3);  // the stage is free again in both CTAs
        }
        if (ok) tc_commit_pair(&acc_full[acc], 0x3);
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // =============================== epilogue (warps 2..5 of both CTAs) ===============================
    const int q = warp & 3;
    uint32_t local_tile = 0;
    bool ok = true;
    for (int t = pair; t < num_tiles && ok; t += stride, ++local_tile) {
      int tm, tn, shard, row_in_shard;
      pair_tile_map<kGatherWait, kScatterOut>(p, t, tm, tn, shard, row_in_shard);
      uint32_t acc = local_tile & 1;
      uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!mbar_wait(&acc_full[acc], acc_ph, p.wait_ns)) {
        if (lane == 0) report(p, kTimeoutPairEpilogue);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int row0 = tm * kPairBM + (int)cta_rank * BM + q * 32;
      OutT* cbase;
      if constexpr (kScatterOut) {
        const int owner = (tm * kPairBM) / p.scatter_rows;  // scatter_rows is a multiple of 256 here
        cbase = reinterpret_cast<OutT*>(p.scatter_dst[owner]) + (int64_t)(row0 - owner * p.scatter_rows) * p.ldc;
      } else {
        cbase = reinterpret_cast<OutT*>(p.C) + (int64_t)row0 * p.ldc;
      }
      uint8_t* patch = epi_patch + (warp - 2) * kEpiPatchBytes;
      const uint32_t taddr = tmem_base + acc * kAccCols + ((uint32_t)(q * 32) << 16);
      constexpr int kColsPerPass = 128 / (int)sizeof(OutT);
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
      // both CTAs' epilogue warps release the accumulator on the leader's barrier
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[acc]), 0));
      if constexpr (kScatterOut) {
        // this warp's 32 rows are on their way: one arrival on the owner's counter of their 128-row block
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const int owner = (tm * kPairBM) / p.scatter_rows;
          const int blk = (tm * kPairBM + (int)cta_rank * BM - owner * p.scatter_rows) / BM;
          red_add_release_sys(p.scatter_cnt[owner] + blk, 1u);
        }
      }
    }
    if (!ok && lane == 0) *abort_flag = 1;
  }

  body_sync();
  if (*abort_flag) {
    // a wait ran out somewhere in this CTA: give copies that may still be in flight towards this CTA's
    // shared memory time to land before it is released
    for (int i = 0; i < 64; ++i) __nanosleep(20000);
  }
  tc_fence_before_sync();
  cluster_sync_all();  // the peer no longer reads this CTA's shared memory or signals its barriers
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

}  // namespace gemm
}  // namespace mb
