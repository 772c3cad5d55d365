// C entry points of the sm_100a kernel library (libmoodist_b200.so). Everything here takes raw device
// pointers and a CUDA stream handle, allocates nothing unless stated, and returns one of the MB_* codes;
// failures detected on the device (a wait that ran out) are written to the caller's status word.
#pragma once

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  MB_OK = 0,
  MB_ERR_ARG = 1,     // bad size / null pointer / unsupported combination
  MB_ERR_ALIGN = 2,   // pointer or pitch not 16-byte aligned where required
  MB_ERR_DRIVER = 3,  // a driver entry point is missing or failed
  MB_ERR_LAUNCH = 4,  // the launch itself was rejected
  MB_ERR_TOO_BIG = 5, // beyond a fixed capacity (no-allocation entry points)
};

// dtype codes shared with the host library (values follow torch's ScalarType like the reference's
// DType enum, api/moodist_api.h:29-44)
enum {
  MB_U8 = 0,
  MB_I8 = 1,
  MB_I16 = 2,
  MB_I32 = 3,
  MB_I64 = 4,
  MB_F16 = 5,
  MB_F32 = 6,
  MB_F64 = 7,
  MB_BF16 = 15,
};

// reduction codes (torch ReduceOp values: SUM 0, AVG 1, PRODUCT 2, MIN 3, MAX 4, ..., PREMUL_SUM 8)
enum { MB_SUM = 0, MB_AVG = 1, MB_MIN = 3, MB_MAX = 4, MB_PREMUL_SUM = 8 };

#define MB_MAX_RANKS 8

// Everything a collective kernel needs to know about the group's symmetric memory. All pointers are
// addresses valid on THIS device: peer[r] is rank r's staging buffer mapped here (peer[rank] is the
// local one), flags[r] is rank r's flag page mapped here. mc_* are NVLS multicast mappings or null.
typedef struct {
  int rank;
  int world;
  void* peer[MB_MAX_RANKS];
  uint32_t* flags[MB_MAX_RANKS];
  void* mc_buf;         // multicast alias of the staging buffers (same offsets), or null
  uint32_t* mc_flags;   // multicast alias of the flag pages, or null
  uint32_t* status;     // local device word: 0 ok, else first failure code
  uint64_t wait_ns;     // cap for device-side waits
} mb_comm_t;

// Flag page layout (uint32 words). Each rank owns one page of MB_FLAG_WORDS words.
#define MB_FLAG_WORDS 4096
#define MB_FLAG_BARRIER 0      // [MB_MAX_RANKS] arrival words written by peers (barrier "in")
#define MB_FLAG_BARRIER2 16    // second bank for the exit barrier
#define MB_FLAG_CHUNK 64       // [..] per-chunk / per-shard arrival words for fused ops
#define MB_FLAG_LOCAL 1024     // CTA-arrival counters private to the local grid

// --- GEMM ------------------------------------------------------------------------------------
// C[M,N] = A·B^T, bf16 inputs, fp32 accumulate. a_mn_major: A is given as [K,M] row-major instead of
// [M,K]; b_mn_major: B is given as [K,N] row-major instead of [N,K]. epilogue: 0 none, 1 SiLU.
int mb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                 int a_mn_major, int b_mn_major, int out_fp32, int epilogue, uint32_t* status, uint64_t wait_ns,
                 void* stream);

// --- collectives over symmetric staging buffers ------------------------------------------------
// seq: per-group launch counter (monotone, same on every rank) used as the flag epoch.
// variant: 0 = P2P (pull), 1 = NVLS multimem.
int mb_barrier(const mb_comm_t* c, uint32_t seq, void* stream);

// out[r*count .. (r+1)*count) = rank r's in[0..count). `in` may be null: then the input is already in
// this rank's staging buffer at in_off. out is local memory; src/dst dtypes may differ (fused cast).
int mb_all_gather(const mb_comm_t* c, uint32_t seq, const void* in, size_t in_off, void* out, size_t count,
                  int in_dtype, int out_dtype, int variant, void* stream);

// out[0..count) = reduce over ranks r of (rank r's in[rank*count ..]) * scale, accumulated in fp32
// (fp64 for f64, exact for ints). `in` is copied to staging first unless null (already at in_off).
int mb_reduce_scatter(const mb_comm_t* c, uint32_t seq, const void* in, size_t in_off, void* out, size_t count,
                      int in_dtype, int out_dtype, int op, float scale, int variant, void* stream);

// in-place capable all-reduce of `count` elements. variant 0: one-shot (every rank reads all peers),
// 1: two-shot in one launch (reduce-scatter then all-gather through staging), 2: NVLS.
int mb_all_reduce(const mb_comm_t* c, uint32_t seq, const void* in, void* out, size_t count, int dtype, int op,
                  float scale, int variant, void* stream);

int mb_broadcast(const mb_comm_t* c, uint32_t seq, void* data, size_t bytes, int root, int variant, void* stream);

// Uneven all-to-all of bytes: this rank sends send_bytes[r] from in+send_off[r] to rank r, which stores
// it at out+recv_off (receiver's table). Tables live in device memory (8 entries each).
typedef struct {
  uint64_t send_off[MB_MAX_RANKS];
  uint64_t send_bytes[MB_MAX_RANKS];
  uint64_t recv_off[MB_MAX_RANKS];
  uint64_t recv_bytes[MB_MAX_RANKS];
} mb_a2a_table_t;
int mb_all_to_all(const mb_comm_t* c, uint32_t seq, const void* in, void* out, const mb_a2a_table_t* host_table,
                  void* stream);

// compile_op lowering: a list of 2-D pieces, each copied from (possibly peer) src to local dst.
typedef struct {
  const void* src;
  void* dst;
  uint32_t rows;
  uint32_t row_bytes;
  uint64_t src_pitch;
  uint64_t dst_pitch;
} mb_piece_t;
// pieces: device array. Runs entry barrier, copies, exit barrier.
int mb_gather_scatter(const mb_comm_t* c, uint32_t seq, const mb_piece_t* pieces, int num_pieces, void* stream);

// plain local helpers (also used as world==1 paths)
int mb_copy_cast(const void* in, void* out, size_t count, int in_dtype, int out_dtype, float scale, void* stream);

#ifdef __cplusplus
}
#endif
