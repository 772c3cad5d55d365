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
// addresses valid on THIS device: peer[r] is the base of rank r's symmetric heap as mapped here
// (peer[rank] is the local heap), stage[r] / flags[r] are rank r's staging area and flag page mapped
// here. The staging area has two halves used alternately by consecutive collectives.
typedef struct {
  int rank;
  int world;
  void* peer[MB_MAX_RANKS];   // heap base of each rank
  void* stage[MB_MAX_RANKS];  // staging area of each rank
  uint32_t* flags[MB_MAX_RANKS];
  uint64_t staging_bytes;  // both halves together
  void* mc_stage;          // NVLS multicast alias of the staging areas, or null
  uint32_t* mc_flags;      // NVLS multicast alias of the flag pages, or null
  uint32_t* status;        // word the device can write (may be host-mapped): 0 ok, else code | peer << 16
  uint64_t wait_ns;        // cap for device-side waits
  int max_ctas;            // upper bound on CTAs a collective may occupy (0 = default)
  uint32_t tuning;         // MB_TUNE_* bits
} mb_comm_t;

#define MB_TUNE_STAGGER 1u  // all-gather: CTA b starts its pulls at peer rank-1-b instead of rank-1

#define MB_FLAG_WORDS 4096  // uint32 words per flag page; layout in coll.cuh

size_t mb_dtype_size(int dtype);

// --- GEMM ------------------------------------------------------------------------------------
// C[M,N] = A·B^T, bf16 inputs, fp32 accumulate. a_mn_major: A is given as [K,M] row-major instead of
// [M,K]; b_mn_major: B is given as [K,N] row-major instead of [N,K]. epilogue: 0 none, 1 SiLU.
int mb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                 int a_mn_major, int b_mn_major, int out_fp32, int epilogue, uint32_t* status, uint64_t wait_ns,
                 void* stream);

// Kernel choice of mb_gemm_bf16: 0 by shape (the two-SM cta_group::2 kernel from 256 rows up), 1 always the
// one-SM kernel, 2 same as 0. Initial value from MOODIST_GEMM_VARIANT.
void mb_gemm_set_variant(int v);
int mb_gemm_get_variant(void);

// --- collectives -------------------------------------------------------------------------------
// seq: per-group collective counter (starts at 1, +1 per call, identical on every rank).
// *_heap_off: byte offset of the tensor inside this rank's symmetric heap when it lives there (peers
// then read it in place and the kernel holds until they are done), or -1: the kernel stages it.
int mb_barrier(const mb_comm_t* c, uint32_t seq, void* stream);

// out[r*out_stride .. +count) = rank r's in[0..count), converted to out_dtype while staging.
int mb_all_gather(const mb_comm_t* c, uint32_t seq, const void* in, int64_t in_heap_off, void* out, size_t count,
                  size_t out_stride, int in_dtype, int out_dtype, void* stream);

// out[0..count) = op over ranks r of rank r's in[rank*in_stride .. +count), accumulated in fp32 (fp64
// for f64, int64 for integers), times 1/world for AVG or `premul` for PREMUL_SUM, converted to out_dtype.
int mb_reduce_scatter(const mb_comm_t* c, uint32_t seq, const void* in, int64_t in_heap_off, void* out, size_t count,
                      size_t in_stride, int in_dtype, int out_dtype, int op, float premul, void* stream);

// all-reduce of `count` elements, in place allowed. variant 0: one-shot (each rank receives every
// peer's vector and reduces), 1: two-shot in one launch (reduce at the owner, owner redistributes).
int mb_all_reduce(const mb_comm_t* c, uint32_t seq, const void* in, void* out, size_t count, int dtype, int op,
                  float premul, int variant, void* stream);

int mb_broadcast(const mb_comm_t* c, uint32_t seq, void* data, int64_t heap_off, size_t bytes, int root, void* stream);

// Uneven all-to-all of bytes: this rank sends send_bytes[r] from in+send_off[r] to rank r, and stores
// what rank r sends at out+recv_off[r] (recv_bytes[r] must equal r's send_bytes[rank]).
typedef struct {
  uint64_t send_off[MB_MAX_RANKS];
  uint64_t send_bytes[MB_MAX_RANKS];
  uint64_t recv_off[MB_MAX_RANKS];
  uint64_t recv_bytes[MB_MAX_RANKS];
} mb_a2a_table_t;
// out_heap_off: byte offset of `out` inside this rank's symmetric heap (peers then write into it directly),
// or -1: incoming segments pass through this rank's staging half.
int mb_all_to_all(const mb_comm_t* c, uint32_t seq, const void* in, int64_t out_heap_off, void* out,
                  const mb_a2a_table_t* table, void* stream);

// compile_op lowering. Every rank first stages its inputs (stage_in: local tensor -> offset in its
// staging half), then copies each 2-D piece from the source rank's staging area (or, for pieces whose
// source is this rank, straight from src_local) into local dst.
typedef struct {
  const void* src;
  uint64_t dst_off;
  uint64_t bytes;
} mb_stage_copy_t;
typedef struct {
  int32_t src_rank;
  uint32_t rows;
  uint64_t src_off;       // in the source rank's staging half
  const void* src_local;  // non-null when src_rank == rank: read the input tensor directly
  void* dst;
  uint64_t row_bytes;
  uint64_t src_pitch;
  uint64_t dst_pitch;
} mb_piece_t;
// stage_in / pieces are DEVICE arrays.
int mb_gather_scatter(const mb_comm_t* c, uint32_t seq, const mb_stage_copy_t* stage_in, int num_stage,
                      const mb_piece_t* pieces, int num_pieces, size_t max_bytes, void* stream);

// --- copy-engine variants: the host moves the bytes with stream-ordered DMA copies between these phases ----
// phase 0: wait until this op's staging half is free on every rank; 1: publish "my bytes are in place" and
// wait for every peer's; 2: publish "I am done reading" (what phase 0 of the op after next waits for).
int mb_ce_phase(const mb_comm_t* c, uint32_t seq, int phase, void* stream);
// out[0..count) = op(own[0..count), the world-1 peer slots of this rank's staging half for `seq`), slot p at
// element offset p*count; fp32 accumulation, AVG / PREMUL_SUM scale and dtype conversion as in mb_reduce_scatter.
int mb_reduce_local(const mb_comm_t* c, uint32_t seq, const void* own, void* out, size_t count, int in_dtype,
                    int out_dtype, int op, float premul, void* stream);

// --- point-to-point hand-over between two GPUs (Queue items, send / recv) -------------------------------
// mb_flag_set: once everything queued on `stream` so far is done, *flag = value (release, system scope).
// mb_flag_wait: hold `stream` until *flag >= value (the flag may be a peer's memory); gives up after wait_ns and
// then records `code` in *status instead of hanging.
int mb_flag_set(uint32_t* flag, uint32_t value, void* stream);
int mb_flag_wait(const uint32_t* flag, uint32_t value, uint32_t* status, uint64_t wait_ns, uint32_t code, void* stream);

// --- NVLS variants (collectives_nvls.cu); need the multicast alias (mb_nvls_available) ------------------
int mb_nvls_available(const mb_comm_t* c);
int mb_all_reduce_nvls(const mb_comm_t* c, uint32_t seq, const void* in, void* out, size_t count, int dtype, int op,
                       float premul, void* stream);
int mb_reduce_scatter_nvls(const mb_comm_t* c, uint32_t seq, const void* in, void* out, size_t count, size_t in_stride,
                           int in_dtype, int out_dtype, int op, float premul, void* stream);
int mb_all_gather_nvls(const mb_comm_t* c, uint32_t seq, const void* in, void* out, size_t bytes,
                       size_t out_stride_bytes, void* stream);

// --- fused collective GEMMs (fused_gemm.cu) -------------------------------------------------------
// C = gather(A shards) · B^T (gather_on_b 0) or C = A · gather(B shards)^T (gather_on_b 1); `shard` is this
// rank's [rows/world, K] bf16 slice, `other` the local operand. comm_ctas: copy CTAs (0 = default).
int mb_ag_gemm(const mb_comm_t* c, uint32_t seq, const void* shard, const void* other, void* C, int M, int N, int K,
               int64_t ld_other, int64_t ldc, int gather_on_b, int other_mn_major, int out_fp32, int epilogue,
               int comm_ctas, void* stream);
// Where collective `seq` staged this rank's data (the gathered operand after mb_ag_gemm).
void* mb_stage_pointer(const mb_comm_t* c, uint32_t seq);
// out[M/world, N] = scale * sum_r (A_r · B_r^T)[rows of this rank]; bf16 partials cross NVLink, fp32 sum.
int mb_gemm_rs(const mb_comm_t* c, uint32_t seq, const void* A, const void* B, void* out, int M, int N, int K,
               int64_t lda, int64_t ldb, int64_t ldo, int b_mn_major, int out_fp32, float scale, int use_scale,
               void* stream);

// local cast / scale copy (also the world == 1 path of the collectives)
int mb_copy_cast(const void* in, void* out, size_t count, int in_dtype, int out_dtype, float scale, int use_scale,
                 void* stream);

// --- training-step kernels (train_ops.cu): bf16 tensors, rows contiguous, 16-byte aligned ------------
// Rotary embedding in place on heads [0, n_heads) of x[tokens, row_stride]; pairs are (j, j + head_dim/2),
// position = row % seq, tables are fp32 [seq, head_dim/2]. inverse: rotate by the negative angle.
int mb_rope_bf16(void* x, const float* cos_tab, const float* sin_tab, int64_t tokens, int seq, int n_heads,
                 int head_dim, int64_t row_stride, int inverse, void* stream);
// out[t, j] = silu(gu[t, j]) * gu[t, F + j]; the backward fills dgu[t, 0:2F] from dout[t, 0:F].
int mb_swiglu_fwd_bf16(const void* gu, void* out, int64_t tokens, int F, int64_t gu_stride, int64_t out_stride,
                       void* stream);
int mb_swiglu_bwd_bf16(const void* gu, const void* dout, void* dgu, int64_t tokens, int F, int64_t gu_stride,
                       int64_t dout_stride, int64_t dgu_stride, void* stream);
// loss[row] = logsumexp(logits[row]) - logits[row, target]; lse[row] kept for the backward, which
// overwrites logits with (softmax - onehot) * gscale[0] * inv_count.
int mb_cross_entropy_fwd_bf16(const void* logits, const int64_t* targets, float* lse, float* loss, int64_t rows, int V,
                              int64_t stride, int64_t ignore_index, void* stream);
int mb_cross_entropy_bwd_bf16(void* logits, const int64_t* targets, const float* lse, const float* gscale,
                              float inv_count, int64_t rows, int V, int64_t stride, int64_t ignore_index, void* stream);
// RMSNorm over the last dimension (D a multiple of 8, at most mb_rmsnorm_max_dim()): y = x * rstd * w with rstd saved
// per row; the backward gives dx and dw (partial sums per CTA in `dw_partial`, mb_rmsnorm_bwd_parts(rows) x D fp32).
int mb_rmsnorm_max_dim(void);
int mb_rmsnorm_bwd_parts(int64_t rows);
int mb_rmsnorm_fwd_bf16(const void* x, const void* w, void* y, float* rstd, int64_t rows, int D, int64_t x_stride,
                        int64_t y_stride, float eps, void* stream);
int mb_rmsnorm_bwd_bf16(const void* x, const void* w, const void* dy, const float* rstd, void* dx, float* dw_partial,
                        void* dw, int64_t rows, int D, int64_t x_stride, int64_t dy_stride, int64_t dx_stride,
                        void* stream);
// AdamW (decoupled decay, bias-corrected) on n bf16 parameters with bf16 moments; grad_dtype MB_F32 or MB_BF16.
int mb_adamw_bf16(void* p, const void* g, int grad_dtype, void* m, void* v, int64_t n, float lr, float b1, float b2,
                  float eps, float wd, int step, float grad_scale, void* stream);

#ifdef __cplusplus
}
#endif
