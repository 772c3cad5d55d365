// An entry point for callers that are not allowed to allocate device memory.
//
// This has no counterpart in the reference library.
//
// Who needs it: code that runs inside someone else's memory budget or critical section — a plugin
// loaded into an inference server whose device memory is fully pre-planned, a signal/health handler,
// a teardown or out-of-memory recovery path — cannot call cudaMalloc (it may fail, block on other
// streams, or simply be forbidden by the host application's rules). The regular strided-copy entry point, mb_gather_scatter,
// needs its table of copy pieces in device memory that somebody has to allocate. This variant keeps that
// table in a fixed array compiled into the library instead.
//
//   mb_strided_copy_noalloc(pieces, n, stream)
//     Runs `n` 2-D copy pieces (mb_piece_t with src_local and dst set; src_rank / src_off are ignored)
//     on the current device: for each piece, `rows` rows of `row_bytes` bytes go from src_local to dst
//     with the given pitches. Same result as mb_gather_scatter on a one-rank group.
//
// Limits and rules:
//   * at most MB_NOALLOC_MAX_PIECES pieces per call; more is rejected with MB_ERR_TOO_BIG and nothing runs;
//   * the table lives in a static device array of MB_NOALLOC_MAX_PIECES * sizeof(mb_piece_t) bytes that
//     every GPU which loads this library holds until the process exits;
//   * the first call on each device looks up the array's device address (cudaGetSymbolAddress); make that
//     first call before any stream capture begins. Threads may make first calls at the same time: the
//     address is cached in an atomic, and two threads that both look it up store the same value;
//   * all calls share the one array per device and it keeps the previous call's table, so two calls whose
//     kernels could overlap on the GPU (different streams, no ordering between them) race: order them on
//     one stream or with events. The table upload itself is ordered on `stream` before the kernel;
//   * no cudaMalloc, cudaFree or other allocating call is made, here or in anything this calls. `pieces`
//     is host memory and must stay valid until the copy enqueued on `stream` has read it (pinned memory
//     makes that copy asynchronous; pageable memory is read before the call returns).
#pragma once

#include "kernels_api.h"

#ifdef __cplusplus
extern "C" {
#endif

#define MB_NOALLOC_MAX_PIECES 4096

int mb_strided_copy_noalloc(const mb_piece_t* pieces, int num_pieces, void* stream);

#ifdef __cplusplus
}
#endif
