// mb_strided_copy_noalloc: strided 2-D copies with the piece table in a static device array, for
// callers that must not allocate (see no_alloc.h for who they are and the rules).
#include "no_alloc.h"

#include <cuda_runtime.h>

#include <atomic>

#include "coll.cuh"

namespace {

// The scratch the regular entry point gets from its caller: one table of copy pieces.
// Fixed capacity; held by every GPU that loads the library until the process exits.
static __device__ __align__(256) unsigned char g_piece_table[MB_NOALLOC_MAX_PIECES * sizeof(mb_piece_t)];

constexpr int kThreads = 512;

// Same copy logic as the one-rank path of gather_scatter_kernel: contiguous pieces are split over the
// grid by bytes, strided ones by rows (one warp per row).
__global__ void __launch_bounds__(kThreads, 1) strided_copy_kernel(const mb_piece_t* pieces, int num_pieces) {
  using namespace mb;
  using namespace mb::coll;
  const int b = blockIdx.x, G = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int i = 0; i < num_pieces; ++i) {
    mb_piece_t pc = pieces[i];
    const uint8_t* sbase = reinterpret_cast<const uint8_t*>(pc.src_local);
    uint8_t* dbase = reinterpret_cast<uint8_t*>(pc.dst);
    if (pc.rows == 1 || (pc.src_pitch == pc.row_bytes && pc.dst_pitch == pc.row_bytes)) {
      size_t begin, len;
      slice_of((size_t)pc.rows * pc.row_bytes, G, b, begin, len);
      cta_copy(dbase + begin, sbase + begin, len);
    } else {
      bool vec = ((pc.row_bytes | pc.src_pitch | pc.dst_pitch | (uintptr_t)sbase | (uintptr_t)dbase) & 15) == 0;
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

// Device address of the table, looked up once per device with that device current. In host code the
// array's name is only a handle for the runtime, never something to hand to a kernel.
mb_piece_t* table_address(int device) {
  static std::atomic<void*> addr[64];  // zero-initialised; concurrent first calls store the same address
  if (device < 0 || device >= 64) return nullptr;
  void* p = addr[device].load(std::memory_order_acquire);
  if (!p) {
    if (cudaGetSymbolAddress(&p, g_piece_table) != cudaSuccess || !p) {
      cudaGetLastError();
      return nullptr;
    }
    addr[device].store(p, std::memory_order_release);
  }
  return static_cast<mb_piece_t*>(p);
}

}  // namespace

extern "C" int mb_strided_copy_noalloc(const mb_piece_t* pieces, int num_pieces, void* stream) {
  if (num_pieces < 0 || (num_pieces > 0 && !pieces)) return MB_ERR_ARG;
  if (num_pieces > MB_NOALLOC_MAX_PIECES) return MB_ERR_TOO_BIG;
  if (num_pieces == 0) return MB_OK;
  size_t biggest = 1;
  for (int i = 0; i < num_pieces; ++i) {
    if (!pieces[i].src_local || !pieces[i].dst) return MB_ERR_ARG;
    size_t b = (size_t)pieces[i].rows * pieces[i].row_bytes;
    if (b > biggest) biggest = b;
  }
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess) return MB_ERR_DRIVER;
  mb_piece_t* table = table_address(device);
  if (!table) return MB_ERR_DRIVER;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // the whole table is rewritten for every call: nothing of the previous call's contents is relied on
  if (cudaMemcpyAsync(table, pieces, (size_t)num_pieces * sizeof(mb_piece_t), cudaMemcpyHostToDevice, s) != cudaSuccess)
    return MB_ERR_LAUNCH;
  size_t g = (biggest + 32767) / 32768;
  int grid = (int)(g < 1 ? 1 : (g > 64 ? 64 : g));
  strided_copy_kernel<<<grid, kThreads, 0, s>>>(table, num_pieces);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}
