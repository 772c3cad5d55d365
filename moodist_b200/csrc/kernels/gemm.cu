// Host side of the tcgen05 GEMM: tensor-map construction, launch, and the exported C entry points.
#include "gemm_tcgen05.cuh"
#include "kernels_api.h"

#include <cstdio>
#include <mutex>

namespace mb {
namespace gemm {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeFn get_encode() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  });
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with row pitch `ld` elements,
// box = [box_rows, 64 columns] with the 128-byte swizzle the MMA descriptors expect.
// cuTensorMapEncodeTiled is a raw driver call and needs a current context. A thread that has only ever
// used another CUDA runtime instance (torch's autograd workers) may not have bound one for this runtime
// yet; any runtime call that initialises the device does it.
void ensure_context() {
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

int make_tmap_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeFn enc = get_encode();
  ensure_context();
  if (!enc) return MB_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return MB_ERR_ALIGN;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MB_OK : MB_ERR_DRIVER;
}

template <bool kAMn, bool kBMn, typename OutT>
__global__ void __launch_bounds__(kNumThreads, 1)
    gemm_kernel(const __grid_constant__ Params p, const __grid_constant__ CUtensorMap tmap_a,
                const __grid_constant__ CUtensorMap tmap_b) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  gemm_body<kAMn, kBMn, OutT, false, false>(p, &tmap_a, &tmap_b, smem_raw);
}

template <bool kAMn, bool kBMn, typename OutT>
static int launch(const Params& p, const CUtensorMap& ta, const CUtensorMap& tb, int grid, cudaStream_t stream) {
  auto kern = gemm_kernel<kAMn, kBMn, OutT>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
      return MB_ERR_LAUNCH;
    configured = true;
  }
  kern<<<grid, kNumThreads, kSmemBytes, stream>>>(p, ta, tb);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

int fill_params_and_maps(Params& p, CUtensorMap& ta, CUtensorMap& tb, const void* A, const void* B, void* C, int M,
                         int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int a_mn, int b_mn, int out_fp32,
                         int epilogue, uint32_t* status, uint64_t wait_ns) {
  if (M <= 0 || N <= 0 || K <= 0) return MB_ERR_ARG;
  if ((N % 8) || (K % 8) || (M % 8 && a_mn)) return MB_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || ((ldc * (out_fp32 ? 4 : 2)) & 15)) return MB_ERR_ALIGN;
  int rc;
  // K-major operand: matrix [MN, K], box 64(k) x tile rows.  MN-major: matrix [K, MN], box 64(mn) x 64(k).
  rc = a_mn ? make_tmap_bf16(&ta, A, K, M, lda, 64) : make_tmap_bf16(&ta, A, M, K, lda, BM);
  if (rc) return rc;
  rc = b_mn ? make_tmap_bf16(&tb, B, K, N, ldb, 64) : make_tmap_bf16(&tb, B, N, K, ldb, BN);
  if (rc) return rc;
  p = Params{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.C = C;
  p.ldc = ldc;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.group_m = 8;
  p.epilogue = epilogue;
  p.status = status;
  p.wait_ns = wait_ns ? wait_ns : kDefaultWaitNs;
  return MB_OK;
}

bool want_pair(int M, int N);
int gemm_pair_launch(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                     int a_mn, int b_mn, int out_fp32, int epilogue, uint32_t* status, uint64_t wait_ns,
                     cudaStream_t stream);

}  // namespace gemm
}  // namespace mb

using namespace mb::gemm;

extern "C" int mb_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb,
                            int64_t ldc, int a_mn_major, int b_mn_major, int out_fp32, int epilogue,
                            uint32_t* status, uint64_t wait_ns, void* stream) {
  if (want_pair(M, N))
    return gemm_pair_launch(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, out_fp32, epilogue, status,
                            wait_ns, static_cast<cudaStream_t>(stream));
  Params p;
  CUtensorMap ta, tb;
  int rc = fill_params_and_maps(p, ta, tb, A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, out_fp32,
                                epilogue, status, wait_ns);
  if (rc) return rc;
  int tiles = p.tiles_m * p.tiles_n;
  int grid = tiles < sm_count() ? tiles : sm_count();
  p.num_gemm_ctas = grid;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int sel = (a_mn_major ? 4 : 0) | (b_mn_major ? 2 : 0) | (out_fp32 ? 1 : 0);
  switch (sel) {
    case 0: return launch<false, false, __nv_bfloat16>(p, ta, tb, grid, s);
    case 1: return launch<false, false, float>(p, ta, tb, grid, s);
    case 2: return launch<false, true, __nv_bfloat16>(p, ta, tb, grid, s);
    case 3: return launch<false, true, float>(p, ta, tb, grid, s);
    case 4: return launch<true, false, __nv_bfloat16>(p, ta, tb, grid, s);
    case 5: return launch<true, false, float>(p, ta, tb, grid, s);
    case 6: return launch<true, true, __nv_bfloat16>(p, ta, tb, grid, s);
    default: return launch<true, true, float>(p, ta, tb, grid, s);
  }
}
