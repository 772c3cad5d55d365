// Host side of the two-SM (cta_group::2) GEMM variant and the variant switch of mb_gemm_bf16.
#include "gemm_pair_tcgen05.cuh"
#include "kernels_api.h"

#include <cstdlib>

namespace mb {
namespace gemm {

int make_tmap_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
int sm_count();

template <bool kAMn, bool kBMn, typename OutT>
__global__ void __launch_bounds__(kNumThreads, 1)
    gemm_pair_kernel(const __grid_constant__ Params p, const __grid_constant__ CUtensorMap tmap_a,
                     const __grid_constant__ CUtensorMap tmap_b) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  gemm_pair_body<kAMn, kBMn, OutT>(p, &tmap_a, &tmap_b, smem_raw);
}

template <bool kAMn, bool kBMn, typename OutT>
static int launch_pair(Params& p, const CUtensorMap& ta, const CUtensorMap& tb, int tiles, cudaStream_t stream) {
  auto kern = gemm_pair_kernel<kAMn, kBMn, OutT>;
  static int max_clusters = 0;  // per instantiation
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.blockDim = dim3(kNumThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (max_clusters == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes) != cudaSuccess)
      return MB_ERR_LAUNCH;
    cfg.gridDim = dim3(sm_count() & ~1, 1, 1);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = sm_count() / 2;
    }
    max_clusters = n < sm_count() / 2 ? n : sm_count() / 2;
  }
  int clusters = tiles < max_clusters ? tiles : max_clusters;
  p.num_gemm_ctas = 2 * clusters;
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p, ta, tb);
  return e == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

// 0: decide by shape, 1: always the one-SM kernel, 2: the pair kernel whenever the shape allows it
static int g_variant = -1;

int gemm_variant() {
  if (g_variant < 0) {
    const char* e = getenv("MOODIST_GEMM_VARIANT");
    g_variant = e ? atoi(e) : 0;
    if (g_variant < 0 || g_variant > 2) g_variant = 0;
  }
  return g_variant;
}

bool want_pair(int M, int N) {
  int v = gemm_variant();
  if (v == 1) return false;
  // a pair tile is 256 rows: below that half of the pair would idle
  return M >= kPairBM && N >= 8;
}

int gemm_pair_launch(const void* A, const void* B, void* C, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc,
                     int a_mn, int b_mn, int out_fp32, int epilogue, uint32_t* status, uint64_t wait_ns,
                     cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return MB_ERR_ARG;
  if ((N % 8) || (K % 8) || (M % 8 && a_mn)) return MB_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(C) & 15) || ((ldc * (out_fp32 ? 4 : 2)) & 15)) return MB_ERR_ALIGN;
  CUtensorMap ta, tb;
  int rc = a_mn ? make_tmap_bf16(&ta, A, K, M, lda, 64) : make_tmap_bf16(&ta, A, M, K, lda, BM);
  if (rc) return rc;
  rc = b_mn ? make_tmap_bf16(&tb, B, K, N, ldb, 64) : make_tmap_bf16(&tb, B, N, K, ldb, BN / 2);
  if (rc) return rc;
  Params p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.C = C;
  p.ldc = ldc;
  p.tiles_m = (M + kPairBM - 1) / kPairBM;
  p.tiles_n = (N + BN - 1) / BN;
  p.group_m = 4;  // 4 pair tiles = 1024 rows, the raster height of the one-SM kernel
  p.epilogue = epilogue;
  p.status = status;
  p.wait_ns = wait_ns ? wait_ns : kDefaultWaitNs;
  int tiles = p.tiles_m * p.tiles_n;
  int sel = (a_mn ? 4 : 0) | (b_mn ? 2 : 0) | (out_fp32 ? 1 : 0);
  switch (sel) {
    case 0: return launch_pair<false, false, __nv_bfloat16>(p, ta, tb, tiles, stream);
    case 1: return launch_pair<false, false, float>(p, ta, tb, tiles, stream);
    case 2: return launch_pair<false, true, __nv_bfloat16>(p, ta, tb, tiles, stream);
    case 3: return launch_pair<false, true, float>(p, ta, tb, tiles, stream);
    case 4: return launch_pair<true, false, __nv_bfloat16>(p, ta, tb, tiles, stream);
    case 5: return launch_pair<true, false, float>(p, ta, tb, tiles, stream);
    case 6: return launch_pair<true, true, __nv_bfloat16>(p, ta, tb, tiles, stream);
    default: return launch_pair<true, true, float>(p, ta, tb, tiles, stream);
  }
}

}  // namespace gemm
}  // namespace mb

extern "C" void mb_gemm_set_variant(int v) { mb::gemm::g_variant = (v < 0 || v > 2) ? 0 : v; }
extern "C" int mb_gemm_get_variant(void) { return mb::gemm::gemm_variant(); }
