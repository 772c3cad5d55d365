// NVLS variants of the collectives: the NVSwitch does the replication (multimem.st) and the reduction
// (multimem.ld_reduce, fp32 accumulation inside the switch), so every byte crosses each link once.
// They work on the group's staging areas through the multicast alias that SymmHeap::attach_group binds
// (cuMulticastCreate / AddDevice / BindMem); the data path of each op is
//   all-reduce     : stage input -> ld_reduce own chunk through the switch -> scale -> multimem.st the result
//                    to every rank -> copy out
//   reduce-scatter : stage input -> ld_reduce own chunk -> scale / cast -> out
//   all-gather     : multimem.st own shard to every rank's staging -> copy out
// The reference has no NVLS path; P2P kernels in collectives.cu are the fallback wherever a
// multicast object cannot be created.
#include <cuda_runtime.h>

#include "coll.cuh"

namespace mb {
namespace coll {

constexpr int kNvlsThreads = 512;

template <typename T>
struct Mc;
template <>
struct Mc<__nv_bfloat16> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) { return multimem_ld_reduce_bf16x8(p); }
};
template <>
struct Mc<float> {
  static __device__ __forceinline__ uint4 ld_reduce(const void* p) { return multimem_ld_reduce_f32x4(p); }
};

__device__ __forceinline__ uint8_t* mc_stage_ptr(const mb_comm_t& c, uint32_t seq) {
  return reinterpret_cast<uint8_t*>(c.mc_stage) + (uint64_t)(seq & 1) * (c.staging_bytes >> 1);
}

template <typename T>
__device__ __forceinline__ uint4 scale_vec(uint4 v, float scale);
template <>
__device__ __forceinline__ uint4 scale_vec<float>(uint4 v, float s) {
  v.x = __float_as_uint(__uint_as_float(v.x) * s);
  v.y = __float_as_uint(__uint_as_float(v.y) * s);
  v.z = __float_as_uint(__uint_as_float(v.z) * s);
  v.w = __float_as_uint(__uint_as_float(v.w) * s);
  return v;
}
template <>
__device__ __forceinline__ uint4 scale_vec<__nv_bfloat16>(uint4 v, float s) {
  float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y), c = unpack_bf16x2(v.z), d = unpack_bf16x2(v.w);
  v.x = pack_bf16x2(a.x * s, a.y * s);
  v.y = pack_bf16x2(b.x * s, b.y * s);
  v.z = pack_bf16x2(c.x * s, c.y * s);
  v.w = pack_bf16x2(d.x * s, d.y * s);
  return v;
}

// wait until CTA b of every peer has published `seq` in the given bank
__device__ __forceinline__ bool wait_all_ready(const mb_comm_t& c, uint32_t seq, int b, int bank) {
  bool ok = true;
  for (int i = 1; i < c.world; ++i) ok = wait_ready_warp(c, seq, (c.rank + i) % c.world, b, bank) && ok;
  return ok;
}

// count elements, chunk = elements per rank (multiple of 64); region A [world*chunk] inputs, region B results
template <typename T>
__global__ void MB_COLL_BOUNDS
    all_reduce_nvls_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq, const void* in, void* out, size_t count,
                           size_t chunk, float scale, int use_scale) {
  constexpr int N = 16 / sizeof(T);
  const int b = blockIdx.x, G = gridDim.x;
  entry_wait(c, seq);
  const T* x = reinterpret_cast<const T*>(in);
  T* y = reinterpret_cast<T*>(out);
  T* mine = reinterpret_cast<T*>(stage_ptr(c, c.rank, seq));
  auto chunk_len = [&](int r) -> size_t {
    size_t s = (size_t)r * chunk;
    return s >= count ? 0 : (count - s < chunk ? count - s : chunk);
  };
  // stage slice b of every chunk (zero-fill the padding so the switch sums zeros there)
  for (int r = 0; r < c.world; ++r) {
    size_t begin, len;
    slice_of(chunk, G, b, begin, len);
    size_t valid = chunk_len(r) > begin ? min(len, chunk_len(r) - begin) : 0;
    cta_copy(mine + (size_t)r * chunk + begin, x + (size_t)r * chunk + begin, valid * sizeof(T));
    for (size_t i = valid + threadIdx.x; i < len; i += blockDim.x) mine[(size_t)r * chunk + begin + i] = T(0.f);
  }
  signal_ready(c, seq, b, 0, -1);
  bool ok = wait_all_ready(c, seq, b, 0);
  // reduce my chunk through the switch, write the result into everyone's region B
  size_t begin, len;
  slice_of(chunk, G, b, begin, len);
  const uint8_t* mc = mc_stage_ptr(c, seq);
  const size_t a_off = ((size_t)c.rank * chunk + begin) * sizeof(T);
  const size_t b_off = ((size_t)(c.world + c.rank) * chunk + begin) * sizeof(T);
  if (ok) {
    for (size_t i = threadIdx.x; i < len / N; i += blockDim.x) {
      uint4 v = Mc<T>::ld_reduce(mc + a_off + i * 16);
      if (use_scale) v = scale_vec<T>(v, scale);
      multimem_st16(const_cast<uint8_t*>(mc) + b_off + i * 16, v);
    }
  }
  signal_ready(c, seq, b, 1, -1);
  ok = wait_all_ready(c, seq, b, 1) && ok;
  if (ok) {
    for (int r = 0; r < c.world; ++r) {
      size_t valid = chunk_len(r) > begin ? min(len, chunk_len(r) - begin) : 0;
      cta_copy(y + (size_t)r * chunk + begin, mine + (size_t)(c.world + r) * chunk + begin, valid * sizeof(T));
    }
  }
  exit_done(c, seq, false);
}

// out[count] = reduce over ranks of in[rank*in_stride ..]; count multiple of 64 handled by padding rules of the caller
template <typename T, typename OutT>
__global__ void MB_COLL_BOUNDS
    reduce_scatter_nvls_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq, const void* in, void* out, size_t count,
                               size_t in_stride, float scale, int use_scale) {
  constexpr int N = 16 / sizeof(T);
  const int b = blockIdx.x, G = gridDim.x;
  entry_wait(c, seq);
  const T* x = reinterpret_cast<const T*>(in);
  T* mine = reinterpret_cast<T*>(stage_ptr(c, c.rank, seq));
  size_t begin, len;
  slice_of(count, G, b, begin, len);
  for (int r = 0; r < c.world; ++r) cta_copy(mine + (size_t)r * count + begin, x + (size_t)r * in_stride + begin, len * sizeof(T));
  signal_ready(c, seq, b, 0, -1);
  bool ok = wait_all_ready(c, seq, b, 0);
  const uint8_t* mc = mc_stage_ptr(c, seq) + ((size_t)c.rank * count + begin) * sizeof(T);
  OutT* o = reinterpret_cast<OutT*>(out) + begin;
  // the staged chunks are 16-byte aligned by construction; the caller's output need not be
  const bool out_vec = ((uintptr_t)o & 15) == 0;
  if (ok) {
    size_t nv = len / N;
    for (size_t i = threadIdx.x; i < nv; i += blockDim.x) {
      uint4 v = Mc<T>::ld_reduce(mc + i * 16);
      if (use_scale) v = scale_vec<T>(v, scale);
      if (!out_vec) {
        Vec<T> e;
        e.u = v;
#pragma unroll
        for (int k = 0; k < N; ++k) o[i * N + k] = from_acc<OutT, float>(to_acc<float, T>(e.e[k]));
      } else if constexpr (sizeof(T) == sizeof(OutT)) {
        st_stream16(o + i * N, v);
      } else if constexpr (sizeof(T) == 2) {  // bf16 in, fp32 out
        float2 p0 = unpack_bf16x2(v.x), p1 = unpack_bf16x2(v.y), p2 = unpack_bf16x2(v.z), p3 = unpack_bf16x2(v.w);
        st_stream16(o + i * N, make_uint4(__float_as_uint(p0.x), __float_as_uint(p0.y), __float_as_uint(p1.x), __float_as_uint(p1.y)));
        st_stream16(o + i * N + 4, make_uint4(__float_as_uint(p2.x), __float_as_uint(p2.y), __float_as_uint(p3.x), __float_as_uint(p3.y)));
      } else {  // fp32 in, bf16 out
        uint2 w;
        w.x = pack_bf16x2(__uint_as_float(v.x), __uint_as_float(v.y));
        w.y = pack_bf16x2(__uint_as_float(v.z), __uint_as_float(v.w));
        *reinterpret_cast<uint2*>(o + i * N) = w;
      }
    }
    // ragged tail (< one vector): plain peer reads
    for (size_t i = nv * N + threadIdx.x; i < len; i += blockDim.x) {
      float acc = 0.f;
      for (int r = 0; r < c.world; ++r)
        acc += to_acc<float, T>(reinterpret_cast<const T*>(stage_ptr(c, r, seq))[(size_t)c.rank * count + begin + i]);
      if (use_scale) acc *= scale;
      o[i] = from_acc<OutT, float>(acc);
    }
  }
  exit_done(c, seq, false);
}

// bytes per rank; every rank's shard goes to all staging areas with one multimem.st stream
__global__ void MB_COLL_BOUNDS
    all_gather_nvls_kernel(const __grid_constant__ mb_comm_t c, uint32_t seq, const void* in, void* out, size_t bytes,
                           size_t out_stride) {
  const int b = blockIdx.x, G = gridDim.x;
  entry_wait(c, seq);
  size_t begin, len;
  slice_of(bytes, G, b, begin, len);
  const uint8_t* x = reinterpret_cast<const uint8_t*>(in);
  uint8_t* o = reinterpret_cast<uint8_t*>(out);
  uint8_t* mc = mc_stage_ptr(c, seq) + (size_t)c.rank * bytes + begin;
  const bool vec = ((uintptr_t)x & 15) == 0 && (bytes & 15) == 0;
  if (vec) {
    for (size_t i = threadIdx.x; i < len / 16; i += blockDim.x) multimem_st16(mc + i * 16, ld_stream16(x + begin + i * 16));
  } else {
    // unaligned source: unicast stores into each staging area
    for (int r = 0; r < c.world; ++r) cta_copy(stage_ptr(c, r, seq) + (size_t)c.rank * bytes + begin, x + begin, len);
  }
  signal_ready(c, seq, b, 0, -1);
  if ((const void*)(o + (size_t)c.rank * out_stride) != in) cta_copy(o + (size_t)c.rank * out_stride + begin, x + begin, len);
  const uint8_t* mine = stage_ptr(c, c.rank, seq);
  for (int i = 1; i < c.world; ++i) {
    int p = (c.rank + i) % c.world;
    if (wait_ready_warp(c, seq, p, b, 0)) cta_copy(o + (size_t)p * out_stride + begin, mine + (size_t)p * bytes + begin, len);
  }
  exit_done(c, seq, false);
}

static inline int nvls_grid(const mb_comm_t* c, size_t bytes) {
  int maxc = c->max_ctas > 0 ? c->max_ctas : 64;
  if (maxc > kMaxCtas) maxc = kMaxCtas;
  size_t g = (bytes + 65535) / 65536;
  return (int)(g < 1 ? 1 : (g > (size_t)maxc ? maxc : g));
}

}  // namespace coll
}  // namespace mb

using namespace mb::coll;

extern "C" int mb_nvls_available(const mb_comm_t* c) { return c->mc_stage != nullptr && c->world > 1; }

extern "C" int mb_all_reduce_nvls(const mb_comm_t* c, uint32_t seq, const void* in, void* out, size_t count, int dtype,
                                  int op, float premul, void* stream) {
  if (!mb_nvls_available(c)) return MB_ERR_ARG;
  float scale = 1.f;
  int use_scale = 0;
  if (op == MB_AVG) {
    scale = 1.f / c->world;
    use_scale = 1;
  } else if (op == MB_PREMUL_SUM) {
    scale = premul;
    use_scale = 1;
  } else if (op != MB_SUM) {
    return MB_ERR_ARG;
  }
  size_t sz = mb_dtype_size(dtype);
  if (dtype != MB_F32 && dtype != MB_BF16) return MB_ERR_ARG;
  // no alignment demand on in / out: the kernel stages and copies out with cta_copy, which falls back to a
  // byte loop for pointers off a 16-byte boundary, and the switch only ever sees the aligned staging area
  size_t chunk = ((count + c->world - 1) / c->world + 63) & ~(size_t)63;
  if (2 * (size_t)c->world * chunk * sz > c->staging_bytes / 2) return MB_ERR_TOO_BIG;
  int grid = nvls_grid(c, chunk * sz);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == MB_F32)
    all_reduce_nvls_kernel<float><<<grid, kNvlsThreads, 0, s>>>(*c, seq, in, out, count, chunk, scale, use_scale);
  else
    all_reduce_nvls_kernel<__nv_bfloat16><<<grid, kNvlsThreads, 0, s>>>(*c, seq, in, out, count, chunk, scale, use_scale);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_reduce_scatter_nvls(const mb_comm_t* c, uint32_t seq, const void* in, void* out, size_t count,
                                      size_t in_stride, int in_dtype, int out_dtype, int op, float premul, void* stream) {
  if (!mb_nvls_available(c)) return MB_ERR_ARG;
  float scale = 1.f;
  int use_scale = 0;
  if (op == MB_AVG) {
    scale = 1.f / c->world;
    use_scale = 1;
  } else if (op == MB_PREMUL_SUM) {
    scale = premul;
    use_scale = 1;
  } else if (op != MB_SUM) {
    return MB_ERR_ARG;
  }
  size_t isz = mb_dtype_size(in_dtype);
  if ((in_dtype != MB_F32 && in_dtype != MB_BF16) || (out_dtype != MB_F32 && out_dtype != MB_BF16)) return MB_ERR_ARG;
  // every rank's staged chunk must start on a 16-byte boundary for the vector ld_reduce; the caller's own
  // pointers may sit anywhere (cta_copy and the store path handle it)
  if ((count * isz) & 15) return MB_ERR_ALIGN;
  if ((size_t)c->world * count * isz > c->staging_bytes / 2) return MB_ERR_TOO_BIG;
  int grid = nvls_grid(c, count * isz);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define RSN(IDT, ODT, IT, OT)                                                                                          \
  if (in_dtype == IDT && out_dtype == ODT) {                                                                           \
    reduce_scatter_nvls_kernel<IT, OT><<<grid, kNvlsThreads, 0, s>>>(*c, seq, in, out, count, in_stride, scale, use_scale); \
    return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;                                                  \
  }
  RSN(MB_F32, MB_F32, float, float)
  RSN(MB_BF16, MB_BF16, __nv_bfloat16, __nv_bfloat16)
  RSN(MB_BF16, MB_F32, __nv_bfloat16, float)
  RSN(MB_F32, MB_BF16, float, __nv_bfloat16)
#undef RSN
  return MB_ERR_ARG;
}

extern "C" int mb_all_gather_nvls(const mb_comm_t* c, uint32_t seq, const void* in, void* out, size_t bytes,
                                  size_t out_stride_bytes, void* stream) {
  if (!mb_nvls_available(c)) return MB_ERR_ARG;
  if ((size_t)c->world * bytes > c->staging_bytes / 2) return MB_ERR_TOO_BIG;
  int grid = nvls_grid(c, bytes);
  all_gather_nvls_kernel<<<grid, kNvlsThreads, 0, static_cast<cudaStream_t>(stream)>>>(*c, seq, in, out, bytes,
                                                                                      out_stride_bytes);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}
