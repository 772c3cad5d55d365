// Memory-bound kernels of the Llama training step that sit between the tcgen05 GEMMs: rotary embedding
// applied in place to the fused QKV activations, SwiGLU forward / backward, cross-entropy over a bf16
// logit matrix with the gradient written back in place, and AdamW over a flat parameter shard. Each one
// makes a single pass over its operands with 16-byte accesses, so its cost is the bytes it must touch.
// The reference library is a communication backend and has no counterpart of these.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "kernels_api.h"

#define MB_STREAM(s) reinterpret_cast<cudaStream_t>(s)

namespace {

inline int check_launch() { return cudaPeekAtLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH; }

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float* f) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ bf16x8 pack8(const float* f) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

// ---- rotary embedding -------------------------------------------------------------------------
// x: [tokens, row_stride] bf16, heads [0, n_heads) of width head_dim start at column 0. Pairs are
// (j, j + head_dim/2). One thread rotates 8 pairs. sign = -1 applies the inverse rotation (backward).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                            int64_t tokens, int seq, int n_heads, int head_dim, int64_t row_stride, float sign) {
  const int half = head_dim / 2;
  const int vec_per_head = half / 8;
  const int64_t total = tokens * n_heads * vec_per_head;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int v = (int)(i % vec_per_head);
    int64_t r = i / vec_per_head;
    int h = (int)(r % n_heads);
    int64_t t = r / n_heads;
    int pos = (int)(t % seq);
    __nv_bfloat16* p = x + t * row_stride + (int64_t)h * head_dim + v * 8;
    bf16x8 a = *reinterpret_cast<const bf16x8*>(p);
    bf16x8 b = *reinterpret_cast<const bf16x8*>(p + half);
    float fa[8], fb[8], c[8], s[8], oa[8], ob[8];
    unpack8(a, fa);
    unpack8(b, fb);
    const float4* cp = reinterpret_cast<const float4*>(cs + (int64_t)pos * half + v * 8);
    const float4* sp = reinterpret_cast<const float4*>(sn + (int64_t)pos * half + v * 8);
    *reinterpret_cast<float4*>(c) = cp[0];
    *reinterpret_cast<float4*>(c + 4) = cp[1];
    *reinterpret_cast<float4*>(s) = sp[0];
    *reinterpret_cast<float4*>(s + 4) = sp[1];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float sk = s[k] * sign;
      oa[k] = fa[k] * c[k] - fb[k] * sk;
      ob[k] = fb[k] * c[k] + fa[k] * sk;
    }
    *reinterpret_cast<bf16x8*>(p) = pack8(oa);
    *reinterpret_cast<bf16x8*>(p + half) = pack8(ob);
  }
}

// ---- SwiGLU -------------------------------------------------------------------------------------
// gu: [tokens, 2F] (gate columns [0,F), up columns [F,2F)); out[t, j] = silu(g) * u.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int64_t tokens,
                                  int F, int64_t gu_stride, int64_t out_stride) {
  const int vec = F / 8;
  const int64_t total = tokens * vec;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t t = i / vec;
    int j = (int)(i % vec) * 8;
    const __nv_bfloat16* row = gu + t * gu_stride;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const bf16x8*>(row + j), g);
    unpack8(*reinterpret_cast<const bf16x8*>(row + F + j), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
    *reinterpret_cast<bf16x8*>(out + t * out_stride + j) = pack8(o);
  }
}

// dgu[t, :F] = dout * u * d silu(g), dgu[t, F:] = dout * silu(g)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                                  __nv_bfloat16* __restrict__ dgu, int64_t tokens, int F, int64_t gu_stride,
                                  int64_t dout_stride, int64_t dgu_stride) {
  const int vec = F / 8;
  const int64_t total = tokens * vec;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t t = i / vec;
    int j = (int)(i % vec) * 8;
    const __nv_bfloat16* row = gu + t * gu_stride;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(*reinterpret_cast<const bf16x8*>(row + j), g);
    unpack8(*reinterpret_cast<const bf16x8*>(row + F + j), u);
    unpack8(*reinterpret_cast<const bf16x8*>(dout + t * dout_stride + j), d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float sig = 1.f / (1.f + __expf(-g[k]));
      float sl = g[k] * sig;
      dg[k] = d[k] * u[k] * (sig + sl * (1.f - sig));
      du[k] = d[k] * sl;
    }
    __nv_bfloat16* orow = dgu + t * dgu_stride;
    *reinterpret_cast<bf16x8*>(orow + j) = pack8(dg);
    *reinterpret_cast<bf16x8*>(orow + F + j) = pack8(du);
  }
}

// ---- cross-entropy ---------------------------------------------------------------------------------
constexpr int kCeThreads = 512;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One CTA per row: online max / sum-of-exponentials over the row in one read, then
// loss[row] = lse - logit[target], lse[row] kept for the backward pass. Rows whose target is
// ignore_index get loss 0.
__global__ void ce_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                              float* __restrict__ lse, float* __restrict__ loss, int V, int64_t stride,
                              int64_t ignore_index) {
  const int64_t row = blockIdx.x;
  const __nv_bfloat16* p = logits + row * stride;
  float m = -INFINITY, s = 0.f;
  const int nvec = V / 8;
  for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(p)[i], f);
    float lm = f[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) lm = fmaxf(lm, f[k]);
    float nm = fmaxf(m, lm);
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc += __expf(f[k] - nm);
    s = s * __expf(m - nm) + acc;
    m = nm;
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += kCeThreads) {
    float f = __bfloat162float(p[i]);
    float nm = fmaxf(m, f);
    s = s * __expf(m - nm) + __expf(f - nm);
    m = nm;
  }
  __shared__ float sm[kCeThreads / 32], ss[kCeThreads / 32];
  float wm = warp_max(m);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - wm);
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) {
    sm[threadIdx.x >> 5] = wm;
    ss[threadIdx.x >> 5] = s;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    float a = threadIdx.x < kCeThreads / 32 ? sm[threadIdx.x] : -INFINITY;
    float b = threadIdx.x < kCeThreads / 32 ? ss[threadIdx.x] : 0.f;
    float gm = warp_max(a);
    b = (a == -INFINITY) ? 0.f : b * __expf(a - gm);
    b = warp_sum(b);
    if (threadIdx.x == 0) {
      float l = gm + __logf(b);
      lse[row] = l;
      int64_t t = targets[row];
      loss[row] = (t == ignore_index || t < 0 || t >= V) ? 0.f : l - __bfloat162float(p[t]);
    }
  }
}

// logits[row, j] <- (exp(logit - lse) - [j == target]) * scale[0] * inv_count   (0 for ignored rows)
__global__ void ce_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int64_t* __restrict__ targets,
                              const float* __restrict__ lse, const float* __restrict__ gscale, float inv_count, int V,
                              int64_t stride, int64_t ignore_index) {
  const int64_t row = blockIdx.x;
  __nv_bfloat16* p = logits + row * stride;
  const int64_t t = targets[row];
  const bool ignored = (t == ignore_index || t < 0 || t >= V);
  const float l = lse[row];
  const float sc = ignored ? 0.f : gscale[0] * inv_count;
  const int nvec = V / 8;
  for (int i = threadIdx.x; i < nvec; i += kCeThreads) {
    float f[8];
    unpack8(reinterpret_cast<const bf16x8*>(p)[i], f);
    int base = i * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = (__expf(f[k] - l) - ((base + k) == t ? 1.f : 0.f)) * sc;
    reinterpret_cast<bf16x8*>(p)[i] = pack8(f);
  }
  for (int i = nvec * 8 + threadIdx.x; i < V; i += kCeThreads) {
    float f = __bfloat162float(p[i]);
    p[i] = __float2bfloat16((__expf(f - l) - (i == t ? 1.f : 0.f)) * sc);
  }
}

// ---- AdamW -----------------------------------------------------------------------------------------
// Decoupled weight decay, bias correction as in torch.optim.AdamW; bf16 parameters and moments, the
// arithmetic in fp32. GradT is float (the reduce-scatter's fp32 result) or bf16 (single-GPU path).
template <typename GradT>
__device__ __forceinline__ void load_grad8(const GradT* g, int64_t i, float* f);
template <>
__device__ __forceinline__ void load_grad8<float>(const float* g, int64_t i, float* f) {
  *reinterpret_cast<float4*>(f) = reinterpret_cast<const float4*>(g + i)[0];
  *reinterpret_cast<float4*>(f + 4) = reinterpret_cast<const float4*>(g + i)[1];
}
template <>
__device__ __forceinline__ void load_grad8<__nv_bfloat16>(const __nv_bfloat16* g, int64_t i, float* f) {
  unpack8(*reinterpret_cast<const bf16x8*>(g + i), f);
}

template <typename GradT>
__global__ void adamw_kernel(__nv_bfloat16* __restrict__ p, const GradT* __restrict__ g, __nv_bfloat16* __restrict__ m,
                             __nv_bfloat16* __restrict__ v, int64_t n, float lr, float b1, float b2, float eps,
                             float wd, float inv_bc1, float inv_sqrt_bc2, float grad_scale) {
  const int64_t nvec = n / 8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    float fp[8], fg[8], fm[8], fv[8];
    unpack8(reinterpret_cast<const bf16x8*>(p)[i], fp);
    load_grad8<GradT>(g, i * 8, fg);
    unpack8(reinterpret_cast<const bf16x8*>(m)[i], fm);
    unpack8(reinterpret_cast<const bf16x8*>(v)[i], fv);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      float gr = fg[k] * grad_scale;
      fm[k] = b1 * fm[k] + (1.f - b1) * gr;
      fv[k] = b2 * fv[k] + (1.f - b2) * gr * gr;
      float denom = sqrtf(fv[k]) * inv_sqrt_bc2 + eps;
      fp[k] = fp[k] * (1.f - lr * wd) - lr * inv_bc1 * fm[k] / denom;
    }
    reinterpret_cast<bf16x8*>(p)[i] = pack8(fp);
    reinterpret_cast<bf16x8*>(m)[i] = pack8(fm);
    reinterpret_cast<bf16x8*>(v)[i] = pack8(fv);
  }
}

// ---- RMSNorm ---------------------------------------------------------------------------------------
// y = x * rsqrt(mean(x^2) + eps) * w, one CTA of 256 threads per row (forward) or per stripe of rows (backward).
// A thread owns the same 8-element column groups in every row (groups tid, tid + 256, ...; at most kMaxGroups),
// so the weight and the weight-gradient partial sums stay in registers across rows.
constexpr int kNormThreads = 256;
constexpr int kMaxGroups = 4;  // D <= 256 * 8 * 4 = 8192

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // red may still be read from the previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = lane < kNormThreads / 32 ? red[lane] : 0.f;
  return warp_sum(t);
}

template <int kG>
__global__ void __launch_bounds__(kNormThreads)
    rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                       __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int64_t rows, int D, int64_t x_stride,
                       int64_t y_stride, float eps) {
  __shared__ float red[kNormThreads / 32];
  const int groups = D / 8;
  float fw[kG][8];
#pragma unroll
  for (int g = 0; g < kG; ++g) {
    const int col = (threadIdx.x + g * kNormThreads) * 8;
    if (threadIdx.x + g * kNormThreads < groups) unpack8(*reinterpret_cast<const bf16x8*>(w + col), fw[g]);
  }
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    float fx[kG][8];
    float ss = 0.f;
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      const int col = (threadIdx.x + g * kNormThreads) * 8;
      if (threadIdx.x + g * kNormThreads < groups) {
        unpack8(*reinterpret_cast<const bf16x8*>(x + r * x_stride + col), fx[g]);
#pragma unroll
        for (int k = 0; k < 8; ++k) ss += fx[g][k] * fx[g][k];
      }
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(ss / (float)D + eps);
    if (threadIdx.x == 0) rstd[r] = rs;
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      const int col = (threadIdx.x + g * kNormThreads) * 8;
      if (threadIdx.x + g * kNormThreads < groups) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = fx[g][k] * rs * fw[g][k];
        *reinterpret_cast<bf16x8*>(y + r * y_stride + col) = pack8(o);
      }
    }
  }
}

// dx = rstd * (dy*w - xhat * mean(dy*w*xhat)),  dw_partial[cta] = sum over the CTA's rows of dy * xhat
template <int kG>
__global__ void __launch_bounds__(kNormThreads)
    rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                       const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd,
                       __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int64_t rows, int D,
                       int64_t x_stride, int64_t dy_stride, int64_t dx_stride) {
  __shared__ float red[kNormThreads / 32];
  const int groups = D / 8;
  float fw[kG][8], acc[kG][8];
#pragma unroll
  for (int g = 0; g < kG; ++g) {
    const int col = (threadIdx.x + g * kNormThreads) * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) acc[g][k] = 0.f;
    if (threadIdx.x + g * kNormThreads < groups) unpack8(*reinterpret_cast<const bf16x8*>(w + col), fw[g]);
  }
  // the next row's operands are requested before the current row's block-wide reduction, so their latency
  // hides behind it
  bf16x8 px[kG], pd[kG];
  auto fetch = [&](int64_t r) {
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      const int col = (threadIdx.x + g * kNormThreads) * 8;
      if (threadIdx.x + g * kNormThreads < groups) {
        px[g] = *reinterpret_cast<const bf16x8*>(x + r * x_stride + col);
        pd[g] = *reinterpret_cast<const bf16x8*>(dy + r * dy_stride + col);
      }
    }
  };
  if ((int64_t)blockIdx.x < rows) fetch(blockIdx.x);
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const float rs = rstd[r];
    float xh[kG][8], gw[kG][8];
    float dot = 0.f;
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      if (threadIdx.x + g * kNormThreads < groups) {
        float fx[8], fd[8];
        unpack8(px[g], fx);
        unpack8(pd[g], fd);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xh[g][k] = fx[k] * rs;
          gw[g][k] = fd[k] * fw[g][k];
          dot += gw[g][k] * xh[g][k];
          acc[g][k] += fd[k] * xh[g][k];
        }
      }
    }
    if (r + gridDim.x < rows) fetch(r + gridDim.x);
    dot = block_sum(dot, red) / (float)D;
#pragma unroll
    for (int g = 0; g < kG; ++g) {
      const int col = (threadIdx.x + g * kNormThreads) * 8;
      if (threadIdx.x + g * kNormThreads < groups) {
        float o[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = rs * (gw[g][k] - xh[g][k] * dot);
        *reinterpret_cast<bf16x8*>(dx + r * dx_stride + col) = pack8(o);
      }
    }
  }
#pragma unroll
  for (int g = 0; g < kG; ++g) {
    const int col = (threadIdx.x + g * kNormThreads) * 8;
    if (threadIdx.x + g * kNormThreads < groups) {
      float* o = dw_partial + (int64_t)blockIdx.x * D + col;
      *reinterpret_cast<float4*>(o) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
      *reinterpret_cast<float4*>(o + 4) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
    }
  }
}

// dw[c] = sum over `parts` rows of dw_partial[:, c]. One CTA per 32 columns: eight warps stride over the
// rows (128-byte coalesced reads), then combine through shared memory.
__global__ void __launch_bounds__(256)
    rmsnorm_dw_kernel(const float* __restrict__ dw_partial, __nv_bfloat16* __restrict__ dw, int parts, int D) {
  __shared__ float sm[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < D) {
    for (int p = ty; p < parts; p += 8) s += dw_partial[(int64_t)p * D + c];
  }
  sm[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < D) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) t += sm[k][tx];
    dw[c] = __float2bfloat16(t);
  }
}

inline int grid_for(int64_t work_items, int threads) {
  int64_t g = (work_items + threads - 1) / threads;
  if (g < 1) g = 1;
  if (g > 148 * 16) g = 148 * 16;
  return (int)g;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace

extern "C" int mb_rope_bf16(void* x, const float* cos_tab, const float* sin_tab, int64_t tokens, int seq, int n_heads,
                            int head_dim, int64_t row_stride, int inverse, void* stream) {
  if (tokens <= 0 || n_heads <= 0) return MB_OK;
  if (head_dim % 16 || seq <= 0) return MB_ERR_ARG;
  if (!aligned16(x) || row_stride % 8 || !aligned16(cos_tab) || !aligned16(sin_tab)) return MB_ERR_ALIGN;
  int64_t work = tokens * n_heads * (head_dim / 16);
  rope_kernel<<<grid_for(work, 256), 256, 0, MB_STREAM(stream)>>>(reinterpret_cast<__nv_bfloat16*>(x), cos_tab, sin_tab,
                                                                   tokens, seq, n_heads, head_dim, row_stride,
                                                                   inverse ? -1.f : 1.f);
  return check_launch();
}

extern "C" int mb_swiglu_fwd_bf16(const void* gu, void* out, int64_t tokens, int F, int64_t gu_stride,
                                  int64_t out_stride, void* stream) {
  if (tokens <= 0 || F <= 0) return MB_OK;
  if (F % 8) return MB_ERR_ARG;
  if (!aligned16(gu) || !aligned16(out) || gu_stride % 8 || out_stride % 8) return MB_ERR_ALIGN;
  swiglu_fwd_kernel<<<grid_for(tokens * (F / 8), 256), 256, 0, MB_STREAM(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(gu), reinterpret_cast<__nv_bfloat16*>(out), tokens, F, gu_stride,
      out_stride);
  return check_launch();
}

extern "C" int mb_swiglu_bwd_bf16(const void* gu, const void* dout, void* dgu, int64_t tokens, int F, int64_t gu_stride,
                                  int64_t dout_stride, int64_t dgu_stride, void* stream) {
  if (tokens <= 0 || F <= 0) return MB_OK;
  if (F % 8) return MB_ERR_ARG;
  if (!aligned16(gu) || !aligned16(dout) || !aligned16(dgu) || gu_stride % 8 || dout_stride % 8 || dgu_stride % 8)
    return MB_ERR_ALIGN;
  swiglu_bwd_kernel<<<grid_for(tokens * (F / 8), 256), 256, 0, MB_STREAM(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(gu), reinterpret_cast<const __nv_bfloat16*>(dout),
      reinterpret_cast<__nv_bfloat16*>(dgu), tokens, F, gu_stride, dout_stride, dgu_stride);
  return check_launch();
}

extern "C" int mb_cross_entropy_fwd_bf16(const void* logits, const int64_t* targets, float* lse, float* loss,
                                         int64_t rows, int V, int64_t stride, int64_t ignore_index, void* stream) {
  if (rows <= 0) return MB_OK;
  if (V <= 0) return MB_ERR_ARG;
  if (!aligned16(logits) || stride % 8) return MB_ERR_ALIGN;
  ce_fwd_kernel<<<(unsigned)rows, kCeThreads, 0, MB_STREAM(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(logits),
                                                                      targets, lse, loss, V, stride, ignore_index);
  return check_launch();
}

extern "C" int mb_cross_entropy_bwd_bf16(void* logits, const int64_t* targets, const float* lse, const float* gscale,
                                         float inv_count, int64_t rows, int V, int64_t stride, int64_t ignore_index,
                                         void* stream) {
  if (rows <= 0) return MB_OK;
  if (V <= 0) return MB_ERR_ARG;
  if (!aligned16(logits) || stride % 8) return MB_ERR_ALIGN;
  ce_bwd_kernel<<<(unsigned)rows, kCeThreads, 0, MB_STREAM(stream)>>>(reinterpret_cast<__nv_bfloat16*>(logits), targets,
                                                                      lse, gscale, inv_count, V, stride, ignore_index);
  return check_launch();
}

extern "C" int mb_adamw_bf16(void* p, const void* g, int grad_dtype, void* m, void* v, int64_t n, float lr, float b1,
                             float b2, float eps, float wd, int step, float grad_scale, void* stream) {
  if (n <= 0) return MB_OK;
  if (n % 8 || step < 1) return MB_ERR_ARG;
  if (!aligned16(p) || !aligned16(g) || !aligned16(m) || !aligned16(v)) return MB_ERR_ALIGN;
  double bc1 = 1.0 - pow((double)b1, (double)step), bc2 = 1.0 - pow((double)b2, (double)step);
  float inv_bc1 = (float)(1.0 / bc1), inv_sqrt_bc2 = (float)(1.0 / sqrt(bc2));
  int grid = grid_for(n / 8, 256);
  if (grad_dtype == MB_F32) {
    adamw_kernel<float><<<grid, 256, 0, MB_STREAM(stream)>>>(
        reinterpret_cast<__nv_bfloat16*>(p), reinterpret_cast<const float*>(g), reinterpret_cast<__nv_bfloat16*>(m),
        reinterpret_cast<__nv_bfloat16*>(v), n, lr, b1, b2, eps, wd, inv_bc1, inv_sqrt_bc2, grad_scale);
  } else if (grad_dtype == MB_BF16) {
    adamw_kernel<__nv_bfloat16><<<grid, 256, 0, MB_STREAM(stream)>>>(
        reinterpret_cast<__nv_bfloat16*>(p), reinterpret_cast<const __nv_bfloat16*>(g),
        reinterpret_cast<__nv_bfloat16*>(m), reinterpret_cast<__nv_bfloat16*>(v), n, lr, b1, b2, eps, wd, inv_bc1,
        inv_sqrt_bc2, grad_scale);
  } else {
    return MB_ERR_ARG;
  }
  return check_launch();
}

extern "C" int mb_rmsnorm_max_dim(void) { return kNormThreads * 8 * kMaxGroups; }
extern "C" int mb_rmsnorm_bwd_parts(int64_t rows) {
  int64_t g = rows < 148 * 8 ? rows : 148 * 8;
  return (int)(g < 1 ? 1 : g);
}

extern "C" int mb_rmsnorm_fwd_bf16(const void* x, const void* w, void* y, float* rstd, int64_t rows, int D,
                                   int64_t x_stride, int64_t y_stride, float eps, void* stream) {
  if (rows <= 0) return MB_OK;
  if (D <= 0 || D % 8 || D > kNormThreads * 8 * kMaxGroups) return MB_ERR_ARG;
  if (!aligned16(x) || !aligned16(w) || !aligned16(y) || x_stride % 8 || y_stride % 8) return MB_ERR_ALIGN;
  int64_t grid = rows < (1 << 20) ? rows : (1 << 20);  // one row per CTA: every load of the row is in flight at once
  const int need = (D / 8 + kNormThreads - 1) / kNormThreads;  // column groups per thread
#define FWD(G)                                                                         \
  rmsnorm_fwd_kernel<G><<<(unsigned)grid, kNormThreads, 0, MB_STREAM(stream)>>>(       \
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w), \
      reinterpret_cast<__nv_bfloat16*>(y), rstd, rows, D, x_stride, y_stride, eps)
  if (need <= 1) FWD(1); else if (need <= 2) FWD(2); else FWD(4);
#undef FWD
  return check_launch();
}

// dw_partial: fp32 scratch of mb_rmsnorm_bwd_parts(rows) x D elements
extern "C" int mb_rmsnorm_bwd_bf16(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                                   float* dw_partial, void* dw, int64_t rows, int D, int64_t x_stride,
                                   int64_t dy_stride, int64_t dx_stride, void* stream) {
  if (rows <= 0) return MB_OK;
  if (D <= 0 || D % 8 || D > kNormThreads * 8 * kMaxGroups) return MB_ERR_ARG;
  if (!aligned16(x) || !aligned16(w) || !aligned16(dy) || !aligned16(dx) || !aligned16(dw_partial) || x_stride % 8 ||
      dy_stride % 8 || dx_stride % 8)
    return MB_ERR_ALIGN;
  const int parts = mb_rmsnorm_bwd_parts(rows);
  const int need = (D / 8 + kNormThreads - 1) / kNormThreads;
#define BWD(G)                                                                                  \
  rmsnorm_bwd_kernel<G><<<parts, kNormThreads, 0, MB_STREAM(stream)>>>(                         \
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w),     \
      reinterpret_cast<const __nv_bfloat16*>(dy), rstd, reinterpret_cast<__nv_bfloat16*>(dx), dw_partial, rows, D, \
      x_stride, dy_stride, dx_stride)
  if (need <= 1) BWD(1); else if (need <= 2) BWD(2); else BWD(4);
#undef BWD
  if (check_launch()) return MB_ERR_LAUNCH;
  rmsnorm_dw_kernel<<<(D + 31) / 32, 256, 0, MB_STREAM(stream)>>>(dw_partial, reinterpret_cast<__nv_bfloat16*>(dw),
                                                                   parts, D);
  return check_launch();
}
