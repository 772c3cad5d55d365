// Element-wise reductions for CPU tensors. Floating types of 16 bits accumulate in fp32, integers in
// their own width (wrapping like the reference's scalar loops, core/cputhread.cc:125-148); bf16 and
// f16 are supported (bf16 on CPU is fatal in the reference, core/cputhread.cc:99-107). AVG and
// PREMUL_SUM are folded into the final pass as a scale instead of a separate multiply over the output.
#pragma once

#include <type_traits>

#include <cstddef>
#include <cstdint>
#include <cstring>

namespace moodist {

enum : int { kDtU8 = 0, kDtI8 = 1, kDtI16 = 2, kDtI32 = 3, kDtI64 = 4, kDtF16 = 5, kDtF32 = 6, kDtF64 = 7, kDtBF16 = 15 };
// the values of c10d::ReduceOp; product and the bitwise three exist on the host path only
enum : int {
  kRedSum = 0, kRedAvg = 1, kRedProduct = 2, kRedMin = 3, kRedMax = 4, kRedBand = 5, kRedBor = 6, kRedBxor = 7,
  kRedPremulSum = 8
};
inline bool cpu_dtype_is_integer(int dtype) {
  return dtype == kDtU8 || dtype == kDtI8 || dtype == kDtI16 || dtype == kDtI32 || dtype == kDtI64;
}
inline bool cpu_reduce_op_supported(int op, int dtype) {
  if (op == kRedBand || op == kRedBor || op == kRedBxor) return cpu_dtype_is_integer(dtype);
  return op == kRedSum || op == kRedAvg || op == kRedProduct || op == kRedMin || op == kRedMax || op == kRedPremulSum;
}

inline size_t cpu_dtype_size(int dt) {
  switch (dt) {
    case kDtU8:
    case kDtI8: return 1;
    case kDtI16:
    case kDtF16:
    case kDtBF16: return 2;
    case kDtI32:
    case kDtF32: return 4;
    case kDtI64:
    case kDtF64: return 8;
    default: return 0;
  }
}

inline float bf16_to_float(uint16_t v) {
  uint32_t u = (uint32_t)v << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t float_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);  // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1);                                             // round to nearest even
  return (uint16_t)(u >> 16);
}
inline float f16_to_float(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000) << 16, exp = (h >> 10) & 0x1f, man = h & 0x3ff, u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while (!(man & 0x400));
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ff) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t float_to_f16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  uint32_t sign = (u >> 16) & 0x8000;
  int32_t exp = (int32_t)((u >> 23) & 0xff) - 127 + 15;
  uint32_t man = u & 0x7fffff;
  if (((u >> 23) & 0xff) == 0xff) return (uint16_t)(sign | 0x7c00 | (man ? 0x200 : 0));
  if (exp >= 31) return (uint16_t)(sign | 0x7c00);
  if (exp <= 0) {
    if (exp < -10) return (uint16_t)sign;
    man |= 0x800000;
    uint32_t shift = (uint32_t)(14 - exp);
    uint32_t half = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1), mid = 1u << (shift - 1);
    if (rem > mid || (rem == mid && (half & 1))) ++half;
    return (uint16_t)(sign | half);
  }
  uint32_t half = ((uint32_t)exp << 10) | (man >> 13);
  uint32_t rem = man & 0x1fff;
  if (rem > 0x1000 || (rem == 0x1000 && (half & 1))) ++half;
  return (uint16_t)(sign | half);
}

namespace detail {
template <typename T>
struct Traits {
  using Acc = T;
  static Acc load(const T* p) { return *p; }
  static void store(T* p, Acc v) { *p = v; }
};
struct Bf16 {};
struct F16 {};
template <>
struct Traits<Bf16> {
  using Acc = float;
  static Acc load(const uint16_t* p) { return bf16_to_float(*p); }
  static void store(uint16_t* p, Acc v) { *p = float_to_bf16(v); }
};
template <>
struct Traits<F16> {
  using Acc = float;
  static Acc load(const uint16_t* p) { return f16_to_float(*p); }
  static void store(uint16_t* p, Acc v) { *p = float_to_f16(v); }
};

// Blocked, source-outer loops with the operation hoisted out of them, so that the compiler vectorises each pass;
// a block's sources are all read before anything is stored, which keeps in-place use (out aliasing a source) valid.
template <typename Tag, typename Elem>
void reduce_typed(void* out, const void* const* srcs, int nsrc, size_t n, int op, double scale, bool use_scale) {
  using Tr = Traits<Tag>;
  using Acc = typename Tr::Acc;
  constexpr size_t kBlock = 2048;
  Elem* o = static_cast<Elem*>(out);
  Acc acc[kBlock];
  for (size_t base = 0; base < n; base += kBlock) {
    const size_t m = n - base < kBlock ? n - base : kBlock;
    const Elem* s0 = static_cast<const Elem*>(srcs[0]) + base;
    for (size_t i = 0; i < m; ++i) acc[i] = Tr::load(s0 + i);
    for (int r = 1; r < nsrc; ++r) {
      const Elem* sr = static_cast<const Elem*>(srcs[r]) + base;
      if (op == kRedMin) {
        for (size_t i = 0; i < m; ++i) {
          Acc b = Tr::load(sr + i);
          acc[i] = b < acc[i] ? b : acc[i];
        }
      } else if (op == kRedMax) {
        for (size_t i = 0; i < m; ++i) {
          Acc b = Tr::load(sr + i);
          acc[i] = b > acc[i] ? b : acc[i];
        }
      } else if (op == kRedProduct) {
        for (size_t i = 0; i < m; ++i) acc[i] = (Acc)(acc[i] * Tr::load(sr + i));
      } else if (op == kRedBand || op == kRedBor || op == kRedBxor) {
        if constexpr (std::is_integral_v<Acc>) {
          if (op == kRedBand)
            for (size_t i = 0; i < m; ++i) acc[i] = (Acc)(acc[i] & Tr::load(sr + i));
          else if (op == kRedBor)
            for (size_t i = 0; i < m; ++i) acc[i] = (Acc)(acc[i] | Tr::load(sr + i));
          else
            for (size_t i = 0; i < m; ++i) acc[i] = (Acc)(acc[i] ^ Tr::load(sr + i));
        }
      } else {
        for (size_t i = 0; i < m; ++i) acc[i] = (Acc)(acc[i] + Tr::load(sr + i));
      }
    }
    if (use_scale) {
      if constexpr (std::is_floating_point_v<Acc>) {
        const Acc sc = (Acc)scale;
        for (size_t i = 0; i < m; ++i) acc[i] *= sc;
      } else {
        for (size_t i = 0; i < m; ++i) acc[i] = (Acc)(acc[i] * scale);
      }
    }
    for (size_t i = 0; i < m; ++i) Tr::store(o + base + i, acc[i]);
  }
}
}  // namespace detail

// out[i] = op_r(srcs[r][i]) (* scale). Sources are combined in the order given.
inline bool cpu_reduce(void* out, const void* const* srcs, int nsrc, size_t n, int dtype, int op, double scale,
                       bool use_scale) {
  using namespace detail;
  switch (dtype) {
    case kDtF32: reduce_typed<float, float>(out, srcs, nsrc, n, op, scale, use_scale); return true;
    case kDtF64: reduce_typed<double, double>(out, srcs, nsrc, n, op, scale, use_scale); return true;
    case kDtI32: reduce_typed<int32_t, int32_t>(out, srcs, nsrc, n, op, scale, use_scale); return true;
    case kDtI64: reduce_typed<int64_t, int64_t>(out, srcs, nsrc, n, op, scale, use_scale); return true;
    case kDtI16: reduce_typed<int16_t, int16_t>(out, srcs, nsrc, n, op, scale, use_scale); return true;
    case kDtI8: reduce_typed<int8_t, int8_t>(out, srcs, nsrc, n, op, scale, use_scale); return true;
    case kDtU8: reduce_typed<uint8_t, uint8_t>(out, srcs, nsrc, n, op, scale, use_scale); return true;
    case kDtBF16: reduce_typed<Bf16, uint16_t>(out, srcs, nsrc, n, op, scale, use_scale); return true;
    case kDtF16: reduce_typed<F16, uint16_t>(out, srcs, nsrc, n, op, scale, use_scale); return true;
    default: return false;
  }
}

}  // namespace moodist
