// Element types and 16-byte vector arithmetic used by every reduction in the library.
//
// Covers the reference's DataType set (include/mscclpp/gpu_data_types.hpp:82-155) and its
// SUM/MIN reductions with an optional wider accumulator (src/core/include/reduce_kernel.hpp:16-189),
// re-written around one idea: every hot loop moves 16-byte words (uint4), so each type provides
// unpack-to-fp32 / pack-from-fp32 for one 16-byte word plus a native packed fast path where the
// hardware has one (add.f32x2 on sm_100a, __hadd2/__hmin2 for 16-bit floats).
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "device/ptx.cuh"

namespace mscclpp {

enum class DataType : int {
  INT32 = 0,
  UINT32 = 1,
  FLOAT16 = 2,
  FLOAT32 = 3,
  BFLOAT16 = 4,
  FLOAT8_E4M3 = 5,   // e4m3fn (OCP), the only e4m3 flavour NVIDIA hardware implements
  FLOAT8_E5M2 = 6,
  UINT8 = 7,
  FLOAT8_E4M3B15 = 8,  // software format: e4m3 with exponent bias 15, no inf/nan
  AUTO = 255,
};

enum ReduceOp : int { SUM = 0, MIN = 1, NOP = 255 };

MSCCLPP_HOST_DEVICE_INLINE int dataTypeSize(DataType t) {
  switch (t) {
    case DataType::INT32:
    case DataType::UINT32:
    case DataType::FLOAT32:
      return 4;
    case DataType::FLOAT16:
    case DataType::BFLOAT16:
      return 2;
    default:
      return 1;
  }
}

// Tag types for the 8-bit formats (distinct C++ types so templates can dispatch on them).
struct f8e4m3 {
  uint8_t bits;
};
struct f8e5m2 {
  uint8_t bits;
};
struct f8e4m3b15 {
  uint8_t bits;
};

// ---------------------------------------------------------------- software fp8_e4m3b15 codec
// value = (-1)^s * 2^(e-15) * (1 + m/8) for e>0, (-1)^s * 2^-14 * (m/8) for e==0. No inf/nan:
// out-of-range inputs clip to the largest finite magnitude (0x7f -> 1.875 * 2^0 = 1.875).
MSCCLPP_HOST_DEVICE_INLINE float e4m3b15ToFloat(uint8_t b) {
  uint32_t s = (b >> 7) & 1u, e = (b >> 3) & 0xfu, m = b & 7u;
  float mag;
  if (e == 0) {
    mag = static_cast<float>(m) * (1.0f / 8.0f) * 6.103515625e-05f;  // 2^-14
  } else {
    union {
      uint32_t u;
      float f;
    } cvt;
    cvt.u = ((e + 127u - 15u) << 23) | (m << 20);
    mag = cvt.f;
  }
  return s ? -mag : mag;
}
MSCCLPP_HOST_DEVICE_INLINE uint8_t floatToE4m3b15(float f) {
  union {
    float f;
    uint32_t u;
  } cvt;
  cvt.f = f;
  uint32_t s = cvt.u >> 31;
  float a = f < 0 ? -f : f;
  if (!(a == a)) a = 1.875f;  // NaN clips to max
  if (a >= 1.875f) return static_cast<uint8_t>((s << 7) | 0x7f);
  // scale into the subnormal grid of 2^-17 and round to nearest even
  float scaled = a * 131072.0f;  // a / 2^-17
  if (scaled < 8.0f) {
    uint32_t m = static_cast<uint32_t>(scaled);
    float r = scaled - static_cast<float>(m);
    if (r > 0.5f || (r == 0.5f && (m & 1u))) m++;
    return static_cast<uint8_t>((s << 7) | m);  // m==8 rolls into e=1,m=0 naturally
  }
  cvt.f = a;
  uint32_t e32 = (cvt.u >> 23) & 0xffu, man = cvt.u & 0x7fffffu;
  uint32_t m = man >> 20, rest = man & 0xfffffu;
  if (rest > 0x80000u || (rest == 0x80000u && (m & 1u))) m++;
  uint32_t e = e32 - 127u + 15u;
  if (m == 8) {
    m = 0;
    e++;
  }
  if (e > 15u) return static_cast<uint8_t>((s << 7) | 0x7f);
  return static_cast<uint8_t>((s << 7) | (e << 3) | m);
}

#if defined(__CUDACC__)

// ---------------------------------------------------------------- per-type traits over one 16-byte word
template <typename T>
struct Vec16;  // kElems, toFloat(uint4, float*), fromFloat(const float*) -> uint4

template <>
struct Vec16<float> {
  static constexpr int kElems = 4;
  MSCCLPP_DEVICE_INLINE static void toFloat(uint4 v, float* f) {
    f[0] = __uint_as_float(v.x);
    f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z);
    f[3] = __uint_as_float(v.w);
  }
  MSCCLPP_DEVICE_INLINE static uint4 fromFloat(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
};

template <>
struct Vec16<__half> {
  static constexpr int kElems = 8;
  MSCCLPP_DEVICE_INLINE static void toFloat(uint4 v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
  MSCCLPP_DEVICE_INLINE static uint4 fromFloat(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int kElems = 8;
  MSCCLPP_DEVICE_INLINE static void toFloat(uint4 v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      // bf16 -> fp32 is a 16-bit shift
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  MSCCLPP_DEVICE_INLINE static uint4 fromFloat(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <>
struct Vec16<int32_t> {
  static constexpr int kElems = 4;
};
template <>
struct Vec16<uint32_t> {
  static constexpr int kElems = 4;
};
template <>
struct Vec16<uint8_t> {
  static constexpr int kElems = 16;
};

template <__nv_fp8_interpretation_t kKind>
struct Fp8Vec16 {
  static constexpr int kElems = 16;
  MSCCLPP_DEVICE_INLINE static void toFloat(uint4 v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
      __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] & 0xffffu), kKind);
      __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(w[i] >> 16), kKind);
      float2 a = __half22float2(*reinterpret_cast<__half2*>(&lo));
      float2 b = __half22float2(*reinterpret_cast<__half2*>(&hi));
      f[4 * i] = a.x;
      f[4 * i + 1] = a.y;
      f[4 * i + 2] = b.x;
      f[4 * i + 3] = b.y;
    }
  }
  MSCCLPP_DEVICE_INLINE static uint4 fromFloat(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i], f[4 * i + 1]), __NV_SATFINITE, kKind);
      uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(f[4 * i + 2], f[4 * i + 3]), __NV_SATFINITE, kKind);
      w[i] = lo | (hi << 16);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};
template <>
struct Vec16<f8e4m3> : Fp8Vec16<__NV_E4M3> {};
template <>
struct Vec16<f8e5m2> : Fp8Vec16<__NV_E5M2> {};

template <>
struct Vec16<f8e4m3b15> {
  static constexpr int kElems = 16;
  MSCCLPP_DEVICE_INLINE static void toFloat(uint4 v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 16; i++) f[i] = e4m3b15ToFloat(static_cast<uint8_t>(w[i >> 2] >> (8 * (i & 3))));
  }
  MSCCLPP_DEVICE_INLINE static uint4 fromFloat(const float* f) {
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 16; i++) w[i >> 2] |= static_cast<uint32_t>(floatToE4m3b15(f[i])) << (8 * (i & 3));
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
};

template <typename T>
struct IsFloatLike {
  static constexpr bool value = true;
};
template <>
struct IsFloatLike<int32_t> {
  static constexpr bool value = false;
};
template <>
struct IsFloatLike<uint32_t> {
  static constexpr bool value = false;
};
template <>
struct IsFloatLike<uint8_t> {
  static constexpr bool value = false;
};

// ---------------------------------------------------------------- native (element-type) 16-byte reduce
template <ReduceOp Op>
MSCCLPP_DEVICE_INLINE float opf(float a, float b) {
  if constexpr (Op == SUM)
    return a + b;
  else
    return fminf(a, b);
}

// a (op) b on one 16-byte word, computed in the element type (what the reference's calVector does).
template <typename T, ReduceOp Op>
MSCCLPP_DEVICE_INLINE uint4 reduce16(uint4 a, uint4 b) {
  if constexpr (sizeof(T) == 4 && IsFloatLike<T>::value) {
    if constexpr (Op == SUM) {
      // packed fp32x2 add (Blackwell): two adds per instruction
      uint64_t a0 = (static_cast<uint64_t>(a.y) << 32) | a.x, b0 = (static_cast<uint64_t>(b.y) << 32) | b.x;
      uint64_t a1 = (static_cast<uint64_t>(a.w) << 32) | a.z, b1 = (static_cast<uint64_t>(b.w) << 32) | b.z;
      uint64_t r0, r1;
      asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r0) : "l"(a0), "l"(b0));
      asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r1) : "l"(a1), "l"(b1));
      return make_uint4(static_cast<uint32_t>(r0), static_cast<uint32_t>(r0 >> 32), static_cast<uint32_t>(r1),
                        static_cast<uint32_t>(r1 >> 32));
    } else {
      return make_uint4(__float_as_uint(fminf(__uint_as_float(a.x), __uint_as_float(b.x))),
                        __float_as_uint(fminf(__uint_as_float(a.y), __uint_as_float(b.y))),
                        __float_as_uint(fminf(__uint_as_float(a.z), __uint_as_float(b.z))),
                        __float_as_uint(fminf(__uint_as_float(a.w), __uint_as_float(b.w))));
    }
  } else if constexpr (sizeof(T) == 4) {
    uint4 r;
    if constexpr (Op == SUM) {
      r.x = a.x + b.x;
      r.y = a.y + b.y;
      r.z = a.z + b.z;
      r.w = a.w + b.w;
    } else if constexpr (static_cast<T>(-1) < static_cast<T>(0)) {
      r.x = min(static_cast<int>(a.x), static_cast<int>(b.x));
      r.y = min(static_cast<int>(a.y), static_cast<int>(b.y));
      r.z = min(static_cast<int>(a.z), static_cast<int>(b.z));
      r.w = min(static_cast<int>(a.w), static_cast<int>(b.w));
    } else {
      r.x = min(a.x, b.x);
      r.y = min(a.y, b.y);
      r.z = min(a.z, b.z);
      r.w = min(a.w, b.w);
    }
    return r;
  } else if constexpr (sizeof(T) == 2) {
    uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w}, rw[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      if constexpr (sizeof(T) == 2 && Op == SUM) {
        if constexpr (__is_same(T, __half)) {
          __half2 r = __hadd2(*reinterpret_cast<__half2*>(&aw[i]), *reinterpret_cast<__half2*>(&bw[i]));
          rw[i] = *reinterpret_cast<uint32_t*>(&r);
        } else {
          __nv_bfloat162 r =
              __hadd2(*reinterpret_cast<__nv_bfloat162*>(&aw[i]), *reinterpret_cast<__nv_bfloat162*>(&bw[i]));
          rw[i] = *reinterpret_cast<uint32_t*>(&r);
        }
      } else {
        if constexpr (__is_same(T, __half)) {
          __half2 r = __hmin2(*reinterpret_cast<__half2*>(&aw[i]), *reinterpret_cast<__half2*>(&bw[i]));
          rw[i] = *reinterpret_cast<uint32_t*>(&r);
        } else {
          __nv_bfloat162 r =
              __hmin2(*reinterpret_cast<__nv_bfloat162*>(&aw[i]), *reinterpret_cast<__nv_bfloat162*>(&bw[i]));
          rw[i] = *reinterpret_cast<uint32_t*>(&r);
        }
      }
    }
    return make_uint4(rw[0], rw[1], rw[2], rw[3]);
  } else if constexpr (__is_same(T, uint8_t)) {
    uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w}, rw[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      if constexpr (Op == SUM)
        rw[i] = __vadd4(aw[i], bw[i]);
      else
        rw[i] = __vminu4(aw[i], bw[i]);
    }
    return make_uint4(rw[0], rw[1], rw[2], rw[3]);
  } else {
    // 8-bit floats: there is no native packed add; go through fp32 and round once.
    float fa[16], fb[16];
    Vec16<T>::toFloat(a, fa);
    Vec16<T>::toFloat(b, fb);
#pragma unroll
    for (int i = 0; i < 16; i++) fa[i] = opf<Op>(fa[i], fb[i]);
    return Vec16<T>::fromFloat(fa);
  }
}

// fp32 accumulator path: acc[i] = acc[i] (op) float(v[i]).
template <typename T, ReduceOp Op>
MSCCLPP_DEVICE_INLINE void accumulate16(float* acc, uint4 v) {
  float f[Vec16<T>::kElems];
  Vec16<T>::toFloat(v, f);
#pragma unroll
  for (int i = 0; i < Vec16<T>::kElems; i++) acc[i] = opf<Op>(acc[i], f[i]);
}

#endif  // __CUDACC__

}  // namespace mscclpp
