// Scalar numeric building blocks of the FFA quantisers: fp8 / e2m1 / NF4 encoders and the
// "one rounding per torch op" arithmetic of the reference quantisers.  Plain C++ that compiles
// both as CUDA device code and as host code, so the same functions can be checked on a CPU
// against the reference's outputs (tests/test_numeric_host.py) and then run inside the kernels.
//
// Reference semantics (paths relative to the reference root):
//   ffa-q2fp8/fused_kproj_rope_q2fp8.py:44-52       2-bit asymmetric, arithmetic in K's dtype
//   ffa-fp8fp8/fused_kproj_rope_fp8fp8.py:62-63     fp8 base + fp8 residual
//   ffa-fp4fp8/fused_kproj_rope_fp4fp8.py:45-62     e2m1 by seven cut points, residual in K's dtype
//   ffa-nf4fp8/fused_kproj_rope_nf4fp8.py:77-85     NF4 by fifteen midpoints, arithmetic in fp32
//   ffa-nvfp4fp8/fused_kproj_rope_nvfp4fp8.py:71-97 e2m1 of K/scale, arithmetic in K's dtype
// torch's float -> float8 casts round to nearest even; float8_e4m3fn has no infinity and maps
// everything that rounds past 448 (and NaN) to its NaN code 0x7F, float8_e5m2 overflows to
// infinity 0x7C like IEEE half.
#pragma once

#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#define FFA_HD __host__ __device__ __forceinline__
#else
#include <math.h>
#define FFA_HD inline
#endif

namespace ffa {
namespace num {

enum { kF16 = 0, kBF16 = 1, kF32 = 2 };
enum { kE5M2 = 0, kE4M3 = 1 };

FFA_HD uint32_t f2u(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}
FFA_HD float u2f(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f; memcpy(&f, &u, 4); return f;
#endif
}

// ---- 16-bit floats --------------------------------------------------------------------------
FFA_HD float bf16_bits_to_f32(uint16_t h) { return u2f(static_cast<uint32_t>(h) << 16); }

FFA_HD uint16_t f32_to_bf16_bits(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);  // quiet NaN
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

FFA_HD float f16_bits_to_f32(uint16_t h) {
#if defined(__CUDA_ARCH__)
  return __half2float(__ushort_as_half(h));
#endif
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  const uint32_t e = (h >> 10) & 0x1fu, m = h & 0x3ffu;
  if (e == 0x1fu) return u2f(sign | 0x7f800000u | (m << 13));
  if (e != 0) return u2f(sign | ((e + 112u) << 23) | (m << 13));
  // subnormal: m * 2^-24, exact in fp32
  const float v = static_cast<float>(m) * 5.9604644775390625e-08f;
  return u2f(f2u(v) | sign);
}

// Round-to-nearest-even narrowing of |x| (given as fp32 bits, finite, below the overflow
// point) to a small float with MB mantissa bits and exponent bias BIAS; returns the magnitude
// code.  Values that round past the largest normal simply carry into the next code.
template <int MB, int BIAS>
FFA_HD uint32_t narrow_rne(uint32_t a) {
  const uint32_t be = a >> 23;
  if (be == 0) return 0;                                   // fp32 subnormal: far below half an ulp
  const int e = static_cast<int>(be) - 127;
  const uint32_t sig = (a & 0x7fffffu) | 0x800000u;
  const int emin = 1 - BIAS;
  int shift = 23 - MB;
  if (e < emin) shift += emin - e;
  if (shift > 25) return 0;
  uint32_t kept = sig >> shift;
  const uint32_t rem = sig & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (kept & 1u))) ++kept;
  return e < emin ? kept : ((static_cast<uint32_t>(e + BIAS - 1) << MB) + kept);
}

FFA_HD uint16_t f32_to_f16_bits(float f) {
  const uint32_t u = f2u(f), a = u & 0x7fffffffu;
  const uint16_t sign = static_cast<uint16_t>((u >> 16) & 0x8000u);
  if (a > 0x7f800000u) return sign | 0x7e00u;
  if (a >= 0x477ff000u) return sign | 0x7c00u;             // >= 65520 rounds to infinity
  return sign | static_cast<uint16_t>(narrow_rne<10, 15>(a));
}

// x rounded to the element type `dt` and widened back: the effect of one torch op on a tensor
// of that dtype.
FFA_HD float round_to(float x, int dt) {
#if defined(__CUDA_ARCH__)
  if (dt == kBF16) return __bfloat162float(__float2bfloat16_rn(x));
  if (dt == kF16) return __half2float(__float2half_rn(x));
  return x;
#else
  if (dt == kBF16) return bf16_bits_to_f32(f32_to_bf16_bits(x));
  if (dt == kF16) return f16_bits_to_f32(f32_to_f16_bits(x));
  return x;
#endif
}

FFA_HD float load_elem(const void* p, int64_t i, int dt) {
  if (dt == kBF16) return bf16_bits_to_f32(static_cast<const uint16_t*>(p)[i]);
  if (dt == kF16) return f16_bits_to_f32(static_cast<const uint16_t*>(p)[i]);
  return static_cast<const float*>(p)[i];
}
FFA_HD void store_elem(void* p, int64_t i, int dt, float x) {
  if (dt == kBF16) static_cast<uint16_t*>(p)[i] = f32_to_bf16_bits(x);
  else if (dt == kF16) static_cast<uint16_t*>(p)[i] = f32_to_f16_bits(x);
  else static_cast<float*>(p)[i] = x;
}

// ---- fp8 ------------------------------------------------------------------------------------
// On the device the narrowing itself is the hardware's round-to-nearest-even conversion; it
// saturates where torch overflows, so everything above the last value that still rounds down to
// the largest finite number (464 for e4m3fn, 61440 for e5m2) is patched to torch's result.
FFA_HD uint8_t f32_to_e4m3(float f) {
  const uint32_t u = f2u(f), a = u & 0x7fffffffu;
  const uint8_t sign = static_cast<uint8_t>((u >> 24) & 0x80u);
#if defined(__CUDA_ARCH__)
  if (a > 0x43e80000u) return sign | 0x7fu;                // |x| > 464, inf, NaN
  uint16_t pair;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(pair) : "f"(0.f), "f"(f));
  return static_cast<uint8_t>(pair & 0xffu);
#else
  if (a >= 0x43f00000u) return sign | 0x7fu;               // |x| >= 480, inf, NaN
  return sign | static_cast<uint8_t>(narrow_rne<3, 7>(a));  // (464, 480) carries into 0x7F too
#endif
}
FFA_HD uint8_t f32_to_e5m2(float f) {
  const uint32_t u = f2u(f), a = u & 0x7fffffffu;
  const uint8_t sign = static_cast<uint8_t>((u >> 24) & 0x80u);
  if (a > 0x7f800000u) return sign | 0x7fu;
#if defined(__CUDA_ARCH__)
  if (a >= 0x47700000u) return sign | 0x7cu;               // |x| >= 61440 rounds to infinity
  uint16_t pair;
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;\n" : "=h"(pair) : "f"(0.f), "f"(f));
  return static_cast<uint8_t>(pair & 0xffu);
#else
  if (a >= 0x47800000u) return sign | 0x7cu;               // |x| >= 65536
  return sign | static_cast<uint8_t>(narrow_rne<2, 15>(a));
#endif
}
FFA_HD uint8_t f32_to_fp8(float f, int fmt) { return fmt == kE4M3 ? f32_to_e4m3(f) : f32_to_e5m2(f); }

FFA_HD float e5m2_to_f32(uint8_t b) {
#if defined(__CUDA_ARCH__)
  return __half2float(__ushort_as_half(static_cast<unsigned short>(b) << 8));
#else
  return f16_bits_to_f32(static_cast<uint16_t>(b) << 8);
#endif
}
FFA_HD float e4m3_to_f32(uint8_t b) {
#if defined(__CUDA_ARCH__)
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h2) : "h"(static_cast<uint16_t>(b)));
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
#endif
  const uint32_t sign = static_cast<uint32_t>(b & 0x80u) << 24;
  const uint32_t e = (b >> 3) & 0xfu, m = b & 7u;
  if ((b & 0x7fu) == 0x7fu) return u2f(sign | 0x7fc00000u);
  if (e != 0) return u2f(sign | ((e + 120u) << 23) | (m << 20));
  const float v = static_cast<float>(m) * 0.001953125f;    // m * 2^-9
  return u2f(f2u(v) | sign);
}
FFA_HD float fp8_to_f32(uint8_t b, int fmt) { return fmt == kE4M3 ? e4m3_to_f32(b) : e5m2_to_f32(b); }

// ---- e2m1 -----------------------------------------------------------------------------------
FFA_HD float e2m1_level(uint32_t mag) {
  // 0, .5, 1, 1.5, 2, 3, 4, 6
  return mag < 4u ? 0.5f * static_cast<float>(mag) : (mag == 4u ? 2.f : (mag == 5u ? 3.f : (mag == 6u ? 4.f : 6.f)));
}
// nibble of x: magnitude index = number of cut points <= |x| (ties go up), sign bit from x < 0
FFA_HD uint32_t e2m1_encode(float x, float* level_signed) {
  const float a = x < 0.f ? -x : x;
  uint32_t mag = 0;
  mag += a >= 0.25f; mag += a >= 0.75f; mag += a >= 1.25f; mag += a >= 1.75f;
  mag += a >= 2.5f;  mag += a >= 3.5f;  mag += a >= 5.0f;
  if (a != a) mag = 7;                                      // NaN sorts after every cut point
  const bool neg = x < 0.f;
  const float lv = e2m1_level(mag);
  *level_signed = neg ? -lv : lv;
  return mag | (neg ? 8u : 0u);
}

// ---- NF4 ------------------------------------------------------------------------------------
FFA_HD float nf4_level(uint32_t i) {
  const float book[16] = {-1.0f, -0.6961928009986877f, -0.5229921340942383f, -0.39491748809814453f,
                          -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
                          0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
                          0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};
  return book[i];
}
// index = number of midpoints strictly below the clamped value
FFA_HD uint32_t nf4_encode(float unit) {
  unit = unit < -1.f ? -1.f : (unit > 1.f ? 1.f : unit);
  uint32_t idx = 0;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (uint32_t i = 0; i < 15; ++i) {
    const float mid = (nf4_level(i) + nf4_level(i + 1)) * 0.5f;
    idx += mid < unit;
  }
  return idx;
}

// ---- per-element quantiser bodies -----------------------------------------------------------
// q2: scale/zero from a channel's min/max, all in K's dtype
FFA_HD void q2_scale_zero(float lo, float hi, int dt, float* scale, float* zero) {
  const float floor_ = round_to(1e-6f, dt);
  float span = round_to(hi - lo, dt);
  span = span < floor_ ? floor_ : span;
  *scale = round_to(span / 3.0f, dt);
  *zero = lo;
}
// Each *_f function returns the code and leaves the residual as a float (already rounded the way
// the reference's dtype arithmetic rounds it); the caller narrows it to fp8.
FFA_HD uint32_t q2_encode_f(float k, float scale, float zero, int dt, float* res_f) {
  const float d = round_to(k - zero, dt);
  const float r = round_to(d / scale, dt);
#if defined(__CUDA_ARCH__)
  float c = rintf(r);
#else
  float c = nearbyintf(r);
#endif
  c = c < 0.f ? 0.f : (c > 3.f ? 3.f : c);
  if (r != r) c = 0.f;
  // product and sum round separately like the two torch ops (they only differ from a fused
  // multiply-add when scale has more than 22 significant bits, i.e. for fp32 K)
#if defined(__CUDA_ARCH__)
  const float deq = __fadd_rn(__fmul_rn(c, scale), zero);
  *res_f = __fsub_rn(k, deq);
#else
  volatile float prod = c * scale;
  const float deq = prod + zero;
  *res_f = k - deq;
#endif
  return static_cast<uint32_t>(c);
}
FFA_HD uint32_t q2_encode(float k, float scale, float zero, int dt, int fp8, uint8_t* res) {
  float rf;
  const uint32_t c = q2_encode_f(k, scale, zero, dt, &rf);
  *res = f32_to_fp8(rf, fp8);
  return c;
}
FFA_HD void fp8fp8_encode(float k, int fp8, uint8_t* base, uint8_t* res) {
  const uint8_t b = f32_to_fp8(k, fp8);
  *base = b;
  *res = f32_to_fp8(k - fp8_to_f32(b, fp8), fp8);
}
FFA_HD uint32_t fp4_encode_f(float k, int dt, float* res_f) {
  float lv;
  const uint32_t nib = e2m1_encode(k, &lv);
  *res_f = round_to(k - lv, dt);
  return nib;
}
FFA_HD uint32_t fp4_encode(float k, int dt, int fp8, uint8_t* res) {
  float rf;
  const uint32_t nib = fp4_encode_f(k, dt, &rf);
  *res = f32_to_fp8(rf, fp8);
  return nib;
}
// `level` is NF4_CODEBOOK[idx], looked up by the caller (a table in registers on the device)
FFA_HD float nf4_residual_f(float k, float level, float absmax) {
  // product and difference round separately (no fused multiply-add), as two torch ops do
#if defined(__CUDA_ARCH__)
  return __fsub_rn(k, __fmul_rn(level, absmax));
#else
  volatile float deq = level * absmax;
  return k - deq;
#endif
}
FFA_HD uint32_t nf4_encode_elem(float k, float absmax, int fp8, uint8_t* res) {
  const uint32_t idx = nf4_encode(k / absmax);
  *res = f32_to_fp8(nf4_residual_f(k, nf4_level(idx), absmax), fp8);
  return idx;
}
FFA_HD float nvfp4_scale(float absmax, int dt) {
  const float floor_ = round_to(1e-6f, dt);
  const float s = round_to(absmax / 6.0f, dt);
  return s < floor_ ? floor_ : s;
}
FFA_HD uint32_t nvfp4_encode_f(float k, float scale, int dt, float* res_f) {
  float lv;
  const uint32_t nib = e2m1_encode(round_to(k / scale, dt), &lv);
  // product and difference are two torch ops: no fused multiply-add
#if defined(__CUDA_ARCH__)
  const float deq = round_to(__fmul_rn(lv, scale), dt);
  *res_f = round_to(__fsub_rn(k, deq), dt);
#else
  volatile float prod = lv * scale;
  const float deq = round_to(prod, dt);
  *res_f = round_to(k - deq, dt);
#endif
  return nib;
}
FFA_HD uint32_t nvfp4_encode(float k, float scale, int dt, int fp8, uint8_t* res) {
  float rf;
  const uint32_t nib = nvfp4_encode_f(k, scale, dt, &rf);
  *res = f32_to_fp8(rf, fp8);
  return nib;
}

#if defined(__CUDACC__)
// Two floats -> two fp8 bytes (a in the low byte) with torch's overflow behaviour, one hardware
// conversion for the pair.
template <int F8>
__device__ __forceinline__ uint32_t f32x2_to_fp8x2(float a, float b) {
  uint16_t pair;
  if (F8 == kE4M3) asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(pair) : "f"(b), "f"(a));
  else asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;\n" : "=h"(pair) : "f"(b), "f"(a));
  uint32_t out = pair;
  const uint32_t ua = __float_as_uint(a), ub = __float_as_uint(b);
  const uint32_t aa = ua & 0x7fffffffu, ab = ub & 0x7fffffffu;
  if (F8 == kE4M3) {
    if (aa > 0x43e80000u) out = (out & 0xff00u) | ((ua >> 24) & 0x80u) | 0x7fu;
    if (ab > 0x43e80000u) out = (out & 0x00ffu) | ((((ub >> 24) & 0x80u) | 0x7fu) << 8);
  } else {
    if (aa >= 0x47700000u) out = (out & 0xff00u) | ((ua >> 24) & 0x80u) | (aa > 0x7f800000u ? 0x7fu : 0x7cu);
    if (ab >= 0x47700000u) out = (out & 0x00ffu) | ((((ub >> 24) & 0x80u) | (ab > 0x7f800000u ? 0x7fu : 0x7cu)) << 8);
  }
  return out;
}
// eight floats -> eight fp8 bytes
template <int F8>
__device__ __forceinline__ uint2 narrow8(const float (&r)[8]) {
  return make_uint2(f32x2_to_fp8x2<F8>(r[0], r[1]) | (f32x2_to_fp8x2<F8>(r[2], r[3]) << 16),
                    f32x2_to_fp8x2<F8>(r[4], r[5]) | (f32x2_to_fp8x2<F8>(r[6], r[7]) << 16));
}
// two fp8 bytes -> two floats
template <int F8>
__device__ __forceinline__ float2 fp8x2_to_f32x2(uint32_t pair) {
  uint32_t h2;
  if (F8 == kE4M3) asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h2) : "h"(static_cast<uint16_t>(pair)));
  else asm("cvt.rn.f16x2.e5m2x2 %0, %1;\n" : "=r"(h2) : "h"(static_cast<uint16_t>(pair)));
  return __half22float2(*reinterpret_cast<const __half2*>(&h2));
}
#endif

}  // namespace num
}  // namespace ffa
