// Host build of the scalar quantiser bodies in ffa_numeric.h, for CPU-side checks of their
// bit-exactness against the reference quantisers.  Test aid only: the Python package never
// loads this library, and the CUDA kernels do not depend on it.
#include <stdint.h>

#include <algorithm>
#include <cmath>
#include <limits>
#include <vector>

#include "ffa_numeric.h"

using namespace ffa::num;

namespace {
constexpr int D = 128;
}

extern "C" {

void ffa_host_f32_to_fp8(const float* x, int64_t n, int fmt, uint8_t* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = f32_to_fp8(x[i], fmt);
}
void ffa_host_fp8_to_f32(const uint8_t* x, int64_t n, int fmt, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = fp8_to_f32(x[i], fmt);
}
void ffa_host_round_to(const float* x, int64_t n, int dt, float* out) {
  for (int64_t i = 0; i < n; ++i) out[i] = round_to(x[i], dt);
}

void ffa_host_quantize_q2(const void* k, int dt, int B, int T, int HKV, int fp8, uint8_t* codes, void* scale,
                          void* zero, uint8_t* res) {
  for (int b = 0; b < B; ++b)
    for (int h = 0; h < HKV; ++h)
      for (int c = 0; c < D; c += 4) {
        float sc[4], ze[4];
        for (int j = 0; j < 4; ++j) {
          float lo = std::numeric_limits<float>::infinity(), hi = -lo;
          for (int t = 0; t < T; ++t) {
            const float v = load_elem(k, ((int64_t(b) * T + t) * HKV + h) * D + c + j, dt);
            lo = std::min(lo, v); hi = std::max(hi, v);
          }
          q2_scale_zero(lo, hi, dt, &sc[j], &ze[j]);
          store_elem(scale, (int64_t(b) * HKV + h) * D + c + j, dt, sc[j]);
          store_elem(zero, (int64_t(b) * HKV + h) * D + c + j, dt, ze[j]);
        }
        for (int t = 0; t < T; ++t) {
          const int64_t e = ((int64_t(b) * T + t) * HKV + h) * D + c;
          uint32_t byte = 0;
          for (int j = 0; j < 4; ++j) byte |= q2_encode(load_elem(k, e + j, dt), sc[j], ze[j], dt, fp8, res + e + j) << (2 * j);
          codes[e / 4] = static_cast<uint8_t>(byte);
        }
      }
}

void ffa_host_quantize_fp8fp8(const void* k, int dt, int64_t n, int fp8, uint8_t* base, uint8_t* res) {
  for (int64_t i = 0; i < n; ++i) fp8fp8_encode(load_elem(k, i, dt), fp8, base + i, res + i);
}

void ffa_host_quantize_fp4(const void* k, int dt, int64_t n, int fp8, uint8_t* codes, uint8_t* res) {
  for (int64_t i = 0; i < n; i += 2) {
    const uint32_t lo = fp4_encode(load_elem(k, i, dt), dt, fp8, res + i);
    const uint32_t hi = fp4_encode(load_elem(k, i + 1, dt), dt, fp8, res + i + 1);
    codes[i / 2] = static_cast<uint8_t>(lo | (hi << 4));
  }
}

void ffa_host_quantize_nf4(const void* k, int dt, int B, int T, int HKV, int fp8, uint8_t* codes, void* scale,
                           uint8_t* res) {
  std::vector<float> amax(size_t(B) * HKV * D, 0.f);
  for (int b = 0; b < B; ++b)
    for (int t = 0; t < T; ++t)
      for (int i = 0; i < HKV * D; ++i) {
        float& a = amax[size_t(b) * HKV * D + i];
        a = std::max(a, std::fabs(load_elem(k, (int64_t(b) * T + t) * HKV * D + i, dt)));
      }
  for (size_t i = 0; i < amax.size(); ++i) {
    amax[i] = std::max(amax[i], 1e-6f);
    store_elem(scale, int64_t(i), dt, amax[i]);
  }
  for (int b = 0; b < B; ++b)
    for (int t = 0; t < T; ++t)
      for (int i = 0; i < HKV * D; i += 2) {
        const int64_t e = (int64_t(b) * T + t) * HKV * D + i;
        const uint32_t lo = nf4_encode_elem(load_elem(k, e, dt), amax[size_t(b) * HKV * D + i], fp8, res + e);
        const uint32_t hi = nf4_encode_elem(load_elem(k, e + 1, dt), amax[size_t(b) * HKV * D + i + 1], fp8, res + e + 1);
        codes[e / 2] = static_cast<uint8_t>(lo | (hi << 4));
      }
}

void ffa_host_quantize_nvfp4(const void* k, int dt, int B, int T, int HKV, int fp8, int page, uint8_t* codes,
                             void* scale, uint8_t* res) {
  const int NPG = (T + page - 1) / page;
  for (int b = 0; b < B; ++b)
    for (int pg = 0; pg < NPG; ++pg)
      for (int h = 0; h < HKV; ++h) {
        float amax = 0.f;
        const int t1 = std::min(T, (pg + 1) * page);
        for (int t = pg * page; t < t1; ++t)
          for (int c = 0; c < D; ++c)
            amax = std::max(amax, std::fabs(load_elem(k, ((int64_t(b) * T + t) * HKV + h) * D + c, dt)));
        const float s = nvfp4_scale(amax, dt);
        store_elem(scale, (int64_t(b) * NPG + pg) * HKV + h, dt, s);
        for (int t = pg * page; t < t1; ++t)
          for (int c = 0; c < D; c += 2) {
            const int64_t e = ((int64_t(b) * T + t) * HKV + h) * D + c;
            const uint32_t lo = nvfp4_encode(load_elem(k, e, dt), s, dt, fp8, res + e);
            const uint32_t hi = nvfp4_encode(load_elem(k, e + 1, dt), s, dt, fp8, res + e + 1);
            codes[e / 2] = static_cast<uint8_t>(lo | (hi << 4));
          }
      }
}

}  // extern "C"
