// Shared device helpers for the FFA B200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ffa_b200.h"

namespace ffa {

constexpr int kPage = 64;        // tokens per page == prune granularity
constexpr int kHeadDim = 128;    // K == V == 128
constexpr float kLog2e = 1.4426950408889634f;

// Records a CUDA runtime failure for ffa_last_cuda_error(); returns FFA_E_LAUNCH.
int note_cuda_error(cudaError_t e, const char* where);

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// 16-byte asynchronous global->shared copy that bypasses L1; src_bytes == 0 writes zeros
// and reads nothing.
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                        uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_h2(uint32_t x) {
  return __half22float2(*reinterpret_cast<__half2*>(&x));
}
__device__ __forceinline__ uint32_t hadd2_u32(uint32_t a, uint32_t b) {
  __half2 r = __hadd2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<uint32_t*>(&r);
}

// two fp8 values (low 16 bits of x) -> f16x2
template <int F8>
__device__ __forceinline__ uint32_t fp8x2_to_h2(uint32_t x) {
  if (F8 == FFA_E5M2) {
    // an e5m2 byte is the high byte of the fp16 with the same value
    return __byte_perm(x, 0u, 0x1404);  // {0, b0, 0, b1}
  } else {
    __half2_raw r = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(x & 0xffffu), __NV_E4M3);
    return static_cast<uint32_t>(r.x) | (static_cast<uint32_t>(r.y) << 16);
  }
}

// two e2m1 nibbles (low byte of x; low nibble first) -> f16x2
__device__ __forceinline__ uint32_t e2m1x2_to_h2(uint32_t x) {
  __half2_raw r = __nv_cvt_fp4x2_to_halfraw2(static_cast<__nv_fp4x2_storage_t>(x & 0xffu), __NV_E2M1);
  return static_cast<uint32_t>(r.x) | (static_cast<uint32_t>(r.y) << 16);
}

// two bf16 values -> f16x2 (round to nearest even, as torch/Triton `.to(float16)`)
__device__ __forceinline__ uint32_t bf16x2_to_h2(uint32_t x) {
  return pack_h2(__uint_as_float(x << 16), __uint_as_float(x & 0xffff0000u));
}

__device__ __forceinline__ float load_as_float(const void* base, int64_t idx, int dtype) {
  if (dtype == FFA_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  if (dtype == FFA_F16) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
  return reinterpret_cast<const float*>(base)[idx];
}

__device__ __forceinline__ void store_from_float(void* base, int64_t idx, int dtype, float x) {
  if (dtype == FFA_BF16) reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(x);
  else if (dtype == FFA_F16) reinterpret_cast<__half*>(base)[idx] = __float2half_rn(x);
  else reinterpret_cast<float*>(base)[idx] = x;
}

}  // namespace ffa
