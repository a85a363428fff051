// Device primitives shared by the TMA-fed decode kernels: mbarrier / TMA wrappers, the fp8, fp16 and
// bf16 tensor-core tiles, and the dot products of one 16-token slice of a K tile against the query
// operands (raw fp8 bytes against exact e4m3 pieces of q; dequantised 2-/4-bit codes against fp16 q).
#pragma once

#include <cuda.h>

#include "ffa_decode_shared.cuh"
#include "ffa_numeric.h"

namespace ffa {

namespace {

constexpr unsigned long long kWaitLimitNs = 200ull * 1000 * 1000;   // 0.2 s per mbarrier wait, then give up

struct ScaleCtx {
  const float* sS;
  const float* sZ;
  const float* book;
  float page_scale;
  // fp16 fast paths, taken only when every scale / zero involved is exactly an fp16 number:
  // q2: value = fma(code, scale, zero) evaluated in fp16 with one rounding.  The reference rounds the
  // exact sum to fp32 and then to fp16; the two differ by one fp16 ulp only when the fp32 rounding
  // lands on an fp16 tie (about 2e-5 of the elements for bf16 scales), far below what the prune band
  // or the output tolerance can see.  nvfp4: e2m1 value (2 significant bits) times a bf16 scale
  // (8 bits) is exact in fp16, so the product needs no fp32 detour at all.
  bool q2_fast;
  uint32_t s2[16], z2[16];     // this thread's channels 32t+2i, 32t+2i+1 as f16x2
  bool page_fast;
  uint32_t page_scale_h2;
};

// two 2-bit codes (bits 0-1 and 2-3 of n) as an f16x2 of their integer values: the high bytes of
// fp16 0, 1, 2, 3 are 0x00, 0x3C, 0x40, 0x42 and the low bytes are zero
// The byte permute picks result bytes (0, hi(c0), 0, hi(c1)), i.e. selector nibbles (4, c0, 4, c1);
// multiplying the four code bits by 0x410 drops c0 at bits 4-5 and c1 at bits 12-13 in one step.
__device__ __forceinline__ uint32_t codes2_to_h2(uint32_t low4) {
  const uint32_t sel = ((low4 * 0x410u) & 0x3030u) | 0x0404u;
  return __byte_perm(0x42403C00u, 0u, sel);
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {
  const __half2 r = __hfma2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b), *reinterpret_cast<__half2*>(&c));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  const __half2 r = __hmul2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ bool exact_in_f16(float x) {
  return __half2float(__float2half_rn(x)) == x;     // false for NaN and for values that overflow
}

// ---- mbarrier / TMA primitives ------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity; returns false if it gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, bool gave_up_before = false) {
  // Bounded in wall-clock time: a wait that has not completed after kWaitLimitNs gives up (the caller
  // records it in the status word and carries on, so the kernel still terminates promptly); a thread
  // that already gave up once does not wait again.
  if (gave_up_before) return false;
  unsigned long long t0 = 0;
  for (int spin = 0;; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spin & 63) == 63) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitNs) return false;
    }
  }
}
// 2-D tiled TMA load: box -> shared memory, completion counted in bytes on `bar`.  x is the byte
// offset inside a token row (a multiple of 16), y the token row.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// D(16x8,f32) += A(16x32, fp8 F8A, row) * B(32x8, e4m3, col)
template <int F8A>
__device__ __forceinline__ void mma_fp8(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
  if (F8A == FFA_E4M3) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e5m2.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// raw fp8 bytes of rows (16*warp+g) and (+8) from a 128B-swizzled [64 x 128 B] tile: this thread's
// channels are [32t, 32t+32), register r holding channels 32t+4r .. 32t+4r+3
__device__ __forceinline__ void load_fp8_rows(uint32_t (&ra)[8], uint32_t (&rb)[8], const uint8_t* tile, int warp,
                                              int g, int t) {
  const uint8_t* rowA = tile + (16 * warp + g) * 128;
  const uint8_t* rowB = rowA + 8 * 128;
  const int c0 = ((2 * t) ^ g) * 16, c1 = ((2 * t + 1) ^ g) * 16;    // (row & 7) == g for both rows
  const uint4 a0 = *reinterpret_cast<const uint4*>(rowA + c0);
  const uint4 a1 = *reinterpret_cast<const uint4*>(rowA + c1);
  const uint4 b0 = *reinterpret_cast<const uint4*>(rowB + c0);
  const uint4 b1 = *reinterpret_cast<const uint4*>(rowB + c1);
  ra[0] = a0.x; ra[1] = a0.y; ra[2] = a0.z; ra[3] = a0.w; ra[4] = a1.x; ra[5] = a1.y; ra[6] = a1.z; ra[7] = a1.w;
  rb[0] = b0.x; rb[1] = b0.y; rb[2] = b0.z; rb[3] = b0.w; rb[4] = b1.x; rb[5] = b1.y; rb[6] = b1.z; rb[7] = b1.w;
}

// 16 token rows in GLOBAL memory (not a staged tile): row r of the block starts at base + r * stride;
// rows >= valid read as zeros.  Used for the two 16-token threshold samples, which are read once.
struct RowsRef {
  const uint8_t* base;
  int64_t stride;
  int valid;
};
__device__ __forceinline__ void load_fp8_rows(uint32_t (&ra)[8], uint32_t (&rb)[8], const RowsRef& rows, int /*slice*/,
                                              int g, int t) {
  const uint4 z = make_uint4(0u, 0u, 0u, 0u);
  const uint4* rowA = reinterpret_cast<const uint4*>(rows.base + g * rows.stride) + 2 * t;
  const uint4* rowB = reinterpret_cast<const uint4*>(rows.base + (g + 8) * rows.stride) + 2 * t;
  const uint4 a0 = g < rows.valid ? __ldg(rowA) : z, a1 = g < rows.valid ? __ldg(rowA + 1) : z;
  const uint4 b0 = g + 8 < rows.valid ? __ldg(rowB) : z, b1 = g + 8 < rows.valid ? __ldg(rowB + 1) : z;
  ra[0] = a0.x; ra[1] = a0.y; ra[2] = a0.z; ra[3] = a0.w; ra[4] = a1.x; ra[5] = a1.y; ra[6] = a1.z; ra[7] = a1.w;
  rb[0] = b0.x; rb[1] = b0.y; rb[2] = b0.z; rb[3] = b0.w; rb[4] = b1.x; rb[5] = b1.y; rb[6] = b1.z; rb[7] = b1.w;
}

// q . k for the warp's 16 tokens from raw fp8 K bytes and the e4m3 pieces of q.
// out[nt][0] : token g, head 4nt+t;  out[nt][1] : token g+8, head 4nt+t   (unscaled dot products)
// QP = 2 (bf16 q): one n-tile per four heads, columns 2t / 2t+1 = pieces hi / lo x16.
// QP = 3 (fp16 q): a second n-tile per four heads whose column 2t is the third piece (x256).
template <int F8, int NT, int QP, typename Tile = const uint8_t*>
__device__ __forceinline__ void dot_fp8(float (&out)[NT][2], const uint32_t (&qb)[NT * (QP - 1)][4][2],
                                        const float (&qinv)[NT], const Tile& tile, int warp, int g, int t) {
  uint32_t ra[8], rb[8];
  load_fp8_rows(ra, rb, tile, warp, g, t);
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      if (s & 1) mma_fp8<F8>(acc1, ra[2 * s], rb[2 * s], ra[2 * s + 1], rb[2 * s + 1], qb[nt][s][0], qb[nt][s][1]);
      else       mma_fp8<F8>(acc0, ra[2 * s], rb[2 * s], ra[2 * s + 1], rb[2 * s + 1], qb[nt][s][0], qb[nt][s][1]);
    }
    float d0 = (acc0[0] + acc1[0]) + (acc0[1] + acc1[1]) * 0.0625f;
    float d1 = (acc0[2] + acc1[2]) + (acc0[3] + acc1[3]) * 0.0625f;
    if (QP == 3) {
      float acc2[4] = {0.f, 0.f, 0.f, 0.f}, acc3[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const uint32_t b0 = qb[(QP - 2) * NT + nt][s][0], b1 = qb[(QP - 2) * NT + nt][s][1];
        if (s & 1) mma_fp8<F8>(acc3, ra[2 * s], rb[2 * s], ra[2 * s + 1], rb[2 * s + 1], b0, b1);
        else       mma_fp8<F8>(acc2, ra[2 * s], rb[2 * s], ra[2 * s + 1], rb[2 * s + 1], b0, b1);
      }
      d0 += (acc2[0] + acc3[0]) * 0.00390625f;
      d1 += (acc2[2] + acc3[2]) * 0.00390625f;
    }
    out[nt][0] = d0 * qinv[nt];
    out[nt][1] = d1 * qinv[nt];
  }
}

// fp16 values of channels kb..kb+3 of one token row of a 2-bit / 4-bit coarse tile
// FAST selects the packed-fp16 route of q2 / nvfp4 (the caller checked that it is exact enough, see
// ScaleCtx); it is a template parameter so that the choice is one branch per page, not one per pair.
template <int FMT, bool FAST>
__device__ __forceinline__ void coarse_pair16(uint32_t& lo, uint32_t& hi, const uint32_t (&r)[4], int s, int kb,
                                              const ScaleCtx& sc) {
  if (FMT == FFA_K_Q2) {
    const uint32_t byte = (r[s >> 2] >> (8 * (s & 3))) & 0xffu;
    if (FAST) {
      lo = hfma2_u32(codes2_to_h2(byte & 0xfu), sc.s2[2 * s], sc.z2[2 * s]);
      hi = hfma2_u32(codes2_to_h2(byte >> 4), sc.s2[2 * s + 1], sc.z2[2 * s + 1]);
      return;
    }
    const float4 S = *reinterpret_cast<const float4*>(sc.sS + kb);
    const float4 Z = *reinterpret_cast<const float4*>(sc.sZ + kb);
    lo = pack_h2(fmaf(static_cast<float>(byte & 3u), S.x, Z.x), fmaf(static_cast<float>((byte >> 2) & 3u), S.y, Z.y));
    hi = pack_h2(fmaf(static_cast<float>((byte >> 4) & 3u), S.z, Z.z), fmaf(static_cast<float>(byte >> 6), S.w, Z.w));
  } else {
    const uint32_t two = (r[s >> 1] >> (16 * (s & 1))) & 0xffffu;
    if (FMT == FFA_K_FP4) {
      lo = e2m1x2_to_h2(two);
      hi = e2m1x2_to_h2(two >> 8);
    } else if (FMT == FFA_K_NVFP4) {
      if (FAST) {
        lo = hmul2_u32(e2m1x2_to_h2(two), sc.page_scale_h2);
        hi = hmul2_u32(e2m1x2_to_h2(two >> 8), sc.page_scale_h2);
        return;
      }
      const float2 a = unpack_h2(e2m1x2_to_h2(two));
      const float2 b = unpack_h2(e2m1x2_to_h2(two >> 8));
      lo = pack_h2(a.x * sc.page_scale, a.y * sc.page_scale);
      hi = pack_h2(b.x * sc.page_scale, b.y * sc.page_scale);
    } else {
      const float4 S = *reinterpret_cast<const float4*>(sc.sS + kb);
      lo = pack_h2(sc.book[two & 15u] * S.x, sc.book[(two >> 4) & 15u] * S.y);
      hi = pack_h2(sc.book[(two >> 8) & 15u] * S.z, sc.book[(two >> 12) & 15u] * S.w);
    }
  }
}

// the raw code bytes of rows (16*warp+g) and (+8) that this thread contracts over: channels [32t, 32t+32)
template <int FMT>
__device__ __forceinline__ void load_code_rows(uint32_t (&ra)[4], uint32_t (&rb)[4], const uint8_t* tile, int warp, int g,
                                               int t) {
  constexpr int ROW = Fmt<FMT>::kRow;
  const uint8_t* rowA = tile + (16 * warp + g) * ROW;
  const uint8_t* rowB = rowA + 8 * ROW;
  if (FMT == FFA_K_Q2) {
    const uint2 a = *reinterpret_cast<const uint2*>(rowA + 8 * t);
    const uint2 b = *reinterpret_cast<const uint2*>(rowB + 8 * t);
    ra[0] = a.x; ra[1] = a.y; rb[0] = b.x; rb[1] = b.y; ra[2] = ra[3] = rb[2] = rb[3] = 0;
  } else {
    const uint4 a = *reinterpret_cast<const uint4*>(rowA + 16 * t);
    const uint4 b = *reinterpret_cast<const uint4*>(rowB + 16 * t);
    ra[0] = a.x; ra[1] = a.y; ra[2] = a.z; ra[3] = a.w; rb[0] = b.x; rb[1] = b.y; rb[2] = b.z; rb[3] = b.w;
  }
}
template <int FMT>
__device__ __forceinline__ void load_code_rows(uint32_t (&ra)[4], uint32_t (&rb)[4], const RowsRef& rows, int /*slice*/,
                                               int g, int t) {
  const uint8_t* rowA = rows.base + g * rows.stride;
  const uint8_t* rowB = rows.base + (g + 8) * rows.stride;
  if (FMT == FFA_K_Q2) {
    const uint2 z = make_uint2(0u, 0u);
    const uint2 a = g < rows.valid ? __ldg(reinterpret_cast<const uint2*>(rowA + 8 * t)) : z;
    const uint2 b = g + 8 < rows.valid ? __ldg(reinterpret_cast<const uint2*>(rowB + 8 * t)) : z;
    ra[0] = a.x; ra[1] = a.y; rb[0] = b.x; rb[1] = b.y; ra[2] = ra[3] = rb[2] = rb[3] = 0;
  } else {
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    const uint4 a = g < rows.valid ? __ldg(reinterpret_cast<const uint4*>(rowA + 16 * t)) : z;
    const uint4 b = g + 8 < rows.valid ? __ldg(reinterpret_cast<const uint4*>(rowB + 16 * t)) : z;
    ra[0] = a.x; ra[1] = a.y; ra[2] = a.z; ra[3] = a.w; rb[0] = b.x; rb[1] = b.y; rb[2] = b.z; rb[3] = b.w;
  }
}

// q . k_coarse for 2-bit / 4-bit formats: codes -> fp16 -> m16n8k16 against fp16 q (odd columns 0)
template <int FMT, int NT, bool FAST, typename Tile = const uint8_t*>
__device__ __forceinline__ void dot_f16(float (&out)[NT][2], const uint32_t (&qh)[NT][8][2], const Tile& tile,
                                        const ScaleCtx& sc, int warp, int g, int t) {
  uint32_t ra[4], rb[4];
  load_code_rows<FMT>(ra, rb, tile, warp, g, t);
  float acc[NT][2][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int h = 0; h < 2; ++h) { acc[nt][h][0] = acc[nt][h][1] = acc[nt][h][2] = acc[nt][h][3] = 0.f; }
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    const int kb = 32 * t + 4 * s;
    uint32_t alo, ahi, blo, bhi;
    coarse_pair16<FMT, FAST>(alo, ahi, ra, s, kb, sc);
    coarse_pair16<FMT, FAST>(blo, bhi, rb, s, kb, sc);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mma_f16(acc[nt][s & 1], alo, blo, ahi, bhi, qh[nt][s][0], qh[nt][s][1]);
  }
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    out[nt][0] = acc[nt][0][0] + acc[nt][1][0];
    out[nt][1] = acc[nt][0][2] + acc[nt][1][2];
  }
}

// two floats -> two e4m3 bytes (round to nearest even), first value in the low byte
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float a, float b) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;\n" : "=h"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint32_t x) {
  return unpack_h2(fp8x2_to_h2<FFA_E4M3>(x));
}

}  // namespace

}  // namespace ffa
