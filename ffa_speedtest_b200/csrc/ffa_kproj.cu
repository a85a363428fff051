// Fused K projection + bias + RoPE for B200 (sm_100a), feeding the cache quantisers.
//
// Replaces the reference's Triton kernels _kproj_rope_minmax_kernel / _kproj_rope_quant_kernel
// (ffa-q2fp8/fused_kproj_rope_q2fp8.py:103-399 and the fp4 / nf4 siblings), which run the GEMM in
// 16x32x16 tiles with even and odd output columns as separate strided dots, and run it twice
// for the formats whose scale needs the whole sequence.  Here:
//
//   K_lin[M, N] = h[M, H] . W_k[N, H]^T  (+ bias)       M = B*T tokens, N = HKV*128, H = hidden
//
// is ONE tcgen05 GEMM: 128x128 output tiles (one kv-head wide, so RoPE pairs stay inside a tile),
// bf16/fp16 operands moved by TMA into a 6-stage 128B-swizzled shared-memory ring, a single
// elected thread issuing tcgen05.mma (M=128, N=128, K=16) with the fp32 accumulator in tensor
// memory, and four epilogue warps that read the accumulator back with tcgen05.ld (one token row
// per thread), add the bias, round to the activation dtype like F.linear, apply RoPE with the
// caller's cos/sin tables in the reference's op order (x*cos + rotate_half(x)*sin, pairs (2j,2j+1))
// and write post-RoPE K.  The quantise-and-scatter pass (ffa_quantize.cu) then reads that K, which
// at T = 8192 is 16-32 MB and still L2-resident.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocator + MMA issuer,
// warps 2..5 = epilogue (TMEM lane quarter = warp % 4).  Every mbarrier wait is bounded.
//
// Up to 24 token rows (one decode step of a batch, a short chunk) take kproj_few_kernel instead: the
// call is then a stream over W_k, so 32-channel column groups times a thread-block cluster that splits
// the hidden dimension read the weight once with plain 16-byte loads, feed it to warp-level MMAs whose
// eight columns are tokens, add the cluster's partial sums through distributed shared memory in a
// fixed order and run the same epilogue: one launch, no partial tiles in global memory, no waits
// other than the hardware cluster barrier.
#include <cooperative_groups.h>
#include <cuda.h>

#include "ffa_common.cuh"
#include "ffa_numeric.h"

namespace ffa {

// defined in ffa_quantize.cu
int quantize_dispatch(int variant, const void* k, int k_dtype, int B, int T, int HKV, int fp8, int page_size,
                      uint8_t* codes, void* scale, void* zero, uint8_t* residual, void* scratch,
                      const int32_t* slot_table, int slot_stride, int slot_pos0, cudaStream_t st);

// same, with the per-channel min/max already reduced per group of 32 token rows by the GEMM's epilogue:
// parts[B * parts_per_b][HKV*128][2] ordered uints (defined in ffa_quantize.cu)
int quantize_from_partials(int variant, const void* k, int k_dtype, int B, int T, int HKV, int fp8, uint8_t* codes,
                           void* scale, void* zero, uint8_t* residual, void* scratch, const uint32_t* parts,
                           int parts_per_b, const int32_t* slot_table, int slot_stride, cudaStream_t st);

namespace {

constexpr int kBM = 128, kBK = 64;                  // tile rows; kBK 16-bit elements = one 128-byte swizzle row
constexpr int kTileBytes = kBM * kBK * 2;           // 16 KiB: the A tile, and each 128 rows of the B tile
constexpr int kThreadsK = 192;
constexpr unsigned long long kWaitLimitNs = 200ull * 1000 * 1000;   // 0.2 s per mbarrier wait, then give up

// Tile width BN: 128 (one kv-head) or 256 (two).  The wider tile halves the A traffic per flop and
// is used whenever there are enough tiles to fill the GPU; shared memory holds as many 128B-swizzled
// stages as fit, tensor memory two BN-column fp32 accumulators.
template <int BN>
struct Tile {
  static constexpr int kStages = BN == 128 ? 6 : 4;
  static constexpr int kBBytes = BN * kBK * 2;
  static constexpr int kStageBytes = kTileBytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kOffBars = kStages * kStageBytes;       // full[], empty[], tmem_full[2], tmem_empty[2]
  static constexpr int kOffTmem = kOffBars + (2 * kStages + 4) * 8;
  static constexpr int kBytes = kOffTmem + 16 + 1024;           // + alignment slack
};

struct KprojParams {
  const void* bias;      // [N] in io dtype or null
  const void* cos;       // [T, 128]
  const void* sin;
  void* k_out;           // [M, N] post-RoPE K in out dtype
  int* status;
  const void* h;         // [M, H] and [N, H] operands as plain pointers (kproj_few_kernel; the GEMM uses TMA maps)
  const void* w;
  int M, T, N, H;
  float* partial;        // [n_split, M, N] fp32 when n_split > 1
  uint32_t* mm_part;     // [M / 32, N, 2] ordered-uint (min, max) of K per 32 token rows, when the epilogue reduces them
  int m_tiles, n_split;
  int io_dtype;          // FFA_F16 | FFA_BF16: h, W, bias
  int rope_dtype;        // dtype of cos/sin; the RoPE arithmetic and k_out use promote(io, rope)
  // quantisation inside the epilogue (elementwise formats with 16-bit K): the codes and residual of
  // token row m go to row slot_table[b][t / 64] * 64 + t % 64 of the pools (row m without a table)
  uint8_t* codes;
  uint8_t* residual;
  const int32_t* slot_table;
  int slot_stride;
  int slot_pos0;
};

// What the epilogue emits besides (or instead of) K: nothing, fp8 base + fp8 residual, or e2m1
// codes + fp8 residual; the fp8 format is part of the mode so the conversions are compile-time.
enum { kQuantNone = 0, kQuantFp8E4 = 1, kQuantFp8E5 = 2, kQuantFp4E4 = 3, kQuantFp4E5 = 4 };

__device__ __forceinline__ int64_t out_row_of(const KprojParams& p, int64_t m) {
  if (!p.slot_table) return m;
  const int64_t b = m / p.T, t = m % p.T + p.slot_pos0;
  return static_cast<int64_t>(p.slot_table[b * p.slot_stride + t / kPage]) * kPage + t % kPage;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
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
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major [rows x 64] 16-bit tile stored with the 128-byte
// swizzle: rows are 128 B apart, groups of 8 rows 1024 B apart (stride byte offset), descriptor
// version 1 (sm_100), layout type 2 (SWIZZLE_128B).  Advancing by UMMA_K = 16 elements inside the
// swizzle row is +32 B on the start address.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);        // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                             // leading byte offset (unused here)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                     // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                             // descriptor version
  d |= static_cast<uint64_t>(2) << 61;                             // SWIZZLE_128B
  return d;
}

// Instruction descriptor for kind::f16: fp32 accumulate, A and B both K-major, 16-bit format
// `fmt` (0 = fp16, 1 = bf16), N = bn, M = 128.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt, uint32_t bn) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((bn >> 3) << 17) | ((kBM >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(float (&v)[32], uint32_t taddr) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Epilogue of one token row x 32 channels (16 RoPE pairs): bias, rounding to the activation dtype
// (F.linear returns it), then RoPE with the interleaved-pair rotate_half of the reference
// (fused_kproj_rope_q2fp8.py:24-37): out = x * cos + rotate_half(x) * sin, every product and the sum
// rounded separately in the promoted dtype like the three torch ops.  IO / ROPE are the FFA_* codes
// of the activation dtype and of the cos/sin tables (ROPE is IO or FFA_F32).
//
// With 16-bit tables the whole rotation runs on packed pairs: the hardware's two-wide 16-bit
// multiply and add round once to the 16-bit result, which is what rounding the exact fp32 product
// (or sum) of two 16-bit numbers gives.
template <int IO> struct Pack16;
template <> struct Pack16<FFA_BF16> {
  using T2 = __nv_bfloat162;
  static __device__ __forceinline__ T2 from_floats(float lo, float hi) { return __floats2bfloat162_rn(lo, hi); }
  static __device__ __forceinline__ float2 to_floats(T2 v) { return __bfloat1622float2(v); }
};
template <> struct Pack16<FFA_F16> {
  using T2 = __half2;
  static __device__ __forceinline__ T2 from_floats(float lo, float hi) { return __floats2half2_rn(lo, hi); }
  static __device__ __forceinline__ float2 to_floats(T2 v) { return __half22float2(v); }
};

// cos / sin of one token for 32 consecutive channels, as loaded (16-byte loads)
template <int ROPE> struct RopeTables;
template <> struct RopeTables<FFA_F32> {
  float4 c[8], s[8];
  __device__ __forceinline__ void load(const KprojParams& p, int64_t tok, int ch0) {
    const float4* c4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.cos) + tok * kHeadDim + ch0);
    const float4* s4 = reinterpret_cast<const float4*>(static_cast<const float*>(p.sin) + tok * kHeadDim + ch0);
#pragma unroll
    for (int i = 0; i < 8; ++i) { c[i] = c4[i]; s[i] = s4[i]; }
  }
};
struct RopeTables16 {
  uint4 c[4], s[4];
  __device__ __forceinline__ void load(const KprojParams& p, int64_t tok, int ch0) {
    const uint4* c4 = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.cos) + tok * kHeadDim + ch0);
    const uint4* s4 = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.sin) + tok * kHeadDim + ch0);
#pragma unroll
    for (int i = 0; i < 4; ++i) { c[i] = c4[i]; s[i] = s4[i]; }
  }
};
template <> struct RopeTables<FFA_BF16> : RopeTables16 {};
template <> struct RopeTables<FFA_F16> : RopeTables16 {};

// MM: 0 = nothing more; 1 = also reduce min and max of each channel over the warp's 32 token rows
// (2-bit format), 2 = max of |K| (NF4), as order-preserving uints, into mm_row[32][2].  With MM every
// lane of the warp must be here (the reductions are warp-wide): the caller uses it only when all
// rows of every tile exist.
enum { kMmNone = 0, kMmMinMax = 1, kMmAbsMax = 2 };

template <int IO, int ROPE, int QUANT, int MM = kMmNone>
__device__ __forceinline__ void rope_apply_store(const float (&acc)[32], const RopeTables<ROPE>& tab,
                                                 const KprojParams& p, int64_t m, int64_t out_row, int n_base,
                                                 int ch0, uint32_t* mm_row = nullptr, int lane = 0) {
  static_assert(QUANT == kQuantNone || ROPE != FFA_F32, "the fused quantisers take 16-bit K");
  static_assert(MM == kMmNone || (ROPE != FFA_F32 && QUANT == kQuantNone), "min/max in the epilogue: 16-bit K, no fused quantiser");
  uint32_t wk[MM != kMmNone ? 16 : 1];             // the row's 32 K values as packed pairs (|K| for NF4)
  using P = Pack16<IO>;
  using T2 = typename P::T2;
  const int64_t o = m * p.N + n_base + ch0;
  // activations: fp32 accumulator (+ bias) rounded to the activation dtype, as packed pairs
  T2 x2[16];
  if (p.bias) {
    const uint4* b4 = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.bias) + n_base + ch0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 b = b4[i];
      const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 bf = P::to_floats(*reinterpret_cast<const T2*>(&bw[j]));
        x2[4 * i + j] = P::from_floats(__fadd_rn(acc[8 * i + 2 * j], bf.x), __fadd_rn(acc[8 * i + 2 * j + 1], bf.y));
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) x2[i] = P::from_floats(acc[2 * i], acc[2 * i + 1]);
  }
  if constexpr (ROPE != FFA_F32) {
    uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.k_out) + o);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t cw[4] = {tab.c[i].x, tab.c[i].y, tab.c[i].z, tab.c[i].w};
      const uint32_t sw[4] = {tab.s[i].x, tab.s[i].y, tab.s[i].z, tab.s[i].w};
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const T2 x = x2[4 * i + j];
        // rotate_half of the pair (x0, x1) is (-x1, x0): swap the halves, flip the sign of the low one
        const uint32_t xr = __byte_perm(*reinterpret_cast<const uint32_t*>(&x), 0u, 0x1032) ^ 0x00008000u;
        const T2 a = __hmul2(x, *reinterpret_cast<const T2*>(&cw[j]));
        const T2 b = __hmul2(*reinterpret_cast<const T2*>(&xr), *reinterpret_cast<const T2*>(&sw[j]));
        const T2 r = __hadd2(a, b);
        w[j] = *reinterpret_cast<const uint32_t*>(&r);
      }
      if (p.k_out) dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
      if constexpr (MM != kMmNone) {
#pragma unroll
        for (int j = 0; j < 4; ++j) wk[4 * i + j] = MM == kMmAbsMax ? (w[j] & 0x7fff7fffu) : w[j];
      }
      if constexpr (QUANT != kQuantNone) {
        // the reference quantisers on these eight K values (ffa_numeric.h has the per-element rules)
        constexpr int kF8 = (QUANT == kQuantFp8E4 || QUANT == kQuantFp4E4) ? num::kE4M3 : num::kE5M2;
        float kf[8], rf[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = P::to_floats(*reinterpret_cast<const T2*>(&w[j]));
          kf[2 * j] = f.x; kf[2 * j + 1] = f.y;
        }
        const int64_t oe = out_row * p.N + n_base + ch0 + 8 * i;       // element index in the pools
        if constexpr (QUANT == kQuantFp8E4 || QUANT == kQuantFp8E5) {
          const uint2 base = num::narrow8<kF8>(kf);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 d = num::fp8x2_to_f32x2<kF8>((j < 2 ? base.x : base.y) >> (16 * (j & 1)));
            rf[2 * j] = kf[2 * j] - d.x;
            rf[2 * j + 1] = kf[2 * j + 1] - d.y;
          }
          *reinterpret_cast<uint2*>(p.codes + oe) = base;
        } else {
          uint32_t c = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) c |= num::fp4_encode_f(kf[j], IO, &rf[j]) << (4 * j);
          *reinterpret_cast<uint32_t*>(p.codes + oe / 2) = c;
        }
        *reinterpret_cast<uint2*>(p.residual + oe) = num::narrow8<kF8>(rf);
      }
    }
    if constexpr (MM != kMmNone) {
      // Transposing butterfly over the warp's 32 rows on packed pairs: at lane bit b a lane keeps one half
      // of its registers and trades the other half with lane ^ (1 << b), so after bits 4..1 lane L holds
      // pair L >> 1 reduced over 16 rows, and bit 0 finishes it: lane L ends with channel L.
      auto mn = [](uint32_t a, uint32_t b) {
        const T2 r = __hmin2(*reinterpret_cast<const T2*>(&a), *reinterpret_cast<const T2*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
      };
      auto mx = [](uint32_t a, uint32_t b) {
        const T2 r = __hmax2(*reinterpret_cast<const T2*>(&a), *reinterpret_cast<const T2*>(&b));
        return *reinterpret_cast<const uint32_t*>(&r);
      };
      uint32_t lo[8], hi[8];
      {
        const bool up = (lane & 16) != 0;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          const uint32_t keep = up ? wk[r + 8] : wk[r];
          const uint32_t got = __shfl_xor_sync(0xffffffffu, up ? wk[r] : wk[r + 8], 16);
          lo[r] = mn(keep, got);
          hi[r] = mx(keep, got);
        }
      }
#pragma unroll
      for (int half = 4; half >= 1; half >>= 1) {   // lane bits 3, 2, 1
        const bool up = (lane & (2 * half)) != 0;
#pragma unroll
        for (int r = 0; r < half; ++r) {
          const uint32_t keep_hi = up ? hi[r + half] : hi[r];
          const uint32_t got_hi = __shfl_xor_sync(0xffffffffu, up ? hi[r] : hi[r + half], 2 * half);
          hi[r] = mx(keep_hi, got_hi);
          if (MM == kMmMinMax) {
            const uint32_t keep_lo = up ? lo[r + half] : lo[r];
            const uint32_t got_lo = __shfl_xor_sync(0xffffffffu, up ? lo[r] : lo[r + half], 2 * half);
            lo[r] = mn(keep_lo, got_lo);
          }
        }
      }
      hi[0] = mx(hi[0], __shfl_xor_sync(0xffffffffu, hi[0], 1));
      if (MM == kMmMinMax) lo[0] = mn(lo[0], __shfl_xor_sync(0xffffffffu, lo[0], 1));
      const float2 flo = P::to_floats(*reinterpret_cast<const T2*>(&lo[0]));
      const float2 fhi = P::to_floats(*reinterpret_cast<const T2*>(&hi[0]));
      const uint32_t ulo = __float_as_uint((lane & 1) ? flo.y : flo.x), uhi = __float_as_uint((lane & 1) ? fhi.y : fhi.x);
      reinterpret_cast<uint2*>(mm_row)[lane] =
          make_uint2(MM == kMmMinMax ? ((ulo & 0x80000000u) ? ~ulo : (ulo | 0x80000000u)) : 0u,
                     (uhi & 0x80000000u) ? ~uhi : (uhi | 0x80000000u));
    }
  } else {
    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(p.k_out) + o);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 c = tab.c[i], s = tab.s[i];
      const float2 xa = P::to_floats(x2[2 * i]), xb = P::to_floats(x2[2 * i + 1]);
      float4 r;
      r.x = __fadd_rn(__fmul_rn(xa.x, c.x), __fmul_rn(-xa.y, s.x));
      r.y = __fadd_rn(__fmul_rn(xa.y, c.y), __fmul_rn(xa.x, s.y));
      r.z = __fadd_rn(__fmul_rn(xb.x, c.z), __fmul_rn(-xb.y, s.z));
      r.w = __fadd_rn(__fmul_rn(xb.y, c.w), __fmul_rn(xb.x, s.w));
      dst[i] = r;
    }
  }
}

template <int IO, int ROPE, int QUANT>
__device__ __forceinline__ void rope_store_32_t(const float (&acc)[32], const KprojParams& p, int64_t m, int n_base,
                                                int ch0) {
  RopeTables<ROPE> tab;
  tab.load(p, m % p.T, ch0);
  rope_apply_store<IO, ROPE, QUANT>(acc, tab, p, m, QUANT != kQuantNone ? out_row_of(p, m) : m, n_base, ch0);
}

// Fused epilogue of one token row of a finished [128, BN] accumulator: the heads of the tile share
// the row's cos/sin, so each 32-channel slice of the tables is loaded once (the next slice while the
// current one is used) and applied to every head.  All 32 lanes run the TMEM loads; rows beyond M
// only skip the global loads and stores.  The accumulator is released once the last TMEM load has landed.
template <int IO, int ROPE, int QUANT, int BN, int MM>
__device__ __forceinline__ void epilogue_row(const KprojParams& p, uint32_t taddr, int64_t m, int n0,
                                             uint32_t bar_release, int lane) {
  constexpr int kHeads = BN / kHeadDim;
  constexpr int kSlices = kHeadDim / 32;
  const bool valid = m < p.M;
  const int64_t tok = valid ? m % p.T : 0;
  const int64_t out_row = (valid && QUANT != kQuantNone) ? out_row_of(p, m) : m;
  auto one_slice = [&](int c, const RopeTables<ROPE>& tab) {
#pragma unroll
    for (int hd = 0; hd < kHeads; ++hd) {
      float v[32];
      tmem_ld32(v, taddr + hd * kHeadDim + 32 * c);
      if (c == kSlices - 1 && hd == kHeads - 1) {
        // everything is in registers: hand the accumulator back to the MMA warp
        asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar_release) : "memory");
      }
      if constexpr (MM != kMmNone) {
        // every row of the tile exists (the host checked): the whole warp takes part in the reductions
        uint32_t* mm_row = p.mm_part + ((m >> 5) * p.N + n0 + hd * kHeadDim + 32 * c) * 2;
        rope_apply_store<IO, ROPE, QUANT, MM>(v, tab, p, m, out_row, n0 + hd * kHeadDim, 32 * c, mm_row, lane);
      } else {
        if (valid) rope_apply_store<IO, ROPE, QUANT>(v, tab, p, m, out_row, n0 + hd * kHeadDim, 32 * c);
      }
    }
  };
  if constexpr (ROPE == FFA_F32) {
    // fp32 tables take 64 registers per slice: one slice at a time
#pragma unroll 1
    for (int c = 0; c < kSlices; ++c) {
      RopeTables<ROPE> tab;
      if (valid) tab.load(p, tok, 32 * c);
      one_slice(c, tab);
    }
  } else {
    // 16-bit tables (32 registers per slice) are double-buffered
    RopeTables<ROPE> tab[2];
    if (valid) tab[0].load(p, tok, 0);
#pragma unroll
    for (int c = 0; c < kSlices; ++c) {
      if (valid && c + 1 < kSlices) tab[(c + 1) & 1].load(p, tok, 32 * (c + 1));
      one_slice(c, tab[c & 1]);
    }
  }
}

// Persistent kernel: work item w -> (m tile, n tile, k split); CTA c takes items c, c + grid, ...
// With n_split == 1 the epilogue is fused (bias, rounding, RoPE, store K); with n_split > 1 (few
// tokens: the GEMM is then a stream over W_k and needs more CTAs than output tiles) each item
// stores its fp32 partial tile and kproj_finish_kernel adds the splits and applies the epilogue.
template <int BN, int IO, int ROPE, int QUANT, int MM>
__global__ void __launch_bounds__(kThreadsK) kproj_rope_kernel(const __grid_constant__ KprojParams p,
                                                               const __grid_constant__ CUtensorMap tm_a,
                                                               const __grid_constant__ CUtensorMap tm_b) {
  using TL = Tile<BN>;
  constexpr int kStages = TL::kStages;
  constexpr int kBN = BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bars = smem_u32(smem + TL::kOffBars);
  const uint32_t bar_full = bars, bar_empty = bars + 8 * kStages;
  const uint32_t bar_tfull = bars + 16 * kStages, bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + TL::kOffTmem);
  auto a_tile = [&](int s) { return smem + s * TL::kStageBytes; };
  auto b_tile = [&](int s) { return smem + s * TL::kStageBytes + kTileBytes; };
  const int n_tiles = p.N / kBN;
  const int k_iters = p.H / kBK / p.n_split;                 // per work item
  const int n_items = p.m_tiles * n_tiles * p.n_split;
  bool timed_out = false;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(bar_tfull + 8 * i, 1); mbar_init(bar_tempty + 8 * i, 4); }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (warp == 1) {   // one warp allocates two accumulators' worth of tensor-memory columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)),
                 "r"(TL::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  auto decode_item = [&](int w, int& m0, int& n0, int& k0) {
    const int split = w % p.n_split;
    const int tile = w / p.n_split;
    n0 = (tile % n_tiles) * kBN;
    m0 = (tile / n_tiles) * kBM;
    k0 = split * k_iters * kBK;
  };

  if (warp == 0) {
    // ---- TMA producer ---------------------------------------------------------------------------
    if (lane == 0) {
      int it = 0;
      for (int w = blockIdx.x; w < n_items; w += gridDim.x) {
        int m0, n0, k0;
        decode_item(w, m0, n0, k0);
        for (int k = 0; k < k_iters; ++k, ++it) {
          const int s = it % kStages;
          if (it >= kStages) timed_out |= !mbar_wait(bar_empty + 8 * s, ((it / kStages) - 1) & 1, timed_out);
          mbar_expect_tx(bar_full + 8 * s, TL::kStageBytes);
          tma_load_2d(smem_u32(a_tile(s)), &tm_a, k0 + k * kBK, m0, bar_full + 8 * s);
          tma_load_2d(smem_u32(b_tile(s)), &tm_b, k0 + k * kBK, n0, bar_full + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -----------------------------------------------------------------------------
    if (lane == 0) {
      const uint32_t idesc = instr_desc(IO == FFA_BF16 ? 1u : 0u, kBN);
      int it = 0, local = 0;
      for (int w = blockIdx.x; w < n_items; w += gridDim.x, ++local) {
        const int buf = local & 1;
        // the epilogue must have drained this accumulator (two items ago)
        if (local >= 2) timed_out |= !mbar_wait(bar_tempty + 8 * buf, ((local >> 1) - 1) & 1, timed_out);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t tmem_d = tmem_base + buf * kBN;
        for (int k = 0; k < k_iters; ++k, ++it) {
          const int s = it % kStages;
          timed_out |= !mbar_wait(bar_full + 8 * s, (it / kStages) & 1, timed_out);
          asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
          const uint64_t da = smem_desc_sw128(smem_u32(a_tile(s)));
          const uint64_t db = smem_desc_sw128(smem_u32(b_tile(s)));
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) umma_f16(tmem_d, da + 2 * kk, db + 2 * kk, idesc, (k | kk) != 0 ? 1u : 0u);
          umma_commit(bar_empty + 8 * s);        // frees the stage once these MMAs have read it
        }
        umma_commit(bar_tfull + 8 * buf);        // accumulator complete
      }
    }
  } else {
    // ---- epilogue: one token row per thread --------------------------------------------------------
    const int q = warp & 3;                      // TMEM lane quarter this warp may read
    const int row = 32 * q + lane;
    int local = 0;
    for (int w = blockIdx.x; w < n_items; w += gridDim.x, ++local) {
      int m0, n0, k0;
      decode_item(w, m0, n0, k0);
      const int buf = local & 1;
      const int64_t m = static_cast<int64_t>(m0) + row;
      timed_out |= !mbar_wait(bar_tfull + 8 * buf, (local >> 1) & 1, timed_out);
      asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(32 * q) << 16) + buf * kBN;
      const uint32_t bar_release = bar_tempty + 8 * buf;
      if (p.n_split == 1) {
        epilogue_row<IO, ROPE, QUANT, kBN, MM>(p, taddr, m, n0, bar_release, lane);
      } else {
        const int split = w % p.n_split;
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
          float v[32];
          tmem_ld32(v, taddr + 32 * c);
          if (c == kBN / 32 - 1) {
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar_release) : "memory");
          }
          if (m < p.M) {
            float4* dst = reinterpret_cast<float4*>(p.partial + (static_cast<int64_t>(split) * p.M + m) * p.N + n0 + 32 * c);
#pragma unroll
            for (int i = 0; i < 8; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          }
        }
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TL::kTmemCols)
                 : "memory");
  }
  if (timed_out && p.status) atomicExch(p.status, 2);
}

// Adds the k-split partial tiles and applies the epilogue.  One warp per (token row, 32 channels):
// lane = (split mod 4, float4 index) so that a warp has four splits of its 32 channels in flight per
// step; the four split lanes are then folded with shuffles, the 32 sums meet in shared memory and
// lane 0 runs the epilogue.  (Few tokens only, so the idle lanes cost nothing; what mattered was the
// chain of dependent loads a single thread per row group used to walk: 13 us at T = 1.)
template <int IO, int ROPE, int QUANT>
__global__ void __launch_bounds__(128) kproj_finish_kernel(const __grid_constant__ KprojParams p) {
  __shared__ float s_sum[4][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = p.N / 32;
  const int64_t idx = blockIdx.x * 4LL + warp;
  const bool live = idx < static_cast<int64_t>(p.M) * groups;
  const int64_t m = live ? idx / groups : 0;
  const int n = live ? static_cast<int>(idx % groups) * 32 : 0;
  const int sub = lane >> 3, v4 = lane & 7;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (live) {
    for (int s = sub; s < p.n_split; s += 4) {
      const float4 x = *reinterpret_cast<const float4*>(p.partial + (static_cast<int64_t>(s) * p.M + m) * p.N + n + 4 * v4);
      acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
    }
  }
#pragma unroll
  for (int off = 8; off < 32; off <<= 1) {
    acc.x += __shfl_xor_sync(0xffffffffu, acc.x, off);
    acc.y += __shfl_xor_sync(0xffffffffu, acc.y, off);
    acc.z += __shfl_xor_sync(0xffffffffu, acc.z, off);
    acc.w += __shfl_xor_sync(0xffffffffu, acc.w, off);
  }
  if (sub == 0) *reinterpret_cast<float4*>(&s_sum[warp][4 * v4]) = acc;
  __syncwarp();
  if (live && lane == 0) {
    float sum[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) sum[i] = s_sum[warp][i];
    rope_store_32_t<IO, ROPE, QUANT>(sum, p, m, (n / kHeadDim) * kHeadDim, n % kHeadDim);
  }
}

// ---- a few token rows (one decode step of a batch, a short chunk): one launch ------------------------
//
// grid = (N / 32 column groups) x (cluster of CS CTAs along the hidden dimension), 256 threads.
// CTA (group, rank) owns channels [32 group, +32) x hidden slice [rank * H/CS, +H/CS), slice <= 1024.
// Warp w: channel half cw = w & 1 (16 channels = the 16 rows of an m16n8k16 A fragment), slice
// quarter kw = w >> 1.  A lane (g = lane / 4, t = lane % 4) loads 16 bytes (8 hidden elements) of
// weight rows g and g + 8 per 32-element step, once, and per block of eight token rows 16 bytes of
// token g's hidden row from shared memory; the eight elements feed two MMAs whose k positions are
// a permutation of the real ones, the same for both operands, so the dot products are the real
// ones.  D[channel][token] (fp32) goes to shared memory; the four slice quarters are added, then
// the ranks share out the blocks of eight rows: the owner of a block adds the CS ranks' [8][32]
// sums in rank order through distributed shared memory (so the result does not depend on timing)
// and one of its threads per token applies bias, rounding, RoPE and the fused quantiser.  NB = 1
// (up to eight rows) compiles the block loops away; NB = kFewBlocks serves up to 24 rows.
constexpr int kFewBlocks = 3;                     // blocks of eight token rows (the MMA's n extent) per call at most
constexpr int kFewRows = 8 * kFewBlocks;          // beyond that the tensor-memory GEMM with split k is faster
constexpr int kFewSlice = 1024;                   // hidden elements per CTA at most
constexpr int kFewPad = 32;                       // 64 bytes between token rows: conflict-free 16-byte reads
constexpr int kFewThreads = 256;

// dynamic shared memory of the few-row kernel: hidden rows, per-quarter sums, CTA sums, cluster sums
constexpr size_t few_smem_bytes(int rows, int slice) {
  return static_cast<size_t>(rows) * ((slice + kFewPad) * 2 + (4 * 32 + 32 + 33) * 4);
}

template <int IO>
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
  if constexpr (IO == FFA_BF16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

template <int IO, int ROPE, int QUANT, int NB>
__global__ void __launch_bounds__(kFewThreads) kproj_few_kernel(const __grid_constant__ KprojParams p) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  extern __shared__ __align__(16) uint8_t few_smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cs = static_cast<int>(cluster.num_blocks());
  const int rank = static_cast<int>(cluster.block_rank());
  const int group = blockIdx.x / cs;
  const int slice = p.H / cs, stride = slice + kFewPad;
  const int k0 = rank * slice;
  const int n0 = group * 32;
  const int cw = warp & 1, kw = warp >> 1;
  const int g = lane >> 2, t = lane & 3;
  const int quarter = slice / 4;                   // a multiple of 32
  const int n_steps = quarter / 32;                // <= 8
  const int nb = NB == 1 ? 1 : (p.M + 7) / 8;      // blocks of eight token rows (NB = 1: known when compiling)
  const int rows = 8 * nb;
  uint16_t* s_h = reinterpret_cast<uint16_t*>(few_smem);                      // [rows][stride]
  float* s_quarter = reinterpret_cast<float*>(few_smem + static_cast<size_t>(rows) * stride * 2);   // [4][32][rows]
  float* s_part = s_quarter + 4 * 32 * rows;       // [rows][32]: this CTA's sums, what the peers read
  float* s_sum = s_part + 32 * rows;               // [rows][33]

  // the weight first: every load of this lane is in flight before anything waits
  const uint16_t* wp = static_cast<const uint16_t*>(p.w);
  const uint16_t* w_lo = wp + static_cast<int64_t>(n0 + 16 * cw + g) * p.H + k0 + kw * quarter + 8 * t;
  const uint16_t* w_hi = w_lo + 8LL * p.H;
  uint4 wx[8], wy[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (j < n_steps) {
      wx[j] = __ldg(reinterpret_cast<const uint4*>(w_lo + 32 * j));
      wy[j] = __ldg(reinterpret_cast<const uint4*>(w_hi + 32 * j));
    }
  }
  // Row block b (eight tokens) is finished by rank b % cs: that rank adds the cluster's sums of the block
  // and runs its epilogue, thread i of the rank taking token 8 (rank + (i / 8) cs) + i % 8.  These threads
  // fetch their RoPE rows and cache slot now, off the tail.
  const int m_fin = 8 * (rank + (tid >> 3) * cs) + (tid & 7);
  const bool finisher = tid < 8 * NB && m_fin < p.M;
  RopeTables<ROPE> tab;
  int64_t out_row = m_fin;
  if (finisher) {
    tab.load(p, m_fin % p.T, n0 % kHeadDim);
    if (QUANT != kQuantNone) out_row = out_row_of(p, m_fin);
  }
  // the token rows' hidden slice (rows beyond M are zero)
  const uint16_t* hp = static_cast<const uint16_t*>(p.h);
  const int vec_per_row = slice / 8;
  const uint32_t s_h_addr = smem_u32(s_h);
  for (int i = tid; i < rows * vec_per_row; i += kFewThreads) {
    const int row = i / vec_per_row, c8 = i % vec_per_row;
    const bool live = row < p.M;                   // asynchronous 16-byte copies, all in flight; zero fill beyond M
    const uint16_t* src = hp + static_cast<int64_t>(live ? row : 0) * p.H + k0 + 8 * c8;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s_h_addr + 2u * (row * stride + 8 * c8)),
                 "l"(src), "r"(live ? 16 : 0)
                 : "memory");
  }
  asm volatile("cp.async.wait_all;\n" ::: "memory");
  __syncthreads();

  // One block of eight token rows at a time (a rolled loop: every instruction of this kernel runs once
  // or twice per warp, so its time follows its code size); two accumulators halve the MMA chain.
  const uint16_t* h_lane = &s_h[g * stride + kw * quarter + 8 * t];
  float* q_lo = s_quarter + (kw * 32 + 16 * cw + g) * rows + 2 * t;     // D[channel g (+8)][token 8 b + 2 t (+1)]
  float* q_hi = q_lo + 8 * rows;
#pragma unroll 1
  for (int b = 0; b < nb; ++b) {
    float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (j < n_steps) {
        const uint4 hv = *reinterpret_cast<const uint4*>(h_lane + 8 * b * stride + 32 * j);
        mma_16816<IO>(d0, wx[j].x, wy[j].x, wx[j].y, wy[j].y, hv.x, hv.y);
        mma_16816<IO>(d1, wx[j].z, wy[j].z, wx[j].w, wy[j].w, hv.z, hv.w);
      }
    }
    *reinterpret_cast<float2*>(q_lo + 8 * b) = make_float2(d0[0] + d1[0], d0[1] + d1[1]);
    *reinterpret_cast<float2*>(q_hi + 8 * b) = make_float2(d0[2] + d1[2], d0[3] + d1[3]);
  }
  __syncthreads();
  const int tok8 = tid >> 5, ch = tid & 31;
#pragma unroll 1
  for (int b = 0; b < nb; ++b) {
    const float* q = s_quarter + ch * rows + 8 * b + tok8;
    s_part[256 * b + tid] = (q[0] + q[32 * rows]) + (q[64 * rows] + q[96 * rows]);
  }
  cluster.sync();                                  // every rank's s_part is complete and visible
  // this rank's blocks: the remote values of a block are loaded together, the sum runs in rank order
#pragma unroll 1
  for (int i = 0, b = rank; b < nb; ++i, b += cs) {
    float v[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) v[r] = r < cs ? cluster.map_shared_rank(s_part, r)[256 * b + tid] : 0.f;
    float acc = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) acc += v[r];
    s_sum[(8 * i + tok8) * 33 + ch] = acc;
  }
  cluster.sync();                                  // the peers' shared memory has been read: they may exit
  if (!finisher) return;
  float sum[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) sum[i] = s_sum[tid * 33 + i];
  rope_apply_store<IO, ROPE, QUANT>(sum, tab, p, m_fin, out_row, (n0 / kHeadDim) * kHeadDim, n0 % kHeadDim);
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      sym = nullptr;
    return reinterpret_cast<EncodeTiledFn>(sym);
  }();
  return fn;
}

// [rows, cols] 16-bit row-major, box = box_rows rows x 64 columns, 128-byte swizzle
bool make_operand_map(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int box_rows) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {kBK, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

size_t elem_size(int dt) { return dt == FFA_F32 ? 4 : 2; }
size_t align256(size_t x) { return (x + 255) / 256 * 256; }

constexpr size_t kPartialCap = 16u << 20;      // k-split partial tiles never take more than this
constexpr int kFewTiles = 74;                  // below half the SMs' worth of tiles, split K

int sm_count() {
  static int sms = [] {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    return n;
  }();
  return sms;
}

// Number of k splits for an [M, N] output with k_total_iters 64-wide k steps.
int plan_split(int64_t M, int N, int k_total_iters) {
  const int64_t tiles = ((M + kBM - 1) / kBM) * (N / 128);
  if (tiles >= kFewTiles) return 1;
  int64_t limit = sm_count() / tiles;
  const int64_t by_mem = static_cast<int64_t>(kPartialCap / (static_cast<size_t>(M) * N * 4));
  if (by_mem < limit) limit = by_mem;
  if (limit > 16) limit = 16;
  int split = 1;
  while (split * 2 <= limit && k_total_iters % (split * 2) == 0) split *= 2;
  return split;
}

size_t partial_reserve(int64_t M, int N) {
  const int64_t tiles = ((M + kBM - 1) / kBM) * (N / 128);
  if (tiles >= kFewTiles) return 0;
  const size_t full = static_cast<size_t>(16) * M * N * 4;
  return align256(full < kPartialCap ? full : kPartialCap);
}

// The epilogue can reduce the per-channel min/max the 2-bit and NF4 scales need (one pair per 32 token
// rows and channel, folded by a small kernel afterwards) when every tile is full and belongs to
// one sequence (T a multiple of the tile height) and the GEMM is not split along k.
bool minmax_in_epilogue(int T, int64_t M, int N) {
  return T % kBM == 0 && ((M + kBM - 1) / kBM) * (N / 128) >= kFewTiles;
}
size_t minmax_part_reserve(int T, int64_t M, int N) {
  return minmax_in_epilogue(T, M, N) ? align256(static_cast<size_t>(M / 32) * N * 2 * sizeof(uint32_t)) : 0;
}

// Cluster size along the hidden dimension for the few-row kernel, or 0 when the shape does not fit it
// (more than kFewRows token rows, or a hidden size it cannot slice):
// the slice of one CTA is at most kFewSlice elements and a multiple of 128 (four warps x 32-element
// steps); more ranks are added while the grid stays within one CTA per SM.
int plan_few(int64_t M, int N, int H) {
  if (M > kFewRows || N % 32 != 0) return 0;
  int cs = 0;
  for (int c = 1; c <= 8; c *= 2)
    if (H % (c * 128) == 0 && H / c <= kFewSlice) { cs = c; break; }
  if (!cs) return 0;
  while (cs < 8 && H % (2 * cs * 128) == 0 && static_cast<int64_t>(N / 32) * 2 * cs <= sm_count()) cs *= 2;
  return cs;
}

}  // namespace
}  // namespace ffa

using namespace ffa;

extern "C" size_t ffa_kproj_workspace_bytes(int32_t B, int32_t T, int32_t HKV, int32_t rope_dtype) {
  if (B <= 0 || T <= 0 || HKV <= 0) return 0;
  const int64_t M = static_cast<int64_t>(B) * T;
  const int N = HKV * kHeadDim;
  const size_t k_bytes = static_cast<size_t>(M) * N * elem_size(rope_dtype == FFA_F32 ? FFA_F32 : FFA_BF16);
  return align256(k_bytes) + align256(ffa_quantize_scratch_bytes(B, HKV)) + partial_reserve(M, N) +
         minmax_part_reserve(T, M, N) + 256;
}

extern "C" int ffa_kproj_rope(const FfaKprojArgs* a, ffa_stream_t stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (!a || !a->h || !a->w || !a->cos || !a->sin) return FFA_E_NULL;
  if (a->B <= 0 || a->T <= 0 || a->HKV <= 0 || a->H <= 0 || a->head_dim != kHeadDim) return FFA_E_SHAPE;
  if (a->H % kBK != 0) return FFA_E_SHAPE;
  if (a->io_dtype != FFA_F16 && a->io_dtype != FFA_BF16) return FFA_E_DTYPE;
  if (a->rope_dtype != FFA_F32 && a->rope_dtype != a->io_dtype) return FFA_E_DTYPE;
  if (!encode_fn()) return FFA_E_LAUNCH;
  if (a->slot_table && a->slot_pos0 != 0 && a->variant != FFA_K_FP8 && a->variant != FFA_K_FP4) return FFA_E_VARIANT;
  if (a->slot_table && a->slot_pos0 < 0) return FFA_E_SHAPE;
  const int64_t M = static_cast<int64_t>(a->B) * a->T;
  const int N = a->HKV * kHeadDim;
  if (M > 0x7fffffffLL) return FFA_E_LIMIT;
  const int out_dt = a->rope_dtype == FFA_F32 ? FFA_F32 : a->io_dtype;

  // workspace: [post-RoPE K][quantiser min/max][k-split partial tiles or per-32-row min/max][status]
  const size_t k_bytes = align256(static_cast<size_t>(M) * N * elem_size(out_dt));
  const size_t q_bytes = align256(ffa_quantize_scratch_bytes(a->B, a->HKV));
  const size_t p_bytes = partial_reserve(M, N) + minmax_part_reserve(a->T, M, N);   // never both
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  if (!ws || a->workspace_bytes < k_bytes + q_bytes + p_bytes + 256) return FFA_E_WORKSPACE;
  void* k_rope = a->k_rope_out ? a->k_rope_out : static_cast<void*>(ws);
  const bool need_quant = a->variant >= 0;

  // two heads per tile when that still leaves at least one tile per SM
  const int64_t m_tiles = (M + kBM - 1) / kBM;
  const int bn = (N % 256 == 0 && m_tiles * (N / 256) >= sm_count()) ? 256 : 128;
  // a handful of token rows (one decode step) go through the one-launch kernel
  const bool aligned16 = ((reinterpret_cast<uintptr_t>(a->h) | reinterpret_cast<uintptr_t>(a->w)) & 15u) == 0;
  const int few_cs = aligned16 ? plan_few(M, N, a->H) : 0;
  alignas(64) CUtensorMap ma, mb;
  if (!few_cs && (!make_operand_map(&ma, a->h, M, a->H, kBM) || !make_operand_map(&mb, a->w, N, a->H, bn)))
    return FFA_E_LAUNCH;

  KprojParams p{};
  p.bias = a->bias; p.cos = a->cos; p.sin = a->sin; p.k_out = k_rope;
  p.h = a->h; p.w = a->w;
  p.status = reinterpret_cast<int*>(ws + k_bytes + q_bytes + p_bytes);
  p.partial = reinterpret_cast<float*>(ws + k_bytes + q_bytes);
  p.M = static_cast<int>(M); p.T = a->T; p.N = N; p.H = a->H;
  p.m_tiles = static_cast<int>(m_tiles);
  p.n_split = bn == 256 ? 1 : plan_split(M, N, a->H / kBK);
  p.io_dtype = a->io_dtype; p.rope_dtype = a->rope_dtype;
  p.mm_part = reinterpret_cast<uint32_t*>(ws + k_bytes + q_bytes);
  int mm_mode = kMmNone;
  if (need_quant && out_dt != FFA_F32 && !few_cs && p.n_split == 1 && minmax_in_epilogue(a->T, M, N) &&
      (a->variant == FFA_K_Q2 || a->variant == FFA_K_NF4))
    mm_mode = a->variant == FFA_K_Q2 ? kMmMinMax : kMmAbsMax;

  // the elementwise formats are quantised inside the epilogue when K is 16-bit; K itself is then
  // written only if the caller asked for it
  int quant = kQuantNone;
  if (need_quant && out_dt != FFA_F32 && (a->variant == FFA_K_FP8 || a->variant == FFA_K_FP4)) {
    if (!a->codes || !a->residual) return FFA_E_NULL;
    if ((reinterpret_cast<uintptr_t>(a->codes) | reinterpret_cast<uintptr_t>(a->residual)) & 15u) return FFA_E_ALIGN;
    quant = a->variant == FFA_K_FP8 ? (a->fp8_format == FFA_E4M3 ? kQuantFp8E4 : kQuantFp8E5)
                                    : (a->fp8_format == FFA_E4M3 ? kQuantFp4E4 : kQuantFp4E5);
    p.codes = static_cast<uint8_t*>(a->codes);
    p.residual = static_cast<uint8_t*>(a->residual);
    p.slot_table = a->slot_table;
    p.slot_stride = a->slot_stride;
    p.slot_pos0 = a->slot_table ? a->slot_pos0 : 0;
    if (!a->k_rope_out) p.k_out = nullptr;
  }

  const int64_t items = static_cast<int64_t>(p.m_tiles) * (N / bn) * p.n_split;
  const unsigned grid = static_cast<unsigned>(items < sm_count() ? items : sm_count());
  const int64_t finish_warps = M * (N / 32);
  const unsigned finish_grid = static_cast<unsigned>((finish_warps + 3) / 4);
  int dev = 0;
  cudaGetDevice(&dev);
  // one kernel per (tile width, activation dtype, table dtype, fused quantiser); each raises its
  // shared-memory limit the first time it runs on a device
#define FFA_KPROJ_LAUNCH(BN_, IO_, ROPE_, Q_, MM_)                                                                  \
  do {                                                                                                             \
    if (few_cs) {                                                                                                  \
      cudaLaunchConfig_t cfg = {};                                                                                 \
      cfg.gridDim = dim3(static_cast<unsigned>(N / 32) * few_cs);                                                  \
      cfg.blockDim = dim3(kFewThreads);                                                                            \
      cfg.stream = st;                                                                                             \
      cudaLaunchAttribute attr[1];                                                                                 \
      attr[0].id = cudaLaunchAttributeClusterDimension;                                                            \
      attr[0].val.clusterDim.x = static_cast<unsigned>(few_cs);                                                    \
      attr[0].val.clusterDim.y = 1;                                                                                \
      attr[0].val.clusterDim.z = 1;                                                                                \
      cfg.attrs = attr;                                                                                            \
      cfg.numAttrs = 1;                                                                                            \
      cfg.dynamicSmemBytes = few_smem_bytes(static_cast<int>((M + 7) / 8 * 8), a->H / few_cs);                     \
      cudaError_t ce;                                                                                              \
      if (M <= 8) {                                                                                                \
        ce = cudaLaunchKernelEx(&cfg, kproj_few_kernel<IO_, ROPE_, Q_, 1>, p);                                     \
      } else {                                                                                                     \
        static bool few_configured[64] = {};                                                                       \
        if (dev >= 0 && dev < 64 && !few_configured[dev]) {                                                        \
          ce = cudaFuncSetAttribute(kproj_few_kernel<IO_, ROPE_, Q_, kFewBlocks>,                                  \
                                    cudaFuncAttributeMaxDynamicSharedMemorySize,                                   \
                                    static_cast<int>(few_smem_bytes(kFewRows, kFewSlice)));                        \
          if (ce != cudaSuccess) return note_cuda_error(ce, "cudaFuncSetAttribute(kproj_few)");                    \
          few_configured[dev] = true;                                                                              \
        }                                                                                                          \
        ce = cudaLaunchKernelEx(&cfg, kproj_few_kernel<IO_, ROPE_, Q_, kFewBlocks>, p);                            \
      }                                                                                                            \
      if (ce != cudaSuccess) return note_cuda_error(ce, "kproj_few launch");                                       \
      break;                                                                                                       \
    }                                                                                                              \
    static bool configured[64] = {};                                                                               \
    if (dev >= 0 && dev < 64 && !configured[dev]) {                                                                \
      cudaError_t ce = cudaFuncSetAttribute(kproj_rope_kernel<BN_, IO_, ROPE_, Q_, MM_>,                            \
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, Tile<BN_>::kBytes);       \
      if (ce != cudaSuccess) return note_cuda_error(ce, "cudaFuncSetAttribute(kproj_rope)");                       \
      configured[dev] = true;                                                                                      \
    }                                                                                                              \
    kproj_rope_kernel<BN_, IO_, ROPE_, Q_, MM_><<<grid, kThreadsK, Tile<BN_>::kBytes, st>>>(p, ma, mb);             \
    if (p.n_split > 1 && cudaPeekAtLastError() == cudaSuccess)                                                     \
      kproj_finish_kernel<IO_, ROPE_, Q_><<<finish_grid, 128, 0, st>>>(p);                                         \
  } while (0)
#define FFA_KPROJ_Q(BN_, IO_)                                                                                      \
  do {                                                                                                             \
    switch (quant) {                                                                                               \
      case kQuantFp8E4: FFA_KPROJ_LAUNCH(BN_, IO_, IO_, kQuantFp8E4, kMmNone); break;                              \
      case kQuantFp8E5: FFA_KPROJ_LAUNCH(BN_, IO_, IO_, kQuantFp8E5, kMmNone); break;                              \
      case kQuantFp4E4: FFA_KPROJ_LAUNCH(BN_, IO_, IO_, kQuantFp4E4, kMmNone); break;                              \
      case kQuantFp4E5: FFA_KPROJ_LAUNCH(BN_, IO_, IO_, kQuantFp4E5, kMmNone); break;                              \
      default:                                                                                                     \
        if (mm_mode == kMmMinMax) FFA_KPROJ_LAUNCH(BN_, IO_, IO_, kQuantNone, kMmMinMax);                          \
        else if (mm_mode == kMmAbsMax) FFA_KPROJ_LAUNCH(BN_, IO_, IO_, kQuantNone, kMmAbsMax);                     \
        else FFA_KPROJ_LAUNCH(BN_, IO_, IO_, kQuantNone, kMmNone);                                                 \
        break;                                                                                                     \
    }                                                                                                              \
  } while (0)
#define FFA_KPROJ_BN(BN_)                                                                                          \
  do {                                                                                                             \
    if (a->io_dtype == FFA_BF16) {                                                                                 \
      if (a->rope_dtype == FFA_F32) FFA_KPROJ_LAUNCH(BN_, FFA_BF16, FFA_F32, kQuantNone, kMmNone);                 \
      else FFA_KPROJ_Q(BN_, FFA_BF16);                                                                             \
    } else {                                                                                                       \
      if (a->rope_dtype == FFA_F32) FFA_KPROJ_LAUNCH(BN_, FFA_F16, FFA_F32, kQuantNone, kMmNone);                  \
      else FFA_KPROJ_Q(BN_, FFA_F16);                                                                              \
    }                                                                                                              \
  } while (0)
  if (bn == 256) FFA_KPROJ_BN(256);
  else FFA_KPROJ_BN(128);
#undef FFA_KPROJ_BN
#undef FFA_KPROJ_Q
#undef FFA_KPROJ_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return note_cuda_error(e, "kproj_rope launch");
  if (!need_quant || quant != kQuantNone) return FFA_OK;
  if (mm_mode != kMmNone)
    return quantize_from_partials(a->variant, k_rope, out_dt, a->B, a->T, a->HKV, a->fp8_format,
                                  static_cast<uint8_t*>(a->codes), a->scale, a->zero,
                                  static_cast<uint8_t*>(a->residual), ws + k_bytes, p.mm_part, a->T / 32,
                                  a->slot_table, a->slot_stride, st);
  return quantize_dispatch(a->variant, k_rope, out_dt, a->B, a->T, a->HKV, a->fp8_format, a->page_size,
                           static_cast<uint8_t*>(a->codes), a->scale, a->zero, static_cast<uint8_t*>(a->residual),
                           ws + k_bytes, a->slot_table, a->slot_stride, a->slot_table ? a->slot_pos0 : 0, st);
}
