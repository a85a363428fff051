// Standalone K-cache quantisers for B200, bit-exact with the reference's torch functions
// (ffa-*/fused_kproj_rope_*.py; see ffa_numeric.h for the per-element arithmetic).
//
// The reference runs ~10 eager torch kernels with full-size temporaries per quantiser; here
// each format is one streaming pass over K (two for the formats whose scale depends on the
// whole sequence: a per-channel min/max reduction, then the encode pass).  All passes are
// HBM-bound: every K element is read once per pass with 8- or 16-byte loads and every output
// byte is written once.
#include "ffa_common.cuh"
#include "ffa_numeric.h"

namespace ffa {
namespace {

using namespace num;

constexpr int D = kHeadDim;

// order-preserving float <-> uint map, so that atomicMin/atomicMax on uint order floats
__device__ __forceinline__ uint32_t ord_encode(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float ord_decode(uint32_t u) {
  return __uint_as_float((u & 0x80000000u) ? (u & 0x7fffffffu) : ~u);
}

// Output token row of input row (b*T + t): identity, or through a slot table [B, stride] of page
// ids (page = 64 tokens) when the codes are scattered straight into a paged cache.
struct RowMap {
  const int32_t* table;
  int stride;
  int T;
  int pos0;     // position in its sequence of token 0 of the input (appending to a cache)
  __device__ __forceinline__ int64_t operator()(int64_t row) const {
    if (!table) return row;
    const int64_t b = row / T, t = row % T + pos0;
    return static_cast<int64_t>(table[b * stride + t / kPage]) * kPage + t % kPage;
  }
};

// ---- eight consecutive elements per thread ------------------------------------------------------
// Every pass moves K in 16-byte (16-bit K) or 2 x 16-byte (fp32 K) loads of eight consecutive
// channels and writes each output with one store of 2 to 8 bytes per thread, so a warp reads and
// writes whole 128-byte lines.  DT and F8 are compile-time so the per-element code has no branches
// on the element type.
template <int DT>
__device__ __forceinline__ void load8(const void* __restrict__ k, int64_t e, float (&x)[8]) {
  if (DT == kF32) {
    const float4 a = *reinterpret_cast<const float4*>(static_cast<const float*>(k) + e);
    const float4 b = *reinterpret_cast<const float4*>(static_cast<const float*>(k) + e + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  } else {
    const uint4 v = *reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(k) + e);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (DT == kBF16) {
        x[2 * i] = __uint_as_float(w[i] << 16);
        x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
        x[2 * i] = f.x; x[2 * i + 1] = f.y;
      }
    }
  }
}

// scratch: [B, HKV*128] x {min, max} as ordered uints
__global__ void minmax_init_kernel(uint32_t* mm, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    mm[2 * i] = ord_encode(INFINITY);
    mm[2 * i + 1] = ord_encode(-INFINITY);
  }
}

// One block per (b, slab of tokens).  A thread owns one group of eight channels and every
// `lanes`-th token of the slab; the block folds its token lanes in shared memory before the
// atomics, so each block issues one atomic pair per channel.
template <bool ABS, int DT>
__global__ void __launch_bounds__(256) minmax_kernel(const void* __restrict__ k, int T, int groups_per_row,
                                                     int tokens_per_block, uint32_t* mm) {
  extern __shared__ float s_fold[];                 // [lanes][groups_per_row * 8][2]
  const int b = blockIdx.y;
  const int t0 = blockIdx.x * tokens_per_block;
  const int t1 = min(T, t0 + tokens_per_block);
  const int row_elems = groups_per_row * 8;
  const int lanes = groups_per_row >= 256 ? 1 : 256 / groups_per_row;
  const int lane = groups_per_row >= 256 ? 0 : threadIdx.x / groups_per_row;
  const int g0 = groups_per_row >= 256 ? threadIdx.x : threadIdx.x % groups_per_row;
  if (lane < lanes) {
    for (int g = g0; g < groups_per_row; g += 256) {
      float lo[8], hi[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { lo[j] = INFINITY; hi[j] = -INFINITY; }
      // four token rows in flight per step
      for (int t = t0 + lane; t < t1; t += 4 * lanes) {
        float x[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int tt = t + u * lanes;
          if (tt < t1) load8<DT>(k, (static_cast<int64_t>(b) * T + tt) * row_elems + 8 * g, x[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (t + u * lanes < t1) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float v = ABS ? fabsf(x[u][j]) : x[u][j];
              lo[j] = fminf(lo[j], v);
              hi[j] = fmaxf(hi[j], v);
            }
          }
        }
      }
      if (lanes == 1) {
        uint32_t* slot = mm + 2 * (static_cast<int64_t>(b) * row_elems + 8 * g);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (!ABS) atomicMin(slot + 2 * j, ord_encode(lo[j]));
          atomicMax(slot + 2 * j + 1, ord_encode(hi[j]));
        }
      } else {
        float* f = s_fold + (static_cast<size_t>(lane) * row_elems + 8 * g) * 2;
#pragma unroll
        for (int j = 0; j < 8; ++j) { f[2 * j] = lo[j]; f[2 * j + 1] = hi[j]; }
      }
    }
  }
  if (lanes > 1) {
    __syncthreads();
    for (int c = threadIdx.x; c < row_elems; c += 256) {
      float lo = INFINITY, hi = -INFINITY;
      for (int l = 0; l < lanes; ++l) {
        lo = fminf(lo, s_fold[(static_cast<size_t>(l) * row_elems + c) * 2]);
        hi = fmaxf(hi, s_fold[(static_cast<size_t>(l) * row_elems + c) * 2 + 1]);
      }
      uint32_t* slot = mm + 2 * (static_cast<int64_t>(b) * row_elems + c);
      if (!ABS) atomicMin(slot, ord_encode(lo));
      atomicMax(slot + 1, ord_encode(hi));
    }
  }
}

// q2: finalise (scale, zero) per channel
__global__ void q2_finalize_kernel(const uint32_t* mm, int n, int dt, void* scale, void* zero) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s, z;
  q2_scale_zero(ord_decode(mm[2 * i]), ord_decode(mm[2 * i + 1]), dt, &s, &z);
  store_elem(scale, i, dt, s);
  store_elem(zero, i, dt, z);
}

__global__ void nf4_finalize_kernel(const uint32_t* mm, int n, int dt, void* scale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) store_elem(scale, i, dt, fmaxf(ord_decode(mm[2 * i + 1]), 1e-6f));
}

// Folds per-slab (min, max) pairs, parts[B * parts_per_b][n_cols][2] ordered uints (what the K-projection's
// epilogue leaves per 32 token rows), into mm[B][n_cols][2] and finalises the scales in the same
// pass.  Block = 32 channels x 32 slab lanes (every load of a thread in flight at once for up to
// 256 slabs), grid = (n_cols / 32, B).
template <bool ABS>
__global__ void __launch_bounds__(1024) minmax_fold_kernel(const uint32_t* __restrict__ parts, int parts_per_b,
                                                           int n_cols, uint32_t* __restrict__ mm, int dt,
                                                           void* scale, void* zero) {
  __shared__ uint32_t s_lo[32][33], s_hi[32][33];
  const int lane = threadIdx.x & 31, pl = threadIdx.x >> 5, b = blockIdx.y;
  const int c = blockIdx.x * 32 + lane;
  uint32_t lo = 0xffffffffu, hi = 0u;
  const uint2* src = reinterpret_cast<const uint2*>(parts) + static_cast<int64_t>(b) * parts_per_b * n_cols + c;
#pragma unroll 8
  for (int q = pl; q < parts_per_b; q += 32) {
    const uint2 v = src[static_cast<int64_t>(q) * n_cols];
    lo = min(lo, v.x);
    hi = max(hi, v.y);
  }
  s_lo[pl][lane] = lo;
  s_hi[pl][lane] = hi;
  __syncthreads();
  if (pl != 0) return;
#pragma unroll
  for (int q = 1; q < 32; ++q) { lo = min(lo, s_lo[q][lane]); hi = max(hi, s_hi[q][lane]); }
  const int64_t i = static_cast<int64_t>(b) * n_cols + c;
  mm[2 * i] = ABS ? ord_encode(0.f) : lo;
  mm[2 * i + 1] = hi;
  if (ABS) {
    store_elem(scale, i, dt, fmaxf(ord_decode(hi), 1e-6f));
  } else {
    float sc, z;
    q2_scale_zero(ord_decode(lo), ord_decode(hi), dt, &sc, &z);
    store_elem(scale, i, dt, sc);
    store_elem(zero, i, dt, z);
  }
}

// nf4 append: the encoder reads absmax as ordered uints; rebuild them from the (frozen) scale tensor
__global__ void nf4_mm_from_scale_kernel(const void* scale, int n, int dt, uint32_t* mm) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    mm[2 * i] = ord_encode(0.f);
    mm[2 * i + 1] = ord_encode(load_elem(scale, i, dt));
  }
}

// Encode pass of q2 / fp8fp8 / fp4 / nf4: a block walks token rows, a thread takes one group of
// eight channels of the row.  Two rows are in flight per thread.
enum { kEncFp8 = 0, kEncFp4 = 1, kEncNf4 = 2, kEncQ2 = 3 };

// NF4 level of idx from a table spread over the lanes of the warp (lane i < 16 holds level i)
__device__ __forceinline__ float nf4_level_shfl(float lane_level, uint32_t idx) {
  return __shfl_sync(0xffffffffu, lane_level, static_cast<int>(idx));
}

template <int KIND, int DT, int F8>
__device__ __forceinline__ void encode8(const float (&x)[8], const float (&p0)[8], const float (&p1)[8],
                                        float lane_level, uint8_t* __restrict__ codes, uint8_t* __restrict__ res,
                                        int64_t out_group, bool active) {
  float r[8];
  uint32_t c = 0, c_hi = 0;
  if (KIND == kEncFp8) {
    const uint2 base = narrow8<F8>(x);
    c = base.x; c_hi = base.y;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 lo = fp8x2_to_f32x2<F8>((j < 2 ? base.x : base.y) >> (16 * (j & 1)));
      r[2 * j] = x[2 * j] - lo.x;
      r[2 * j + 1] = x[2 * j + 1] - lo.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (KIND == kEncFp4) {
        c |= fp4_encode_f(x[j], DT, &r[j]) << (4 * j);
      } else if (KIND == kEncNf4) {
        const uint32_t idx = nf4_encode(x[j] / p0[j]);
        r[j] = nf4_residual_f(x[j], nf4_level_shfl(lane_level, idx), p0[j]);
        c |= idx << (4 * j);
      } else {
        c |= q2_encode_f(x[j], p0[j], p1[j], DT, &r[j]) << (2 * j);
      }
    }
  }
  if (!active) return;
  if (KIND == kEncFp8) reinterpret_cast<uint2*>(codes)[out_group] = make_uint2(c, c_hi);
  else if (KIND == kEncQ2) reinterpret_cast<uint16_t*>(codes)[out_group] = static_cast<uint16_t>(c);
  else reinterpret_cast<uint32_t*>(codes)[out_group] = c;
  reinterpret_cast<uint2*>(res)[out_group] = narrow8<F8>(r);
}

template <int KIND, int DT, int F8>
__global__ void __launch_bounds__(256) encode_rows_kernel(const void* __restrict__ k, uint32_t rows, int T,
                                                          int groups_per_row, const void* __restrict__ aux0,
                                                          const void* __restrict__ aux1, uint8_t* __restrict__ codes,
                                                          uint8_t* __restrict__ res, RowMap map) {
  // aux0 / aux1: q2 scale / zero in K's dtype, nf4 the min/max scratch (ordered uints), else unused.
  // Every thread runs every iteration (idle ones on zeros) so that warp shuffles stay legal.
  const int row_elems = groups_per_row * 8;
  const int rows_per_iter = groups_per_row >= 256 ? 1 : 256 / groups_per_row;
  const int sub = groups_per_row >= 256 ? 0 : threadIdx.x / groups_per_row;
  const int g0 = groups_per_row >= 256 ? threadIdx.x : threadIdx.x % groups_per_row;
  const uint32_t stride = gridDim.x * rows_per_iter;
  const uint32_t n_iter = (rows + 2 * stride - 1) / (2 * stride);
  const float lane_level = KIND == kEncNf4 ? nf4_level(threadIdx.x & 15) : 0.f;
  for (uint32_t it = 0; it < n_iter; ++it) {
    const uint32_t row_a = 2 * it * stride + blockIdx.x * rows_per_iter + sub;
    const uint32_t row_b = row_a + stride;
    for (int gb = 0; gb < groups_per_row; gb += 256) {
      const int g = gb + g0;
      const bool lane_ok = sub < rows_per_iter && g < groups_per_row;
      const bool va = lane_ok && row_a < rows, vb = lane_ok && row_b < rows;
      float xa[8], xb[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) xa[j] = xb[j] = 0.f;
      if (va) load8<DT>(k, static_cast<int64_t>(row_a) * row_elems + 8 * g, xa);
      if (vb) load8<DT>(k, static_cast<int64_t>(row_b) * row_elems + 8 * g, xb);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const uint32_t r = half ? row_b : row_a;
        const bool valid = half ? vb : va;
        const uint32_t b = r / static_cast<uint32_t>(T);
        float p0[8], p1[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { p0[j] = 1.f; p1[j] = 0.f; }
        if (valid && KIND == kEncQ2) {
          load8<DT>(aux0, static_cast<int64_t>(b) * row_elems + 8 * g, p0);
          load8<DT>(aux1, static_cast<int64_t>(b) * row_elems + 8 * g, p1);
        } else if (valid && KIND == kEncNf4) {
          const uint4* mmv = reinterpret_cast<const uint4*>(static_cast<const uint32_t*>(aux0) +
                                                            2 * (static_cast<int64_t>(b) * row_elems + 8 * g));
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint4 v = mmv[j];
            p0[2 * j] = fmaxf(ord_decode(v.y), 1e-6f);
            p0[2 * j + 1] = fmaxf(ord_decode(v.w), 1e-6f);
          }
        }
        encode8<KIND, DT, F8>(half ? xb : xa, p0, p1, lane_level, codes, res,
                              valid ? map(r) * groups_per_row + g : 0, valid);
      }
    }
  }
}

// nvfp4: one block per (b, page, kv-head): absmax over page x 128, then encode.  With the usual
// 64-token page a thread keeps its 32 elements in registers between the two phases.
template <int DT, int F8>
__global__ void __launch_bounds__(256) nvfp4_kernel(const void* __restrict__ k, int T, int HKV, int page,
                                                    uint8_t* __restrict__ codes, void* __restrict__ scale,
                                                    uint8_t* __restrict__ res, RowMap map) {
  const int pg = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n_pages = gridDim.x;
  const int t0 = pg * page, t1 = min(T, t0 + page);
  const int n_groups = (t1 - t0) * (D / 8);
  __shared__ float s_red[8];
  __shared__ float s_scale;
  constexpr int kHeld = 4;                          // groups a thread keeps in registers
  float held[kHeld][8];
  float amax = 0.f;
  for (int i = threadIdx.x, n = 0; i < n_groups; i += blockDim.x, ++n) {
    const int t = t0 + i / (D / 8), c = (i % (D / 8)) * 8;
    float x[8];
    load8<DT>(k, ((static_cast<int64_t>(b) * T + t) * HKV + h) * D + c, x);
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(x[j]));
#pragma unroll
    for (int m = 0; m < kHeld; ++m)
      if (m == n) {
#pragma unroll
        for (int j = 0; j < 8; ++j) held[m][j] = x[j];
      }
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = s_red[0];
    for (int w = 1; w < 8; ++w) m = fmaxf(m, s_red[w]);
    const float s = nvfp4_scale(m, DT);
    s_scale = s;
    store_elem(scale, (static_cast<int64_t>(b) * n_pages + pg) * HKV + h, DT, s);
  }
  __syncthreads();
  const float s = s_scale;
  for (int i = threadIdx.x, n = 0; i < n_groups; i += blockDim.x, ++n) {
    const int t = t0 + i / (D / 8), c = (i % (D / 8)) * 8;
    float x[8];
    if (n < kHeld) {
#pragma unroll
      for (int m = 0; m < kHeld; ++m)
        if (m == n) {
#pragma unroll
          for (int j = 0; j < 8; ++j) x[j] = held[m][j];
        }
    } else {
      load8<DT>(k, ((static_cast<int64_t>(b) * T + t) * HKV + h) * D + c, x);
    }
    float r[8];
    uint32_t cw = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) cw |= nvfp4_encode_f(x[j], s, DT, &r[j]) << (4 * j);
    const int64_t og = ((map(static_cast<int64_t>(b) * T + t) * HKV + h) * D + c) / 8;
    reinterpret_cast<uint32_t*>(codes)[og] = cw;
    reinterpret_cast<uint2*>(res)[og] = narrow8<F8>(r);
  }
}

int check_common(const void* k, int dt, int B, int T, int HKV, int fp8) {
  if (!k) return FFA_E_NULL;
  if (B <= 0 || T <= 0 || HKV <= 0) return FFA_E_SHAPE;
  if (dt != FFA_F16 && dt != FFA_BF16 && dt != FFA_F32) return FFA_E_DTYPE;
  if (fp8 != FFA_E5M2 && fp8 != FFA_E4M3) return FFA_E_DTYPE;
  return FFA_OK;
}

int last_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FFA_OK : note_cuda_error(e, what);
}

// dispatch a kernel template over the runtime element type and fp8 format
#define FFA_DISPATCH_DT_F8(dt, fp8, CALL)                                  \
  do {                                                                      \
    if ((dt) == FFA_BF16) { if ((fp8) == FFA_E4M3) { CALL(kBF16, kE4M3); } else { CALL(kBF16, kE5M2); } } \
    else if ((dt) == FFA_F16) { if ((fp8) == FFA_E4M3) { CALL(kF16, kE4M3); } else { CALL(kF16, kE5M2); } } \
    else { if ((fp8) == FFA_E4M3) { CALL(kF32, kE4M3); } else { CALL(kF32, kE5M2); } }                    \
  } while (0)

void launch_minmax(bool abs_only, const void* k, int dt, int B, int T, int HKV, uint32_t* mm, cudaStream_t st,
                   bool init = true) {
  const int row_elems = HKV * D;
  const int n = B * row_elems;
  if (init) minmax_init_kernel<<<(n + 255) / 256, 256, 0, st>>>(mm, n);   // else: fold into running statistics
  const int gpr = row_elems / 8;
  const int lanes = gpr >= 256 ? 1 : 256 / gpr;
  // enough blocks to fill the GPU, at least 16 tokens per token lane
  int tpb = (T + 148 * 8 - 1) / (148 * 8);
  if (tpb < 16 * lanes) tpb = 16 * lanes;
  dim3 grid((T + tpb - 1) / tpb, B);
  const size_t smem = lanes > 1 ? static_cast<size_t>(lanes) * row_elems * 2 * sizeof(float) : 0;
#define FFA_MINMAX(DT_, F8_)                                                                   \
  if (abs_only) minmax_kernel<true, DT_><<<grid, 256, smem, st>>>(k, T, gpr, tpb, mm);         \
  else minmax_kernel<false, DT_><<<grid, 256, smem, st>>>(k, T, gpr, tpb, mm)
  FFA_DISPATCH_DT_F8(dt, FFA_E4M3, FFA_MINMAX);
#undef FFA_MINMAX
}

template <int KIND>
void launch_encode(const void* k, int dt, int fp8, int B, int T, int HKV, const void* aux0, const void* aux1,
                   uint8_t* codes, uint8_t* residual, RowMap map, cudaStream_t st) {
  const int gpr = HKV * D / 8;
  const int rows_per_iter = gpr >= 256 ? 1 : 256 / gpr;
  const uint32_t rows = static_cast<uint32_t>(B) * static_cast<uint32_t>(T);
  int64_t blocks = (static_cast<int64_t>(rows) + 2 * rows_per_iter - 1) / (2 * rows_per_iter);
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
#define FFA_ENCODE(DT_, F8_)                                                                              \
  encode_rows_kernel<KIND, DT_, F8_><<<static_cast<unsigned>(blocks), 256, 0, st>>>(k, rows, T, gpr, aux0, aux1, codes, \
                                                                                    residual, map)
  FFA_DISPATCH_DT_F8(dt, fp8, FFA_ENCODE);
#undef FFA_ENCODE
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int quantize_impl(int variant, const void* k, int dt, int B, int T, int HKV, int fp8, int page_size, uint8_t* codes,
                  void* scale, void* zero, uint8_t* residual, void* scratch, RowMap map, cudaStream_t st) {
  int rc = check_common(k, dt, B, T, HKV, fp8);
  if (rc) return rc;
  if (!codes || !residual) return FFA_E_NULL;
  if (static_cast<int64_t>(B) * T >= (int64_t{1} << 31)) return FFA_E_LIMIT;
  if (!aligned16(k) || !aligned16(codes) || !aligned16(residual) || !aligned16(scale) || !aligned16(zero) ||
      !aligned16(scratch))
    return FFA_E_ALIGN;
  const int row_elems = HKV * D, n = B * row_elems;
  uint32_t* mm = static_cast<uint32_t*>(scratch);
  switch (variant) {
    case FFA_K_Q2:
      if (!scale || !zero || !scratch) return FFA_E_NULL;
      launch_minmax(false, k, dt, B, T, HKV, mm, st);
      q2_finalize_kernel<<<(n + 255) / 256, 256, 0, st>>>(mm, n, dt, scale, zero);
      launch_encode<kEncQ2>(k, dt, fp8, B, T, HKV, scale, zero, codes, residual, map, st);
      return last_launch("ffa_quantize_q2");
    case FFA_K_FP8:
      launch_encode<kEncFp8>(k, dt, fp8, B, T, HKV, nullptr, nullptr, codes, residual, map, st);
      return last_launch("ffa_quantize_fp8fp8");
    case FFA_K_FP4:
      launch_encode<kEncFp4>(k, dt, fp8, B, T, HKV, nullptr, nullptr, codes, residual, map, st);
      return last_launch("ffa_quantize_fp4");
    case FFA_K_NF4:
      if (!scale || !scratch) return FFA_E_NULL;
      launch_minmax(true, k, dt, B, T, HKV, mm, st);
      nf4_finalize_kernel<<<(n + 255) / 256, 256, 0, st>>>(mm, n, dt, scale);
      launch_encode<kEncNf4>(k, dt, fp8, B, T, HKV, mm, nullptr, codes, residual, map, st);
      return last_launch("ffa_quantize_nf4");
    case FFA_K_NVFP4: {
      if (!scale) return FFA_E_NULL;
      if (page_size <= 0) return FFA_E_SHAPE;
      if (HKV > 65535 || B > 65535) return FFA_E_LIMIT;
      dim3 grid((T + page_size - 1) / page_size, HKV, B);
#define FFA_NVFP4(DT_, F8_) nvfp4_kernel<DT_, F8_><<<grid, 256, 0, st>>>(k, T, HKV, page_size, codes, scale, residual, map)
      FFA_DISPATCH_DT_F8(dt, fp8, FFA_NVFP4);
#undef FFA_NVFP4
      return last_launch("ffa_quantize_nvfp4");
    }
    default:
      return FFA_E_VARIANT;
  }
}

}  // namespace

// Copies rows of `vec_per_row` 16-byte pieces to the rows the map names (V into its page slots).
__global__ void __launch_bounds__(256) scatter_rows_kernel(const uint4* __restrict__ src, int64_t n_vec, int vec_per_row,
                                                           uint4* __restrict__ dst, RowMap map) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row, c = i % vec_per_row;
    dst[map(r) * vec_per_row + c] = src[i];
  }
}

int quantize_dispatch(int variant, const void* k, int k_dtype, int B, int T, int HKV, int fp8, int page_size,
                      uint8_t* codes, void* scale, void* zero, uint8_t* residual, void* scratch,
                      const int32_t* slot_table, int slot_stride, int slot_pos0, cudaStream_t st) {
  if (slot_pos0 != 0 && (!slot_table || (variant != FFA_K_FP8 && variant != FFA_K_FP4))) return FFA_E_VARIANT;
  return quantize_impl(variant, k, k_dtype, B, T, HKV, fp8, page_size, codes, scale, zero, residual, scratch,
                       RowMap{slot_table, slot_stride, T, slot_pos0}, st);
}

// q2 / nf4 with the min/max already reduced per slab of token rows (by the K-projection's epilogue):
// fold + finalise in one small kernel, then the usual encode pass.
int quantize_from_partials(int variant, const void* k, int k_dtype, int B, int T, int HKV, int fp8, uint8_t* codes,
                           void* scale, void* zero, uint8_t* residual, void* scratch, const uint32_t* parts,
                           int parts_per_b, const int32_t* slot_table, int slot_stride, cudaStream_t st) {
  int rc = check_common(k, k_dtype, B, T, HKV, fp8);
  if (rc) return rc;
  if (variant != FFA_K_Q2 && variant != FFA_K_NF4) return FFA_E_VARIANT;
  if (!codes || !residual || !scale || !scratch || !parts || (variant == FFA_K_Q2 && !zero)) return FFA_E_NULL;
  if (parts_per_b <= 0 || B > 65535) return FFA_E_SHAPE;
  if (static_cast<int64_t>(B) * T >= (int64_t{1} << 31)) return FFA_E_LIMIT;
  if (!aligned16(k) || !aligned16(codes) || !aligned16(residual) || !aligned16(scale) || !aligned16(zero) ||
      !aligned16(scratch) || !aligned16(parts))
    return FFA_E_ALIGN;
  const int n_cols = HKV * D;
  uint32_t* mm = static_cast<uint32_t*>(scratch);
  const RowMap map{slot_table, slot_stride, T, 0};
  const dim3 grid(n_cols / 32, B);
  if (variant == FFA_K_Q2) {
    minmax_fold_kernel<false><<<grid, 1024, 0, st>>>(parts, parts_per_b, n_cols, mm, k_dtype, scale, zero);
    launch_encode<kEncQ2>(k, k_dtype, fp8, B, T, HKV, scale, zero, codes, residual, map, st);
  } else {
    minmax_fold_kernel<true><<<grid, 1024, 0, st>>>(parts, parts_per_b, n_cols, mm, k_dtype, scale, nullptr);
    launch_encode<kEncNf4>(k, k_dtype, fp8, B, T, HKV, mm, nullptr, codes, residual, map, st);
  }
  return last_launch("ffa_quantize (min/max from the projection)");
}

}  // namespace ffa

using namespace ffa;

extern "C" size_t ffa_quantize_scratch_bytes(int32_t B, int32_t HKV) {
  if (B <= 0 || HKV <= 0) return 0;
  return static_cast<size_t>(B) * HKV * D * 2 * sizeof(uint32_t);
}

extern "C" int ffa_quantize_q2(const void* k, int32_t dt, int32_t B, int32_t T, int32_t HKV, int32_t fp8,
                               uint8_t* codes, void* scale, void* zero, uint8_t* residual, void* scratch,
                               ffa_stream_t stream) {
  return quantize_impl(FFA_K_Q2, k, dt, B, T, HKV, fp8, 0, codes, scale, zero, residual, scratch, RowMap{nullptr, 0, T, 0},
                       reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ffa_quantize_fp8fp8(const void* k, int32_t dt, int32_t B, int32_t T, int32_t HKV, int32_t fp8,
                                   uint8_t* base, uint8_t* residual, ffa_stream_t stream) {
  return quantize_impl(FFA_K_FP8, k, dt, B, T, HKV, fp8, 0, base, nullptr, nullptr, residual, nullptr,
                       RowMap{nullptr, 0, T, 0}, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ffa_quantize_fp4(const void* k, int32_t dt, int32_t B, int32_t T, int32_t HKV, int32_t fp8,
                                uint8_t* codes, uint8_t* residual, ffa_stream_t stream) {
  return quantize_impl(FFA_K_FP4, k, dt, B, T, HKV, fp8, 0, codes, nullptr, nullptr, residual, nullptr,
                       RowMap{nullptr, 0, T, 0}, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ffa_quantize_nf4(const void* k, int32_t dt, int32_t B, int32_t T, int32_t HKV, int32_t fp8,
                                uint8_t* codes, void* scale, uint8_t* residual, void* scratch, ffa_stream_t stream) {
  return quantize_impl(FFA_K_NF4, k, dt, B, T, HKV, fp8, 0, codes, scale, nullptr, residual, scratch,
                       RowMap{nullptr, 0, T, 0}, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ffa_quantize_nvfp4(const void* k, int32_t dt, int32_t B, int32_t T, int32_t HKV, int32_t fp8,
                                  int32_t page_size, uint8_t* codes, void* scale, uint8_t* residual,
                                  ffa_stream_t stream) {
  return quantize_impl(FFA_K_NVFP4, k, dt, B, T, HKV, fp8, page_size, codes, scale, nullptr, residual, nullptr,
                       RowMap{nullptr, 0, T, 0}, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ffa_cache_append(int32_t variant, const void* k, const void* v, int32_t dt, int32_t B, int32_t T_new,
                                int32_t HKV, int32_t fp8, uint8_t* codes_pool, uint8_t* residual_pool, void* v_pool,
                                const int32_t* block_table, int32_t bt_stride, int32_t pos0, ffa_stream_t stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (!block_table || (!k && !v)) return FFA_E_NULL;
  if (B <= 0 || T_new <= 0 || HKV <= 0 || pos0 < 0 || bt_stride < (pos0 + T_new + kPage - 1) / kPage) return FFA_E_SHAPE;
  if (variant != FFA_K_FP8 && variant != FFA_K_FP4) return FFA_E_VARIANT;     // formats without per-sequence statistics
  if (k) {
    const int rc = quantize_dispatch(variant, k, dt, B, T_new, HKV, fp8, kPage, codes_pool, nullptr, nullptr, residual_pool,
                                     nullptr, block_table, bt_stride, pos0, st);
    if (rc != FFA_OK) return rc;
  }
  if (v) {
    if (!v_pool) return FFA_E_NULL;
    if (dt != FFA_F16 && dt != FFA_BF16) return FFA_E_DTYPE;
    if (!aligned16(v) || !aligned16(v_pool)) return FFA_E_ALIGN;
    const int vec_per_row = HKV * D * 2 / 16;
    const int64_t n_vec = static_cast<int64_t>(B) * T_new * vec_per_row;
    int64_t blocks = (n_vec + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    scatter_rows_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(static_cast<const uint4*>(v), n_vec, vec_per_row,
                                                                      static_cast<uint4*>(v_pool),
                                                                      RowMap{block_table, bt_stride, T_new, pos0});
    return last_launch("ffa_cache_append");
  }
  return FFA_OK;
}

extern "C" int ffa_quantize_append(int32_t variant, const void* k, int32_t dt, int32_t B, int32_t T_new, int32_t HKV,
                                   int32_t fp8, uint8_t* codes_pool, const void* scale, const void* zero,
                                   uint8_t* residual_pool, void* running_minmax, void* scratch,
                                   const int32_t* block_table, int32_t bt_stride, int32_t pos0, ffa_stream_t stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc = check_common(k, dt, B, T_new, HKV, fp8);
  if (rc) return rc;
  if (!codes_pool || !residual_pool || !block_table) return FFA_E_NULL;
  if (pos0 < 0 || bt_stride < (pos0 + T_new + kPage - 1) / kPage) return FFA_E_SHAPE;
  if (!aligned16(k) || !aligned16(codes_pool) || !aligned16(residual_pool) || !aligned16(scale) || !aligned16(zero) ||
      !aligned16(running_minmax) || !aligned16(scratch))
    return FFA_E_ALIGN;
  const RowMap map{block_table, bt_stride, T_new, pos0};
  const int n = B * HKV * D;
  switch (variant) {
    case FFA_K_FP8:
      launch_encode<kEncFp8>(k, dt, fp8, B, T_new, HKV, nullptr, nullptr, codes_pool, residual_pool, map, st);
      break;
    case FFA_K_FP4:
      launch_encode<kEncFp4>(k, dt, fp8, B, T_new, HKV, nullptr, nullptr, codes_pool, residual_pool, map, st);
      break;
    case FFA_K_Q2:
      if (!scale || !zero) return FFA_E_NULL;
      if (running_minmax) launch_minmax(false, k, dt, B, T_new, HKV, static_cast<uint32_t*>(running_minmax), st, false);
      launch_encode<kEncQ2>(k, dt, fp8, B, T_new, HKV, scale, zero, codes_pool, residual_pool, map, st);
      break;
    case FFA_K_NF4:
      if (!scale || !scratch) return FFA_E_NULL;
      if (running_minmax) launch_minmax(true, k, dt, B, T_new, HKV, static_cast<uint32_t*>(running_minmax), st, false);
      nf4_mm_from_scale_kernel<<<(n + 255) / 256, 256, 0, st>>>(scale, n, dt, static_cast<uint32_t*>(scratch));
      launch_encode<kEncNf4>(k, dt, fp8, B, T_new, HKV, scratch, nullptr, codes_pool, residual_pool, map, st);
      break;
    default:
      return FFA_E_VARIANT;       // nvfp4: page-local scales, re-encode the open page with ffa_quantize_nvfp4
  }
  return last_launch("ffa_quantize_append");
}
