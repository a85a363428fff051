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
  __device__ __forceinline__ int64_t operator()(int64_t row) const {
    if (!table) return row;
    const int64_t b = row / T, t = row % T;
    return static_cast<int64_t>(table[b * stride + t / kPage]) * kPage + t % kPage;
  }
};

// scratch: [B, HKV*128] x {min, max} as ordered uints
__global__ void minmax_init_kernel(uint32_t* mm, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    mm[2 * i] = ord_encode(INFINITY);
    mm[2 * i + 1] = ord_encode(-INFINITY);
  }
}

// One block per (b, slab of tokens); thread i owns channels i, i+256, ... of the HKV*128 row.
template <bool ABS>
__global__ void __launch_bounds__(256) minmax_kernel(const void* __restrict__ k, int dt, int T, int row_elems,
                                                     int tokens_per_block, uint32_t* mm) {
  const int b = blockIdx.y;
  const int t0 = blockIdx.x * tokens_per_block;
  const int t1 = min(T, t0 + tokens_per_block);
  for (int c = threadIdx.x; c < row_elems; c += blockDim.x) {
    float lo = INFINITY, hi = -INFINITY;
    for (int t = t0; t < t1; ++t) {
      float v = load_elem(k, (static_cast<int64_t>(b) * T + t) * row_elems + c, dt);
      if (ABS) v = fabsf(v);
      lo = fminf(lo, v);
      hi = fmaxf(hi, v);
    }
    uint32_t* slot = mm + 2 * (static_cast<int64_t>(b) * row_elems + c);
    if (!ABS) atomicMin(slot, ord_encode(lo));
    atomicMax(slot + 1, ord_encode(hi));
  }
}

// q2: finalise (scale, zero) per channel, then encode four channels per thread
__global__ void q2_finalize_kernel(const uint32_t* mm, int n, int dt, void* scale, void* zero) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s, z;
  q2_scale_zero(ord_decode(mm[2 * i]), ord_decode(mm[2 * i + 1]), dt, &s, &z);
  store_elem(scale, i, dt, s);
  store_elem(zero, i, dt, z);
}

__global__ void __launch_bounds__(256) q2_encode_kernel(const void* __restrict__ k, int dt, int T, int row_elems,
                                                        int64_t n_quads, int fp8, const void* __restrict__ scale,
                                                        const void* __restrict__ zero, uint8_t* __restrict__ codes,
                                                        uint8_t* __restrict__ res, RowMap map) {
  const int quads_per_row = row_elems / 4;
  for (int64_t qd = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; qd < n_quads;
       qd += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = qd / quads_per_row;          // b*T + t
    const int c = static_cast<int>(qd % quads_per_row) * 4;
    const int64_t b = row / T;
    const int64_t e = row * row_elems + c;
    const int64_t sidx = b * row_elems + c;
    uint32_t byte = 0;
    uint32_t r4 = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint8_t r;
      byte |= q2_encode(load_elem(k, e + j, dt), load_elem(scale, sidx + j, dt), load_elem(zero, sidx + j, dt), dt, fp8,
                        &r) << (2 * j);
      r4 |= static_cast<uint32_t>(r) << (8 * j);
    }
    const int64_t oq = map(row) * quads_per_row + c / 4;
    codes[oq] = static_cast<uint8_t>(byte);
    reinterpret_cast<uint32_t*>(res)[oq] = r4;
  }
}

// element-pair kernels (fp8fp8, fp4, nf4): thread handles 4 consecutive elements
template <int KIND>   // 0 fp8fp8, 1 fp4, 2 nf4
__global__ void __launch_bounds__(256) quad_encode_kernel(const void* __restrict__ k, int dt, int T, int row_elems,
                                                          int64_t n_quads, int fp8, const uint32_t* __restrict__ mm,
                                                          uint8_t* __restrict__ codes, uint8_t* __restrict__ res,
                                                          RowMap map) {
  const int quads_per_row = row_elems / 4;
  for (int64_t qd = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; qd < n_quads;
       qd += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t row = qd / quads_per_row;
    const int c = static_cast<int>(qd % quads_per_row) * 4;
    const int64_t e = row * row_elems + c;
    uint32_t r4 = 0, c4 = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float x = load_elem(k, e + j, dt);
      uint8_t r;
      if (KIND == 0) {
        uint8_t base;
        fp8fp8_encode(x, fp8, &base, &r);
        c4 |= static_cast<uint32_t>(base) << (8 * j);
      } else if (KIND == 1) {
        c4 |= fp4_encode(x, dt, fp8, &r) << (4 * j);
      } else {
        const int64_t b = row / T;
        const float amax = fmaxf(ord_decode(mm[2 * (b * row_elems + c + j) + 1]), 1e-6f);
        c4 |= nf4_encode_elem(x, amax, fp8, &r) << (4 * j);
      }
      r4 |= static_cast<uint32_t>(r) << (8 * j);
    }
    const int64_t oq = map(row) * quads_per_row + c / 4;
    if (KIND == 0) reinterpret_cast<uint32_t*>(codes)[oq] = c4;
    else reinterpret_cast<uint16_t*>(codes)[oq] = static_cast<uint16_t>(c4);
    reinterpret_cast<uint32_t*>(res)[oq] = r4;
  }
}

__global__ void nf4_finalize_kernel(const uint32_t* mm, int n, int dt, void* scale) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) store_elem(scale, i, dt, fmaxf(ord_decode(mm[2 * i + 1]), 1e-6f));
}

// nvfp4: one block per (b, page, kv-head): absmax over page x 128, then encode
__global__ void __launch_bounds__(256) nvfp4_kernel(const void* __restrict__ k, int dt, int T, int HKV, int page,
                                                    int fp8, uint8_t* __restrict__ codes, void* __restrict__ scale,
                                                    uint8_t* __restrict__ res, RowMap map) {
  const int pg = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n_pages = gridDim.x;
  const int t0 = pg * page, t1 = min(T, t0 + page);
  const int n_pairs = (t1 - t0) * (D / 2);
  __shared__ float s_red[8];
  __shared__ float s_scale;
  float amax = 0.f;
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int t = t0 + i / (D / 2), c = (i % (D / 2)) * 2;
    const int64_t e = ((static_cast<int64_t>(b) * T + t) * HKV + h) * D + c;
    amax = fmaxf(amax, fmaxf(fabsf(load_elem(k, e, dt)), fabsf(load_elem(k, e + 1, dt))));
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = s_red[0];
    for (int w = 1; w < 8; ++w) m = fmaxf(m, s_red[w]);
    const float s = nvfp4_scale(m, dt);
    s_scale = s;
    store_elem(scale, (static_cast<int64_t>(b) * n_pages + pg) * HKV + h, dt, s);
  }
  __syncthreads();
  const float s = s_scale;
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) {
    const int t = t0 + i / (D / 2), c = (i % (D / 2)) * 2;
    const int64_t e = ((static_cast<int64_t>(b) * T + t) * HKV + h) * D + c;
    uint8_t r0, r1;
    const uint32_t lo = nvfp4_encode(load_elem(k, e, dt), s, dt, fp8, &r0);
    const uint32_t hi = nvfp4_encode(load_elem(k, e + 1, dt), s, dt, fp8, &r1);
    const int64_t oe = (map(static_cast<int64_t>(b) * T + t) * HKV + h) * D + c;
    codes[oe / 2] = static_cast<uint8_t>(lo | (hi << 4));
    reinterpret_cast<uint16_t*>(res)[oe / 2] = static_cast<uint16_t>(r0 | (static_cast<uint32_t>(r1) << 8));
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

unsigned stream_grid(int64_t n_threads) {
  const int64_t blocks = (n_threads + 255) / 256;
  return static_cast<unsigned>(blocks < 148 * 16 ? (blocks < 1 ? 1 : blocks) : 148 * 16);
}

void launch_minmax(bool abs_only, const void* k, int dt, int B, int T, int HKV, uint32_t* mm, cudaStream_t st) {
  const int row_elems = HKV * D;
  const int n = B * row_elems;
  minmax_init_kernel<<<(n + 255) / 256, 256, 0, st>>>(mm, n);
  // enough blocks to fill the GPU, at least 16 tokens per block
  int tpb = (T + 148 * 8 - 1) / (148 * 8);
  if (tpb < 16) tpb = 16;
  dim3 grid((T + tpb - 1) / tpb, B);
  if (abs_only) minmax_kernel<true><<<grid, 256, 0, st>>>(k, dt, T, row_elems, tpb, mm);
  else minmax_kernel<false><<<grid, 256, 0, st>>>(k, dt, T, row_elems, tpb, mm);
}

int quantize_impl(int variant, const void* k, int dt, int B, int T, int HKV, int fp8, int page_size, uint8_t* codes,
                  void* scale, void* zero, uint8_t* residual, void* scratch, RowMap map, cudaStream_t st) {
  int rc = check_common(k, dt, B, T, HKV, fp8);
  if (rc) return rc;
  if (!codes || !residual) return FFA_E_NULL;
  const int row_elems = HKV * D, n = B * row_elems;
  const int64_t n_quads = static_cast<int64_t>(B) * T * row_elems / 4;
  uint32_t* mm = static_cast<uint32_t*>(scratch);
  switch (variant) {
    case FFA_K_Q2:
      if (!scale || !zero || !scratch) return FFA_E_NULL;
      launch_minmax(false, k, dt, B, T, HKV, mm, st);
      q2_finalize_kernel<<<(n + 255) / 256, 256, 0, st>>>(mm, n, dt, scale, zero);
      q2_encode_kernel<<<stream_grid(n_quads), 256, 0, st>>>(k, dt, T, row_elems, n_quads, fp8, scale, zero, codes,
                                                             residual, map);
      return last_launch("ffa_quantize_q2");
    case FFA_K_FP8:
      quad_encode_kernel<0><<<stream_grid(n_quads), 256, 0, st>>>(k, dt, T, row_elems, n_quads, fp8, nullptr, codes,
                                                                  residual, map);
      return last_launch("ffa_quantize_fp8fp8");
    case FFA_K_FP4:
      quad_encode_kernel<1><<<stream_grid(n_quads), 256, 0, st>>>(k, dt, T, row_elems, n_quads, fp8, nullptr, codes,
                                                                  residual, map);
      return last_launch("ffa_quantize_fp4");
    case FFA_K_NF4:
      if (!scale || !scratch) return FFA_E_NULL;
      launch_minmax(true, k, dt, B, T, HKV, mm, st);
      nf4_finalize_kernel<<<(n + 255) / 256, 256, 0, st>>>(mm, n, dt, scale);
      quad_encode_kernel<2><<<stream_grid(n_quads), 256, 0, st>>>(k, dt, T, row_elems, n_quads, fp8, mm, codes, residual,
                                                                  map);
      return last_launch("ffa_quantize_nf4");
    case FFA_K_NVFP4: {
      if (!scale) return FFA_E_NULL;
      if (page_size <= 0) return FFA_E_SHAPE;
      if (HKV > 65535 || B > 65535) return FFA_E_LIMIT;
      dim3 grid((T + page_size - 1) / page_size, HKV, B);
      nvfp4_kernel<<<grid, 256, 0, st>>>(k, dt, T, HKV, page_size, fp8, codes, scale, residual, map);
      return last_launch("ffa_quantize_nvfp4");
    }
    default:
      return FFA_E_VARIANT;
  }
}

}  // namespace

int quantize_dispatch(int variant, const void* k, int k_dtype, int B, int T, int HKV, int fp8, int page_size,
                      uint8_t* codes, void* scale, void* zero, uint8_t* residual, void* scratch,
                      const int32_t* slot_table, int slot_stride, cudaStream_t st) {
  return quantize_impl(variant, k, k_dtype, B, T, HKV, fp8, page_size, codes, scale, zero, residual, scratch,
                       RowMap{slot_table, slot_stride, T}, st);
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
  return quantize_impl(FFA_K_Q2, k, dt, B, T, HKV, fp8, 0, codes, scale, zero, residual, scratch, RowMap{nullptr, 0, T},
                       reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ffa_quantize_fp8fp8(const void* k, int32_t dt, int32_t B, int32_t T, int32_t HKV, int32_t fp8,
                                   uint8_t* base, uint8_t* residual, ffa_stream_t stream) {
  return quantize_impl(FFA_K_FP8, k, dt, B, T, HKV, fp8, 0, base, nullptr, nullptr, residual, nullptr,
                       RowMap{nullptr, 0, T}, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ffa_quantize_fp4(const void* k, int32_t dt, int32_t B, int32_t T, int32_t HKV, int32_t fp8,
                                uint8_t* codes, uint8_t* residual, ffa_stream_t stream) {
  return quantize_impl(FFA_K_FP4, k, dt, B, T, HKV, fp8, 0, codes, nullptr, nullptr, residual, nullptr,
                       RowMap{nullptr, 0, T}, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ffa_quantize_nf4(const void* k, int32_t dt, int32_t B, int32_t T, int32_t HKV, int32_t fp8,
                                uint8_t* codes, void* scale, uint8_t* residual, void* scratch, ffa_stream_t stream) {
  return quantize_impl(FFA_K_NF4, k, dt, B, T, HKV, fp8, 0, codes, scale, nullptr, residual, scratch,
                       RowMap{nullptr, 0, T}, reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int ffa_quantize_nvfp4(const void* k, int32_t dt, int32_t B, int32_t T, int32_t HKV, int32_t fp8,
                                  int32_t page_size, uint8_t* codes, void* scale, uint8_t* residual,
                                  ffa_stream_t stream) {
  return quantize_impl(FFA_K_NVFP4, k, dt, B, T, HKV, fp8, page_size, codes, scale, nullptr, residual, nullptr,
                       RowMap{nullptr, 0, T}, reinterpret_cast<cudaStream_t>(stream));
}
