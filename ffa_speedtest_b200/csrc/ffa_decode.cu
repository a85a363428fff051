// FFA decode attention for B200 (sm_100a): coarse score -> page prune -> fp8-residual refine ->
// online softmax * V, fused in one streaming kernel, followed by a small split-KV merge.
//
// Mirrors the semantics of the reference's two Triton kernels
//   attn_forward_stage1_fused_threshold_*  (ffa-q2fp8/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8.py:10-139
//                                           and the fp8fp8 / fp4fp8 / nf4fp8 / nvfp4fp8 siblings)
//   attn_forward_stage2_masked             (same file :142-171)
// with a different decomposition:
//   * a CTA owns a run of consecutive pages ("chunk") of one (batch, kv-head) and keeps the
//     running (max, sum, output) of that run in registers, so the per-page fp32 partial output
//     the reference writes to and re-reads from global memory never leaves the SM;
//   * tokens sit on the M dimension of the tensor-core tile (S^T = K_tile * Q^T), so a page of
//     64 tokens fills four m16n8k16 tiles whatever the GQA group size is (G <= 8 on N);
//   * every byte is moved once by 16-byte cp.async copies into a shared-memory ring; coarse K of
//     page j+DA is in flight while page j is scored and page j-DA is refined, and the residual
//     and V of a page are only requested after the page survived the prune test.
//
// Rounding sequence kept from the reference: q and the coarse K tile are fp16, the dot accumulates
// in fp32 and is multiplied by sm_scale and then by log2(e); the residual is added to the coarse
// tile in fp16; p = exp2(s - page max) is rounded to fp16 for the P*V product while its fp32 sum is
// kept; V is converted to fp16; pages merge in order with the reference's stage-2 recurrence.

#include "ffa_decode_shared.cuh"

namespace ffa {

namespace {

constexpr int kThreads = kDecodeThreads;
constexpr int kWarps = kDecodeWarps;

// Dynamic shared memory layout
template <int FMT, int DA>
struct Smem {
  static constexpr int kNB = 2 * DA + 1;                  // coarse slots: scored .. refined
  static constexpr int kNR = DA + 1;                      // residual+V slots
  static constexpr int kBaseSlot = kPage * Fmt<FMT>::kRow;
  static constexpr int kOffRv = kNB * kBaseSlot;
  static constexpr int kOffAux = kOffRv + kNR * kRvSlot;
  // aux: xchg[2][2][4][8] f32 | th[2][8] f32 | (q2, nf4 only) sS[128] | sZ[128] | book[16]
  // kept small: the fp8 variant needs 2 x (112 KiB + aux + 1 KiB reserved) <= 228 KiB per SM
  static constexpr bool kHasChannelScale = (FMT == FFA_K_Q2 || FMT == FFA_K_NF4);
  static constexpr int kOffXchg = kOffAux;
  static constexpr int kOffTh = kOffXchg + 2 * 2 * 4 * 8 * 4;
  static constexpr int kOffS = kOffTh + 2 * 8 * 4;
  static constexpr int kOffZ = kOffS + 128 * 4;
  static constexpr int kOffBook = kOffZ + 128 * 4;
  static constexpr int kBytes = kHasChannelScale ? kOffBook + 16 * 4 : kOffS;
  static_assert(kNR * kRvSlot >= kWarps * 8 * 128 * 4 + 256, "epilogue scratch must fit in the rv ring");
};

struct ScaleCtx {
  const float* sS;    // per-channel scale (q2, nf4)
  const float* sZ;    // per-channel zero (q2)
  const float* book;  // nf4 code book
  float page_scale;   // nvfp4
};

// Copy 16 token rows (row_bytes each, for one kv-head) into rows [16*warp, 16*warp+16) of a
// shared tile.  Rows whose token index is >= T are zero-filled and read nothing.
template <int ROW, int SWZ_MASK>
__device__ __forceinline__ void issue_rows(uint8_t* tile, const uint8_t* gbase, int64_t pitch, int64_t first_row,
                                           int64_t safe_row, int tok_first, int T, int warp, int lane) {
  constexpr int CH = ROW / 16;
  constexpr int PER_LANE = (16 * CH) / 32;
  static_assert(PER_LANE >= 1, "row too short");
#pragma unroll
  for (int i = 0; i < PER_LANE; ++i) {
    const int idx = i * 32 + lane;
    const int row = idx / CH;
    const int ch = idx % CH;
    const bool ok = (tok_first + row) < T;
    const uint8_t* src = gbase + (ok ? (first_row + row) : safe_row) * pitch + ch * 16;
    const int prow = 16 * warp + row;
    const uint32_t dst = smem_u32(tile + prow * ROW + ((ch ^ (prow & SWZ_MASK)) * 16));
    cp_async16(dst, src, ok ? 16u : 0u);
  }
}

// Raw coarse bytes of token rows (16*warp + g) and (+8) that this thread contracts over:
// channels [32t, 32t+32) in every format.
template <int FMT>
__device__ __forceinline__ void load_raw(uint32_t (&ra)[8], uint32_t (&rb)[8], const uint8_t* tile, int warp, int g,
                                         int t) {
  const int rowA = 16 * warp + g, rowB = rowA + 8;
  if (FMT == FFA_K_FP8) {
    const uint4 a0 = *reinterpret_cast<const uint4*>(tile + rowA * 128 + (((2 * t) ^ (rowA & 1)) * 16));
    const uint4 a1 = *reinterpret_cast<const uint4*>(tile + rowA * 128 + (((2 * t + 1) ^ (rowA & 1)) * 16));
    const uint4 b0 = *reinterpret_cast<const uint4*>(tile + rowB * 128 + (((2 * t) ^ (rowB & 1)) * 16));
    const uint4 b1 = *reinterpret_cast<const uint4*>(tile + rowB * 128 + (((2 * t + 1) ^ (rowB & 1)) * 16));
    ra[0] = a0.x; ra[1] = a0.y; ra[2] = a0.z; ra[3] = a0.w; ra[4] = a1.x; ra[5] = a1.y; ra[6] = a1.z; ra[7] = a1.w;
    rb[0] = b0.x; rb[1] = b0.y; rb[2] = b0.z; rb[3] = b0.w; rb[4] = b1.x; rb[5] = b1.y; rb[6] = b1.z; rb[7] = b1.w;
  } else if (FMT == FFA_K_Q2) {
    const uint2 a = *reinterpret_cast<const uint2*>(tile + rowA * 32 + 8 * t);
    const uint2 b = *reinterpret_cast<const uint2*>(tile + rowB * 32 + 8 * t);
    ra[0] = a.x; ra[1] = a.y; rb[0] = b.x; rb[1] = b.y;
  } else {
    const uint4 a = *reinterpret_cast<const uint4*>(tile + rowA * 64 + 16 * t);
    const uint4 b = *reinterpret_cast<const uint4*>(tile + rowB * 64 + 16 * t);
    ra[0] = a.x; ra[1] = a.y; ra[2] = a.z; ra[3] = a.w; rb[0] = b.x; rb[1] = b.y; rb[2] = b.z; rb[3] = b.w;
  }
}

// fp16 values of channels kb..kb+3 (kb = 32t + 4s) of one token row, as two f16x2 registers.
template <int FMT, int F8>
__device__ __forceinline__ void coarse_pair(uint32_t& lo, uint32_t& hi, const uint32_t (&r)[8], int s, int kb,
                                            const ScaleCtx& sc) {
  if (FMT == FFA_K_FP8) {
    lo = fp8x2_to_h2<F8>(r[s]);
    hi = fp8x2_to_h2<F8>(r[s] >> 16);
  } else if (FMT == FFA_K_Q2) {
    // fp16(fp32(code) * scale + zero): code*scale is exact in fp32, so the fused form rounds once
    // exactly like the reference's separate multiply and add.
    const uint32_t byte = (r[s >> 2] >> (8 * (s & 3))) & 0xffu;
    const float4 S = *reinterpret_cast<const float4*>(sc.sS + kb);
    const float4 Z = *reinterpret_cast<const float4*>(sc.sZ + kb);
    const float c0 = static_cast<float>(byte & 3u), c1 = static_cast<float>((byte >> 2) & 3u);
    const float c2 = static_cast<float>((byte >> 4) & 3u), c3 = static_cast<float>(byte >> 6);
    lo = pack_h2(fmaf(c0, S.x, Z.x), fmaf(c1, S.y, Z.y));
    hi = pack_h2(fmaf(c2, S.z, Z.z), fmaf(c3, S.w, Z.w));
  } else {
    const uint32_t two = (r[s >> 1] >> (16 * (s & 1))) & 0xffffu;   // 4 nibbles: kb, kb+1 | kb+2, kb+3
    if (FMT == FFA_K_FP4) {
      lo = e2m1x2_to_h2(two);
      hi = e2m1x2_to_h2(two >> 8);
    } else if (FMT == FFA_K_NVFP4) {
      const float2 a = unpack_h2(e2m1x2_to_h2(two));
      const float2 b = unpack_h2(e2m1x2_to_h2(two >> 8));
      lo = pack_h2(a.x * sc.page_scale, a.y * sc.page_scale);
      hi = pack_h2(b.x * sc.page_scale, b.y * sc.page_scale);
    } else {  // NF4
      const float4 S = *reinterpret_cast<const float4*>(sc.sS + kb);
      lo = pack_h2(sc.book[two & 15u] * S.x, sc.book[(two >> 4) & 15u] * S.y);
      hi = pack_h2(sc.book[(two >> 8) & 15u] * S.z, sc.book[(two >> 12) & 15u] * S.w);
    }
  }
}

// Scores of the warp's 16 tokens against the (up to 8) query heads of the group, in log2 units.
// out[0], out[1]: token g, heads 2t, 2t+1;  out[2], out[3]: token g+8, heads 2t, 2t+1.
template <int FMT, int F8>
__device__ __forceinline__ void score_tile(float (&out)[4], const uint32_t (&qf)[8][2], const uint8_t* base_tile,
                                           const uint8_t* res_tile, const ScaleCtx& sc, float sm_scale, int warp,
                                           int g, int t) {
  uint32_t ra[8], rb[8];
  load_raw<FMT>(ra, rb, base_tile, warp, g, t);
  uint32_t qa[8], qb[8];
  const bool with_res = res_tile != nullptr;
  if (with_res) load_raw<FFA_K_FP8>(qa, qb, res_tile, warp, g, t);
  float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int s = 0; s < 8; ++s) {
    const int kb = 32 * t + 4 * s;
    uint32_t alo, ahi, blo, bhi;
    coarse_pair<FMT, F8>(alo, ahi, ra, s, kb, sc);
    coarse_pair<FMT, F8>(blo, bhi, rb, s, kb, sc);
    if (with_res) {
      alo = hadd2_u32(alo, fp8x2_to_h2<F8>(qa[s]));
      ahi = hadd2_u32(ahi, fp8x2_to_h2<F8>(qa[s] >> 16));
      blo = hadd2_u32(blo, fp8x2_to_h2<F8>(qb[s]));
      bhi = hadd2_u32(bhi, fp8x2_to_h2<F8>(qb[s] >> 16));
    }
    if (s & 1) mma_f16(acc1, alo, blo, ahi, bhi, qf[s][0], qf[s][1]);
    else       mma_f16(acc0, alo, blo, ahi, bhi, qf[s][0], qf[s][1]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = ((acc0[i] + acc1[i]) * sm_scale) * kLog2e;
}

// max over the 16 tokens of the warp for heads 2t and 2t+1 (result valid in every lane)
__device__ __forceinline__ void warp_token_max(float& m0, float& m1, const float (&s)[4]) {
  m0 = fmaxf(s[0], s[2]);
  m1 = fmaxf(s[1], s[3]);
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, off));
    m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, off));
  }
}

template <int FMT, int F8, int DA>
__global__ void __launch_bounds__(kThreads) decode_stage1_kernel(const __grid_constant__ DecodeParams p) {
  using L = Smem<FMT, DA>;
  constexpr int ROW = Fmt<FMT>::kRow;
  constexpr int BSWZ = (FMT == FFA_K_FP8) ? 1 : 0;
  extern __shared__ __align__(128) uint8_t smem[];

  const int chunk = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int G = p.G, T = p.T;
  const int h0 = 2 * t, h1 = 2 * t + 1;

  float* xchg = reinterpret_cast<float*>(smem + L::kOffXchg);       // [parity][kind][warp][head]
  float* sTh = reinterpret_cast<float*>(smem + L::kOffTh);          // [2][8]
  float* sS = reinterpret_cast<float*>(smem + L::kOffS);
  float* sZ = reinterpret_cast<float*>(smem + L::kOffZ);
  float* sBook = reinterpret_cast<float*>(smem + L::kOffBook);

  const int64_t pitch_c = static_cast<int64_t>(p.HKV) * ROW;
  const int64_t pitch_r = static_cast<int64_t>(p.HKV) * kResRow;
  const int64_t pitch_v = static_cast<int64_t>(p.HKV) * kVRow;
  const uint8_t* gkc = p.kc + static_cast<int64_t>(hkv) * ROW;
  const uint8_t* gkr = p.kr ? p.kr + static_cast<int64_t>(hkv) * kResRow : nullptr;
  const uint8_t* gv = p.v + static_cast<int64_t>(hkv) * kVRow;
  const bool use_res = p.use_res != 0;

  auto page_row0 = [&](int page) -> int64_t {
    return p.bt ? static_cast<int64_t>(p.bt[static_cast<int64_t>(b) * p.bt_stride + page]) * kPage
                : static_cast<int64_t>(b) * T + static_cast<int64_t>(page) * kPage;
  };

  // ---- per-(b, kv-head) constants -------------------------------------------------------------
  if (FMT == FFA_K_Q2 || FMT == FFA_K_NF4) {
    const int64_t o = (static_cast<int64_t>(b) * p.HKV + hkv) * kHeadDim + tid;
    sS[tid] = load_as_float(p.ks, o, p.scale_dtype);
    if (FMT == FFA_K_Q2) sZ[tid] = load_as_float(p.kz, o, p.scale_dtype);
    if (FMT == FFA_K_NF4 && tid < 16) sBook[tid] = c_nf4_book[tid];
  }
  ScaleCtx sc{sS, sZ, sBook, 1.0f};
  auto block_scale = [&](int blk) -> float {
    return load_as_float(p.ks, (static_cast<int64_t>(b) * p.NTB + blk) * p.HKV + hkv, p.scale_dtype);
  };

  // q fragments (B operand): head n = g, channels 32t+4s .. +3
  uint32_t qf[8][2];
  {
    const int64_t qo = (static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G + g) * kHeadDim;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const int kb = 32 * t + 4 * s;
      float x0 = 0.f, x1 = 0.f, x2 = 0.f, x3 = 0.f;
      if (g < G) {
        x0 = load_as_float(p.q, qo + kb, p.q_dtype);
        x1 = load_as_float(p.q, qo + kb + 1, p.q_dtype);
        x2 = load_as_float(p.q, qo + kb + 2, p.q_dtype);
        x3 = load_as_float(p.q, qo + kb + 3, p.q_dtype);
      }
      qf[s][0] = pack_h2(x0, x1);
      qf[s][1] = pack_h2(x2, x3);
    }
  }
  __syncthreads();

  // ---- prune thresholds (…q2fp8.py:55-82) -------------------------------------------------------
  float th0, th1;
  if (p.th_in) {
    const int64_t o = static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G;
    th0 = h0 < G ? p.th_in[o + h0] : 0.f;
    th1 = h1 < G ? p.th_in[o + h1] : 0.f;
  } else {
    if (warp < 2) {
      const int blk = warp == 0 ? 0 : p.NTB - 1;
      const int tok0 = blk * kSample;
      const int page = tok0 / kPage;
      const int64_t r0 = page_row0(page);
      issue_rows<ROW, BSWZ>(smem, gkc, pitch_c, r0 + (tok0 % kPage), r0, tok0, T, warp, lane);
      cp_async_commit();
      cp_async_wait<0>();
      __syncwarp();
      if (FMT == FFA_K_NVFP4) sc.page_scale = block_scale(blk);
      float s[4];
      score_tile<FMT, F8>(s, qf, smem, nullptr, sc, p.sm_scale, warp, g, t);
      if (tok0 + g >= T) { s[0] = -INFINITY; s[1] = -INFINITY; }
      if (tok0 + g + 8 >= T) { s[2] = -INFINITY; s[3] = -INFINITY; }
      float m0, m1;
      warp_token_max(m0, m1, s);
      if (g == 0) { sTh[warp * 8 + h0] = m0; sTh[warp * 8 + h1] = m1; }
    }
    __syncthreads();
    th0 = fmaxf(sTh[h0], sTh[8 + h0]) - p.delta;
    th1 = fmaxf(sTh[h1], sTh[8 + h1]) - p.delta;
  }
  if (p.th_out && chunk == 0 && warp == 0 && g == 0) {
    const int64_t o = static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G;
    if (h0 < G) p.th_out[o + h0] = th0;
    if (h1 < G) p.th_out[o + h1] = th1;
  }

  // ---- page pipeline ---------------------------------------------------------------------------
  const int page_begin = chunk * p.ppc;
  const int n = min(p.ppc, p.NP - page_begin);

  auto issue_base = [&](int j) {
    const int page = page_begin + j;
    const int64_t r0 = page_row0(page);
    uint8_t* tile = smem + (j % L::kNB) * L::kBaseSlot;
    issue_rows<ROW, BSWZ>(tile, gkc, pitch_c, r0 + 16 * warp, r0, page * kPage + 16 * warp, T, warp, lane);
  };
  auto issue_rv = [&](int j) {
    const int page = page_begin + j;
    const int64_t r0 = page_row0(page);
    uint8_t* slot = smem + L::kOffRv + (j % L::kNR) * kRvSlot;
    if (use_res)
      issue_rows<kResRow, 1>(slot, gkr, pitch_r, r0 + 16 * warp, r0, page * kPage + 16 * warp, T, warp, lane);
    issue_rows<kVRow, 7>(slot + kPage * kResRow, gv, pitch_v, r0 + 16 * warp, r0, page * kPage + 16 * warp, T, warp,
                         lane);
  };

  float run_m0 = -INFINITY, run_m1 = -INFINITY, run_l0 = 0.f, run_l1 = 0.f;
  float run_o[8][4];
#pragma unroll
  for (int i = 0; i < 8; ++i) { run_o[i][0] = run_o[i][1] = run_o[i][2] = run_o[i][3] = 0.f; }
  uint32_t keepq = 0;   // bit i: decision for the page scored i+1 iterations ago

#pragma unroll
  for (int j = 0; j < DA; ++j) {
    if (j < n) issue_base(j);
    cp_async_commit();
  }

  for (int it = 0; it < n + DA; ++it) {
    const int j = it, r = it - DA;
    if (j + DA < n) issue_base(j + DA);
    cp_async_commit();
    // the first DA pages were committed by the prologue and have fewer groups behind them
    if (it < DA) cp_async_wait<DA>();
    else cp_async_wait<2 * DA - 1>();
    __syncwarp();

    const bool do_score = j < n;
    const bool do_refine = r >= 0 && ((keepq >> (DA - 1)) & 1u);
    float cm0 = -INFINITY, cm1 = -INFINITY, rm0 = -INFINITY, rm1 = -INFINITY;
    float s_ref[4] = {0.f, 0.f, 0.f, 0.f};

    if (do_score) {
      const int page = page_begin + j;
      if (FMT == FFA_K_NVFP4) sc.page_scale = block_scale((page * kPage) / p.BS);
      float s[4];
      score_tile<FMT, F8>(s, qf, smem + (j % L::kNB) * L::kBaseSlot, nullptr, sc, p.sm_scale, warp, g, t);
      const int tok = page * kPage + 16 * warp + g;
      if (tok >= T) { s[0] = -INFINITY; s[1] = -INFINITY; }
      if (tok + 8 >= T) { s[2] = -INFINITY; s[3] = -INFINITY; }
      warp_token_max(cm0, cm1, s);
    }
    if (do_refine) {
      const int page = page_begin + r;
      if (FMT == FFA_K_NVFP4) sc.page_scale = block_scale((page * kPage) / p.BS);
      const uint8_t* slot = smem + L::kOffRv + (r % L::kNR) * kRvSlot;
      score_tile<FMT, F8>(s_ref, qf, smem + (r % L::kNB) * L::kBaseSlot, use_res ? slot : nullptr, sc, p.sm_scale,
                          warp, g, t);
      const int tok = page * kPage + 16 * warp + g;
      if (tok >= T) { s_ref[0] = -INFINITY; s_ref[1] = -INFINITY; }
      if (tok + 8 >= T) { s_ref[2] = -INFINITY; s_ref[3] = -INFINITY; }
      warp_token_max(rm0, rm1, s_ref);
    }
    float* xb = xchg + (it & 1) * 64;
    if (g == 0) {
      xb[warp * 8 + h0] = cm0; xb[warp * 8 + h1] = cm1;
      xb[32 + warp * 8 + h0] = rm0; xb[32 + warp * 8 + h1] = rm1;
    }
    __syncthreads();
    cm0 = fmaxf(fmaxf(xb[h0], xb[8 + h0]), fmaxf(xb[16 + h0], xb[24 + h0]));
    cm1 = fmaxf(fmaxf(xb[h1], xb[8 + h1]), fmaxf(xb[16 + h1], xb[24 + h1]));
    rm0 = fmaxf(fmaxf(xb[32 + h0], xb[40 + h0]), fmaxf(xb[48 + h0], xb[56 + h0]));
    rm1 = fmaxf(fmaxf(xb[32 + h1], xb[40 + h1]), fmaxf(xb[48 + h1], xb[56 + h1]));

    // prune test: every valid head of the group strictly below its threshold (…q2fp8.py:99-102)
    bool keep = false;
    if (do_score) {
      const bool below = (h0 >= G || cm0 < th0) && (h1 >= G || cm1 < th1);
      keep = !__all_sync(0xffffffffu, below);
      if (keep) issue_rv(j);
      if (p.mask && tid == 0)
        p.mask[(static_cast<int64_t>(b) * p.HKV + hkv) * p.NTBS + page_begin + j] = keep ? 1 : 0;
    }
    cp_async_commit();

    if (do_refine) {
      // p = exp2(s - page max), l = fp32 sum, o_page = fp16(p) * fp16(V)  (…q2fp8.py:123-131)
      const float p0 = s_ref[0] == -INFINITY ? 0.f : exp2f(s_ref[0] - rm0);
      const float p1 = s_ref[1] == -INFINITY ? 0.f : exp2f(s_ref[1] - rm1);
      const float p2 = s_ref[2] == -INFINITY ? 0.f : exp2f(s_ref[2] - rm0);
      const float p3 = s_ref[3] == -INFINITY ? 0.f : exp2f(s_ref[3] - rm1);
      const float l0 = p0 + p2, l1 = p1 + p3;
      // P^T fragment (B operand of O^T = V^T P^T): this lane needs tokens 2t, 2t+1, 2t+8, 2t+9 of
      // head g; they live in lanes 8t + g/2 and 8t + 4 + g/2, in the half selected by g & 1.
      const uint32_t pa = pack_h2(p0, p1), pb = pack_h2(p2, p3);
      const int src = 8 * t + (g >> 1);
      const uint32_t x0 = __shfl_sync(0xffffffffu, pa, src), x1 = __shfl_sync(0xffffffffu, pa, src + 4);
      const uint32_t y0 = __shfl_sync(0xffffffffu, pb, src), y1 = __shfl_sync(0xffffffffu, pb, src + 4);
      const uint32_t sel = (g & 1) ? 0x7632u : 0x5410u;
      const uint32_t pb0 = __byte_perm(x0, x1, sel);
      const uint32_t pb1 = __byte_perm(y0, y1, sel);

      const uint8_t* vt = smem + L::kOffRv + (r % L::kNR) * kRvSlot + kPage * kResRow;
      const int vrow = 16 * warp + (lane & 7) + ((lane >> 4) & 1) * 8;
      const int vsel = (lane >> 3) & 1;
      // stage-2 recurrence in page order (…q2fp8.py:162-167)
      const float nm0 = fmaxf(run_m0, rm0), nm1 = fmaxf(run_m1, rm1);
      const float rp0 = nm0 == -INFINITY ? 0.f : exp2f(run_m0 - nm0);
      const float rp1 = nm1 == -INFINITY ? 0.f : exp2f(run_m1 - nm1);
      const float rb0 = nm0 == -INFINITY ? 0.f : exp2f(rm0 - nm0);
      const float rb1 = nm1 == -INFINITY ? 0.f : exp2f(rm1 - nm1);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint32_t a[4];
        ldmatrix_x4_trans(a, smem_u32(vt + vrow * kVRow + (((2 * i + vsel) ^ (vrow & 7)) * 16)));
        if (p.v_bf16) {
          a[0] = bf16x2_to_h2(a[0]); a[1] = bf16x2_to_h2(a[1]); a[2] = bf16x2_to_h2(a[2]); a[3] = bf16x2_to_h2(a[3]);
        }
        float o[4] = {0.f, 0.f, 0.f, 0.f};
        mma_f16(o, a[0], a[1], a[2], a[3], pb0, pb1);
        run_o[i][0] = run_o[i][0] * rp0 + o[0] * rb0;
        run_o[i][1] = run_o[i][1] * rp1 + o[1] * rb1;
        run_o[i][2] = run_o[i][2] * rp0 + o[2] * rb0;
        run_o[i][3] = run_o[i][3] * rp1 + o[3] * rb1;
      }
      run_l0 = run_l0 * rp0 + l0 * rb0;
      run_l1 = run_l1 * rp1 + l1 * rb1;
      run_m0 = nm0;
      run_m1 = nm1;
    }
    keepq = (keepq << 1) | (keep ? 1u : 0u);
  }

  // ---- chunk epilogue: add the four warps' token slices and write one partial ------------------
  cp_async_wait<0>();
  __syncthreads();
  float* red = reinterpret_cast<float*>(smem + L::kOffRv);          // [warp][head 8][128]
  float* lred = red + kWarps * 8 * 128;                              // [warp][8]
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    run_l0 += __shfl_xor_sync(0xffffffffu, run_l0, off);
    run_l1 += __shfl_xor_sync(0xffffffffu, run_l1, off);
  }
  if (g == 0) { lred[warp * 8 + h0] = run_l0; lred[warp * 8 + h1] = run_l1; }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float* w = red + warp * 1024;
    w[h0 * 128 + 16 * i + g] = run_o[i][0];
    w[h1 * 128 + 16 * i + g] = run_o[i][1];
    w[h0 * 128 + 16 * i + g + 8] = run_o[i][2];
    w[h1 * 128 + 16 * i + g + 8] = run_o[i][3];
  }
  // the running max is identical in all warps: lanes t of warp 0 publish it
  float* mred = lred + kWarps * 8;
  if (warp == 0 && g == 0) { mred[h0] = run_m0; mred[h1] = run_m1; }
  __syncthreads();
  const int64_t row0 = static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G;
  for (int h = 0; h < G; ++h) {
    const float o = red[h * 128 + tid] + red[1024 + h * 128 + tid] + red[2048 + h * 128 + tid] +
                    red[3072 + h * 128 + tid];
    p.part_o[((row0 + h) * p.nch + chunk) * kHeadDim + tid] = o;
  }
  if (tid < G) {
    const float l = lred[tid] + lred[8 + tid] + lred[16 + tid] + lred[24 + tid];
    p.part_m[(row0 + tid) * p.nch + chunk] = mred[tid];
    p.part_l[(row0 + tid) * p.nch + chunk] = l;
  }
  // mask entries past the last real page (padding blocks count as pruned)
  if (p.mask && chunk == p.nch - 1) {
    for (int i = p.NP + tid; i < p.NTBS; i += kThreads)
      p.mask[(static_cast<int64_t>(b) * p.HKV + hkv) * p.NTBS + i] = 0;
  }
}

// Stage 2: merge the chunk partials of one q head in chunk order; one thread per output channel.
// `nch` is the stride of the partial arrays.  With wc == 0 every row has nch partials; with wc > 0
// (page ranges of wc pages cut across the flattened (b, kv-head, page) space) a row's kv-head has
// one partial per range that overlaps its NP pages.
__global__ void __launch_bounds__(kHeadDim) decode_merge_kernel(const float* __restrict__ part_m,
                                                                const float* __restrict__ part_l,
                                                                const float* __restrict__ part_o, int nch, int wc,
                                                                int NP, int G, void* out, int out_dtype,
                                                                float* partial_out) {
  const int64_t row = blockIdx.x;
  const int c = threadIdx.x;
  int count = nch;
  if (wc > 0) {
    const int64_t u0 = (row / G) * NP;
    count = static_cast<int>((u0 + NP - 1) / wc - u0 / wc) + 1;
  }
  float m = -INFINITY, acc = 0.f, o = 0.f;
  for (int i = 0; i < count; ++i) {
    const float mi = part_m[row * nch + i];
    const float li = part_l[row * nch + i];
    if (li == 0.f || mi == -INFINITY) continue;
    const float oi = part_o[(row * nch + i) * kHeadDim + c];
    const float nm = fmaxf(m, mi);
    const float rp = exp2f(m - nm), rb = exp2f(mi - nm);
    acc = acc * rp + li * rb;
    o = o * rp + oi * rb;
    m = nm;
  }
  const float res = acc == 0.f ? 0.f : o / acc;
  if (out) store_from_float(out, row * kHeadDim + c, out_dtype, res);
  if (partial_out) {
    partial_out[row * (kHeadDim + 1) + c] = res;
    if (c == 0) partial_out[row * (kHeadDim + 1) + kHeadDim] = acc == 0.f ? -INFINITY : m + log2f(acc);
  }
}

// Merge R normalised partials with base-2 LSE: parts [R, rows, 129].
__global__ void __launch_bounds__(kHeadDim) merge_partials_kernel(const float* __restrict__ parts, int R, int rows,
                                                                  void* out, int out_dtype) {
  const int64_t row = blockIdx.x;
  const int c = threadIdx.x;
  float top = -INFINITY;
  for (int r = 0; r < R; ++r) top = fmaxf(top, parts[(static_cast<int64_t>(r) * rows + row) * 129 + 128]);
  float den = 0.f, num = 0.f;
  if (top != -INFINITY) {
    for (int r = 0; r < R; ++r) {
      const float* pr = parts + (static_cast<int64_t>(r) * rows + row) * 129;
      const float lse = pr[128];
      if (lse == -INFINITY) continue;
      const float w = exp2f(lse - top);
      den += w;
      num += w * pr[c];
    }
  }
  store_from_float(out, row * kHeadDim + c, out_dtype, den == 0.f ? 0.f : num / den);
}

template <int FMT, int F8, int DA>
int launch_stage1(const DecodeParams& p, cudaStream_t stream) {
  using L = Smem<FMT, DA>;
  auto kern = decode_stage1_kernel<FMT, F8, DA>;
  static bool configured[64] = {};   // per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
    if (e != cudaSuccess) return note_cuda_error(e, "cudaFuncSetAttribute(decode_stage1)");
    configured[dev] = true;
  }
  dim3 grid(p.nch, p.HKV, p.B);
  kern<<<grid, kThreads, L::kBytes, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FFA_OK : note_cuda_error(e, "decode_stage1 launch");
}

template <int FMT>
int launch_stage1_fmt(const DecodeParams& p, int f8, cudaStream_t stream) {
  constexpr int DA = 2;
  return f8 == FFA_E4M3 ? launch_stage1<FMT, FFA_E4M3, DA>(p, stream) : launch_stage1<FMT, FFA_E5M2, DA>(p, stream);
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

}  // namespace

}  // namespace ffa

using namespace ffa;

extern "C" int ffa_decode_plan(int32_t B, int32_t T, int32_t HKV, int32_t ppc_in, int32_t* ppc_out,
                               int32_t* nch_out) {
  if (B <= 0 || T <= 0 || HKV <= 0) return FFA_E_SHAPE;
  const int NP = (T + kPage - 1) / kPage;
  int ppc = ppc_in;
  if (ppc <= 0) {
    // about eight waves of CTAs over 148 SMs x 2 resident CTAs, at least 4 pages per CTA
    const long long units = static_cast<long long>(B) * HKV;
    long long want = (148LL * 2 * 8 + units - 1) / units;
    if (want < 1) want = 1;
    ppc = static_cast<int>((NP + want - 1) / want);
    if (ppc < 4) ppc = 4;
  }
  if (ppc > NP) ppc = NP;
  if (ppc_out) *ppc_out = ppc;
  if (nch_out) *nch_out = (NP + ppc - 1) / ppc;
  return FFA_OK;
}

extern "C" size_t ffa_decode_workspace_bytes(int32_t B, int32_t T, int32_t HQ, int32_t HKV, int32_t ppc_in) {
  if (B <= 0 || T <= 0 || HKV <= 0 || HQ <= 0) return 0;
  // sized for the most partials either kernel can produce per (b, kv-head); the bound does not
  // shrink when T grows, so a workspace made for a maximum length serves every shorter one
  const int nch = decode_nch_bound(B, HKV, (T + kPage - 1) / kPage, ppc_in);
  const size_t rows = static_cast<size_t>(B) * HQ;
  return kArrivalBytes + align_up(rows * nch * sizeof(float), 256) * 4 +
         align_up(rows * nch * kHeadDim * sizeof(float), 256) + 256;
}

// fp8 coarse K goes to the warp-specialised kernel from this many pages (batch x kv-heads x pages per
// sequence) up: 2^20 cached tokens at 8 kv-heads
constexpr long long kFp8WsPages = 131072;
// NF4 (the format with the most scoring work per page) does better on the page-pipeline kernel between
// about 96K and a million cached tokens
constexpr long long kNf4PipePages = 12288;

namespace {
int decode_impl(const FfaDecodeArgs* a, const FfaPeerArgs* peer, ffa_stream_t stream_);
}

extern "C" int ffa_decode(const FfaDecodeArgs* a, ffa_stream_t stream_) { return decode_impl(a, nullptr, stream_); }

extern "C" int ffa_decode_peer(const FfaDecodeArgs* a, const FfaPeerArgs* peer, ffa_stream_t stream_) {
  if (!peer) return FFA_E_NULL;
  return decode_impl(a, peer, stream_);
}

namespace {
int decode_impl(const FfaDecodeArgs* a, const FfaPeerArgs* peer, ffa_stream_t stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (!a || !a->q || !a->k_codes || !a->v || !a->out || !a->workspace) return FFA_E_NULL;
  if (a->B <= 0 || a->T <= 0 || a->HKV <= 0 || a->HQ <= 0 || a->HQ % a->HKV != 0) return FFA_E_SHAPE;
  const int G = a->HQ / a->HKV;
  if (G > 8 || a->head_dim != kHeadDim) return FFA_E_SHAPE;
  // prune blocks of whole pages (SBS = 64 m), or of a half / a quarter of a page (SBS 32 / 16, BS whole pages)
  const bool sub_page = a->SBS == 32 || a->SBS == 16;
  if (sub_page ? (a->BS < kPage || a->BS % kPage != 0)
               : (a->SBS < kPage || a->SBS % kPage != 0 || a->BS < a->SBS || a->BS % a->SBS != 0))
    return FFA_E_SHAPE;
  if (a->q_dtype < FFA_F16 || a->q_dtype > FFA_F32) return FFA_E_DTYPE;
  if (a->v_dtype != FFA_F16 && a->v_dtype != FFA_BF16) return FFA_E_DTYPE;
  if (a->fp8_format != FFA_E5M2 && a->fp8_format != FFA_E4M3) return FFA_E_DTYPE;
  if (a->use_residual && !a->k_residual) return FFA_E_NULL;
  const bool needs_scale = a->variant == FFA_K_Q2 || a->variant == FFA_K_NF4 || a->variant == FFA_K_NVFP4;
  if (needs_scale && (!a->k_scale || a->scale_dtype < FFA_F16 || a->scale_dtype > FFA_F32)) return FFA_E_NULL;
  if (a->variant == FFA_K_Q2 && !a->k_zero) return FFA_E_NULL;
  if (a->block_table && a->bt_stride < (a->T + kPage - 1) / kPage) return FFA_E_SHAPE;

  DecodeParams p{};
  p.q = static_cast<const uint8_t*>(a->q);
  p.kc = static_cast<const uint8_t*>(a->k_codes);
  p.ks = a->k_scale;
  p.kz = a->k_zero;
  p.kr = a->use_residual ? static_cast<const uint8_t*>(a->k_residual) : nullptr;
  p.v = static_cast<const uint8_t*>(a->v);
  p.bt = a->block_table;
  p.bt_stride = a->bt_stride;
  p.th_in = a->threshold_in;
  p.mask = a->kept_mask;
  p.th_out = a->threshold_out;
  p.B = a->B; p.T = a->T; p.HQ = a->HQ; p.HKV = a->HKV; p.G = G;
  p.NP = (a->T + kPage - 1) / kPage;
  p.NTB = (a->T + a->BS - 1) / a->BS;
  p.NTBS = p.NTB * (a->BS / a->SBS);
  p.BS = a->BS;
  p.sm_scale = a->sm_scale; p.delta = a->delta;
  p.q_dtype = a->q_dtype; p.scale_dtype = a->scale_dtype;
  p.use_res = a->use_residual ? 1 : 0;
  p.v_bf16 = a->v_dtype == FFA_BF16 ? 1 : 0;
  // Kernel choice.  reserved = 0 picks by measurement (both TMA kernels timed over batch 1-16,
  // 4K-128K tokens, kept fractions 0.2-0.98): the warp-specialised kernel for the 2- and 4-bit coarse
  // formats, for prune groups of more than one page, for the dtype pairs only it takes, and for fp8
  // coarse K from about a million cached tokens up; below that fp8 coarse K runs on the page-pipeline
  // kernel (three CTAs per SM, every warp scores and refines), which keeps more loads in flight per
  // SM when the coarse pass is cheap and is 3-10 % faster there; NF4 takes the page-pipeline kernel
  // between about 96K and a million cached tokens (2-11 % faster there at high kept fractions).  Bit 0
  // forces the fp16 tensor-core kernel, bit 1 the page-pipeline kernel, bit 2 the warp-specialised kernel.
  const int m = sub_page ? 1 : a->SBS / kPage;  // pages per prune group
  p.sub = sub_page ? kPage / a->SBS : 1;
  const bool want_fp16 = (a->reserved & 1) != 0;
  const bool want_v1 = (a->reserved & 2) != 0;
  const bool want_ws = (a->reserved & 4) != 0 || (peer != nullptr && (a->reserved & 3) == 0);   // the fused exchange lives in this kernel
  p.refine_lag = 1;
  p.group = m;
  const bool v1_ok = m == 1 && !sub_page && decode_tma_supported(p);
  const bool ws_ok = decode_ws_supported(p, m);
  bool use_ws = false, use_tma = false;
  const long long total_pages = static_cast<long long>(a->B) * a->HKV * p.NP;
  if (!want_fp16) {
    if (want_v1) use_tma = v1_ok;
    else if (want_ws) use_ws = ws_ok;
    else if (a->variant == FFA_K_FP8 && v1_ok && total_pages < kFp8WsPages) use_tma = true;
    else if (a->variant == FFA_K_NF4 && v1_ok && total_pages >= kNf4PipePages && total_pages < kFp8WsPages) use_tma = true;
    else use_ws = ws_ok;
    if (!use_ws && !use_tma && !want_v1 && !want_ws) use_tma = v1_ok;
    if ((want_v1 || want_ws) && !use_ws && !use_tma) return m > 1 ? FFA_E_SHAPE : FFA_E_DTYPE;   // asked for by name
  }
  if (use_ws) decode_ws_plan(a->B, a->HKV, p.NP, m, a->pages_per_chunk, &p.NPp, &p.ppc, &p.nseg, &p.grid);
  else if (use_tma)
    decode_tma_plan(a->B, a->HKV, p.NP, a->pages_per_chunk, decode_tma_residency(p, a->variant, a->fp8_format), &p.ppc,
                    &p.nch);
  else ffa_decode_plan(a->B, a->T, a->HKV, a->pages_per_chunk, &p.ppc, &p.nch);
  if (use_ws) p.nch = p.nseg;                              // one partial per chunk

  const size_t rows = static_cast<size_t>(a->B) * a->HQ;
  const size_t ml = align_up(rows * p.nch * sizeof(float), 256);
  const size_t po = align_up(rows * p.nch * kHeadDim * sizeof(float), 256);
  const size_t need = kArrivalBytes + ml * 4 + po + 256;          // m, l, mean-V (m, l), o
  if (a->workspace_bytes < need) return FFA_E_WORKSPACE;
  if (static_cast<size_t>(a->B) * a->HKV > static_cast<size_t>(kWorkCounterIndex)) return FFA_E_LIMIT;
  uint8_t* ws = static_cast<uint8_t*>(a->workspace);
  p.arrivals = reinterpret_cast<int*>(ws);
  p.work = p.arrivals + kWorkCounterIndex;
  p.part_m = reinterpret_cast<float*>(ws + kArrivalBytes);
  p.part_l = reinterpret_cast<float*>(ws + kArrivalBytes + ml);
  p.part_o = reinterpret_cast<float*>(ws + kArrivalBytes + 2 * ml);
  p.status = reinterpret_cast<int*>(ws + kArrivalBytes - 256);      // fixed place: end of the counter block
  p.out = a->out;
  p.partial_out = a->partial_out;
  p.part_pm = reinterpret_cast<float*>(ws + kArrivalBytes + 2 * ml + po + 256);
  p.part_pl = reinterpret_cast<float*>(ws + kArrivalBytes + 3 * ml + po + 256);
  p.v_mean = a->v_mean;
  if (a->v_mean) {
    // mean-V: 2-bit format, final output only (a partial would need the mass too)
    if (a->variant != FFA_K_Q2 || !(use_ws || use_tma) || a->partial_out) return FFA_E_SHAPE;
  }
  if ((m > 1 || sub_page) && !use_ws) return FFA_E_SHAPE;     // the other kernels prune page by page only
  if (sub_page && a->v_mean) return FFA_E_SHAPE;              // mean-V keeps whole pages' mass

  if (peer) {
    // the fused exchange lives in the warp-specialised kernel's merge
    if (!use_ws || !a->partial_out || a->v_mean) return FFA_E_SHAPE;
    if (peer->world < 1 || peer->world > kMaxPeerRanks || peer->rank < 0 || peer->rank >= peer->world || peer->step <= 0 ||
        !peer->peer_gathered || !peer->peer_flags)
      return FFA_E_SHAPE;
    p.peer_world = peer->world; p.peer_rank = peer->rank; p.peer_step = peer->step;
    const int64_t n_part = static_cast<int64_t>(rows) * (kHeadDim + 1);
    for (int r = 0; r < peer->world; ++r) {
      if (!peer->peer_gathered[r] || !peer->peer_flags[r]) return FFA_E_NULL;
      p.peer_slot[r] = peer->peer_gathered[r] + (static_cast<int64_t>(peer->step & 1) * peer->world + peer->rank) * n_part;
      p.peer_flag[r] = peer->peer_flags[r] + peer->rank;
    }
    if (a->partial_out != p.peer_slot[peer->rank]) return FFA_E_SHAPE;      // the local partial is this rank's own slot
  }
  int rc;
  const int64_t kv_rows = a->kv_rows > 0 ? a->kv_rows : static_cast<int64_t>(a->B) * a->T;
  p.kv_rows = kv_rows;
  if (use_ws) rc = launch_decode_ws(p, a->variant, a->fp8_format, kv_rows, stream);
  else if (use_tma) rc = launch_decode_tma(p, a->variant, a->fp8_format, kv_rows, stream);
  else
  switch (a->variant) {
    case FFA_K_FP8:   rc = launch_stage1_fmt<FFA_K_FP8>(p, a->fp8_format, stream); break;
    case FFA_K_Q2:    rc = launch_stage1_fmt<FFA_K_Q2>(p, a->fp8_format, stream); break;
    case FFA_K_FP4:   rc = launch_stage1_fmt<FFA_K_FP4>(p, a->fp8_format, stream); break;
    case FFA_K_NF4:   rc = launch_stage1_fmt<FFA_K_NF4>(p, a->fp8_format, stream); break;
    case FFA_K_NVFP4: rc = launch_stage1_fmt<FFA_K_NVFP4>(p, a->fp8_format, stream); break;
    default: return FFA_E_VARIANT;
  }
  if (rc != FFA_OK) return rc;
  if (use_ws || use_tma) return FFA_OK;          // the last segment of every (b, kv-head) merged in-kernel
  decode_merge_kernel<<<static_cast<unsigned>(rows), kHeadDim, 0, stream>>>(
      p.part_m, p.part_l, p.part_o, p.nch, 0, p.NP, G, a->out, a->q_dtype, a->partial_out);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FFA_OK : note_cuda_error(e, "decode_merge launch");
}
}  // namespace

extern "C" int ffa_merge_partials(const float* parts, int32_t R, int32_t rows, void* out, int32_t out_dtype,
                                  ffa_stream_t stream_) {
  if (!parts || !out) return FFA_E_NULL;
  if (R <= 0 || rows <= 0) return FFA_E_SHAPE;
  if (out_dtype < FFA_F16 || out_dtype > FFA_F32) return FFA_E_DTYPE;
  merge_partials_kernel<<<static_cast<unsigned>(rows), kHeadDim, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      parts, R, rows, out, out_dtype);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FFA_OK : note_cuda_error(e, "merge_partials launch");
}
