// FFA decode attention for B200, bf16-query fast path: TMA-fed shared-memory ring, fp8 tensor-core
// tiles consumed without any per-element conversion.
//
// Same math and same reference semantics as ffa_decode.cu (coarse score -> page prune -> residual
// refine -> online softmax * V; see the citations there), restructured around what bounds the
// step on B200: the stream of K/V bytes from HBM.  The fp16 path spends ~1400 instructions per warp
// per page, most of them address arithmetic for 16-byte copies and fp8->fp16 conversions; this
// kernel removes both:
//
//   * One elected thread moves every tile with cp.async.bulk.tensor (TMA): the coarse tile of
//     page j+3 is requested while page j is scored, residual + V of a page only after it survived
//     the prune test.  Completion is tracked by mbarriers; tiles land 128B-swizzled so that the
//     tensor-core fragment loads are bank-conflict free.
//   * q is bf16 (8 significant bits).  Per head it is scaled by a power of two and split into two
//     e4m3 "pieces" q*2^s = hi + lo/16, both exact.  The pieces sit on the N dimension of an
//     m16n8k32 fp8 MMA whose A operand is the raw fp8 K bytes (e4m3 or e5m2), so
//     acc_hi + acc_lo/16 = 2^s * (q . k) with every product exact and fp32 accumulation: the coarse
//     score equals the reference's fp16 x fp16 -> fp32 dot up to summation order.
//   * The refined score is (q . k_coarse) + (q . k_residual), the second dot again an fp8 MMA on
//     the raw residual bytes.  The reference rounds (k_coarse + k_residual) to fp16 before its
//     second dot; skipping that rounding changes a refined score by < 2^-11 of |q||k| (it cannot
//     change the kept set, which only depends on the coarse scores).
//   * P is rounded to fp16 like the reference, then split exactly into two bf16 pieces on the N
//     dimension of a bf16 MMA whose A operand is V^T straight from ldmatrix - no V conversion.
//
// 2-bit / 4-bit coarse formats still dequantise their codes to fp16 for the coarse dot (their
// values are not fp8 numbers) but share everything else.
#include "ffa_decode_prims.cuh"

namespace ffa {

namespace {

constexpr int kThreads = kDecodeThreads;
constexpr int kWarps = kDecodeWarps;
// Coarse tiles requested ahead of the page being scored, and the slots that takes (one more).  The
// fp8 coarse format with a refine lag of 1 keeps 3 slots so that three CTAs fit on an SM
// (3 x 8 + 2 x 24 KiB); everything else keeps 4.
constexpr int n_base_slots(int fmt, int lag) { return (fmt == FFA_K_FP8 && lag == 1) ? 3 : 4; }

// DA = pages between scoring a page and refining it; DA + 1 residual+V slots
template <int FMT, int DA>
struct SmemT {
  static constexpr int kNRv = DA + 1;
  static constexpr int kNBase = n_base_slots(FMT, DA);
  static constexpr int kPB = kNBase - 1;
  static constexpr int kBaseSlot = kPage * Fmt<FMT>::kRow;            // 8 KiB / 2 KiB / 4 KiB
  static constexpr int kOffRv = kNBase * kBaseSlot;
  static constexpr int kOffAux = kOffRv + kNRv * kRvSlot;
  static constexpr bool kHasChannelScale = (FMT == FFA_K_Q2 || FMT == FFA_K_NF4);
  static constexpr int kOffBars = kOffAux;                              // (kNBase + kNRv) x 8 B
  static constexpr int kOffXchg = kOffBars + 64;                        // [2][2][4][8] f32
  static constexpr int kOffTh = kOffXchg + 512;                         // [2][8] f32
  static constexpr int kOffQinv = kOffTh + 64;                          // [8] f32
  static constexpr int kOffS = kOffQinv + 32;
  static constexpr int kOffZ = kOffS + 512;
  static constexpr int kOffBook = kOffZ + 512;
  static constexpr int kBytes = (kHasChannelScale ? kOffBook + 64 : kOffS) + 1024;   // + alignment slack
};


// One CTA walks a contiguous range of the flattened (batch x kv-head, page) space, `wc` pages
// long; the part of the range inside one (b, kv-head) is a "segment" and produces one partial.
// QP: e4m3 pieces per q value (2 for bf16 q, 3 for fp16 q: 4 + 4 + 3 significant bits).
// Three CTAs per SM for up to four q heads per kv head (at most 168 registers), two beyond that.
// MV: the mean-V variant (pruned pages keep their coarse softmax mass; see DecodeParams::v_mean).
template <int FMT, int F8, int NT, bool VBF, int kDA, int QP, bool MV>
__global__ void __launch_bounds__(kThreads, NT == 1 ? 3 : 2) decode_tma_kernel(const __grid_constant__ DecodeParams p,
                                                              const __grid_constant__ CUtensorMap tm_c,
                                                              const __grid_constant__ CUtensorMap tm_r,
                                                              const __grid_constant__ CUtensorMap tm_v) {
  using L = SmemT<FMT, kDA>;
  constexpr int kNRv = L::kNRv;
  constexpr int kNBase = L::kNBase;
  constexpr int kPB = L::kPB;
  constexpr int ROW = Fmt<FMT>::kRow;
  constexpr bool kFp8Coarse = (FMT == FFA_K_FP8);
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled TMA tiles need 1024-byte alignment
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int G = p.G, T = p.T;

  const uint32_t bars = smem_u32(smem + L::kOffBars);          // [0,kNBase): coarse, then kNRv: res+V
  float* xchg = reinterpret_cast<float*>(smem + L::kOffXchg);
  float* sTh = reinterpret_cast<float*>(smem + L::kOffTh);
  float* sQinv = reinterpret_cast<float*>(smem + L::kOffQinv);
  float* sS = reinterpret_cast<float*>(smem + L::kOffS);
  float* sZ = reinterpret_cast<float*>(smem + L::kOffZ);
  float* sBook = reinterpret_cast<float*>(smem + L::kOffBook);
  const bool use_res = p.use_res != 0;
  const bool sampled = p.th_in == nullptr;
  bool timed_out = false;
  // diagnostics of the first wait that gave up: site (1 sample, 2 coarse tile, 3 residual+V),
  // iteration, pages in the segment, segment ordinal within the CTA
  int gave_up_site = 0, gave_up_it = 0, gave_up_n = 0, gave_up_seg = 0;
  int seg_n = 0, seg_ord = -1;
  auto wait_or_note = [&](uint32_t bar, uint32_t parity, int site, int it) {
    if (!mbar_wait(bar, parity, timed_out)) {
      if (!timed_out) { gave_up_site = site; gave_up_it = it; gave_up_n = seg_n; gave_up_seg = seg_ord; }
      timed_out = true;
    }
  };

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < kNBase + kNRv; ++i) mbar_init(bars + 8 * i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  __syncthreads();
  uint32_t fills = 0;          // bit i: parity of the number of loads issued on barrier i

  const int64_t total_pages = static_cast<int64_t>(p.B) * p.HKV * p.NP;
  int64_t g0 = static_cast<int64_t>(blockIdx.x) * p.ppc;
  const int64_t g1 = min(total_pages, g0 + p.ppc);

  for (bool first = true; g0 < g1; first = false) {
    // ---- segment geometry ------------------------------------------------------------------------
    const int unit = static_cast<int>(g0 / p.NP);
    const int b = unit / p.HKV, hkv = unit % p.HKV;
    const int64_t unit0 = static_cast<int64_t>(unit) * p.NP;
    const int page_begin = static_cast<int>(g0 - unit0);
    const int n = static_cast<int>(min(g1 - g0, static_cast<int64_t>(p.NP - page_begin)));
    const int part = static_cast<int>(g0 / p.ppc - unit0 / p.ppc);     // partial slot of this segment
    g0 += n;
    seg_n = n; ++seg_ord;

    auto page_row0 = [&](int page) -> int {
      return p.bt ? p.bt[static_cast<int64_t>(b) * p.bt_stride + page] * kPage : b * T + page * kPage;
    };
    // local page j lives in coarse slot (j + 2) % kNBase: slots 2 and 3 are free while slots 0 and
    // 1 hold the two threshold samples, so the first two pages are requested at once.  Every thread
    // keeps `fills` (bit i: parity of the number of loads issued on barrier i so far), so the
    // barriers live for the whole kernel and the phase to wait for is the bit at the time of waiting:
    // no barrier gets a second load before every thread has waited for the first.
    auto base_slot = [&](int j) -> int { return (j + 2) % kNBase; };
    auto issue_tile = [&](int slot, int page) {       // called by all threads
      fills ^= 1u << slot;
      if (tid == 0) {
        mbar_expect_tx(bars + 8 * slot, L::kBaseSlot);
        tma_load_2d(smem_u32(smem + slot * L::kBaseSlot), &tm_c, hkv * ROW, page_row0(page), bars + 8 * slot);
      }
    };
    auto issue_base = [&](int j) { issue_tile(base_slot(j), page_begin + j); };
    auto wait_fill = [&](int i, int site, int it) { wait_or_note(bars + 8 * i, ((fills >> i) & 1u) ^ 1u, site, it); };

    if (!first) __syncthreads();        // the previous segment is done with shared memory
    // get the first tiles moving before anything else
    if (sampled) {
      issue_tile(0, 0);
      issue_tile(1, ((p.NTB - 1) * kSample) / kPage);
    }
    for (int j = 0; j < kNBase - 2 && j < n; ++j) issue_base(j);     // the slots the samples do not use

    if (L::kHasChannelScale) {
      const int64_t o = (static_cast<int64_t>(b) * p.HKV + hkv) * kHeadDim + tid;
      sS[tid] = load_as_float(p.ks, o, p.scale_dtype);
      if (FMT == FFA_K_Q2) sZ[tid] = load_as_float(p.kz, o, p.scale_dtype);
      if (FMT == FFA_K_NF4 && tid < 16) sBook[tid] = c_nf4_book[tid];
    }
    ScaleCtx sc;
    sc.sS = sS; sc.sZ = sZ; sc.book = sBook; sc.page_scale = 1.0f;
    sc.q2_fast = false; sc.page_fast = false; sc.page_scale_h2 = 0u;
    if (FMT == FFA_K_Q2) {
      // uniform over the CTA: all 128 (scale, zero) pairs of this (b, kv-head) are fp16 numbers
      sc.q2_fast = __syncthreads_and(exact_in_f16(sS[tid]) && exact_in_f16(sZ[tid])) != 0;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        sc.s2[i] = pack_h2(sS[32 * t + 2 * i], sS[32 * t + 2 * i + 1]);
        sc.z2[i] = pack_h2(sZ[32 * t + 2 * i], sZ[32 * t + 2 * i + 1]);
      }
    }
    // nvfp4: the scale of a BS-token block, and (apply) whether the fp16 product is exact for it.  The
    // main loop loads the next page's scale one iteration ahead so the global load is off the path
    // to the prune decision.
    auto load_block_scale = [&](int blk) -> float {
      return load_as_float(p.ks, (static_cast<int64_t>(b) * p.NTB + blk) * p.HKV + hkv, p.scale_dtype);
    };
    auto apply_block_scale = [&](float x) {
      sc.page_scale = x;
      // e2m1 (2 significant bits) x scale fits fp16's 11 bits if the scale has at most 9 (bf16 has 8),
      // and stays a normal fp16 number if the scale is within [2^-13, 2^13)
      sc.page_fast = (__float_as_uint(x) & 0x7fffu) == 0u && fabsf(x) >= 1.220703125e-4f && fabsf(x) < 8192.f;
      sc.page_scale_h2 = pack_h2(x, x);
    };
    auto set_block_scale = [&](int blk) { apply_block_scale(load_block_scale(blk)); };

    // ---- q operands ------------------------------------------------------------------------------
    // q . 2^e = hi + mid / 16 (+ lo / 256 for fp16 q), every piece an e4m3 number: exact for bf16's 8
    // and fp16's 11 significant bits as long as the value stays above e4m3's underflow.
    // B-fragment column n = g of n-tile nt is head 4nt + g/2, piece g&1 (hi / mid); with three pieces
    // n-tile NT + nt holds (lo / zero) in the same columns.  The fp16 MMA of the 2-bit / 4-bit coarse
    // formats takes (q as fp16 / zero).
    uint32_t qb[NT * (QP - 1)][4][2];
    uint32_t qh[kFp8Coarse ? 1 : NT][kFp8Coarse ? 1 : 8][2];
    auto q_pair = [&](uint32_t w) -> float2 {               // two consecutive q values as floats
      if (QP == 2) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
      return unpack_h2(w);
    };
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int hc = 4 * nt + (g >> 1);
      const bool second = (g & 1) != 0;                        // column of the mid piece / of zeros
      uint32_t raw[16];                                       // 32 16-bit channels 32t .. 32t+31
      if (hc < G) {
        const uint4* src = reinterpret_cast<const uint4*>(
            p.q + ((static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G + hc) * kHeadDim + 32 * t) * 2);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 v4 = src[i];
          raw[4 * i] = v4.x; raw[4 * i + 1] = v4.y; raw[4 * i + 2] = v4.z; raw[4 * i + 3] = v4.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) raw[i] = 0u;
      }
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 f = q_pair(raw[i]);
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      // power of two that brings the head's largest |q| into [128, 256)
      int e = 0;
      if (amax > 0.f && amax < INFINITY) e = 134 - static_cast<int>((__float_as_uint(amax) >> 23) & 0xffu);
      e = max(-100, min(100, e));
      const float up = __int_as_float((127 + e) << 23), down = __int_as_float((127 - e) << 23);
      if (warp == 0 && t == 0 && !second) sQinv[hc] = down;
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const float2 fa = q_pair(raw[2 * r]), fb = q_pair(raw[2 * r + 1]);
        const float x0 = fa.x * up, x1 = fa.y * up, x2 = fb.x * up, x3 = fb.y * up;
        const uint32_t h01 = f32x2_to_e4m3x2(x0, x1), h23 = f32x2_to_e4m3x2(x2, x3);
        const float2 d01 = e4m3x2_to_f32x2(h01), d23 = e4m3x2_to_f32x2(h23);
        const float r0 = (x0 - d01.x) * 16.f, r1 = (x1 - d01.y) * 16.f, r2 = (x2 - d23.x) * 16.f, r3 = (x3 - d23.y) * 16.f;
        const uint32_t m01 = f32x2_to_e4m3x2(r0, r1), m23 = f32x2_to_e4m3x2(r2, r3);
        qb[nt][r >> 1][r & 1] = second ? (m01 | (m23 << 16)) : (h01 | (h23 << 16));   // register r: channels 32t+4r .. +3
        if (QP == 3) {
          const float2 e01 = e4m3x2_to_f32x2(m01), e23 = e4m3x2_to_f32x2(m23);
          const uint32_t l01 = f32x2_to_e4m3x2((r0 - e01.x) * 16.f, (r1 - e01.y) * 16.f);
          const uint32_t l23 = f32x2_to_e4m3x2((r2 - e23.x) * 16.f, (r3 - e23.y) * 16.f);
          qb[(QP - 2) * NT + nt][r >> 1][r & 1] = second ? 0u : (l01 | (l23 << 16));
        }
      }
      if (!kFp8Coarse) {
#pragma unroll
        for (int s = 0; s < 8; ++s) {
          // the reference's q.to(float16)
          qh[kFp8Coarse ? 0 : nt][kFp8Coarse ? 0 : s][0] = second ? 0u : (QP == 2 ? bf16x2_to_h2(raw[2 * s]) : raw[2 * s]);
          qh[kFp8Coarse ? 0 : nt][kFp8Coarse ? 0 : s][1] = second ? 0u : (QP == 2 ? bf16x2_to_h2(raw[2 * s + 1]) : raw[2 * s + 1]);
        }
      }
    }
    __syncthreads();
    float qinv[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) qinv[nt] = sQinv[4 * nt + t];

    // unscaled coarse dots of one tile -> [nt][token g / g+8]; `slice` selects which 16 rows
    auto coarse_dots = [&](float (&out)[NT][2], const uint8_t* tile, int slice) {
      if constexpr (kFp8Coarse) dot_fp8<F8, NT, QP>(out, qb, qinv, tile, slice, g, t);
      else if (FMT == FFA_K_Q2 ? sc.q2_fast : (FMT == FFA_K_NVFP4 && sc.page_fast))
        dot_f16<FMT, NT, true>(out, qh, tile, sc, slice, g, t);
      else dot_f16<FMT, NT, false>(out, qh, tile, sc, slice, g, t);
    };
    auto to_log2 = [&](float d) -> float { return (d * p.sm_scale) * kLog2e; };

    // ---- prune thresholds (reference ...q2fp8.py:55-82) ---------------------------------------------
    // Two 16-token samples of the coarse K: tokens [0,16) and [(NTB-1)*16, +16).
    float th[NT];
    if (!sampled) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int h = 4 * nt + t;
        th[nt] = h < G ? p.th_in[static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G + h] : 0.f;
      }
    } else {
      if (warp < 2) {
        wait_fill(warp, 1, 0);
        const int blk = warp == 0 ? 0 : p.NTB - 1;
        const int tok0 = blk * kSample;
        if (FMT == FFA_K_NVFP4) set_block_scale(blk);
        float d[NT][2];
        coarse_dots(d, smem + warp * L::kBaseSlot, (tok0 % kPage) / 16);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const float s0 = tok0 + g < T ? to_log2(d[nt][0]) : -INFINITY;
          const float s1 = tok0 + g + 8 < T ? to_log2(d[nt][1]) : -INFINITY;
          float mm = fmaxf(s0, s1);
#pragma unroll
          for (int off = 4; off < 32; off <<= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));
          if (g == 0) sTh[warp * 8 + 4 * nt + t] = mm;
        }
      }
      __syncthreads();
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) th[nt] = fmaxf(sTh[4 * nt + t], sTh[8 + 4 * nt + t]) - p.delta;
    }
    if (p.th_out && page_begin == 0 && warp == 0 && g == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int h = 4 * nt + t;
        if (h < G) p.th_out[static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G + h] = th[nt];
      }
    }

    // ---- page pipeline -----------------------------------------------------------------------------
    auto issue_rv = [&](int j) {                      // thread 0 only; all threads toggle the bit
      const int slot = j % kNRv;
      const uint32_t bar = bars + 8 * (kNBase + slot);
      const uint32_t dst = smem_u32(smem + L::kOffRv + slot * kRvSlot);
      const int row = page_row0(page_begin + j);
      mbar_expect_tx(bar, (use_res ? kPage * kResRow : 0) + kPage * kVRow);
      if (use_res) tma_load_2d(dst, &tm_r, hkv * kResRow, row, bar);
      tma_load_2d(dst + kPage * kResRow, &tm_v, hkv * kVRow, row, bar);
      tma_load_2d(dst + kPage * kResRow + kPage * 128, &tm_v, hkv * kVRow + 128, row, bar);
    };

    float run_m[NT], run_l[NT], run_o[NT][8][2];
    float hist[kDA][NT][2];          // unscaled coarse dots of the last kDA scored pages
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      run_m[nt] = -INFINITY;
      run_l[nt] = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) run_o[nt][i][0] = run_o[nt][i][1] = 0.f;
#pragma unroll
      for (int d = 0; d < kDA; ++d) hist[d][nt][0] = hist[d][nt][1] = 0.f;
    }
    uint32_t keepq = 0;
    float apx_m[NT], apx_l[NT], cs[NT][2];       // mean-V: running max / mass of the pruned pages, page scores
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) { apx_m[nt] = -INFINITY; apx_l[nt] = 0.f; cs[nt][0] = cs[nt][1] = -INFINITY; }

    // (the __syncthreads after the sample scoring, or after the q set-up, orders every warp's reads
    // of slots 0 and 1 before they are refilled)
    for (int j = kNBase - 2; j < kPB && j < n; ++j) issue_base(j);

    float ks_next = 0.f;
    if (FMT == FFA_K_NVFP4) ks_next = load_block_scale((page_begin * kPage) / p.BS);
    for (int it = 0; it < n + kDA; ++it) {
      const int j = it, r = it - kDA;
      if (j + kPB < n) issue_base(j + kPB);

      const bool do_score = j < n;
      const bool do_refine = r >= 0 && ((keepq >> (kDA - 1)) & 1u);
      float cm[NT], rm[NT], dc[NT][2], sref[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) { cm[nt] = rm[nt] = -INFINITY; dc[nt][0] = dc[nt][1] = 0.f; sref[nt][0] = sref[nt][1] = 0.f; }

      if (do_score) {
        const int page = page_begin + j;
        wait_fill(base_slot(j), 2, it);
        if (FMT == FFA_K_NVFP4) {
          apply_block_scale(ks_next);
          if (j + 1 < n) ks_next = load_block_scale(((page + 1) * kPage) / p.BS);
        }
        coarse_dots(dc, smem + base_slot(j) * L::kBaseSlot, warp);
        const int tok = page * kPage + 16 * warp + g;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const float s0 = tok < T ? to_log2(dc[nt][0]) : -INFINITY;
          const float s1 = tok + 8 < T ? to_log2(dc[nt][1]) : -INFINITY;
          if (MV) { cs[nt][0] = s0; cs[nt][1] = s1; }
          float mm = fmaxf(s0, s1);
#pragma unroll
          for (int off = 4; off < 32; off <<= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));
          cm[nt] = mm;
        }
      }
      if (do_refine) {
        const int page = page_begin + r;
        const uint8_t* slot = smem + L::kOffRv + (r % kNRv) * kRvSlot;
        wait_fill(kNBase + r % kNRv, 3, it);      // pruned pages issue no load and toggle no bit
        float dr[NT][2];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) dr[nt][0] = dr[nt][1] = 0.f;
        if (use_res) dot_fp8<F8, NT, QP>(dr, qb, qinv, slot, warp, g, t);
        const int tok = page * kPage + 16 * warp + g;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          sref[nt][0] = tok < T ? to_log2(hist[kDA - 1][nt][0] + dr[nt][0]) : -INFINITY;
          sref[nt][1] = tok + 8 < T ? to_log2(hist[kDA - 1][nt][1] + dr[nt][1]) : -INFINITY;
          float mm = fmaxf(sref[nt][0], sref[nt][1]);
#pragma unroll
          for (int off = 4; off < 32; off <<= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));
          rm[nt] = mm;
        }
      }
      // shift the history of coarse dots
#pragma unroll
      for (int d = kDA - 1; d > 0; --d)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) { hist[d][nt][0] = hist[d - 1][nt][0]; hist[d][nt][1] = hist[d - 1][nt][1]; }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) { hist[0][nt][0] = dc[nt][0]; hist[0][nt][1] = dc[nt][1]; }

      float* xb = xchg + (it & 1) * 64;
      if (g == 0) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          xb[warp * 8 + 4 * nt + t] = cm[nt];
          xb[32 + warp * 8 + 4 * nt + t] = rm[nt];
        }
      }
      __syncthreads();
      bool below = true;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const int h = 4 * nt + t;
        cm[nt] = fmaxf(fmaxf(xb[h], xb[8 + h]), fmaxf(xb[16 + h], xb[24 + h]));
        rm[nt] = fmaxf(fmaxf(xb[32 + h], xb[40 + h]), fmaxf(xb[48 + h], xb[56 + h]));
        below = below && (h >= G || cm[nt] < th[nt]);
      }

      bool keep = false;
      if (do_score) {
        keep = !__all_sync(0xffffffffu, below);     // pruned only if every head is strictly below
        if (MV && !keep) {
          // pruned page: its coarse scores relative to the page maximum join the running mass
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            const float mc = cm[nt];
            if (mc != -INFINITY) {
              const float pp = (cs[nt][0] == -INFINITY ? 0.f : ex2_approx(cs[nt][0] - mc)) +
                               (cs[nt][1] == -INFINITY ? 0.f : ex2_approx(cs[nt][1] - mc));
              const float nm = fmaxf(apx_m[nt], mc);
              const float rp = apx_m[nt] == -INFINITY ? 0.f : ex2_approx(apx_m[nt] - nm);
              apx_l[nt] = apx_l[nt] * rp + pp * ex2_approx(mc - nm);
              apx_m[nt] = nm;
            }
          }
        }
        if (keep) fills ^= 1u << (kNBase + j % kNRv);
        if (tid == 0) {
          if (keep) issue_rv(j);
          if (p.mask) p.mask[(static_cast<int64_t>(b) * p.HKV + hkv) * p.NTBS + page_begin + j] = keep ? 1 : 0;
        }
      }

      if (do_refine) {
        const int page = page_begin + r;
        const uint8_t* vt = smem + L::kOffRv + (r % kNRv) * kRvSlot + kPage * kResRow;
        const int vrow = 16 * warp + (lane & 7) + ((lane >> 4) & 1) * 8;
        const int vsel = (lane >> 3) & 1;
        const int valid = T - (page * kPage + 16 * warp);       // valid tokens in this warp's slice
        const bool partial = (page + 1) * kPage > T;
        uint32_t m01 = 0xffffffffu, m23 = 0xffffffffu;
        if (partial) {
          m01 = (2 * t < valid ? 0xffffu : 0u) | (2 * t + 1 < valid ? 0xffff0000u : 0u);
          m23 = (2 * t + 8 < valid ? 0xffffu : 0u) | (2 * t + 9 < valid ? 0xffff0000u : 0u);
        }
        const int src = 8 * t + (g >> 1);
        const uint32_t sel = (g & 1) ? 0x7632u : 0x5410u;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          // p = exp2(s - page max), fp32 sum, fp16 rounding for the P.V product (...q2fp8.py:123-131)
          const float p0 = sref[nt][0] == -INFINITY ? 0.f : ex2_approx(sref[nt][0] - rm[nt]);
          const float p1 = sref[nt][1] == -INFINITY ? 0.f : ex2_approx(sref[nt][1] - rm[nt]);
          const float l = p0 + p1;
          uint32_t w0, w1;
          if (VBF) {
            // fp16(p) = hi + lo exactly, both bf16
            const float f0 = __half2float(__float2half_rn(p0)), f1 = __half2float(__float2half_rn(p1));
            const __nv_bfloat16 h0 = __float2bfloat16_rn(f0), h1 = __float2bfloat16_rn(f1);
            const __nv_bfloat16 l0 = __float2bfloat16_rn(f0 - __bfloat162float(h0));
            const __nv_bfloat16 l1 = __float2bfloat16_rn(f1 - __bfloat162float(h1));
            w0 = static_cast<uint32_t>(__bfloat16_as_ushort(h0)) | (static_cast<uint32_t>(__bfloat16_as_ushort(l0)) << 16);
            w1 = static_cast<uint32_t>(__bfloat16_as_ushort(h1)) | (static_cast<uint32_t>(__bfloat16_as_ushort(l1)) << 16);
          } else {
            w0 = static_cast<uint32_t>(__half_as_ushort(__float2half_rn(p0)));
            w1 = static_cast<uint32_t>(__half_as_ushort(__float2half_rn(p1)));
          }
          // P^T fragment: tokens 2t, 2t+1 (and +8) of column g = (head 4nt + g/2, piece g&1)
          const uint32_t x0 = __shfl_sync(0xffffffffu, w0, src), x1 = __shfl_sync(0xffffffffu, w0, src + 4);
          const uint32_t y0 = __shfl_sync(0xffffffffu, w1, src), y1 = __shfl_sync(0xffffffffu, w1, src + 4);
          const uint32_t pb0 = __byte_perm(x0, x1, sel), pb1 = __byte_perm(y0, y1, sel);

          // stage-2 recurrence in page order (...q2fp8.py:162-167)
          const float nm = fmaxf(run_m[nt], rm[nt]);
          const float rp = nm == -INFINITY ? 0.f : ex2_approx(run_m[nt] - nm);
          const float rb = nm == -INFINITY ? 0.f : ex2_approx(rm[nt] - nm);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            uint32_t a[4];
            const int ch = 2 * i + vsel;
            ldmatrix_x4_trans(a, smem_u32(vt + (ch >> 3) * (kPage * 128) + vrow * 128 + (((ch & 7) ^ (vrow & 7)) * 16)));
            if (partial) { a[0] &= m01; a[1] &= m01; a[2] &= m23; a[3] &= m23; }
            float o[4] = {0.f, 0.f, 0.f, 0.f};
            if (VBF) mma_bf16(o, a[0], a[1], a[2], a[3], pb0, pb1);
            else mma_f16(o, a[0], a[1], a[2], a[3], pb0, pb1);
            run_o[nt][i][0] = run_o[nt][i][0] * rp + (o[0] + o[1]) * rb;
            run_o[nt][i][1] = run_o[nt][i][1] * rp + (o[2] + o[3]) * rb;
          }
          run_l[nt] = run_l[nt] * rp + l * rb;
          run_m[nt] = nm;
        }
      }
      keepq = (keepq << 1) | (keep ? 1u : 0u);
    }

    // ---- segment epilogue: add the four warps' token slices and write one partial -------------------
    __syncthreads();
    float* red = reinterpret_cast<float*>(smem + L::kOffRv);          // [warp][head 8][128]
    float* lred = red + kWarps * 8 * 128;                              // [warp][8]
    float* mred = lred + kWarps * 8;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float l = run_l[nt];
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
      const int h = 4 * nt + t;
      if (g == 0) lred[warp * 8 + h] = l;
      if (warp == 0 && g == 0) mred[h] = run_m[nt];
      if (MV) {
        // every thread folded the same page maxima, so only the masses need adding up
        float al = apx_l[nt];
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) al += __shfl_xor_sync(0xffffffffu, al, off);
        if (g == 0) mred[16 + warp * 8 + h] = al;
        if (warp == 0 && g == 0) mred[48 + h] = apx_m[nt];
      }
      float* w = red + warp * 1024 + h * 128;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        w[16 * i + g] = run_o[nt][i][0];
        w[16 * i + g + 8] = run_o[nt][i][1];
      }
    }
    // A segment one of whose waits gave up computed on tiles that may never have landed: its mass is
    // published as NaN, so the merged rows of this (b, kv-head) are NaN rather than plausible numbers.
    const bool seg_bad = __syncthreads_or(timed_out ? 1 : 0) != 0;
    if (seg_bad && tid < 32) lred[tid] = __int_as_float(0x7fc00000);
    __syncthreads();
    const int64_t row0 = static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G;
    for (int h = 0; h < G; ++h) {
      const float o = red[h * 128 + tid] + red[1024 + h * 128 + tid] + red[2048 + h * 128 + tid] +
                      red[3072 + h * 128 + tid];
      p.part_o[((row0 + h) * p.nch + part) * kHeadDim + tid] = o;
    }
    if (tid < G) {
      p.part_m[(row0 + tid) * p.nch + part] = mred[tid];
      p.part_l[(row0 + tid) * p.nch + part] = lred[tid] + lred[8 + tid] + lred[16 + tid] + lred[24 + tid];
      if (MV) {
        p.part_pm[(row0 + tid) * p.nch + part] = mred[48 + tid];
        p.part_pl[(row0 + tid) * p.nch + part] = mred[16 + tid] + mred[24 + tid] + mred[32 + tid] + mred[40 + tid];
      }
    }
    if (p.mask && page_begin + n == p.NP) {
      for (int i = p.NP + tid; i < p.NTBS; i += kThreads)
        p.mask[(static_cast<int64_t>(b) * p.HKV + hkv) * p.NTBS + i] = 0;
    }

    // ---- merge by the last segment of this (b, kv-head) to finish (stage 2, ...q2fp8.py:142-171) -----
    // Every segment publishes its partial, then bumps the unit's arrival counter; whoever sees all the
    // others already there merges the partials in page order and resets the counter for the next launch.
    const int n_seg = static_cast<int>((unit0 + p.NP - 1) / p.ppc - unit0 / p.ppc) + 1;
    int* s_flag = reinterpret_cast<int*>(mred + 8);       // mred + 16 .. + 56 belong to the mean-V sums
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int prev = atomicAdd(p.arrivals + unit, 1);
      *s_flag = (prev == n_seg - 1);
      if (prev == n_seg - 1) p.arrivals[unit] = 0;
    }
    __syncthreads();
    if (*s_flag) {
      __threadfence();
      // (m, l) of every (head, segment) into shared memory, then one warp per head with four
      // channels per lane: all loads of a head are independent, so the merge costs two round trips
      float* sm_m = red;
      float* sm_l = red + 8 * 64;
      const int per_head = n_seg;                       // <= 64 by construction of the page ranges
      for (int idx = tid; idx < G * per_head; idx += kThreads) {
        const int h = idx / per_head, i = idx % per_head;
        sm_m[h * 64 + i] = __ldcg(p.part_m + (row0 + h) * p.nch + i);
        sm_l[h * 64 + i] = __ldcg(p.part_l + (row0 + h) * p.nch + i);
        if (MV) {
          sm_l[8 * 64 + h * 64 + i] = __ldcg(p.part_pm + (row0 + h) * p.nch + i);
          sm_l[16 * 64 + h * 64 + i] = __ldcg(p.part_pl + (row0 + h) * p.nch + i);
        }
      }
      __syncthreads();
      for (int h = warp; h < G; h += kWarps) {
        const int64_t row = row0 + h;
        float top = -INFINITY;
        for (int i = 0; i < per_head; ++i)
          if (sm_l[h * 64 + i] != 0.f) top = fmaxf(top, sm_m[h * 64 + i]);
        float acc = 0.f;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int i0 = 0; i0 < per_head; i0 += 8) {
          float4 v[8];
          float w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int i = i0 + j;
            const bool live = i < per_head && sm_l[h * 64 + i] != 0.f && sm_m[h * 64 + i] != -INFINITY;
            w[j] = live ? exp2f(sm_m[h * 64 + i] - top) : 0.f;
            v[j] = live ? __ldcg(reinterpret_cast<const float4*>(p.part_o + (row * p.nch + i) * kHeadDim) + lane)
                        : make_float4(0.f, 0.f, 0.f, 0.f);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int i = i0 + j;
            if (i < per_head) acc += sm_l[h * 64 + i] * w[j];
            o.x += v[j].x * w[j]; o.y += v[j].y * w[j]; o.z += v[j].z * w[j]; o.w += v[j].w * w[j];
          }
        }
        if (MV) {
          // fold the pruned pages in: mass x mean of V (...meanv_bsz_q2fp8.py:188-200)
          const float* sm_pm = sm_l + 8 * 64;
          const float* sm_pl = sm_l + 16 * 64;
          float p_top = -INFINITY, p_acc = 0.f;
          for (int i = 0; i < per_head; ++i)
            if (sm_pl[h * 64 + i] != 0.f) p_top = fmaxf(p_top, sm_pm[h * 64 + i]);
          for (int i = 0; i < per_head; ++i)
            if (sm_pl[h * 64 + i] != 0.f) p_acc += sm_pl[h * 64 + i] * exp2f(sm_pm[h * 64 + i] - p_top);
          if (acc > 0.f || p_acc > 0.f) {
            const float nm = fmaxf(top, p_top);
            const float rb = acc > 0.f ? exp2f(top - nm) : 0.f, rp = p_acc > 0.f ? exp2f(p_top - nm) : 0.f;
            const int64_t ve = (static_cast<int64_t>(b) * p.HKV + hkv) * kHeadDim + 4 * lane;
            const float wv = p_acc * rp;
            o.x = o.x * rb + load_as_float(p.v_mean, ve, p.v_bf16 ? FFA_BF16 : FFA_F16) * wv;
            o.y = o.y * rb + load_as_float(p.v_mean, ve + 1, p.v_bf16 ? FFA_BF16 : FFA_F16) * wv;
            o.z = o.z * rb + load_as_float(p.v_mean, ve + 2, p.v_bf16 ? FFA_BF16 : FFA_F16) * wv;
            o.w = o.w * rb + load_as_float(p.v_mean, ve + 3, p.v_bf16 ? FFA_BF16 : FFA_F16) * wv;
            acc = acc * rb + wv;
          }
        }
        const float inv = acc == 0.f ? 0.f : 1.f / acc;
        const float r0 = o.x * inv, r1 = o.y * inv, r2 = o.z * inv, r3 = o.w * inv;
        const int64_t e = row * kHeadDim + 4 * lane;
        if (p.out) {
          store_from_float(p.out, e, p.q_dtype, r0);
          store_from_float(p.out, e + 1, p.q_dtype, r1);
          store_from_float(p.out, e + 2, p.q_dtype, r2);
          store_from_float(p.out, e + 3, p.q_dtype, r3);
        }
        if (p.partial_out) {
          float* po = p.partial_out + row * (kHeadDim + 1);
          po[4 * lane] = r0; po[4 * lane + 1] = r1; po[4 * lane + 2] = r2; po[4 * lane + 3] = r3;
          if (lane == 0) po[kHeadDim] = acc == 0.f ? -INFINITY : top + log2f(acc);
        }
      }
    }
  }
  if (timed_out && p.status && atomicCAS(p.status, 0, 1) == 0) {
    p.status[1] = gave_up_site; p.status[2] = gave_up_it; p.status[3] = gave_up_n; p.status[4] = gave_up_seg;
    p.status[5] = static_cast<int>(blockIdx.x); p.status[6] = tid;
  }
}

// ---- host side ------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
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

// [rows, HKV*row_bytes] bytes, box = 64 rows x box_bytes
bool make_map(CUtensorMap* m, const void* base, int64_t rows, int64_t row_bytes_all_heads, int box_bytes,
              bool swizzle128, int promo) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes_all_heads), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes_all_heads)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes), static_cast<cuuint32_t>(kPage)};
  const cuuint32_t estr[2] = {1, 1};
  return encode_tiled_fn()(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE,
                           swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                           static_cast<CUtensorMapL2promotion>(promo), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Launches the kernel, or (stream == kQueryResidency) returns how many of its CTAs fit on an SM.
const cudaStream_t kQueryResidency = reinterpret_cast<cudaStream_t>(static_cast<intptr_t>(-16));

template <int FMT, int F8, int NT, bool VBF, int DA, int QP, bool MV = false>
int launch_one(const DecodeParams& p, const CUtensorMap& mc, const CUtensorMap& mr, const CUtensorMap& mv,
               cudaStream_t stream) {
  using L = SmemT<FMT, DA>;
  auto kern = decode_tma_kernel<FMT, F8, NT, VBF, DA, QP, MV>;
  static bool configured[64] = {};
  static int resident[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const bool slot = dev >= 0 && dev < 64;
  if (!slot || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
    if (e != cudaSuccess) return note_cuda_error(e, "cudaFuncSetAttribute(decode_tma)");
    if (slot) configured[dev] = true;
  }
  if (stream == kQueryResidency) {
    if (slot && resident[dev] > 0) return resident[dev];
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kThreads, L::kBytes) != cudaSuccess || n < 1) n = 1;
    if (slot) resident[dev] = n;
    return n;
  }
  const int64_t total_pages = static_cast<int64_t>(p.B) * p.HKV * p.NP;
  const unsigned grid = static_cast<unsigned>((total_pages + p.ppc - 1) / p.ppc);
  kern<<<grid, kThreads, L::kBytes, stream>>>(p, mc, mr, mv);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FFA_OK : note_cuda_error(e, "decode_tma launch");
}

// bf16 q goes with either V type; fp16 q with fp16 V (decode_tma_supported admits nothing else)
template <int FMT, int F8, int NT>
int launch_types(const DecodeParams& p, const CUtensorMap& mc, const CUtensorMap& mr, const CUtensorMap& mv,
                 cudaStream_t stream) {
  if constexpr (FMT == FFA_K_Q2) {
    if (p.v_mean) {                                  // mean-V variant: 2-bit format only, like the reference
      if (p.q_dtype == FFA_F16) return launch_one<FMT, F8, NT, false, 1, 3, true>(p, mc, mr, mv, stream);
      return p.v_bf16 ? launch_one<FMT, F8, NT, true, 1, 2, true>(p, mc, mr, mv, stream)
                      : launch_one<FMT, F8, NT, false, 1, 2, true>(p, mc, mr, mv, stream);
    }
  }
  if (p.q_dtype == FFA_F16) return launch_one<FMT, F8, NT, false, 1, 3>(p, mc, mr, mv, stream);
  return p.v_bf16 ? launch_one<FMT, F8, NT, true, 1, 2>(p, mc, mr, mv, stream)
                  : launch_one<FMT, F8, NT, false, 1, 2>(p, mc, mr, mv, stream);
}

template <int FMT>
int launch_fmt(const DecodeParams& p, int f8, const CUtensorMap& mc, const CUtensorMap& mr, const CUtensorMap& mv,
               cudaStream_t stream) {
  if (p.G <= 4)
    return f8 == FFA_E4M3 ? launch_types<FMT, FFA_E4M3, 1>(p, mc, mr, mv, stream)
                          : launch_types<FMT, FFA_E5M2, 1>(p, mc, mr, mv, stream);
  return f8 == FFA_E4M3 ? launch_types<FMT, FFA_E4M3, 2>(p, mc, mr, mv, stream)
                        : launch_types<FMT, FFA_E5M2, 2>(p, mc, mr, mv, stream);
}

}  // namespace

void decode_tma_plan(int B, int HKV, int NP, int wc_in, int ctas_per_sm, int* wc_out, int* nch_out) {
  static int sms = [] {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    return n;
  }();
  const long long total = static_cast<long long>(B) * HKV * NP;
  long long wc = wc_in;
  if (wc <= 0) {
    const long long slots = static_cast<long long>(ctas_per_sm) * sms;   // resident CTAs: one wave
    wc = (total + slots - 1) / slots;
    if (wc < 4) wc = 4;                               // a CTA's set-up is worth a few pages
  }
  // the in-kernel merge holds at most 64 partials per q head
  if (wc < (NP + 62) / 63) wc = (NP + 62) / 63;
  if (wc > total) wc = total;
  if (wc < 1) wc = 1;
  *wc_out = static_cast<int>(wc);
  *nch_out = static_cast<int>((NP + wc - 1) / wc) + 1;
}

int decode_tma_residency(const DecodeParams& p, int variant, int f8) {
  // ask the runtime how many CTAs of the kernel that would run fit on an SM (shared memory and
  // registers both count); the page ranges are cut so that the grid is exactly one such wave
  CUtensorMap none{};
  int n;
  switch (variant) {
    case FFA_K_FP8:   n = launch_fmt<FFA_K_FP8>(p, f8, none, none, none, kQueryResidency); break;
    case FFA_K_Q2:    n = launch_fmt<FFA_K_Q2>(p, f8, none, none, none, kQueryResidency); break;
    case FFA_K_FP4:   n = launch_fmt<FFA_K_FP4>(p, f8, none, none, none, kQueryResidency); break;
    case FFA_K_NF4:   n = launch_fmt<FFA_K_NF4>(p, f8, none, none, none, kQueryResidency); break;
    case FFA_K_NVFP4: n = launch_fmt<FFA_K_NVFP4>(p, f8, none, none, none, kQueryResidency); break;
    default: n = 1;
  }
  return n < 1 ? 1 : (n > 4 ? 4 : n);
}

bool decode_tma_supported(const DecodeParams& p) {
  // the query is split into exact e4m3 pieces: two for bf16, three for fp16 (fp16 q comes with
  // fp16 V in practice; the mixed case is left to the fp16 tensor-core kernel)
  const bool types_ok = p.q_dtype == FFA_BF16 || (p.q_dtype == FFA_F16 && !p.v_bf16);
  return types_ok && encode_tiled_fn() != nullptr;
}

namespace {
// The three tensor maps of the last call on this thread: a decode loop calls with the same tensors step
// after step, and encoding the maps (three driver calls) is most of an eager call's host time.
struct TmaMapCache {
  bool valid = false;
  const void *kc = nullptr, *kr = nullptr, *v = nullptr;
  int64_t rows = 0;
  int hkv = 0, variant = 0;
  alignas(64) CUtensorMap mc, mr, mv;
};
thread_local TmaMapCache g_tma_maps;
}  // namespace

int launch_decode_tma(const DecodeParams& p, int variant, int f8, int64_t kv_rows, cudaStream_t stream) {
  if (kv_rows <= 0 || kv_rows > 0x7fffffffLL) return FFA_E_LIMIT;
  TmaMapCache& c = g_tma_maps;
  if (!(c.valid && c.kc == p.kc && c.kr == p.kr && c.v == p.v && c.rows == kv_rows && c.hkv == p.HKV &&
        c.variant == variant)) {
    c.valid = false;
    const int row_c = variant == FFA_K_FP8 ? 128 : (variant == FFA_K_Q2 ? 32 : 64);
    // L2 promotion no wider than one head's row: a 256-byte promotion on 128-byte rows pulled the
    // neighbouring head's bytes from DRAM too early to be reused (+15 % DRAM traffic, -11 % speed).
    const int promo_c = row_c >= 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                     : (row_c >= 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B : CU_TENSOR_MAP_L2_PROMOTION_NONE);
    const int promo_r = CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
    const int promo_v = CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
    if (!make_map(&c.mc, p.kc, kv_rows, static_cast<int64_t>(p.HKV) * row_c, row_c, variant == FFA_K_FP8, promo_c))
      return FFA_E_LAUNCH;
    // without a residual the map is never used; point it at the coarse tensor to keep it valid
    if (!make_map(&c.mr, p.kr ? p.kr : p.kc, kv_rows, static_cast<int64_t>(p.HKV) * (p.kr ? kResRow : row_c),
                  p.kr ? kResRow : row_c, p.kr != nullptr, p.kr ? promo_r : promo_c))
      return FFA_E_LAUNCH;
    if (!make_map(&c.mv, p.v, kv_rows, static_cast<int64_t>(p.HKV) * kVRow, 128, true, promo_v)) return FFA_E_LAUNCH;
    c.kc = p.kc; c.kr = p.kr; c.v = p.v; c.rows = kv_rows; c.hkv = p.HKV; c.variant = variant;
    c.valid = true;
  }
  const CUtensorMap &mc = c.mc, &mr = c.mr, &mv = c.mv;
  switch (variant) {
    case FFA_K_FP8:   return launch_fmt<FFA_K_FP8>(p, f8, mc, mr, mv, stream);
    case FFA_K_Q2:    return launch_fmt<FFA_K_Q2>(p, f8, mc, mr, mv, stream);
    case FFA_K_FP4:   return launch_fmt<FFA_K_FP4>(p, f8, mc, mr, mv, stream);
    case FFA_K_NF4:   return launch_fmt<FFA_K_NF4>(p, f8, mc, mr, mv, stream);
    case FFA_K_NVFP4: return launch_fmt<FFA_K_NVFP4>(p, f8, mc, mr, mv, stream);
    default: return FFA_E_VARIANT;
  }
}

}  // namespace ffa
