// FFA decode attention for B200: warp-specialised kernel, one persistent CTA per SM.
//
// Same math and reference semantics as the fp16 kernel in ffa_decode.cu (coarse score -> prune ->
// residual refine -> online softmax * V -> merge; reference ffa-q2fp8/attn_kernel/
// attn_kernel_v1210_fused_bsz_q2fp8.py:30-171), organised so that a pruned page costs only its
// coarse bytes and its share of the scoring arithmetic:
//
//   warp 0        coarse producer: streams the coarse K tile of every page of the CTA's range into a
//                 ring of shared-memory slots with TMA, as far ahead as the ring allows.
//   warps 2..5    scoring: each takes whole pages (64 tokens = four m16 tiles) round robin, computes
//                 the coarse q.k of every token against all heads of the group on the tensor cores
//                 and publishes the page's per-head maximum plus the raw dots.  No CTA barrier, no
//                 exchange between warps: a page's statistic is complete inside one warp.
//   warp 1        dispatcher: walks the published pages in order, applies the prune rule (a group of
//                 SBS/64 pages is dropped only if every head's maximum over the group is strictly
//                 below that head's threshold), writes the kept mask and, for kept pages, requests
//                 residual + V with TMA into the next free slot of a second ring.
//   warps 6..9    refine: kept page number k goes to refine warp k mod 4, which adds the residual
//                 dot to the coarse dots, does the page's softmax and accumulates P.V for all 64
//                 tokens.  Again nothing leaves the warp until the segment ends.
//
// Scoring runs ahead of refining by the depth of the rings, so the residual + V of several kept
// pages are in flight while earlier pages are refined and later ones are scored; when most pages
// are pruned the step moves at the speed of the scoring warps instead of paying a per-page barrier.
//
// A CTA walks a contiguous range of the flattened (batch x kv-head, page) space; the part inside
// one (batch, kv-head) is a segment and ends in one partial (m, l, o[128]) per q head; the segment
// that arrives last for a (batch, kv-head) merges its partials (stage 2, ...q2fp8.py:142-171).
//
// Numerics are those of the TMA kernel this replaces: q split into exact e4m3 pieces against raw
// fp8 K bytes (fp8 coarse and the residual), fp16 q against dequantised codes (2-/4-bit coarse),
// P rounded to fp16 and split into exact bf16 pieces for bf16 V.  The refined score is
// q.k_coarse + q.k_residual (the reference rounds k_coarse + k_residual to fp16 first).
//
// Every wait is bounded in wall-clock time.  A wait that gives up raises a CTA-wide flag; every role
// then leaves its loop, the CTA publishes NaN partials for its remaining segments (so the merged
// output of the affected heads is NaN, not a plausible number) and sets the status word.
#pragma once

#include "ffa_decode_prims.cuh"

namespace ffa {

namespace {

constexpr int kNS = 4;                     // scoring warps
constexpr int kNR = 4;                     // refine warps (the first four also run the segment epilogue)
constexpr int kWsWarps = 2 + kNS + kNR;
constexpr int kWsThreads = 32 * kWsWarps;
constexpr int kBatch = kMaxPruneGroup;     // pages the dispatcher decides per trip; a whole prune group must fit (SBS <= 512)
constexpr int kND = 2 * kBatch;            // published-page ring: scoring runs a trip ahead of the pages still being refined
constexpr int kSampleRows = kSample;       // rows of a threshold sample tile

template <int FMT, int NT>
struct WsSmem {
  static constexpr int kRow = Fmt<FMT>::kRow;
  static constexpr int kCoarseSlot = kPage * kRow;                                  // 8 / 2 / 4 KiB
  // coarse ring: each scoring warp should find its next tile already landed, i.e. more than one slot
  // per warp in flight; the residual + V ring takes what is left of the 227 KiB
  static constexpr int kNC = FMT == FFA_K_FP8 ? (NT == 2 ? 5 : 7) : (FMT == FFA_K_Q2 ? 16 : 8);
  static constexpr int kNRV = (NT == 2 || FMT == FFA_K_FP8) ? 6 : 7;                // residual + V slots
  static constexpr int kSampleSlot = kSampleRows * kRow < 1024 ? 1024 : kSampleRows * kRow;
  static constexpr int kHist = NT * 1024;                                           // raw dots of one page
  static constexpr bool kHasChannelScale = (FMT == FFA_K_Q2 || FMT == FFA_K_NF4);
  static constexpr int kOffRv = 0;
  static constexpr int kOffCoarse = kOffRv + kNRV * kRvSlot;
  static constexpr int kOffSample = kOffCoarse + kNC * kCoarseSlot;
  static constexpr int kOffDHist = kOffSample + 2 * kSampleSlot;
  static constexpr int kOffDMax = kOffDHist + kND * kHist;      // [kND][8] page maxima
  static constexpr int kOffDPl = kOffDMax + kND * 32;           // [kND][8] mean-V: mass relative to the maximum
  static constexpr int kOffBars = kOffDPl + kND * 32;
  static constexpr int kNBars = 2 * kNC + 2 + 2 * kND + 2 * kNRV + 1;
  static constexpr int kOffMisc = kOffBars + ((kNBars * 8 + 63) / 64) * 64;
  // misc: sTh[16] | sApx[16] | kq_page[8] | kq_ds[8] | abort, flag, pad[6] | sS[128] | sZ[128] | book[16]
  static constexpr int kOffTh = kOffMisc;
  static constexpr int kOffApx = kOffTh + 64;
  static constexpr int kOffKq = kOffApx + 64;
  static constexpr int kOffFlags = kOffKq + 64;
  static constexpr int kOffS = kOffFlags + 32;
  static constexpr int kOffZ = kOffS + 512;
  static constexpr int kOffBook = kOffZ + 512;
  static constexpr int kOffProf = kOffBook + 64;
  static constexpr int kBytes = kOffProf + 1024;                // + alignment slack
  // the epilogue's reduction buffers reuse the coarse ring (idle once a segment's pages are scored)
  static constexpr int kRedBytes = kNR * 8 * 128 * 4 + 2 * kNR * 8 * 4 + 64;
  static_assert(kRedBytes <= kNC * kCoarseSlot, "epilogue buffers must fit the coarse ring");
  static_assert(kBytes <= 232448, "shared memory of one CTA");
  static_assert(kNRV >= 4, "the dispatcher issues up to four requests per round");
  // a ring shared by several consumer warps stays phase-safe only if it has at least as many slots
  static_assert(kNC >= kNS && kNRV >= kNR, "rings must not be smaller than the number of their consumers");
};

// Profiling builds (-DFFA_WS_PROFILE) time, per warp and in SM cycles, the waits of each role and a few
// stretches of work; lane 0 keeps the sums in registers and adds them to the status block at the end.
#ifdef FFA_WS_PROFILE
#define PROF_T(name) const uint32_t name = static_cast<uint32_t>(clock())
#define PROF_ADD(idx, since) do { pacc[idx] += static_cast<uint32_t>(clock()) - (since); } while (0)
#define PROF_INC(idx) do { pacc[idx] += 1u; } while (0)
#define WS_WAIT(bar, par, site, idx) ws_wait_timed(bar, par, sAbort, site, pacc[idx])
#else
#define PROF_T(name)
#define PROF_ADD(idx, since)
#define PROF_INC(idx)
#define WS_WAIT(bar, par, site, idx) ws_wait(bar, par, sAbort, site)
#endif

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;\n" ::"r"(id), "r"(count) : "memory");
}

// Bounded wait of one lane that also ends when another role has given up (abort flag).  Returns
// false without the phase having completed in both cases; the first thread to run out of time sets
// the flag to `site` (a small code naming the wait) so that the status block can say where.
__device__ __forceinline__ bool ws_wait_lane(uint32_t bar, uint32_t parity, int* abort_flag, int site) {
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
      if (*reinterpret_cast<volatile int*>(abort_flag) != 0) return false;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > kWaitLimitNs) {
        atomicCAS(abort_flag, 0, site);
        return false;
      }
    }
  }
}

// The whole (converged) warp waits, every lane on its own; the answer is made the same in every lane
// so that the loops around the waits stay warp-uniform even when one lane runs out of time a moment
// before the others.  (Polling with one lane and broadcasting measured slower.)
__device__ __forceinline__ bool ws_wait_warp(uint32_t bar, uint32_t parity, int* abort_flag, int site) {
  return __all_sync(0xffffffffu, ws_wait_lane(bar, parity, abort_flag, site)) != 0;
}

__device__ __forceinline__ bool ws_wait(uint32_t bar, uint32_t parity, int* abort_flag, int site) {
  return ws_wait_warp(bar, parity, abort_flag, site);
}
#ifdef FFA_WS_PROFILE
__device__ __forceinline__ bool ws_wait_timed(uint32_t bar, uint32_t parity, int* abort_flag, int site, uint32_t& acc) {
  const uint32_t t0 = static_cast<uint32_t>(clock());
  const bool r = ws_wait_warp(bar, parity, abort_flag, site);
  acc += static_cast<uint32_t>(clock()) - t0;
  return r;
}
#endif

// q operands of one (batch, kv-head) for a warp (every lane ends up with its MMA B fragments).
//   qb: e4m3 pieces of q * 2^e (hi, mid [, lo]), for the fp8 tiles;  qinv: 2^-e per head column
//   qh: q as fp16 (odd columns zero), for the dequantised 2-/4-bit tiles
// B-fragment column n = g of n-tile nt is head 4nt + g/2, piece g&1.  q is bf16 (QP = 2: two pieces
// are exact), fp16 (QP = 3) or fp32 rounded to fp16 first like the reference's q.to(float16) (QP = 3).
template <int NT, int QP, bool WANT_QH>
__device__ __forceinline__ void prep_q(const DecodeParams& p, int b, int hkv, int G, int g, int t,
                                       uint32_t (&qb)[NT * (QP - 1)][4][2], uint32_t (&qh)[NT][8][2], float (&qinv)[NT]) {
  auto q_pair = [&](uint32_t w) -> float2 {
    if (QP == 2) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
    return unpack_h2(w);
  };
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    const int hc = 4 * nt + (g >> 1);
    const bool second = (g & 1) != 0;
    uint32_t raw[16];
    if (hc < G) {
      const int64_t e0 = (static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G + hc) * kHeadDim + 32 * t;
      if (QP == 3 && p.q_dtype == FFA_F32) {
        const float4* src = reinterpret_cast<const float4*>(p.q + e0 * 4);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 v4 = src[i];
          raw[2 * i] = pack_h2(v4.x, v4.y);
          raw[2 * i + 1] = pack_h2(v4.z, v4.w);
        }
      } else {
        const uint4* src = reinterpret_cast<const uint4*>(p.q + e0 * 2);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 v4 = src[i];
          raw[4 * i] = v4.x; raw[4 * i + 1] = v4.y; raw[4 * i + 2] = v4.z; raw[4 * i + 3] = v4.w;
        }
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
    // this lane needs 2^-e of head 4nt + t, which the lanes with g>>1 == t computed
    qinv[nt] = __shfl_sync(0xffffffffu, down, 8 * t);
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const float2 fa = q_pair(raw[2 * r]), fb = q_pair(raw[2 * r + 1]);
      const float x0 = fa.x * up, x1 = fa.y * up, x2 = fb.x * up, x3 = fb.y * up;
      const uint32_t h01 = f32x2_to_e4m3x2(x0, x1), h23 = f32x2_to_e4m3x2(x2, x3);
      const float2 d01 = e4m3x2_to_f32x2(h01), d23 = e4m3x2_to_f32x2(h23);
      const float r0 = (x0 - d01.x) * 16.f, r1 = (x1 - d01.y) * 16.f, r2 = (x2 - d23.x) * 16.f, r3 = (x3 - d23.y) * 16.f;
      const uint32_t m01 = f32x2_to_e4m3x2(r0, r1), m23 = f32x2_to_e4m3x2(r2, r3);
      qb[nt][r >> 1][r & 1] = second ? (m01 | (m23 << 16)) : (h01 | (h23 << 16));
      if (QP == 3) {
        const float2 e01 = e4m3x2_to_f32x2(m01), e23 = e4m3x2_to_f32x2(m23);
        const uint32_t l01 = f32x2_to_e4m3x2((r0 - e01.x) * 16.f, (r1 - e01.y) * 16.f);
        const uint32_t l23 = f32x2_to_e4m3x2((r2 - e23.x) * 16.f, (r3 - e23.y) * 16.f);
        qb[(QP - 2) * NT + nt][r >> 1][r & 1] = second ? 0u : (l01 | (l23 << 16));
      }
    }
    if (WANT_QH) {
#pragma unroll
      for (int s = 0; s < 8; ++s) {
        qh[nt][s][0] = second ? 0u : (QP == 2 ? bf16x2_to_h2(raw[2 * s]) : raw[2 * s]);
        qh[nt][s][1] = second ? 0u : (QP == 2 ? bf16x2_to_h2(raw[2 * s + 1]) : raw[2 * s + 1]);
      }
    }
  }
}

// FMT: coarse format; F8: fp8 encoding of the residual (and of the fp8 coarse base); NT: n-tiles of
// four q heads (1: group <= 4, 2: group <= 8); VBF: V is bf16 (else fp16); QP: e4m3 pieces per q value;
// MV: mean-V variant (pruned pages keep their coarse softmax mass; DecodeParams::v_mean).
template <int FMT, int F8, int NT, bool VBF, int QP, bool MV>
__global__ void __launch_bounds__(kWsThreads, 1) decode_ws_kernel(const __grid_constant__ DecodeParams p,
                                                                  const __grid_constant__ CUtensorMap tm_c,
                                                                  const __grid_constant__ CUtensorMap tm_s,
                                                                  const __grid_constant__ CUtensorMap tm_r,
                                                                  const __grid_constant__ CUtensorMap tm_v) {
  using L = WsSmem<FMT, NT>;
  constexpr int ROW = L::kRow;
  constexpr int kNC = L::kNC;
  constexpr int kNRV = L::kNRV;
  constexpr bool kFp8Coarse = (FMT == FFA_K_FP8);
  constexpr uint32_t kFull = 0xffffffffu;
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled TMA tiles need 1024-byte alignment
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int G = p.G, T = p.T;
  const int m_grp = p.group;                       // pages per prune group (SBS / 64)

  const uint32_t bars = smem_u32(smem + L::kOffBars);
  auto cfull = [&](int i) { return bars + 8u * i; };
  auto cempty = [&](int i) { return bars + 8u * (kNC + i); };
  auto sfull = [&](int i) { return bars + 8u * (2 * kNC + i); };
  auto dfull = [&](int i) { return bars + 8u * (2 * kNC + 2 + i); };
  auto dempty = [&](int i) { return bars + 8u * (2 * kNC + 2 + kND + i); };
  auto rvfull = [&](int i) { return bars + 8u * (2 * kNC + 2 + 2 * kND + i); };
  auto rvempty = [&](int i) { return bars + 8u * (2 * kNC + 2 + 2 * kND + kNRV + i); };
  const uint32_t thfull = bars + 8u * (2 * kNC + 2 + 2 * kND + 2 * kNRV);

  float* dhist = reinterpret_cast<float*>(smem + L::kOffDHist);
  float* dmax = reinterpret_cast<float*>(smem + L::kOffDMax);
  float* dpl = reinterpret_cast<float*>(smem + L::kOffDPl);
  float* sTh = reinterpret_cast<float*>(smem + L::kOffTh);
  float* sApx = reinterpret_cast<float*>(smem + L::kOffApx);
  int* kq_page = reinterpret_cast<int*>(smem + L::kOffKq);      // per residual+V slot: page of the (b, kv-head), -1 = end marker
  int* kq_ds = kq_page + 8;                                      // ... and the published-page entry that holds its dots
  int* sAbort = reinterpret_cast<int*>(smem + L::kOffFlags);
  int* sFlag = sAbort + 1;
  float* sS = reinterpret_cast<float*>(smem + L::kOffS);
  float* sZ = reinterpret_cast<float*>(smem + L::kOffZ);
  float* sBook = reinterpret_cast<float*>(smem + L::kOffBook);
  // epilogue buffers, on top of the coarse ring
  float* red = reinterpret_cast<float*>(smem + L::kOffCoarse);      // [kNR][8 heads][128]
  float* lred = red + kNR * 8 * 128;                                // [kNR][8]
  float* mred = lred + kNR * 8;                                     // [kNR][8]

  const bool use_res = p.use_res != 0;
  const bool sampled = p.th_in == nullptr;
  const uint32_t rv_bytes = (use_res ? kPage * kResRow : 0) + kPage * kVRow;

#ifdef FFA_WS_PROFILE
  uint32_t pacc[6] = {0u, 0u, 0u, 0u, 0u, 0u};     // per-role meaning, see the end of the kernel
  const long long prof_c0 = clock64();
  unsigned long long prof_g0;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(prof_g0));
  uint32_t prof_role = 0, prof_epi = 0;
#endif
  if (tid == 0) {
    for (int i = 0; i < L::kNBars - 1; ++i) mbar_init(bars + 8 * i, 1);
    mbar_init(thfull, 2);                          // the two scoring warps that score the samples
    *sAbort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  __syncthreads();

  enum { kRoleCoarse = 0, kRoleDispatch = 1, kRoleScore = 2, kRoleRefine = 3 };
  const int role = warp == 0 ? kRoleCoarse : (warp == 1 ? kRoleDispatch : (warp < 2 + kNS ? kRoleScore : kRoleRefine));
  const int sw = warp - 2;                         // scoring warp index
  const int rw = warp - 2 - kNS;                   // refine warp index

  // running counters that keep ring positions and mbarrier phases consistent across segments
  uint32_t gc = 0;                                 // pages of earlier segments (all roles)
  uint32_t kk = 0;                                 // dispatcher: kept pages + end markers issued so far
  uint32_t myk = rw;                               // refine warp: ordinal of its next kept page
  uint32_t act_ord = 0;                            // segments that ran the pipeline (phase of the per-segment barriers)

  const int NPp = p.NPp;                           // pages per (b, kv-head) rounded up to whole prune groups
  const int64_t total_pages = static_cast<int64_t>(p.B) * p.HKV * NPp;
  int64_t g0 = static_cast<int64_t>(blockIdx.x) * p.ppc;
  const int64_t g1 = min(total_pages, g0 + p.ppc);

  while (g0 < g1) {
    // ---- segment geometry ------------------------------------------------------------------------
    const int unit = static_cast<int>(g0 / NPp);
    const int b = unit / p.HKV, hkv = unit % p.HKV;
    const int64_t unit0 = static_cast<int64_t>(unit) * NPp;
    const int page_begin = static_cast<int>(g0 - unit0);
    const int n_pad = static_cast<int>(min(g1 - g0, static_cast<int64_t>(NPp - page_begin)));
    const int n = max(0, min(n_pad, p.NP - page_begin));              // real pages of the segment
    const int part = static_cast<int>(g0 / p.ppc - unit0 / p.ppc);    // partial slot of this segment
    g0 += n_pad;
    const int64_t row0 = static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G;
    const bool aborted = *reinterpret_cast<volatile int*>(sAbort) != 0;   // uniform: read between CTA barriers
    const bool active = n > 0 && !aborted;
    const uint32_t seg_par = act_ord & 1u;

    auto row_of_page = [&](int page, int bt_val) -> int {
      return p.bt ? bt_val * kPage : b * T + page * kPage;
    };
    auto to_log2 = [&](float d) -> float { return (d * p.sm_scale) * kLog2e; };

#ifdef FFA_WS_PROFILE
    const uint32_t prof_seg0 = static_cast<uint32_t>(clock());
#endif
    if (active && role == kRoleCoarse) {
      // ================= coarse producer ===========================================================
      if (sampled && lane == 0) {
        const int tok1 = (p.NTB - 1) * kSample;
        const int r0 = p.bt ? p.bt[static_cast<int64_t>(b) * p.bt_stride] * kPage : b * T;
        const int r1 = (p.bt ? p.bt[static_cast<int64_t>(b) * p.bt_stride + tok1 / kPage] * kPage
                             : b * T + (tok1 / kPage) * kPage) + tok1 % kPage;
        mbar_expect_tx(sfull(0), kSampleRows * ROW);
        tma_load_2d(smem_u32(smem + L::kOffSample), &tm_s, hkv * ROW, r0, sfull(0));
        mbar_expect_tx(sfull(1), kSampleRows * ROW);
        tma_load_2d(smem_u32(smem + L::kOffSample + L::kSampleSlot), &tm_s, hkv * ROW, r1, sfull(1));
      }
      int btv = 0;
      for (int c = 0; c < n; ++c) {
        const uint32_t gcc = gc + c;
        const int slot = gcc % kNC;
        if ((c & 31) == 0 && p.bt && c + lane < n)
          btv = p.bt[static_cast<int64_t>(b) * p.bt_stride + page_begin + c + lane];
        const int row = row_of_page(page_begin + c, __shfl_sync(kFull, btv, c & 31));
        if (gcc >= kNC && !WS_WAIT(cempty(slot), ((gcc / kNC) - 1u) & 1u, 1, 0)) break;
        if (lane == 0) {
          mbar_expect_tx(cfull(slot), L::kCoarseSlot);
          tma_load_2d(smem_u32(smem + L::kOffCoarse + slot * L::kCoarseSlot), &tm_c, hkv * ROW, row, cfull(slot));
        }
      }
    } else if (active && role == kRoleDispatch) {
      // ================= dispatcher ================================================================
      // Eight pages per trip, four lanes per page (lane = 4 * page + hq, heads 2hq and 2hq + 1): one
      // chain of wait -> compare -> vote decides eight pages, and the lanes that lead a kept page
      // request its residual + V side by side.  (One page per trip made this warp the slowest stage:
      // the chain is a few hundred cycles of latency however little it computes.)
      const int pj = lane >> 2, hq = lane & 3;
      float th0 = 0.f, th1 = 0.f;
      bool ok = true;
      if (sampled) {
        ok = WS_WAIT(thfull, seg_par, 2, 0);
        th0 = fmaxf(sTh[2 * hq], sTh[8 + 2 * hq]) - p.delta;
        th1 = fmaxf(sTh[2 * hq + 1], sTh[8 + 2 * hq + 1]) - p.delta;
      } else {
        if (2 * hq < G) th0 = p.th_in[row0 + 2 * hq];
        if (2 * hq + 1 < G) th1 = p.th_in[row0 + 2 * hq + 1];
      }
      if (ok && p.th_out && page_begin == 0 && pj == 0) {
        if (2 * hq < G) p.th_out[row0 + 2 * hq] = th0;
        if (2 * hq + 1 < G) p.th_out[row0 + 2 * hq + 1] = th1;
      }
      // mean-V: running maximum / mass of the pruned pages, heads 2hq and 2hq + 1 (meaningful in lanes 0-3)
      float apx_m0 = -INFINITY, apx_l0 = 0.f, apx_m1 = -INFINITY, apx_l1 = 0.f;
      int8_t* mask_row = p.mask ? p.mask + (static_cast<int64_t>(b) * p.HKV + hkv) * p.NTBS : nullptr;
      const int gsz = 4 * m_grp;                                   // lanes of one prune group (4 ... 32)
      const uint32_t gmask = gsz >= 32 ? kFull : (((1u << gsz) - 1u) << ((lane / gsz) * gsz));
      for (int c0 = 0; ok && c0 < n; c0 += kBatch) {
        const int c = c0 + pj;
        const bool valid = c < n;
        const uint32_t gcc = gc + c;
        const int ds = gcc % kND;
        // the page's row in the pool, asked for before the wait so that the table lookup hides behind it
        int btv = 0;
        if (p.bt && valid && hq == 0) btv = p.bt[static_cast<int64_t>(b) * p.bt_stride + page_begin + c];
#ifdef FFA_WS_PROFILE
        const uint32_t tw0 = static_cast<uint32_t>(clock());
#endif
        ok = __all_sync(kFull, !valid || ws_wait_lane(dfull(ds), (gcc / kND) & 1u, sAbort, 3)) != 0;
#ifdef FFA_WS_PROFILE
        pacc[1] += static_cast<uint32_t>(clock()) - tw0;
#endif
        if (!ok) break;
        float mx0 = valid ? dmax[ds * 8 + 2 * hq] : -INFINITY, mx1 = valid ? dmax[ds * 8 + 2 * hq + 1] : -INFINITY;
        // pruned only if every head's maximum over the whole group is strictly below its threshold
        // (...q2fp8.py:97-102 with SBS = 64 x group)
        float gx0 = mx0, gx1 = mx1;
        for (int off = 4; off < gsz; off <<= 1) {
          gx0 = fmaxf(gx0, __shfl_xor_sync(kFull, gx0, off));
          gx1 = fmaxf(gx1, __shfl_xor_sync(kFull, gx1, off));
        }
        const bool reaches = valid && ((2 * hq < G && !(gx0 < th0)) || (2 * hq + 1 < G && !(gx1 < th1)));
        const bool keep = (__ballot_sync(kFull, reaches) & gmask) != 0u;
        if (mask_row && valid && (lane % gsz) == 0) mask_row[(page_begin + c) / m_grp] = keep ? 1 : 0;
        const bool lead = valid && hq == 0;
        const uint32_t kept_bits = __ballot_sync(kFull, lead && keep);
        PROF_T(t_keep);
        bool lane_ok = true;
        const uint32_t rank = __popc(kept_bits & ((1u << lane) - 1u));
        // Two rounds of at most four requests: a request may have to wait for the slot of a page that is
        // kNRV places ahead of it, and within one round no lane may depend on another lane of the round
        // (lanes that are done wait for the others where the branches join).
#pragma unroll 1
        for (uint32_t round = 0; round < 2; ++round) {
          if (lead && keep && (rank >> 2) == round) {
            const uint32_t ord = kk + rank;
            const int slot = ord % kNRV;
            const int row = row_of_page(page_begin + c, btv);
            if (ord >= kNRV) lane_ok = ws_wait_lane(rvempty(slot), ((ord / kNRV) - 1u) & 1u, sAbort, 4);
            if (lane_ok) {
              kq_page[slot] = page_begin + c;
              kq_ds[slot] = ds;
              const uint32_t bar = rvfull(slot);
              const uint32_t dst = smem_u32(smem + L::kOffRv + slot * kRvSlot);
              mbar_expect_tx(bar, rv_bytes);
              if (use_res) tma_load_2d(dst, &tm_r, hkv * kResRow, row, bar);
              tma_load_2d(dst + kPage * kResRow, &tm_v, hkv * kVRow, row, bar);
              tma_load_2d(dst + kPage * kResRow + kPage * 128, &tm_v, hkv * kVRow + 128, row, bar);
            }
          }
          __syncwarp();
        }
        kk += __popc(kept_bits);
        PROF_ADD(3, t_keep);
        if (MV) {
          // pruned pages: their coarse mass, relative to their own maximum, joins the running pair of
          // each head; the eight pages of the trip are combined across the lanes first
          float m0 = -INFINITY, l0 = 0.f, m1 = -INFINITY, l1 = 0.f;
          if (valid && !keep) {
            m0 = mx0; l0 = m0 == -INFINITY ? 0.f : dpl[ds * 8 + 2 * hq];
            m1 = mx1; l1 = m1 == -INFINITY ? 0.f : dpl[ds * 8 + 2 * hq + 1];
          }
          auto join = [](float& ma, float& la, float mb, float lb) {
            const float nm = fmaxf(ma, mb);
            if (nm != -INFINITY) {
              la = (ma == -INFINITY ? 0.f : la * ex2_approx(ma - nm)) + (mb == -INFINITY ? 0.f : lb * ex2_approx(mb - nm));
              ma = nm;
            }
          };
          for (int off = 4; off < 32; off <<= 1) {
            const float om0 = __shfl_xor_sync(kFull, m0, off), ol0 = __shfl_xor_sync(kFull, l0, off);
            const float om1 = __shfl_xor_sync(kFull, m1, off), ol1 = __shfl_xor_sync(kFull, l1, off);
            join(m0, l0, om0, ol0);
            join(m1, l1, om1, ol1);
          }
          join(apx_m0, apx_l0, m0, l0);
          join(apx_m1, apx_l1, m1, l1);
        }
        // a pruned page's entry is free again; a kept page's is released by the refine warp that reads it
        if (lead && !keep) mbar_arrive(dempty(ds));
        ok = __all_sync(kFull, lane_ok) != 0;
      }
      // end markers: one per refine warp (kept page k goes to warp k mod kNR, so kNR consecutive
      // ordinals reach every warp once)
      for (int i = 0; ok && i < kNR; ++i) {
        const int slot = kk % kNRV;
        if (kk >= kNRV && !WS_WAIT(rvempty(slot), ((kk / kNRV) - 1u) & 1u, 5, 2)) { ok = false; break; }
        if (lane == 0) {
          kq_page[slot] = -1;
          mbar_arrive(rvfull(slot));
        }
        ++kk;
      }
      if (MV && lane < 4) {
        sApx[2 * hq] = apx_m0; sApx[8 + 2 * hq] = apx_l0;
        sApx[2 * hq + 1] = apx_m1; sApx[8 + 2 * hq + 1] = apx_l1;
      }
    } else if (active && role == kRoleScore) {
      // ================= scoring warps =============================================================
      const int stid = sw * 32 + lane;
      if (L::kHasChannelScale) {
        const int64_t o = (static_cast<int64_t>(b) * p.HKV + hkv) * kHeadDim + stid;
        sS[stid] = load_as_float(p.ks, o, p.scale_dtype);
        if (FMT == FFA_K_Q2) sZ[stid] = load_as_float(p.kz, o, p.scale_dtype);
        if (FMT == FFA_K_NF4 && stid < 16) sBook[stid] = c_nf4_book[stid];
        bar_sync(1, kNS * 32);
      }
      ScaleCtx sc;
      sc.sS = sS; sc.sZ = sZ; sc.book = sBook; sc.page_scale = 1.0f;
      sc.q2_fast = false; sc.page_fast = false; sc.page_scale_h2 = 0u;
      if (FMT == FFA_K_Q2) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          sc.s2[i] = pack_h2(sS[32 * t + 2 * i], sS[32 * t + 2 * i + 1]);
          sc.z2[i] = pack_h2(sZ[32 * t + 2 * i], sZ[32 * t + 2 * i + 1]);
        }
        // The packed-fp16 route (one fused multiply-add per pair of codes) is taken only when it gives,
        // for all four codes of all 128 channels, the very bits of the reference's sequence (fp32
        // code * scale + zero, then rounded to fp16); each lane checks four channels.
        bool same = true;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float s = sS[lane + 32 * i], z = sZ[lane + 32 * i];
          same = same && exact_in_f16(s) && exact_in_f16(z);
          const __half hs = __float2half_rn(s), hz = __float2half_rn(z);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const __half fast = __hfma(__float2half_rn(static_cast<float>(c)), hs, hz);
            const __half ref = __float2half_rn(fmaf(static_cast<float>(c), s, z));
            same = same && (__half_as_ushort(fast) == __half_as_ushort(ref));
          }
        }
        sc.q2_fast = __all_sync(kFull, same) != 0;
      }
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

      uint32_t qb[NT * (QP - 1)][4][2];
      uint32_t qh[NT][8][2];
      float qinv[NT];
      prep_q<NT, QP, !kFp8Coarse>(p, b, hkv, G, g, t, qb, qh, qinv);
      auto coarse_dots = [&](float (&out)[NT][2], const uint8_t* tile, int slice) {
        if constexpr (kFp8Coarse) dot_fp8<F8, NT, QP>(out, qb, qinv, tile, slice, g, t);
        else if (FMT == FFA_K_Q2 ? sc.q2_fast : (FMT == FFA_K_NVFP4 && sc.page_fast))
          dot_f16<FMT, NT, true>(out, qh, tile, sc, slice, g, t);
        else dot_f16<FMT, NT, false>(out, qh, tile, sc, slice, g, t);
      };

      bool ok = true;
      // ---- prune thresholds (reference ...q2fp8.py:55-82): two 16-token samples of the coarse K,
      // tokens [0,16) and [(NTB-1)*16, +16), scored by the first two scoring warps
      if (sampled && sw < 2) {
        ok = WS_WAIT(sfull(sw), seg_par, 6, 0);
        const int blk = sw == 0 ? 0 : p.NTB - 1;
        const int tok0 = blk * kSample;
        if (FMT == FFA_K_NVFP4) apply_block_scale(load_block_scale(blk));
        float d[NT][2];
        coarse_dots(d, smem + L::kOffSample + sw * L::kSampleSlot, 0);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const float s0 = tok0 + g < T ? to_log2(d[nt][0]) : -INFINITY;
          const float s1 = tok0 + g + 8 < T ? to_log2(d[nt][1]) : -INFINITY;
          float mm = fmaxf(s0, s1);
#pragma unroll
          for (int off = 4; off < 32; off <<= 1) mm = fmaxf(mm, __shfl_xor_sync(kFull, mm, off));
          if (g == 0) sTh[sw * 8 + 4 * nt + t] = mm;
        }
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(thfull);
      }

      float ks_batch = 0.f;         // nvfp4: block scales of this warp's next 32 pages, one per lane
      for (int c = sw; ok && c < n; c += kNS) {
        const uint32_t gcc = gc + c;
        const int slot = gcc % kNC, ds = gcc % kND;
        const int page = page_begin + c;
        if (FMT == FFA_K_NVFP4) {
          // one global load per 32 pages: a load per page would be waited for by every arrive below
          const int it = (c - sw) / kNS;
          if ((it & 31) == 0) {
            const int cc = c + lane * kNS;
            ks_batch = cc < n ? load_block_scale(((page_begin + cc) * kPage) / p.BS) : 0.f;
          }
          apply_block_scale(__shfl_sync(kFull, ks_batch, it & 31));
        }
        // Several warps take turns on a coarse slot, and a parity wait is only meaningful for the phase
        // right after the last completed one: were the tile of page gcc - kNC still on its way, a wait
        // for page gcc's tile would pass at once.  Waiting first for that earlier page's release (its
        // reader is done, so its tile did land) pins the phase.
        if (gcc >= kNC && !WS_WAIT(cempty(slot), ((gcc / kNC) - 1u) & 1u, 7, 1)) { ok = false; break; }
        if (!WS_WAIT(cfull(slot), (gcc / kNC) & 1u, 7, 1)) { ok = false; break; }
        if (gcc >= kND && !WS_WAIT(dempty(ds), ((gcc / kND) - 1u) & 1u, 8, 2)) { ok = false; break; }
        PROF_T(t_dots);
        PROF_INC(5);
        const uint8_t* tile = smem + L::kOffCoarse + slot * L::kCoarseSlot;
        float* hd = dhist + ds * (NT * 256);
        float cm[NT];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) cm[nt] = -INFINITY;
        // One 16-token tile per trip of a rolled loop: the four roles run different code on the same
        // SM, and with the page's four tiles unrolled the instruction cache missed on a third of its
        // requests.  The raw dots go to the published entry as they are produced.
#pragma unroll 1
        for (int mt = 0; mt < 4; ++mt) {
          float d[NT][2];
          coarse_dots(d, tile, mt);
          const int tok = page * kPage + 16 * mt + g;
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            hd[((mt * NT + nt) * 2 + 0) * 32 + lane] = d[nt][0];
            hd[((mt * NT + nt) * 2 + 1) * 32 + lane] = d[nt][1];
            const float s0 = tok < T ? to_log2(d[nt][0]) : -INFINITY;
            const float s1 = tok + 8 < T ? to_log2(d[nt][1]) : -INFINITY;
            cm[nt] = fmaxf(cm[nt], fmaxf(s0, s1));
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(cempty(slot));          // every lane has read its rows: the slot can be refilled
        PROF_ADD(3, t_dots);
        PROF_T(t_pub);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
          for (int off = 4; off < 32; off <<= 1) cm[nt] = fmaxf(cm[nt], __shfl_xor_sync(kFull, cm[nt], off));
        }
        float pl[NT];
        if (MV) {
          // mass of the page relative to its maximum, from the dots just stored (each lane reads its own)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) pl[nt] = 0.f;
#pragma unroll 1
          for (int mt = 0; mt < 4; ++mt) {
            const int tok = page * kPage + 16 * mt + g;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              if (cm[nt] != -INFINITY) {
                const float s0 = to_log2(hd[((mt * NT + nt) * 2 + 0) * 32 + lane]);
                const float s1 = to_log2(hd[((mt * NT + nt) * 2 + 1) * 32 + lane]);
                pl[nt] += (tok < T ? ex2_approx(s0 - cm[nt]) : 0.f) + (tok + 8 < T ? ex2_approx(s1 - cm[nt]) : 0.f);
              }
            }
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) pl[nt] += __shfl_xor_sync(kFull, pl[nt], off);
          }
        }
        if (g == 0) {
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            dmax[ds * 8 + 4 * nt + t] = cm[nt];
            if (MV) dpl[ds * 8 + 4 * nt + t] = pl[nt];
          }
          if (NT == 1) { dmax[ds * 8 + 4 + t] = -INFINITY; }
        }
        PROF_ADD(4, t_pub);
        __syncwarp();
        if (lane == 0) mbar_arrive(dfull(ds));
      }
    } else if (role == kRoleRefine) {
      // ================= refine warps ==============================================================
      float run_m[NT], run_l[NT], run_o[NT][8][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        run_m[nt] = -INFINITY;
        run_l[nt] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) run_o[nt][i][0] = run_o[nt][i][1] = 0.f;
      }
      if (active) {
        uint32_t qb[NT * (QP - 1)][4][2];
        uint32_t qh[NT][8][2];
        float qinv[NT];
        prep_q<NT, QP, false>(p, b, hkv, G, g, t, qb, qh, qinv);
        const int src = 8 * t + (g >> 1);
        const uint32_t sel = (g & 1) ? 0x7632u : 0x5410u;
        const int vsel = (lane >> 3) & 1;
        for (;;) {
          const int slot = myk % kNRV;
          // as for the coarse ring: the slot's previous page (another warp's) must have been released
          // before this wait can tell the phase it wants from the one before it
          if (myk >= kNRV && !WS_WAIT(rvempty(slot), ((myk / kNRV) - 1u) & 1u, 9, 0)) break;
          if (!WS_WAIT(rvfull(slot), (myk / kNRV) & 1u, 9, 0)) break;
          const int page = kq_page[slot];
          const int ds = kq_ds[slot];
          myk += kNR;
          if (page < 0) {                                  // end of the segment
            __syncwarp();
            if (lane == 0) mbar_arrive(rvempty(slot));
            break;
          }
          PROF_T(t_page);
          PROF_INC(2);
          const uint8_t* rtile = smem + L::kOffRv + slot * kRvSlot;
          const uint8_t* vt = rtile + kPage * kResRow;
          float* hs = dhist + ds * (NT * 256);
          const bool partial = (page + 1) * kPage > T;
          float rm[NT];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) rm[nt] = -INFINITY;
          // pass 1 (rolled, one 16-token tile per trip): refined scores = coarse dots + residual dots,
          // written back over the dots (each lane owns its entries), and the page maximum
#pragma unroll 1
          for (int mt = 0; mt < 4; ++mt) {
            float dr[NT][2];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) dr[nt][0] = dr[nt][1] = 0.f;
            if (use_res) dot_fp8<F8, NT, QP>(dr, qb, qinv, rtile, mt, g, t);
            const int tok = page * kPage + 16 * mt + g;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              float* e = hs + ((mt * NT + nt) * 2) * 32 + lane;
              const float s0 = tok < T ? to_log2(e[0] + dr[nt][0]) : -INFINITY;
              const float s1 = tok + 8 < T ? to_log2(e[32] + dr[nt][1]) : -INFINITY;
              e[0] = s0;
              e[32] = s1;
              rm[nt] = fmaxf(rm[nt], fmaxf(s0, s1));
            }
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) rm[nt] = fmaxf(rm[nt], __shfl_xor_sync(kFull, rm[nt], off));
          }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            // pass 2 (rolled): p = exp2(s - page max), fp32 sum, fp16 rounding for the P.V product
            // (...q2fp8.py:123-131); the eight 16-channel accumulators of P.V live across the trips
            float oacc[8][4];
#pragma unroll
            for (int i = 0; i < 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
            float l = 0.f;
#pragma unroll 1
            for (int mt = 0; mt < 4; ++mt) {
              const float* e = hs + ((mt * NT + nt) * 2) * 32 + lane;
              const float s0 = e[0], s1 = e[32];
              const float p0 = s0 == -INFINITY ? 0.f : ex2_approx(s0 - rm[nt]);
              const float p1 = s1 == -INFINITY ? 0.f : ex2_approx(s1 - rm[nt]);
              l += p0 + p1;
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
              const uint32_t x0 = __shfl_sync(kFull, w0, src), x1 = __shfl_sync(kFull, w0, src + 4);
              const uint32_t y0 = __shfl_sync(kFull, w1, src), y1 = __shfl_sync(kFull, w1, src + 4);
              const uint32_t pb0 = __byte_perm(x0, x1, sel), pb1 = __byte_perm(y0, y1, sel);
              const int vrow = 16 * mt + (lane & 7) + ((lane >> 4) & 1) * 8;
              uint32_t m01 = 0xffffffffu, m23 = 0xffffffffu;
              if (partial) {
                const int valid = T - (page * kPage + 16 * mt);       // valid tokens in this 16-token tile
                m01 = (2 * t < valid ? 0xffffu : 0u) | (2 * t + 1 < valid ? 0xffff0000u : 0u);
                m23 = (2 * t + 8 < valid ? 0xffffu : 0u) | (2 * t + 9 < valid ? 0xffff0000u : 0u);
              }
              const uint32_t vbase = smem_u32(vt + vrow * 128);
#pragma unroll
              for (int half = 0; half < 2; ++half) {
                uint32_t a[4][4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const int ch = 2 * (4 * half + j) + vsel;
                  ldmatrix_x4_trans(a[j], vbase + (ch >> 3) * (kPage * 128) + (((ch & 7) ^ (vrow & 7)) * 16));
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (partial) { a[j][0] &= m01; a[j][1] &= m01; a[j][2] &= m23; a[j][3] &= m23; }
                  if (VBF) mma_bf16(oacc[4 * half + j], a[j][0], a[j][1], a[j][2], a[j][3], pb0, pb1);
                  else mma_f16(oacc[4 * half + j], a[j][0], a[j][1], a[j][2], a[j][3], pb0, pb1);
                }
              }
            }
            // stage-2 recurrence over the warp's pages in page order (...q2fp8.py:162-167)
            const float nm = fmaxf(run_m[nt], rm[nt]);
            const float rp = nm == -INFINITY ? 0.f : ex2_approx(run_m[nt] - nm);
            const float rb = nm == -INFINITY ? 0.f : ex2_approx(rm[nt] - nm);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              run_o[nt][i][0] = run_o[nt][i][0] * rp + (oacc[i][0] + oacc[i][1]) * rb;
              run_o[nt][i][1] = run_o[nt][i][1] * rp + (oacc[i][2] + oacc[i][3]) * rb;
            }
            run_l[nt] = run_l[nt] * rp + l * rb;
            run_m[nt] = nm;
          }
          __syncwarp();
          if (lane == 0) {                                 // residual, V and the dots of this page are consumed
            mbar_arrive(rvempty(slot));
            mbar_arrive(dempty(ds));
          }
          PROF_ADD(1, t_page);
        }
      }
      // this warp's share of the segment: waits for the other roles to leave the coarse ring alone.
      // A refine warp holds its end marker only after the dispatcher has consumed every published page,
      // which is after the scoring warps read their last tile: the ring is idle and can hold `red`.
      // (An aborted or empty segment has nothing in flight either.)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float l = run_l[nt];
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) l += __shfl_xor_sync(kFull, l, off);
        const int h = 4 * nt + t;
        if (g == 0) { lred[rw * 8 + h] = l; mred[rw * 8 + h] = run_m[nt]; }
        float* w = red + rw * 1024 + h * 128;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          w[16 * i + g] = run_o[nt][i][0];
          w[16 * i + g + 8] = run_o[nt][i][1];
        }
      }
    }

#ifdef FFA_WS_PROFILE
    prof_role += static_cast<uint32_t>(clock()) - prof_seg0;
    const uint32_t prof_a = static_cast<uint32_t>(clock());
#endif
    bar_sync(0, kWsThreads);               // A: every role is done with the segment's pipeline

    if (role == kRoleRefine && rw < 4) {
      // ---- segment epilogue (128 threads): add the refine warps' shares, write one partial ----------
      const int ftid = rw * 32 + lane;
      const bool bad = *reinterpret_cast<volatile int*>(sAbort) != 0;
      const float qnan = __int_as_float(0x7fc00000);
      for (int h = 0; h < G; ++h) {
        float top = -INFINITY;
#pragma unroll
        for (int r = 0; r < kNR; ++r) top = fmaxf(top, mred[r * 8 + h]);
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < kNR; ++r) {
          const float mr = mred[r * 8 + h];
          if (mr != -INFINITY) o += red[r * 1024 + h * 128 + ftid] * exp2f(mr - top);
        }
        p.part_o[((row0 + h) * p.nch + part) * kHeadDim + ftid] = bad ? qnan : o;
      }
      if (ftid < G) {
        float top = -INFINITY, l = 0.f;
#pragma unroll
        for (int r = 0; r < kNR; ++r) top = fmaxf(top, mred[r * 8 + ftid]);
#pragma unroll
        for (int r = 0; r < kNR; ++r) {
          const float mr = mred[r * 8 + ftid];
          if (mr != -INFINITY) l += lred[r * 8 + ftid] * exp2f(mr - top);
        }
        p.part_m[(row0 + ftid) * p.nch + part] = bad ? 0.f : top;
        p.part_l[(row0 + ftid) * p.nch + part] = bad ? qnan : l;
        if (MV) {
          p.part_pm[(row0 + ftid) * p.nch + part] = (bad || n == 0) ? -INFINITY : sApx[ftid];
          p.part_pl[(row0 + ftid) * p.nch + part] = bad ? qnan : (n == 0 ? 0.f : sApx[8 + ftid]);
        }
      }
      if (p.mask && page_begin + n_pad == NPp) {
        // mask entries past the last group that holds tokens (padding blocks count as pruned)
        for (int i = (p.NP + m_grp - 1) / m_grp + ftid; i < p.NTBS; i += 128)
          p.mask[(static_cast<int64_t>(b) * p.HKV + hkv) * p.NTBS + i] = 0;
      }

      // ---- merge by the last segment of this (b, kv-head) to finish (stage 2, ...q2fp8.py:142-171) ---
      const int n_seg = static_cast<int>((unit0 + NPp - 1) / p.ppc - unit0 / p.ppc) + 1;
      __threadfence();
      bar_sync(2, 128);
      if (ftid == 0) {
        const int prev = atomicAdd(p.arrivals + unit, 1);
        *sFlag = (prev == n_seg - 1);
        if (prev == n_seg - 1) p.arrivals[unit] = 0;
      }
      bar_sync(2, 128);
      if (*sFlag) {
        __threadfence();
        float* sm_m = red;                  // [8][64]
        float* sm_l = red + 8 * 64;         // [8][64], then mean-V: pm [8][64], pl [8][64]
        const int per_head = n_seg;         // <= 64 by construction of the page ranges
        for (int idx = ftid; idx < G * per_head; idx += 128) {
          const int h = idx / per_head, i = idx % per_head;
          sm_m[h * 64 + i] = __ldcg(p.part_m + (row0 + h) * p.nch + i);
          sm_l[h * 64 + i] = __ldcg(p.part_l + (row0 + h) * p.nch + i);
          if (MV) {
            sm_l[8 * 64 + h * 64 + i] = __ldcg(p.part_pm + (row0 + h) * p.nch + i);
            sm_l[16 * 64 + h * 64 + i] = __ldcg(p.part_pl + (row0 + h) * p.nch + i);
          }
        }
        bar_sync(2, 128);
        for (int h = rw; h < G; h += 4) {
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
              if (i < per_head && sm_l[h * 64 + i] != 0.f) acc += sm_l[h * 64 + i] * w[j];
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
              const int vd = p.v_bf16 ? FFA_BF16 : FFA_F16;
              o.x = o.x * rb + load_as_float(p.v_mean, ve, vd) * wv;
              o.y = o.y * rb + load_as_float(p.v_mean, ve + 1, vd) * wv;
              o.z = o.z * rb + load_as_float(p.v_mean, ve + 2, vd) * wv;
              o.w = o.w * rb + load_as_float(p.v_mean, ve + 3, vd) * wv;
              acc = acc * rb + wv;
            }
          }
          // a NaN mass marks a segment whose waits gave up: the head's output is NaN, not a guess
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

    bar_sync(0, kWsThreads);               // B: the coarse ring may be refilled
#ifdef FFA_WS_PROFILE
    prof_epi += static_cast<uint32_t>(clock()) - prof_a;
#endif
    if (active) { gc += static_cast<uint32_t>(n); ++act_ord; }
  }
#ifdef FFA_WS_PROFILE
  // 64-bit sums over all CTAs, kept in the middle of the arrival-counter block (byte 32768 of the
  // workspace; profiling builds serve at most 8192 (batch x kv-head) units): [role * 8 + i] = pacc[i] of the role's
  // warps (i < 6), [role * 8 + 6] = the role's pipeline cycles, [role * 8 + 7] = cycles between the two
  // segment barriers; [32] = kernel cycles of a CTA, [33] = its nanoseconds, [34] = the longest CTA's ns.
  //   coarse producer: 0 wait for a free coarse slot
  //   dispatcher:      0 thresholds, 1 published page, 2 free residual+V slot, 3 kept-page branch
  //   scoring:         0 sample tile, 1 coarse tile, 2 free entry, 3 dots, 4 publish, 5 pages
  //   refine:          0 residual+V landed, 1 page work, 2 pages
  if (p.arrivals) {
    unsigned long long* gp = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(p.arrivals) + 32768);
    if (lane == 0) {
      for (int i = 0; i < 6; ++i) atomicAdd(gp + role * 8 + i, static_cast<unsigned long long>(pacc[i]));
      atomicAdd(gp + role * 8 + 6, static_cast<unsigned long long>(prof_role));
      atomicAdd(gp + role * 8 + 7, static_cast<unsigned long long>(prof_epi));
    }
    if (tid == 0) {
      unsigned long long g1;
      asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(g1));
      atomicAdd(gp + 32, static_cast<unsigned long long>(clock64() - prof_c0));
      atomicAdd(gp + 33, g1 - prof_g0);
      atomicMax(gp + 34, g1 - prof_g0);
    }
  }
#endif
  if (tid == 0 && *sAbort != 0 && p.status && atomicCAS(p.status, 0, 1) == 0) {
    p.status[1] = *sAbort;                 // which wait gave up first in this CTA
    p.status[5] = static_cast<int>(blockIdx.x);
  }
}

// Launches the kernel, or (stream == kWsQueryOnly) only configures it.
template <int FMT, int F8, int NT, bool VBF, int QP, bool MV = false>
int launch_ws_one(const DecodeParams& p, const CUtensorMap* maps, cudaStream_t stream) {
  using L = WsSmem<FMT, NT>;
  auto kern = decode_ws_kernel<FMT, F8, NT, VBF, QP, MV>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const bool slot = dev >= 0 && dev < 64;
  if (!slot || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
    if (e != cudaSuccess) return note_cuda_error(e, "cudaFuncSetAttribute(decode_ws)");
    if (slot) configured[dev] = true;
  }
  const int64_t total_pages = static_cast<int64_t>(p.B) * p.HKV * p.NPp;
  const unsigned grid = static_cast<unsigned>((total_pages + p.ppc - 1) / p.ppc);
  kern<<<grid, kWsThreads, L::kBytes, stream>>>(p, maps[0], maps[1], maps[2], maps[3]);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FFA_OK : note_cuda_error(e, "decode_ws launch");
}

// q bf16: two e4m3 pieces; q fp16 or fp32 (rounded to fp16 like the reference): three.  Either V type.
template <int FMT, int F8, int NT>
int launch_ws_types(const DecodeParams& p, const CUtensorMap* maps, cudaStream_t stream) {
  if constexpr (FMT == FFA_K_Q2) {
    if (p.v_mean) {                                  // mean-V variant: 2-bit format only, like the reference
      if (p.q_dtype != FFA_BF16)
        return p.v_bf16 ? launch_ws_one<FMT, F8, NT, true, 3, true>(p, maps, stream)
                        : launch_ws_one<FMT, F8, NT, false, 3, true>(p, maps, stream);
      return p.v_bf16 ? launch_ws_one<FMT, F8, NT, true, 2, true>(p, maps, stream)
                      : launch_ws_one<FMT, F8, NT, false, 2, true>(p, maps, stream);
    }
  }
  if (p.q_dtype != FFA_BF16)
    return p.v_bf16 ? launch_ws_one<FMT, F8, NT, true, 3>(p, maps, stream)
                    : launch_ws_one<FMT, F8, NT, false, 3>(p, maps, stream);
  return p.v_bf16 ? launch_ws_one<FMT, F8, NT, true, 2>(p, maps, stream)
                  : launch_ws_one<FMT, F8, NT, false, 2>(p, maps, stream);
}

template <int FMT>
int launch_ws_fmt_impl(const DecodeParams& p, int f8, const CUtensorMap* maps, cudaStream_t stream) {
  if (p.G <= 4)
    return f8 == FFA_E4M3 ? launch_ws_types<FMT, FFA_E4M3, 1>(p, maps, stream)
                          : launch_ws_types<FMT, FFA_E5M2, 1>(p, maps, stream);
  return f8 == FFA_E4M3 ? launch_ws_types<FMT, FFA_E4M3, 2>(p, maps, stream)
                        : launch_ws_types<FMT, FFA_E5M2, 2>(p, maps, stream);
}

}  // namespace

}  // namespace ffa
