// FFA decode attention for B200: warp-specialised kernel, one persistent CTA per SM.
//
// Same math and reference semantics as the fp16 kernel in ffa_decode.cu (coarse score -> prune ->
// residual refine -> online softmax * V -> merge; reference ffa-q2fp8/attn_kernel/
// attn_kernel_v1210_fused_bsz_q2fp8.py:30-171), organised so that a pruned page costs only its
// coarse bytes and its share of the scoring arithmetic:
//
//   warp 0        coarse producer: claims chunks of work (a run of pages of one (batch, kv-head)) from
//                 a global counter, publishes them to the other warps and streams the coarse K tile of
//                 every page into a ring of shared-memory slots with TMA, as far ahead as the ring
//                 allows - across chunk boundaries, so the pipeline never drains between chunks.
//   warps 2..5    scoring: each takes whole pages (64 tokens = four m16 tiles) round robin, computes
//                 the coarse q.k of every token against all heads of the group on the tensor cores
//                 and publishes the page's per-head maximum plus the raw dots.  No CTA barrier, no
//                 exchange between warps: a page's statistic is complete inside one warp.
//   warp 1        dispatcher: walks the published pages in order, eight per trip, applies the prune
//                 rule (a group of SBS/64 pages is dropped only if every head's maximum over the group
//                 is strictly below that head's threshold), writes the kept mask and, for kept pages,
//                 requests residual + V with TMA into the next free slot of a second ring.
//   warps 6..9    refine, in pairs: kept page number k goes to pair k mod 2, each warp of the pair
//                 taking 32 of its 64 tokens (a page leaves its shared-memory slot twice as fast as
//                 with one warp, which leaves more of the ring for loads in flight).  A warp adds the
//                 residual dot to the coarse dots, the pair agrees on the page maximum through shared
//                 memory, and each warp does the softmax and P.V of its tokens.  At the end of a
//                 chunk the four warps add their (m, l, o[128]) per q head in shared memory and write
//                 one partial for the chunk; whichever CTA arrives last for a (batch, kv-head) merges
//                 all its partials (stage 2, ...q2fp8.py:142-171), the heads split over the four warps.
//
// Chunks are handed out dynamically, so an SM whose pages are mostly pruned simply takes more of
// them; the kept fraction differs a lot between (batch, kv-head)s, and equal page ranges per SM left
// the slowest SM 40 % behind the average.
//
// Numerics are those of the page-pipeline kernel (ffa_decode_tma.cu): q split into exact e4m3 pieces against raw
// fp8 K bytes (fp8 coarse and the residual), fp16 q against dequantised codes (2-/4-bit coarse),
// P rounded to fp16 and split into exact bf16 pieces for bf16 V.  The refined score is
// q.k_coarse + q.k_residual (the reference rounds k_coarse + k_residual to fp16 first).
//
// Every wait is bounded in wall-clock time.  A wait that gives up raises a CTA-wide flag; every role
// then leaves its loops, the refine warps publish NaN partials for the chunk they were on (so the
// merged output of the affected heads is NaN, not a plausible number) and the status word is set.
#pragma once

#include "ffa_decode_prims.cuh"

namespace ffa {

namespace {

constexpr int kNS = 4;                     // scoring warps
constexpr int kNR = kWsRefineWarps;        // refine warps, working in pairs: a kept page is refined by two warps, 32 tokens each
constexpr int kNP = kNR / 2;               // (a page is out of its shared-memory slot twice as fast as with one warp,
                                           // which leaves more of the ring for loads in flight)
constexpr int kWsWarps = 2 + kNS + kNR;
constexpr int kWsThreads = 32 * kWsWarps;
constexpr int kBatch = kMaxPruneGroup;     // pages the dispatcher decides per trip; a whole prune group must fit (SBS <= 512)
constexpr int kSampleRows = kSample;       // rows of a threshold sample tile
constexpr int kNSeg = 4;                   // published chunks the consumers may lag behind the producer

// SUBP: the kernel prunes blocks smaller than a page (SBS 32 or 16) and keeps per-tile maxima for that
template <int FMT, int NT, bool SUBP = false>
struct WsSmem {
  static constexpr int kRow = Fmt<FMT>::kRow;
  static constexpr int kCoarseSlot = kPage * kRow;                                  // 8 / 2 / 4 KiB
  // coarse ring: each scoring warp should find its next tile already landed, i.e. more than one slot
  // per warp in flight; the residual + V ring takes what is left of the 227 KiB
  // (sub-page pruning: the formats with per-channel scales give up one slot for the per-tile maxima)
  static constexpr int kNC = FMT == FFA_K_FP8 ? 6
                             : (FMT == FFA_K_Q2 ? (SUBP && NT == 1 ? 15 : 16) : ((SUBP && FMT == FFA_K_NF4 && NT == 1) ? 7 : 8));
  static constexpr int kNRV = NT == 2 ? 5 : 6;                                      // residual + V slots (24 KiB each)
  // published-page ring (the page's raw dots and maxima).  At least two dispatcher trips; the 2-/4-bit
  // formats, whose scoring is the expensive stage, get four: while the dispatcher waits for a free
  // residual + V slot the scoring warps keep scoring ahead, and the pruned pages behind the wait are
  // then decided in a burst, so scoring time and refine time overlap instead of adding up (-3 to -5 %
  // at kept fractions below 0.5)
  static constexpr int kND = (FMT != FFA_K_FP8 && NT == 1) ? 4 * kBatch : 2 * kBatch;
  static constexpr int kHist = NT * 1024;                                           // raw dots of one page
  static constexpr bool kHasChannelScale = (FMT == FFA_K_Q2 || FMT == FFA_K_NF4);
  static constexpr int kOffRv = 0;
  static constexpr int kOffCoarse = kOffRv + kNRV * kRvSlot;
  static constexpr int kOffDHist = kOffCoarse + kNC * kCoarseSlot;
  static constexpr int kOffDMax = kOffDHist + kND * kHist;      // [kND][8] page maxima
  static constexpr int kOffDPl = kOffDMax + kND * 32;           // [kND][8] mean-V: mass relative to the maximum
  // [kND][4 tiles][8]: maxima per 16-token tile (SBS below 64).  Shares its first quarter with the
  // mean-V masses: the mean-V variant prunes whole pages only, the two are never used together.
  static constexpr int kOffDSub = kOffDPl;
  static constexpr int kOffBars = kOffDSub + kND * (SUBP ? 128 : 32);
  // barriers: chunk full/empty | coarse full/empty | threshold full/empty |
  //           page full/empty | residual+V full/empty
  //           | three chunk-end meeting points of the refine warps | one meeting point per refine pair
  static constexpr int kNBars = 2 * kNSeg + 2 * kNC + 4 + 2 * kND + 2 * kNRV + 3 + kNP;
  static constexpr int kOffMisc = kOffBars + ((kNBars * 8 + 63) / 64) * 64;
  // misc: sTh[2][16] | seg[kNSeg][4] | kq_page[8] | kq_ds[8] | kq_sub[8] | abort, last, pad[6] | book[16] | per scoring warp sS[128], sZ[128]
  static constexpr int kOffTh = kOffMisc;
  static constexpr int kOffSeg = kOffTh + 128;
  static constexpr int kOffKq = kOffSeg + kNSeg * 16;
  static constexpr int kOffFlags = kOffKq + 96;
  static constexpr int kOffBook = kOffFlags + 32;
  static constexpr int kOffS = kOffBook + 64;
  // chunk end: every refine warp's (o[heads][128], m, l), added up before one partial is written
  static constexpr int kRedWarp = NT * 4 * 128 * 4;
  static constexpr int kOffRed = kOffS + (kHasChannelScale ? kNS * 1024 : 0);
  static constexpr int kOffRedML = kOffRed + kNR * kRedWarp;                          // [kNR][2][8] f32
  static constexpr int kOffPairMax = kOffRedML + kNR * 64;                            // [kNP][2 pages][2 warps][8] f32
  static constexpr int kBytes = kOffPairMax + kNP * 128 + 1024;                       // + alignment slack
#ifndef FFA_SKIP_SMEM_ASSERT
  static_assert(kBytes <= 232448, "shared memory of one CTA");
#endif
  static_assert(kNRV >= 4, "the dispatcher issues up to four requests per round");
  // a ring shared by several consumer warps stays phase-safe only if it has at least as many slots
  static_assert(kNC >= kNS && kNRV >= kNP, "rings must not be smaller than the number of their consumers");
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
__device__ __forceinline__ void mbar_arrive_n(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
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
__device__ __forceinline__ bool ws_wait(uint32_t bar, uint32_t parity, int* abort_flag, int site) {
  return __all_sync(0xffffffffu, ws_wait_lane(bar, parity, abort_flag, site)) != 0;
}
#ifdef FFA_WS_PROFILE
__device__ __forceinline__ bool ws_wait_timed(uint32_t bar, uint32_t parity, int* abort_flag, int site, uint32_t& acc) {
  const uint32_t t0 = static_cast<uint32_t>(clock());
  const bool r = ws_wait(bar, parity, abort_flag, site);
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

// Stage 2 for the q heads h0, h0 + hstep, ... of one (batch, kv-head), by one warp: merges the n_seg
// partials each of them has received, one per chunk (reference ...q2fp8.py:142-171; the mean-V fold
// ...meanv_bsz_q2fp8.py:188-200) and writes the output rows.  Run by the warps of the CTA whose chunk
// completed the (batch, kv-head).
template <bool MV>
__device__ __forceinline__ void ws_merge_unit(const DecodeParams& p, int b, int hkv, int n_seg, int h0, int hstep, int lane) {
  constexpr uint32_t kFull = 0xffffffffu;
  const int G = p.G;
  const int64_t row0 = static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G;
  for (int h = h0; h < G; h += hstep) {
    const int64_t row = row0 + h;
    // lane i holds (m, l) of partial i (n_seg <= kWsMaxParts = 32)
    const float pm = lane < n_seg ? __ldcg(p.part_m + row * p.nch + lane) : -INFINITY;
    const float pl = lane < n_seg ? __ldcg(p.part_l + row * p.nch + lane) : 0.f;
    float top = pl != 0.f ? pm : -INFINITY;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(kFull, top, off));
    const bool live_l = pl != 0.f && pm != -INFINITY;
    const float wl = live_l ? exp2f(pm - top) : 0.f;
    float acc = pl != 0.f ? pl * wl : 0.f;                   // a NaN mass (a chunk whose waits gave up) stays NaN
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(kFull, acc, off);
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int i0 = 0; i0 < n_seg; i0 += 8) {
      float4 v[8];
      float w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = i0 + j;
        w[j] = __shfl_sync(kFull, wl, i & 31);
        const bool live = i < n_seg && w[j] != 0.f;
        if (!live) w[j] = 0.f;
        v[j] = live ? __ldcg(reinterpret_cast<const float4*>(p.part_o + (row * p.nch + i) * kHeadDim) + lane)
                    : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) { o.x += v[j].x * w[j]; o.y += v[j].y * w[j]; o.z += v[j].z * w[j]; o.w += v[j].w * w[j]; }
    }
    if (MV) {
      // fold the pruned pages in: mass x mean of V; one (maximum, mass) pair per chunk
      const float qm = lane < n_seg ? __ldcg(p.part_pm + row * p.nch + lane) : -INFINITY;
      const float ql = lane < n_seg ? __ldcg(p.part_pl + row * p.nch + lane) : 0.f;
      float p_top = ql != 0.f ? qm : -INFINITY;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) p_top = fmaxf(p_top, __shfl_xor_sync(kFull, p_top, off));
      float p_acc = ql != 0.f ? ql * exp2f(qm - p_top) : 0.f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) p_acc += __shfl_xor_sync(kFull, p_acc, off);
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
      const float lse = acc == 0.f ? -INFINITY : top + log2f(acc);
      float* po = p.partial_out + row * (kHeadDim + 1);
      po[4 * lane] = r0; po[4 * lane + 1] = r1; po[4 * lane + 2] = r2; po[4 * lane + 3] = r3;
      if (lane == 0) po[kHeadDim] = lse;
      if (p.peer_world > 0) {
        // sequence split: the finished row goes to this rank's slot on every peer as soon as it exists, so
        // the exchange overlaps the rest of the kernel; the fence orders the stores before the flag that
        // the last CTA raises when the whole kernel is done
        for (int pr = 0; pr < p.peer_world; ++pr) {
          if (pr == p.peer_rank) continue;
          float* pp = p.peer_slot[pr] + row * (kHeadDim + 1);
          pp[4 * lane] = r0; pp[4 * lane + 1] = r1; pp[4 * lane + 2] = r2; pp[4 * lane + 3] = r3;
          if (lane == 0) pp[kHeadDim] = lse;
        }
        __threadfence_system();
      }
    }
  }
}

// One arrival for a (batch, kv-head): the caller has published its partial.  Returns true in every
// lane of the warp that completes the count (and has reset the counter for the next launch).
__device__ __forceinline__ bool ws_arrive_unit(const DecodeParams& p, int unit, int target, int lane) {
  __threadfence();
  __syncwarp();
  int last = 0;
  if (lane == 0) {
    const int prev = atomicAdd(p.arrivals + unit, 1);
    last = prev == target - 1;
    if (last) p.arrivals[unit] = 0;
  }
  last = __shfl_sync(0xffffffffu, last, 0);
  if (last) __threadfence();
  return last != 0;
}

// Prune blocks smaller than a page (SBS 32 or 16; the whole warp calls this, four lanes per page, lane
// hq of a page holding heads 2hq and 2hq + 1): the rule "dropped only if every head's maximum is
// strictly below its threshold" is applied to every sub-block's own maxima (`sub_max` = the page's
// [4 tiles][8 heads]).  Returns the page's kept sub-blocks as a bit mask, the same in the page's four
// lanes, and writes the mask entries.  The page is fetched if any sub-block is kept; the refine warps
// skip the tiles of the others.  Kept out of line: it is rare, and the dispatcher's loop is latency
// critical and shares the instruction cache with three other roles.
__device__ __noinline__ uint32_t ws_decide_sub_blocks(const float* sub_max, int n_sub, int tps_shift, int hq, int G,
                                                      float th0, float th1, bool valid, uint32_t gmask, int8_t* mask_out) {
  uint32_t kept = 0u;
  for (int sb = 0; sb < n_sub; ++sb) {
    float a0 = -INFINITY, a1 = -INFINITY;
    for (int tt = 0; tt < (1 << tps_shift); ++tt) {
      const float* e = sub_max + ((sb << tps_shift) + tt) * 8;
      if (valid) { a0 = fmaxf(a0, e[2 * hq]); a1 = fmaxf(a1, e[2 * hq + 1]); }
    }
    const bool r = valid && ((2 * hq < G && !(a0 < th0)) || (2 * hq + 1 < G && !(a1 < th1)));
    const bool ks = (__ballot_sync(0xffffffffu, r) & gmask) != 0u;
    if (ks) kept |= 1u << sb;
    if (mask_out && valid && hq == 0) mask_out[sb] = ks ? 1 : 0;
  }
  return kept;
}

// FMT: coarse format; F8: fp8 encoding of the residual (and of the fp8 coarse base); NT: n-tiles of
// four q heads (1: group <= 4, 2: group <= 8); VBF: V is bf16 (else fp16); QP: e4m3 pieces per q value;
// MV: mean-V variant (pruned pages keep their coarse softmax mass; DecodeParams::v_mean).
template <int FMT, int F8, int NT, bool VBF, int QP, bool MV, bool SUBP>
__global__ void __launch_bounds__(kWsThreads, 1) decode_ws_kernel(const __grid_constant__ DecodeParams p,
                                                                  const __grid_constant__ CUtensorMap tm_c,
                                                                  const __grid_constant__ CUtensorMap tm_r,
                                                                  const __grid_constant__ CUtensorMap tm_v) {
  using L = WsSmem<FMT, NT, SUBP>;
  constexpr int ROW = L::kRow;
  constexpr int kNC = L::kNC;
  constexpr int kNRV = L::kNRV;
  constexpr int kND = L::kND;
  constexpr bool kFp8Coarse = (FMT == FFA_K_FP8);
  constexpr uint32_t kFull = 0xffffffffu;
  extern __shared__ uint8_t smem_raw[];
  // 128B-swizzled TMA tiles need 1024-byte alignment
  uint8_t* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int G = p.G, T = p.T;
  const int m_grp = p.group;                       // pages per prune group (SBS / 64)
  const int CH = p.ppc;                            // pages per chunk (whole prune groups)
  const int n_seg = p.nseg;                        // chunks per (batch, kv-head)
  const int total_chunks = p.B * p.HKV * n_seg;
  const int arrive_target = n_seg * (MV ? 2 : 1);           // arrivals that complete a (batch, kv-head): one per chunk
                                                            // (mean-V: one more per chunk, by the dispatcher)

  const uint32_t bars = smem_u32(smem + L::kOffBars);
  auto segfull = [&](int i) { return bars + 8u * i; };
  auto segempty = [&](int i) { return bars + 8u * (kNSeg + i); };
  constexpr int kB0 = 2 * kNSeg;
  auto cfull = [&](int i) { return bars + 8u * (kB0 + i); };
  auto cempty = [&](int i) { return bars + 8u * (kB0 + kNC + i); };
  constexpr int kB1 = kB0 + 2 * kNC;
  auto thfull = [&](int i) { return bars + 8u * (kB1 + i); };          // 2 chunks
  auto thempty = [&](int i) { return bars + 8u * (kB1 + 2 + i); };
  constexpr int kB2 = kB1 + 4;
  auto dfull = [&](int i) { return bars + 8u * (kB2 + i); };
  auto dempty = [&](int i) { return bars + 8u * (kB2 + kND + i); };
  constexpr int kB3 = kB2 + 2 * kND;
  auto rvfull = [&](int i) { return bars + 8u * (kB3 + i); };
  auto rvempty = [&](int i) { return bars + 8u * (kB3 + kNRV + i); };
  constexpr int kB4 = kB3 + 2 * kNRV;
  auto rfmeet = [&](int i) { return bars + 8u * (kB4 + i); };
  auto pairmeet = [&](int i) { return bars + 8u * (kB4 + 3 + i); };
  static_assert(kB4 + 3 + kNP == L::kNBars, "barrier table");

  float* dhist = reinterpret_cast<float*>(smem + L::kOffDHist);
  float* dmax = reinterpret_cast<float*>(smem + L::kOffDMax);
  float* dpl = reinterpret_cast<float*>(smem + L::kOffDPl);
  float* sTh = reinterpret_cast<float*>(smem + L::kOffTh);          // [2 chunks][2 samples][8 heads]
  int* sSeg = reinterpret_cast<int*>(smem + L::kOffSeg);            // [kNSeg][4]: unit, first page, pages, chunk of the unit
  int* kq_page = reinterpret_cast<int*>(smem + L::kOffKq);      // per residual+V slot: page of the (b, kv-head), -1 = end marker
  int* kq_ds = kq_page + 8;                                      // ... and the published-page entry that holds its dots
  int* kq_sub = kq_page + 16;                                    // ... and which of its sub-blocks are kept (SBS below 64)
  float* dsub = reinterpret_cast<float*>(smem + L::kOffDSub);
  // SBS below one page: `n_sub` prune blocks of 64 / n_sub tokens per page (2 or 4), else 1
  const int n_sub = SUBP && p.sub > 1 ? p.sub : 1;
  const int tps_shift = n_sub == 4 ? 0 : (n_sub == 2 ? 1 : 2);   // log2 of the 16-token tiles per prune block
  int* sAbort = reinterpret_cast<int*>(smem + L::kOffFlags);
  float* sBook = reinterpret_cast<float*>(smem + L::kOffBook);
  int* sLast = sAbort + 1;                                       // the chunk just finished completed its (batch, kv-head)
  float* red = reinterpret_cast<float*>(smem + L::kOffRed);      // [kNR][4 NT heads][128]
  float* redml = reinterpret_cast<float*>(smem + L::kOffRedML);  // [kNR][m: 8, l: 8]
  float* pairmax = reinterpret_cast<float*>(smem + L::kOffPairMax);

  const bool use_res = p.use_res != 0;
  const bool sampled = p.th_in == nullptr;
  const uint32_t rv_bytes = (use_res ? kPage * kResRow : 0) + kPage * kVRow;

#ifdef FFA_WS_PROFILE
  uint32_t pacc[6] = {0u, 0u, 0u, 0u, 0u, 0u};     // per-role meaning, see the end of the kernel
  const long long prof_c0 = clock64();
  unsigned long long prof_g0;
  asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(prof_g0));
#endif
  if (tid == 0) {
    for (int i = 0; i < L::kNBars; ++i) mbar_init(bars + 8 * i, 1);
    for (int i = 0; i < kNSeg; ++i) mbar_init(segempty(i), 1 + kNS + kNR);      // every consumer warp has read the chunk
    for (int i = 0; i < 2; ++i) mbar_init(thfull(i), 2);                        // the two scoring warps that score the samples
    for (int i = 0; i < 3; ++i) mbar_init(rfmeet(i), kNR);                      // every refine warp
    for (int i = 0; i < kNP; ++i) mbar_init(pairmeet(i), 2);                    // the two warps of a refine pair
    for (int i = 0; i < kND; ++i) mbar_init(dempty(i), 2);                      // both warps of the pair (or the dispatcher, twice)
    for (int i = 0; i < kNRV; ++i) mbar_init(rvempty(i), 2);
    *sAbort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
  }
  if (FMT == FFA_K_NF4 && tid < 16) sBook[tid] = c_nf4_book[tid];
  __syncthreads();

  enum { kRoleCoarse = 0, kRoleDispatch = 1, kRoleScore = 2, kRoleRefine = 3 };
  const int role = warp == 0 ? kRoleCoarse : (warp == 1 ? kRoleDispatch : (warp < 2 + kNS ? kRoleScore : kRoleRefine));
  const int sw = warp - 2;                         // scoring warp index
  const int rw = warp - 2 - kNS;                   // refine warp index

  // Every consumer warp walks the published chunks in order.  `gc` counts the pages of earlier chunks:
  // ring positions and mbarrier phases follow from it and are the same in every role.
  uint32_t gc = 0;
  int seg_unit = -1, seg_page0 = 0, seg_n = 0, seg_part = 0;
  auto next_chunk = [&](uint32_t seg_i) -> bool {          // false: no more work (or a wait gave up)
    const int slot = seg_i % kNSeg;
    if (!WS_WAIT(segfull(slot), (seg_i / kNSeg) & 1u, 10, 5)) return false;
    seg_unit = sSeg[slot * 4 + 0]; seg_page0 = sSeg[slot * 4 + 1]; seg_n = sSeg[slot * 4 + 2]; seg_part = sSeg[slot * 4 + 3];
    __syncwarp();
    if (lane == 0) mbar_arrive(segempty(slot));
    return seg_unit >= 0;
  };
  auto to_log2 = [&](float d) -> float { return (d * p.sm_scale) * kLog2e; };

  if (role == kRoleCoarse) {
    // ================= coarse producer ===============================================================
    // The first chunk of a CTA is its own number; further ones come from a global counter.  Lane 0 asks
    // for the next chunk a few pages before the current one has been streamed - early enough that the
    // round trip of the atomic and the first loads of the new chunk hide behind the pages the other
    // warps still hold, late enough that no CTA sits on a chunk it will not start for a long time
    // (asking a whole chunk ahead let the CTAs that started first take two chunks each and left
    // others with none).
    constexpr int kClaimLead = 8;
    int next_raw = 0;
    for (uint32_t seg_i = 0;; ++seg_i) {
      const int chunk = seg_i == 0 ? static_cast<int>(blockIdx.x)
                                   : __shfl_sync(kFull, next_raw, 0) + static_cast<int>(gridDim.x);
      const bool end = chunk >= total_chunks || *reinterpret_cast<volatile int*>(sAbort) != 0;
      const int slot = seg_i % kNSeg;
      if (seg_i >= kNSeg && !WS_WAIT(segempty(slot), ((seg_i / kNSeg) - 1u) & 1u, 11, 1)) break;
      // chunk numbering: kv-head fastest, then the chunk of the sequence, then the batch.  Chunks that
      // are claimed one after the other - and so are in flight together - then cover the same token
      // rows of the same sequence for all kv-heads: a token row holds the heads side by side, and DRAM
      // serves the pieces of one row together far better than pieces of unrelated rows
      const int c_hkv = chunk % p.HKV, c_rest = chunk / p.HKV;
      const int part = end ? 0 : c_rest % n_seg;
      const int unit = end ? -1 : (c_rest / n_seg) * p.HKV + c_hkv;
      const int page_begin = part * CH;
      const int n = end ? 0 : min(CH, p.NP - page_begin);             // real pages (>= 1: a chunk never holds padding only)
      if (lane == 0) {
        sSeg[slot * 4 + 0] = unit; sSeg[slot * 4 + 1] = page_begin; sSeg[slot * 4 + 2] = n; sSeg[slot * 4 + 3] = part;
        mbar_arrive(segfull(slot));
      }
      if (end) break;
      const int b = unit / p.HKV, hkv = unit % p.HKV;
      int btv = 0;
      bool ok = true;
      const int claim_at = n > kClaimLead ? n - kClaimLead : 0;
      for (int c = 0; c < n; ++c) {
        const uint32_t gcc = gc + c;
        const int cslot = gcc % kNC;
        if (c == claim_at && lane == 0) next_raw = atomicAdd(p.work, 1);
        if ((c & 31) == 0 && p.bt && c + lane < n)
          btv = p.bt[static_cast<int64_t>(b) * p.bt_stride + page_begin + c + lane];
        const int bv = __shfl_sync(kFull, btv, c & 31);
        const int row = p.bt ? bv * kPage : b * T + (page_begin + c) * kPage;
        if (gcc >= kNC && !WS_WAIT(cempty(cslot), ((gcc / kNC) - 1u) & 1u, 1, 0)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(cfull(cslot), L::kCoarseSlot);
          tma_load_2d(smem_u32(smem + L::kOffCoarse + cslot * L::kCoarseSlot), &tm_c, hkv * ROW, row, cfull(cslot));
        }
      }
      if (!ok) break;
      gc += static_cast<uint32_t>(n);
    }
  } else if (role == kRoleDispatch) {
    // ================= dispatcher ====================================================================
    // Eight pages per trip, four lanes per page (lane = 4 * page + hq, heads 2hq and 2hq + 1): one
    // chain of wait -> compare -> vote decides eight pages, and the lanes that lead a kept page
    // request its residual + V side by side.  (One page per trip made this warp the slowest stage:
    // the chain is a few hundred cycles of latency however little it computes.)
    const int pj = lane >> 2, hq = lane & 3;
    const int gsz = 4 * m_grp;                                   // lanes of one prune group (4 ... 32)
    const uint32_t gmask = gsz >= 32 ? kFull : (((1u << gsz) - 1u) << ((lane / gsz) * gsz));
    uint32_t kk = 0;                                             // kept pages + end markers issued so far
    bool ok = true;
    for (uint32_t seg_i = 0; ok && next_chunk(seg_i); ++seg_i) {
      const int unit = seg_unit, page_begin = seg_page0, n = seg_n, part = seg_part;
      const int b = unit / p.HKV, hkv = unit % p.HKV;
      const int64_t row0 = static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G;
      float th0 = 0.f, th1 = 0.f;
      if (sampled) {
        const int ss = seg_i & 1;
        ok = WS_WAIT(thfull(ss), (seg_i / 2) & 1u, 2, 0);
        if (!ok) break;
        th0 = fmaxf(sTh[ss * 16 + 2 * hq], sTh[ss * 16 + 8 + 2 * hq]) - p.delta;
        th1 = fmaxf(sTh[ss * 16 + 2 * hq + 1], sTh[ss * 16 + 8 + 2 * hq + 1]) - p.delta;
        __syncwarp();
        if (lane == 0) mbar_arrive(thempty(ss));
      } else {
        if (2 * hq < G) th0 = p.th_in[row0 + 2 * hq];
        if (2 * hq + 1 < G) th1 = p.th_in[row0 + 2 * hq + 1];
      }
      if (p.th_out && page_begin == 0 && pj == 0) {
        if (2 * hq < G) p.th_out[row0 + 2 * hq] = th0;
        if (2 * hq + 1 < G) p.th_out[row0 + 2 * hq + 1] = th1;
      }
      // mean-V: running maximum / mass of the pruned pages, heads 2hq and 2hq + 1 (the same in every page's lanes)
      float apx_m0 = -INFINITY, apx_l0 = 0.f, apx_m1 = -INFINITY, apx_l1 = 0.f;
      int8_t* mask_row = p.mask ? p.mask + (static_cast<int64_t>(b) * p.HKV + hkv) * p.NTBS : nullptr;
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
        bool keep = (__ballot_sync(kFull, reaches) & gmask) != 0u;
        uint32_t sub_kept = 0xfu;
        if (n_sub > 1) {
          sub_kept = ws_decide_sub_blocks(dsub + ds * 32, n_sub, tps_shift, hq, G, th0, th1, valid, gmask,
                                          mask_row ? mask_row + (page_begin + c) * n_sub : nullptr);
          keep = sub_kept != 0u;
        } else if (mask_row && valid && (lane % gsz) == 0) {
          mask_row[(page_begin + c) / m_grp] = keep ? 1 : 0;
        }
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
            const int row = p.bt ? btv * kPage : b * T + (page_begin + c) * kPage;
            if (ord >= kNRV) lane_ok = ws_wait_lane(rvempty(slot), ((ord / kNRV) - 1u) & 1u, sAbort, 4);
            if (lane_ok) {
              kq_page[slot] = page_begin + c;
              kq_ds[slot] = ds;
              kq_sub[slot] = static_cast<int>(sub_kept);
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
        if (lead && !keep) mbar_arrive_n(dempty(ds), 2);
        ok = __all_sync(kFull, lane_ok) != 0;
      }
      if (!ok) break;
      // end markers: one per refine pair (kept page k goes to pair k mod kNP, so kNP consecutive
      // ordinals reach every pair once)
      for (int i = 0; ok && i < kNP; ++i) {
        const int slot = kk % kNRV;
        if (kk >= kNRV && !WS_WAIT(rvempty(slot), ((kk / kNRV) - 1u) & 1u, 5, 2)) { ok = false; break; }
        if (lane == 0) {
          kq_page[slot] = -1;
          mbar_arrive(rvfull(slot));
        }
        ++kk;
      }
      if (!ok) break;
      if (mask_row && page_begin + CH >= p.NPp) {
        // mask entries past the last group that holds tokens (padding blocks count as pruned)
        for (int i = (n_sub > 1 ? p.NP * n_sub : (p.NP + m_grp - 1) / m_grp) + lane; i < p.NTBS; i += 32) mask_row[i] = 0;
      }
      if (MV) {
        // this chunk's pruned mass; the dispatcher is one more party to the (batch, kv-head)'s arrival count
        if (pj == 0) {
          if (2 * hq < G) {
            p.part_pm[(row0 + 2 * hq) * p.nch + part] = apx_m0;
            p.part_pl[(row0 + 2 * hq) * p.nch + part] = apx_l0;
          }
          if (2 * hq + 1 < G) {
            p.part_pm[(row0 + 2 * hq + 1) * p.nch + part] = apx_m1;
            p.part_pl[(row0 + 2 * hq + 1) * p.nch + part] = apx_l1;
          }
        }
        if (ws_arrive_unit(p, unit, arrive_target, lane)) ws_merge_unit<MV>(p, b, hkv, n_seg, 0, 1, lane);
      }
      gc += static_cast<uint32_t>(n);
    }
  } else if (role == kRoleScore) {
    // ================= scoring warps =================================================================
    float* sS = reinterpret_cast<float*>(smem + L::kOffS) + sw * 256;   // this warp's copy of the channel scales
    float* sZ = sS + 128;
    bool ok = true;
    for (uint32_t seg_i = 0; ok && next_chunk(seg_i); ++seg_i) {
      const int unit = seg_unit, page_begin = seg_page0, n = seg_n;
      const int b = unit / p.HKV, hkv = unit % p.HKV;
      if (L::kHasChannelScale) {
        __syncwarp();                              // the previous chunk's reads of sS / sZ are done
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int64_t o = (static_cast<int64_t>(b) * p.HKV + hkv) * kHeadDim + lane + 32 * i;
          sS[lane + 32 * i] = load_as_float(p.ks, o, p.scale_dtype);
          if (FMT == FFA_K_Q2) sZ[lane + 32 * i] = load_as_float(p.kz, o, p.scale_dtype);
        }
        __syncwarp();
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
          for (int cc = 0; cc < 4; ++cc) {
            const __half fast = __hfma(__float2half_rn(static_cast<float>(cc)), hs, hz);
            const __half ref = __float2half_rn(fmaf(static_cast<float>(cc), s, z));
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

      // ---- prune thresholds (reference ...q2fp8.py:55-82): two 16-token samples of the coarse K,
      // tokens [0,16) and [(NTB-1)*16, +16), scored by the first two scoring warps
      if (sampled && sw < 2) {
        const int ss = seg_i & 1;
        if (seg_i >= 2) ok = WS_WAIT(thempty(ss), ((seg_i / 2) - 1u) & 1u, 13, 0);
        if (!ok) break;
        const int blk = sw == 0 ? 0 : p.NTB - 1;
        const int tok0 = blk * kSample;
        if (FMT == FFA_K_NVFP4) apply_block_scale(load_block_scale(blk));
        // the 16 sample rows are read straight from global memory (once per chunk: not worth a slot)
        const int64_t row = (p.bt ? static_cast<int64_t>(p.bt[static_cast<int64_t>(b) * p.bt_stride + tok0 / kPage]) * kPage
                                  : static_cast<int64_t>(b) * T + (tok0 / kPage) * kPage) + tok0 % kPage;
        RowsRef rows;
        rows.stride = static_cast<int64_t>(p.HKV) * ROW;
        rows.base = p.kc + row * rows.stride + hkv * ROW;
        rows.valid = static_cast<int>(min(static_cast<int64_t>(kSampleRows), p.kv_rows - row));
        float d[NT][2];
        if constexpr (kFp8Coarse) dot_fp8<F8, NT, QP, RowsRef>(d, qb, qinv, rows, 0, g, t);
        else if (FMT == FFA_K_Q2 ? sc.q2_fast : (FMT == FFA_K_NVFP4 && sc.page_fast))
          dot_f16<FMT, NT, true, RowsRef>(d, qh, rows, sc, 0, g, t);
        else dot_f16<FMT, NT, false, RowsRef>(d, qh, rows, sc, 0, g, t);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const float s0 = tok0 + g < T ? to_log2(d[nt][0]) : -INFINITY;
          const float s1 = tok0 + g + 8 < T ? to_log2(d[nt][1]) : -INFINITY;
          float mm = fmaxf(s0, s1);
#pragma unroll
          for (int off = 4; off < 32; off <<= 1) mm = fmaxf(mm, __shfl_xor_sync(kFull, mm, off));
          if (g == 0) sTh[ss * 16 + sw * 8 + 4 * nt + t] = mm;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(thfull(ss));
      }

      float ks_batch = 0.f;         // nvfp4: block scales of this warp's next 32 pages, one per lane
      for (int c = sw; c < n; c += kNS) {
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
            if (n_sub > 1) {
              // the tile's own maximum per head, for prune blocks smaller than a page
              float tm = fmaxf(s0, s1);
#pragma unroll
              for (int off = 4; off < 32; off <<= 1) tm = fmaxf(tm, __shfl_xor_sync(kFull, tm, off));
              if (g == 0) {
                dsub[ds * 32 + mt * 8 + 4 * nt + t] = tm;
                if (NT == 1) dsub[ds * 32 + mt * 8 + 4 + t] = -INFINITY;
              }
            }
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
      gc += static_cast<uint32_t>(n);
    }
  } else {
    // ================= refine warps ==================================================================
    const int pair = rw >> 1, sub = rw & 1;        // this warp refines tokens [32 sub, 32 sub + 32) of its pair's pages
    uint32_t myk = pair;                           // ordinal of the pair's next kept page (or end marker)
    uint32_t pair_pages = 0;                       // pages the pair has refined: phase of its meeting point
    const int src = 8 * t + (g >> 1);
    const uint32_t sel = (g & 1) ? 0x7632u : 0x5410u;
    const int vsel = (lane >> 3) & 1;
    const float qnan = __int_as_float(0x7fc00000);
    for (uint32_t seg_i = 0; next_chunk(seg_i); ++seg_i) {
      const int unit = seg_unit, part = seg_part;
      const int b = unit / p.HKV, hkv = unit % p.HKV;
      const int64_t row0 = static_cast<int64_t>(b) * p.HQ + static_cast<int64_t>(hkv) * G;
      float run_m[NT], run_l[NT], run_o[NT][8][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        run_m[nt] = -INFINITY;
        run_l[nt] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) run_o[nt][i][0] = run_o[nt][i][1] = 0.f;
      }
      uint32_t qb[NT * (QP - 1)][4][2];
      uint32_t qh[NT][8][2];
      float qinv[NT];
      prep_q<NT, QP, false>(p, b, hkv, G, g, t, qb, qh, qinv);
      bool ok = true;
      for (;;) {
        const int slot = myk % kNRV;
        // as for the coarse ring: the slot's previous page (another warp's) must have been released
        // before this wait can tell the phase it wants from the one before it
        if (myk >= kNRV && !WS_WAIT(rvempty(slot), ((myk / kNRV) - 1u) & 1u, 9, 0)) { ok = false; break; }
        if (!WS_WAIT(rvfull(slot), (myk / kNRV) & 1u, 9, 0)) { ok = false; break; }
        const int page = kq_page[slot];
        const int ds = kq_ds[slot];
        const uint32_t sub_kept = SUBP ? static_cast<uint32_t>(kq_sub[slot]) : 0xfu;
        myk += kNP;
        if (page < 0) {                                  // end of the chunk
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
        // pass 1 (this warp's two 16-token tiles): refined scores = coarse dots + residual dots, written
        // back over the dots (each lane owns its entries), and the maximum of its half of the page
#pragma unroll
        for (int mt = 2 * sub; mt < 2 * sub + 2; ++mt) {
          float dr[NT][2];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) dr[nt][0] = dr[nt][1] = 0.f;
          if (use_res) dot_fp8<F8, NT, QP>(dr, qb, qinv, rtile, mt, g, t);
          const int tok = page * kPage + 16 * mt + g;
          const bool on = ((sub_kept >> (mt >> tps_shift)) & 1u) != 0u;         // the tile's prune block is kept
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            float* e = hs + ((mt * NT + nt) * 2) * 32 + lane;
            const float s0 = on && tok < T ? to_log2(e[0] + dr[nt][0]) : -INFINITY;
            const float s1 = on && tok + 8 < T ? to_log2(e[32] + dr[nt][1]) : -INFINITY;
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
        {
          // the page maximum (...q2fp8.py:121) is over both halves: the two warps swap theirs
          float* pm = pairmax + (pair * 2 + (pair_pages & 1u)) * 16;
          if (g == 0) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) pm[sub * 8 + 4 * nt + t] = rm[nt];
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(pairmeet(pair));
          if (!WS_WAIT(pairmeet(pair), pair_pages & 1u, 17, 3)) { ok = false; break; }
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) rm[nt] = fmaxf(rm[nt], pm[(sub ^ 1) * 8 + 4 * nt + t]);
          ++pair_pages;
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          // pass 2 (this warp's two tiles): p = exp2(s - page max), fp32 sum, fp16 rounding for the P.V product
          // (...q2fp8.py:123-131); the eight 16-channel accumulators of P.V live across the trips
          float oacc[8][4];
#pragma unroll
          for (int i = 0; i < 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
          float l = 0.f;
#pragma unroll
          for (int mt = 2 * sub; mt < 2 * sub + 2; ++mt) {
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
      // ---- chunk end: the refine warps add up their shares and write ONE partial per q head ----------
      // (separate partials per warp made the merge of a (batch, kv-head) read four times as many rows,
      // one L2 round trip per eight of them, on a single warp)
      {
        float* myred = red + rw * (L::kRedWarp / 4);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          float l = run_l[nt];
#pragma unroll
          for (int off = 4; off < 32; off <<= 1) l += __shfl_xor_sync(kFull, l, off);
          const int h = 4 * nt + t;
          float* w = myred + h * 128;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            w[16 * i + g] = run_o[nt][i][0];
            w[16 * i + g + 8] = run_o[nt][i][1];
          }
          if (g == 0) { redml[rw * 16 + h] = run_m[nt]; redml[rw * 16 + 8 + h] = l; }
        }
      }
      const uint32_t mpar = seg_i & 1u;
      __syncwarp();
      if (lane == 0) mbar_arrive(rfmeet(0));
      if (ok) ok = WS_WAIT(rfmeet(0), mpar, 14, 4);
      // heads rw, rw + 4: sum over the warps, rescaled to the common maximum
      const bool bad = !ok || *reinterpret_cast<volatile int*>(sAbort) != 0;
      for (int h = rw; h < G; h += kNR) {
        float top = -INFINITY;
#pragma unroll
        for (int r = 0; r < kNR; ++r) top = fmaxf(top, redml[r * 16 + h]);
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
        float l = 0.f;
#pragma unroll
        for (int r = 0; r < kNR; ++r) {
          const float mr = redml[r * 16 + h];
          if (mr != -INFINITY) {
            const float sc = exp2f(mr - top);
            const float4 v = *reinterpret_cast<const float4*>(red + r * (L::kRedWarp / 4) + h * 128 + 4 * lane);
            o.x += v.x * sc; o.y += v.y * sc; o.z += v.z * sc; o.w += v.w * sc;
            l += redml[r * 16 + 8 + h] * sc;
          }
        }
        // a chunk whose waits gave up publishes NaN, so that the merged rows are NaN rather than plausible numbers
        if (bad) { o = make_float4(qnan, qnan, qnan, qnan); l = qnan; top = 0.f; }
        *reinterpret_cast<float4*>(p.part_o + ((row0 + h) * p.nch + part) * kHeadDim + 4 * lane) = o;
        if (lane == 0) {
          p.part_m[(row0 + h) * p.nch + part] = top;
          p.part_l[(row0 + h) * p.nch + part] = l;
        }
      }
      __threadfence();
      __syncwarp();
      if (lane == 0) mbar_arrive(rfmeet(1));
      if (ok) ok = WS_WAIT(rfmeet(1), mpar, 15, 4);      // every head's partial is written; `red` may be reused
      if (rw == 0) {
        const bool last = ws_arrive_unit(p, unit, arrive_target, lane);
        if (lane == 0) *sLast = last ? 1 : 0;
        __syncwarp();
      }
      if (lane == 0) mbar_arrive(rfmeet(2));
      if (ok) ok = WS_WAIT(rfmeet(2), mpar, 16, 4);
      if (ok && *reinterpret_cast<volatile int*>(sLast) != 0) ws_merge_unit<MV>(p, b, hkv, n_seg, rw, kNR, lane);
      if (!ok) break;
    }
  }

  __syncthreads();
#ifdef FFA_WS_PROFILE
  // 64-bit sums over all CTAs, kept in the middle of the arrival-counter block (byte 32768 of the
  // workspace; profiling builds serve at most 8192 (batch x kv-head) units): [role * 8 + i] = pacc[i]
  // of the role's warps (i < 6); [32] = kernel cycles of a CTA, [33] = its nanoseconds, [34] = the
  // longest CTA's ns.
  //   coarse producer: 0 wait for a free coarse slot, 1 free chunk entry
  //   dispatcher:      0 thresholds, 1 published page, 2 free residual+V slot, 3 kept-page branch, 5 next chunk
  //   scoring:         0 thresholds read, 1 coarse tile, 2 free entry, 3 dots, 4 publish, 5 next chunk
  //   refine:          0 residual+V landed, 1 page work, 2 pages, 4 chunk-end meetings, 5 next chunk
  if (p.arrivals) {
    unsigned long long* gp = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(p.arrivals) + 32768);
    if (lane == 0) {
      for (int i = 0; i < 6; ++i) atomicAdd(gp + role * 8 + i, static_cast<unsigned long long>(pacc[i]));
    }
    if (tid == 0) {
      unsigned long long g1;
      asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(g1));
      atomicAdd(gp + 32, static_cast<unsigned long long>(clock64() - prof_c0));
      atomicAdd(gp + 33, g1 - prof_g0);
      atomicMax(gp + 34, g1 - prof_g0);
      // per CTA: SM id, start and end time (ns), from byte 36864 of the workspace on
      unsigned long long* pc = reinterpret_cast<unsigned long long*>(reinterpret_cast<char*>(p.arrivals) + 36864) + 3 * blockIdx.x;
      uint32_t smid;
      asm volatile("mov.u32 %0, %%smid;\n" : "=r"(smid));
      pc[0] = smid; pc[1] = prof_g0; pc[2] = g1;
    }
  }
#endif
  if (tid == 0) {
    if (*sAbort != 0 && p.status && atomicCAS(p.status, 0, 1) == 0) {
      p.status[1] = *sAbort;                 // which wait gave up first in this CTA
      p.status[5] = static_cast<int>(blockIdx.x);
    }
    // the last CTA to leave puts the work counter back to zero for the next launch
    if (p.peer_world > 0) __threadfence_system();
    else __threadfence();
    if (atomicAdd(p.work + 1, 1) == static_cast<int>(gridDim.x) - 1) {
      p.work[0] = 0;
      p.work[1] = 0;
      if (p.peer_world > 0) {
        // every CTA's rows are out (each fenced its stores before it was counted): tell the peers
        __threadfence_system();
        for (int pr = 0; pr < p.peer_world; ++pr) *reinterpret_cast<volatile int*>(p.peer_flag[pr]) = p.peer_step;
      }
    }
  }
}

// Configures (once per device) and launches the kernel.
template <int FMT, int F8, int NT, bool VBF, int QP, bool MV = false, bool SUBP = false>
int launch_ws_one(const DecodeParams& p, const CUtensorMap* maps, cudaStream_t stream) {
  if constexpr (!MV && !SUBP) {
    if (p.sub > 1) return launch_ws_one<FMT, F8, NT, VBF, QP, false, true>(p, maps, stream);
  }
  using L = WsSmem<FMT, NT, SUBP>;
  auto kern = decode_ws_kernel<FMT, F8, NT, VBF, QP, MV, SUBP>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const bool slot = dev >= 0 && dev < 64;
  if (!slot || !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes);
    if (e != cudaSuccess) return note_cuda_error(e, "cudaFuncSetAttribute(decode_ws)");
    if (slot) configured[dev] = true;
  }
  kern<<<static_cast<unsigned>(p.grid), kWsThreads, L::kBytes, stream>>>(p, maps[0], maps[2], maps[3]);   // coarse K, residual, V (maps[1] is unused)
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
