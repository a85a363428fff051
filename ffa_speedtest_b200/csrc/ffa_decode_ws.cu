// Host side of the warp-specialised decode kernel (ffa_decode_ws.cuh): page-range plan, TMA
// descriptors and the dispatch to the per-format translation units.
#include "ffa_decode_ws_launch.h"

namespace ffa {

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
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

// [rows, HKV * row_bytes] bytes seen as a 2-D byte tensor; box = box_rows x box_bytes
bool make_map(CUtensorMap* m, const void* base, int64_t rows, int64_t row_bytes_all_heads, int box_bytes,
              int box_rows, bool swizzle128, int promo) {
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes_all_heads), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes_all_heads)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_bytes), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  return encode_tiled()(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        static_cast<CUtensorMapL2promotion>(promo), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

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

// The four descriptors of a call depend on the tensor addresses, the row count and the format only;
// a decode loop calls with the same ones every step, so the last set is kept per thread and the
// driver is not asked to encode them again.
struct MapKey {
  const void *kc, *kr, *v;
  int64_t rows;
  int hkv, variant;
  bool operator==(const MapKey& o) const {
    return kc == o.kc && kr == o.kr && v == o.v && rows == o.rows && hkv == o.hkv && variant == o.variant;
  }
};
struct MapCache {
  bool valid = false;
  MapKey key{};
  alignas(64) CUtensorMap maps[4];
};
thread_local MapCache g_maps;

}  // namespace

void decode_ws_plan(int B, int HKV, int NP, int group, int chunk_in, int* NPp_out, int* chunk_out, int* nseg_out,
                    int* grid_out) {
  const int m = group < 1 ? 1 : group;
  const long long NPp = (static_cast<long long>(NP) + m - 1) / m * m;
  const long long units = static_cast<long long>(B) * HKV;
  const long long total = units * NPp;
  const long long sms = sm_count();
  long long ch = chunk_in;
  if (ch <= 0) {
    // Plenty of work: about six chunks per SM, handed out dynamically - fine enough for the SMs to even
    // out their different kept fractions, coarse enough that a chunk's set-up (q operands, scales,
    // thresholds, one partial) stays small beside its pages.  Less work: the set-up and the hand-over
    // between chunks weigh more than the imbalance, so the chunks are cut to fill `waves` x SMs as
    // exactly as whole chunks per (batch, kv-head) allow - one chunk per SM for the smallest cases.
    const long long per_cta = (total + sms - 1) / sms;
    if (per_cta >= 256) ch = (per_cta + 5) / 6;
    else {
      const long long waves = per_cta < 64 ? 1 : (per_cta < 128 ? 2 : 3);
      ch = (per_cta + waves - 1) / waves;
      if (ch < 4) ch = 4;
      if (ch > NPp) ch = NPp;
      while (ch < NPp && units * ((NPp + ch - 1) / ch) > sms * waves) ++ch;
    }
  }
  // the merge of a (b, kv-head) holds at most kWsMaxParts partials per q head, one per chunk
  const long long max_seg = kWsMaxParts;
  if (ch < (NPp + max_seg - 1) / max_seg) ch = (NPp + max_seg - 1) / max_seg;
  ch = (ch + m - 1) / m * m;                         // whole prune groups
  if (ch > NPp) ch = NPp;
  const long long nseg = (NPp + ch - 1) / ch;
  const long long chunks = units * nseg;
  *NPp_out = static_cast<int>(NPp);
  *chunk_out = static_cast<int>(ch);
  *nseg_out = static_cast<int>(nseg);
  *grid_out = static_cast<int>(chunks < sms ? chunks : sms);
}

int decode_nch_bound(int B, int HKV, int NP, int wc_in) {
  const long long units = static_cast<long long>(B) * HKV;
  const long long NPp = static_cast<long long>(NP) + kMaxPruneGroup - 1;     // whatever the prune group
  // warp-specialised kernel: one partial per chunk; chunks of at least 4 pages (or the caller's size)
  // and at most kWsMaxParts partials per q head
  long long ws = (NPp + (wc_in > 0 ? wc_in : 4) - 1) / (wc_in > 0 ? wc_in : 4);
  if (ws > kWsMaxParts) ws = kWsMaxParts;
  // fp16 kernel (ffa_decode_plan): ceil(NP / ppc) with ppc >= max(4, NP / want)
  long long f16;
  if (wc_in > 0) f16 = (static_cast<long long>(NP) + wc_in - 1) / wc_in;
  else {
    long long want = (148LL * 2 * 8 + units - 1) / units;
    if (want < 1) want = 1;
    f16 = (static_cast<long long>(NP) + 3) / 4;
    if (f16 > want) f16 = want;
  }
  if (f16 < 1) f16 = 1;
  // page-pipeline kernel (decode_tma_plan): ceil(NP / wc) + 1 with wc >= max(4 or the caller's size, ceil(NP / 63))
  long long pipe = (static_cast<long long>(NP) + (wc_in > 0 ? wc_in : 4) - 1) / (wc_in > 0 ? wc_in : 4);
  if (pipe > 63) pipe = 63;
  pipe += 1;
  long long best = ws > f16 ? ws : f16;
  if (pipe > best) best = pipe;
  return static_cast<int>(best);
}

bool decode_ws_supported(const DecodeParams& p, int group) {
  // groups of 1, 2, 4 or 8 pages: a trip of the dispatcher (8 pages) holds whole groups
  return group >= 1 && group <= kMaxPruneGroup && (group & (group - 1)) == 0 && encode_tiled() != nullptr;
}

int launch_decode_ws(const DecodeParams& p, int variant, int f8, int64_t kv_rows, cudaStream_t stream) {
  if (kv_rows <= 0 || kv_rows > 0x7fffffffLL) return FFA_E_LIMIT;
  const int row_c = variant == FFA_K_FP8 ? 128 : (variant == FFA_K_Q2 ? 32 : 64);
  const MapKey key{p.kc, p.kr, p.v, kv_rows, p.HKV, variant};
  MapCache& mc = g_maps;
  if (!mc.valid || !(mc.key == key)) {
    mc.valid = false;
    // L2 promotion no wider than one head's row: a 256-byte promotion on 128-byte rows pulled the
    // neighbouring head's bytes from DRAM too early to be reused (+15 % DRAM traffic, -11 % speed).
    const int promo_c = row_c >= 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                     : (row_c >= 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B : CU_TENSOR_MAP_L2_PROMOTION_NONE);
    const int64_t all_c = static_cast<int64_t>(p.HKV) * row_c;
    const bool swz = variant == FFA_K_FP8;
    if (!make_map(&mc.maps[0], p.kc, kv_rows, all_c, row_c, kPage, swz, promo_c)) return FFA_E_LAUNCH;
    mc.maps[1] = mc.maps[0];              // (second descriptor unused)
    // without a residual the map is never used; point it at the coarse tensor to keep it valid
    if (p.kr) {
      if (!make_map(&mc.maps[2], p.kr, kv_rows, static_cast<int64_t>(p.HKV) * kResRow, kResRow, kPage, true,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B))
        return FFA_E_LAUNCH;
    } else {
      mc.maps[2] = mc.maps[0];
    }
    if (!make_map(&mc.maps[3], p.v, kv_rows, static_cast<int64_t>(p.HKV) * kVRow, 128, kPage, true,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B))
      return FFA_E_LAUNCH;
    mc.key = key;
    mc.valid = true;
  }
  switch (variant) {
    case FFA_K_FP8:   return launch_ws_fp8(p, f8, mc.maps, stream);
    case FFA_K_Q2:    return launch_ws_q2(p, f8, mc.maps, stream);
    case FFA_K_FP4:   return launch_ws_fp4(p, f8, mc.maps, stream);
    case FFA_K_NF4:   return launch_ws_nf4(p, f8, mc.maps, stream);
    case FFA_K_NVFP4: return launch_ws_nvfp4(p, f8, mc.maps, stream);
    default: return FFA_E_VARIANT;
  }
}

}  // namespace ffa
