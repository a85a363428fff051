// Declarations shared by the two decode kernels (ffa_decode.cu: fp16 tensor-core path fed by
// cp.async; ffa_decode_tma.cu: fp8 tensor-core path fed by TMA).
#pragma once

#include "ffa_common.cuh"

namespace ffa {

constexpr int kDecodeThreads = 128;
constexpr int kDecodeWarps = 4;   // each warp owns 16 tokens of every page
constexpr int kSample = 16;       // threshold sample width (T_BS in the reference)
constexpr int kMaxPruneGroup = 8; // largest prune group of the warp-specialised kernel, in pages (SBS <= 512)
constexpr int kWsRefineWarps = 4; // refine warps of the warp-specialised kernel
constexpr int kWsMaxParts = 32;   // partials (one per chunk) per q head that its merge handles
// ints of the arrival-counter block that the warp-specialised kernel uses as its work counter (next
// chunk to hand out) and as the count of CTAs that have left; both are zero between launches
constexpr int kMaxPeerRanks = 16;
constexpr int kWorkCounterIndex = 16000;
constexpr int kResRow = 128;      // fp8 residual bytes per token per head
constexpr int kVRow = 256;        // V bytes per token per head (fp16 / bf16)
constexpr int kRvSlot = kPage * (kResRow + kVRow);
// The first kArrivalBytes of a decode workspace hold the per-(b, kv-head) arrival counters of the TMA
// kernel (zero before the first launch; every launch leaves them zero again); its last 256 bytes hold
// the status word that a kernel sets when a bounded wait gave up.
constexpr int kArrivalBytes = 64 * 1024;

static __constant__ float c_nf4_book[16] = {
    -1.0f, -0.6961928009986877f, -0.5229921340942383f, -0.39491748809814453f,
    -0.28444138169288635f, -0.18477343022823334f, -0.09105003625154495f, 0.0f,
    0.07958029955625534f, 0.16093020141124725f, 0.24611230194568634f, 0.33791524171829224f,
    0.44070982933044434f, 0.5626170039176941f, 0.7229568362236023f, 1.0f};

template <int FMT> struct Fmt;
template <> struct Fmt<FFA_K_FP8>   { static constexpr int kRow = 128; };
template <> struct Fmt<FFA_K_Q2>    { static constexpr int kRow = 32; };
template <> struct Fmt<FFA_K_FP4>   { static constexpr int kRow = 64; };
template <> struct Fmt<FFA_K_NF4>   { static constexpr int kRow = 64; };
template <> struct Fmt<FFA_K_NVFP4> { static constexpr int kRow = 64; };

struct DecodeParams {
  const uint8_t* q;
  const uint8_t* kc;
  const void* ks;
  const void* kz;
  const uint8_t* kr;
  const uint8_t* v;
  const int32_t* bt;
  const float* th_in;
  float* part_m;     // [B*HQ, nch]
  float* part_l;     // [B*HQ, nch]
  float* part_o;     // [B*HQ, nch, 128]
  int8_t* mask;      // [B, HKV, NTBS] or null
  float* th_out;     // [B, HQ] or null
  int* status;       // device status word: set to 1 when a bounded wait gave up
  int* arrivals;     // TMA kernel: per-(b, kv-head) count of finished segments; zero between launches
  void* out;         // TMA kernel: final output [B*HQ, 128] in q_dtype (the last segment merges)
  float* partial_out;  // optional [B*HQ, 129]
  int bt_stride;
  int B, T, HQ, HKV, G;
  int NP;            // real pages = ceil(T/64)
  int NTB;           // ceil(T/BS)
  int NTBS;          // mask entries per (b, hkv)
  int BS;
  int ppc;           // pages per chunk
  int nch;           // chunks per (b, hkv)
  float sm_scale, delta;
  int q_dtype, scale_dtype;
  int use_res, v_bf16;
  int refine_lag;    // TMA kernel: pages between scoring and refining a page (1 or 2)
  // mean-V variant (q2 only): pruned pages contribute their coarse softmax mass times the mean of V.
  // Every segment adds the running maximum and mass of its pruned pages to its partial.
  const void* v_mean;        // [B*HKV, 128] in V's dtype, or null
  // warp-specialised kernel: pages per prune group (SBS / 64) and pages per (b, kv-head) rounded up
  // to whole groups; page ranges are cut in that padded space so that no group straddles two CTAs
  int group;
  int sub;           // prune blocks per page when SBS is below 64 (2 or 4), else 1
  int NPp;
  int nseg;          // chunks per (b, kv-head); `ppc` is the pages of a chunk
  int grid;          // CTAs to launch
  int* work;         // [0] next chunk to hand out, [1] CTAs that have left
  int64_t kv_rows;   // token rows of the K/V tensors
  float* part_pm;            // [B*HQ, nch]
  float* part_pl;            // [B*HQ, nch]
  // sequence split over the GPUs of one box (warp-specialised kernel): every partial_out row is also
  // stored into this rank's slot on each peer, and the last CTA to leave raises this rank's flag on
  // every peer to `peer_step` (see ffa_peer.cu).  peer_world = 0: off.
  int peer_world, peer_rank, peer_step;
  float* peer_slot[kMaxPeerRanks];     // peer p's copy of this rank's [B*HQ, 129] slot for this step (mapped memory)
  int* peer_flag[kMaxPeerRanks];       // this rank's flag on peer p
};


// ffa_decode_ws.cu (warp-specialised kernel: bf16 / fp16 / fp32 q, prune groups of up to 8 pages):
// plan and launch.  Every (b, kv-head) is cut into `nseg` chunks of `chunk` pages (whole prune groups,
// the last one shorter); CTAs take chunks from a counter until none is left.
void decode_ws_plan(int B, int HKV, int NP, int group, int chunk_in, int* NPp, int* chunk, int* nseg, int* grid);
bool decode_ws_supported(const DecodeParams& p, int group);
int launch_decode_ws(const DecodeParams& p, int variant, int f8, int64_t kv_rows, cudaStream_t stream);
// Upper bound, monotonic in NP, of the partials any (b, kv-head) receives under either kernel's plan:
// the stride of the partial arrays and what the workspace is sized for.
int decode_nch_bound(int B, int HKV, int NP, int wc_in);

// ffa_decode_tma.cu: returns FFA_OK after enqueueing stage 1, or a negative FFA_E_* code.
// `kv_rows` is the number of token rows in the K/V tensors (B*T, or pages*64 for a pool).
int launch_decode_tma(const DecodeParams& p, int variant, int f8, int64_t kv_rows, cudaStream_t stream);
// Page ranges of the TMA kernel: `wc` pages per CTA over the flattened (b, kv-head, page) space
// (about one CTA per resident slot: 2 per SM), `nch` = most partials any kv-head can receive.
void decode_tma_plan(int B, int HKV, int NP, int wc_in, int ctas_per_sm, int* wc, int* nch);
// resident CTAs per SM of the TMA kernel for a coarse format and refine lag
int decode_tma_residency(const DecodeParams& p, int variant, int f8);   // CTAs per SM of the kernel that would run
// true when the TMA path handles these arguments (bf16 q, driver entry point available)
bool decode_tma_supported(const DecodeParams& p);

}  // namespace ffa
