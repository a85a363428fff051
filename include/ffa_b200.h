/*
 * C ABI of libffa_b200.so: FFA quantised, pruned decode attention and its quantisers for
 * NVIDIA B200 (sm_100a).
 *
 * The reference project (qluoluo/ffa-speedtest) has no FFI: its boundary for this path is a
 * set of Python entry points that validate tensors and launch two Triton kernels.  Every
 * function below is what a binding for one of those entry points calls after it has done
 * the reference's own validation; each comment cites the reference interface it replaces
 * (paths relative to the reference root).
 *
 * Conventions: all pointers are device pointers unless stated; all tensors are contiguous;
 * nothing here allocates, synchronises or throws; every call only enqueues work on `stream`
 * and is safe to record into a CUDA graph.  Return value 0 = enqueued, negative = FFA_E_*.
 */
#ifndef FFA_B200_H_
#define FFA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* ffa_stream_t; /* a cudaStream_t */

enum {
  FFA_OK = 0,
  FFA_E_NULL = -1,        /* a required pointer is NULL */
  FFA_E_SHAPE = -2,       /* unsupported dimension (head_dim != 128, G > 8, page != 64, ...) */
  FFA_E_DTYPE = -3,       /* unsupported element type code */
  FFA_E_WORKSPACE = -4,   /* workspace too small */
  FFA_E_LAUNCH = -5,      /* the CUDA runtime refused the launch (see ffa_last_cuda_error) */
  FFA_E_VARIANT = -6,     /* unknown coarse-K format */
  FFA_E_LIMIT = -7,       /* size beyond a compiled-in maximum */
  FFA_E_ALIGN = -8        /* a tensor pointer is not 16-byte aligned */
};

/* element types */
enum { FFA_F16 = 0, FFA_BF16 = 1, FFA_F32 = 2 };
/* fp8 encodings (torch.float8_e5m2 / torch.float8_e4m3fn) */
enum { FFA_E5M2 = 0, FFA_E4M3 = 1 };
/* coarse K formats, one per reference variant directory */
enum {
  FFA_K_FP8 = 0,   /* ffa-fp8fp8   : fp8 cast of K, 128 B per token per kv-head           */
  FFA_K_Q2 = 1,    /* ffa-q2fp8    : 2-bit codes + (scale, zero) per (b, kv-head, channel) */
  FFA_K_FP4 = 2,   /* ffa-fp4fp8   : unscaled e2m1 nibbles                                 */
  FFA_K_NF4 = 3,   /* ffa-nf4fp8   : NF4 nibbles + absmax per (b, kv-head, channel)        */
  FFA_K_NVFP4 = 4  /* ffa-nvfp4fp8 : e2m1 nibbles + one scale per (b, BS-block, kv-head)   */
};

/*
 * Arguments of one decode step.  Token rows of the K/V tensors are addressed as
 *     row(b, t) = block_table ? block_table[b*bt_stride + t/64]*64 + t%64 : b*T + t
 * and a row holds HKV heads back to back, i.e. the reference layout [B, T, HKV, D] when
 * block_table is NULL and a paged pool [n_pages, 64, HKV, D] otherwise.
 */
typedef struct FfaDecodeArgs {
  int32_t variant;          /* FFA_K_*                                                          */
  int32_t B, T, HQ, HKV;    /* batch, context length, query heads, kv heads (G = HQ/HKV <= 8)   */
  int32_t head_dim;         /* K = V = 128                                                      */
  int32_t BS, SBS;          /* reference block sizes: SBS (prune granularity) 16, 32, 64, 128, 256 or
                               512, BS a multiple of SBS and of 64; always one launch.  SBS 16 / 32
                               (blocks inside a page): warp-specialised kernel only, not with v_mean */
  float sm_scale;           /* softmax scale, reference default 1/sqrt(K)                       */
  float delta;              /* threshold offset in log2 units                                   */
  int32_t q_dtype;          /* FFA_F16 | FFA_BF16 | FFA_F32; the output has the same type       */
  int32_t v_dtype;          /* FFA_F16 | FFA_BF16                                               */
  int32_t scale_dtype;      /* type of k_scale / k_zero                                         */
  int32_t fp8_format;       /* FFA_E5M2 | FFA_E4M3: residual (and fp8 base) encoding            */
  int32_t use_residual;     /* 0: refine == coarse scores (reference use_fp8_residual=False)    */
  const void* q;            /* [B, HQ, 128]                                                     */
  const void* k_codes;      /* coarse K rows: 128 B (fp8), 32 B (q2) or 64 B (4-bit) per head   */
  const void* k_scale;      /* q2, nf4: [B, HKV, 128]; nvfp4: [B, ceil(T/BS), HKV]; else NULL   */
  const void* k_zero;       /* q2: [B, HKV, 128]; else NULL                                     */
  const void* k_residual;   /* fp8 rows, 128 B per head; may be NULL when use_residual == 0     */
  const void* v;            /* V rows, 256 B per head                                           */
  const int32_t* block_table; /* [B, bt_stride] page ids, or NULL for the contiguous layout     */
  int32_t bt_stride;
  const float* threshold_in;  /* [B, HQ] precomputed thresholds, or NULL to derive them          */
  void* out;                /* [B, HQ, 128] in q_dtype                                          */
  int8_t* kept_mask;        /* optional [B, HKV, NTBS] (NTBS = ceil(T/BS)*(BS/SBS)), 1 = kept   */
  float* threshold_out;     /* optional [B, HQ]: thresholds actually used                       */
  float* partial_out;       /* optional [B, HQ, 129] fp32: normalised output followed by the
                               base-2 log-sum-exp of the kept scores (-inf if none kept), the
                               form ffa_merge_partials consumes                                 */
  void* workspace;          /* >= ffa_decode_workspace_bytes(...) bytes, 256-byte aligned.  Its
                               first 64 KiB (per-(batch, kv-head) arrival counters) must be zero
                               before the first call; every call that returns FFA_OK and runs to
                               completion leaves them zero.  Zero them again (cudaMemsetAsync)
                               after a call that failed or whose stream was torn down mid-kernel:
                               with stale counters the merge of a (batch, kv-head) never runs and
                               its output rows keep their old contents.  The int at byte 65280 is
                               set by a kernel when one of its bounded waits gave up; the outputs
                               of the heads it touched are then NaN                             */
  size_t workspace_bytes;
  int32_t pages_per_chunk;  /* 0 = choose automatically                                         */
  int32_t reserved;         /* kernel choice.  0: by measurement - the warp-specialised TMA kernel,
                               except for fp8 coarse K with SBS = 64, bf16 q (or fp16 q and V) and
                               fewer than 131072 pages in all (B x HKV x pages per sequence), where
                               the page-pipeline TMA kernel is the faster one (NF4: likewise between
                               12288 and 131072 pages).  Bit 0: the fp16
                               tensor-core kernel (the reference's rounding sequence to the letter;
                               SBS = 64 only).  Bit 1: the page-pipeline kernel (SBS = 64, bf16 q
                               or fp16 q with fp16 V).  Bit 2: the warp-specialised kernel.  A
                               kernel asked for by bit that cannot take the call is an error  */
  int64_t kv_rows;          /* token rows in the K/V tensors: pages*64 of a pool, 0 = B*T       */
  const void* v_mean;       /* optional [B, HKV, 128] in V's type: the mean-V variant
                               (ffa-q2fp8-meanv/attn_kernel/attn_kernel_v1210_meanv_bsz_q2fp8.py): pruned
                               pages contribute their coarse softmax mass times this vector.  2-bit
                               format, no partial_out.  NULL = pruned pages are dropped */
} FfaDecodeArgs;

/* Replaces attn_forward_decode_quantized / _fp8fp8 / _fp4 / _nf4 / _nvfp4fp8 after validation:
 *   ffa-q2fp8/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8.py:264-304 (allocate, stage 1, stage 2)
 *   ffa-fp8fp8/attn_kernel/attn_kernel_v1210_fused_bsz_fp8fp8.py:243-308
 *   ffa-fp4fp8/attn_kernel/attn_kernel_v1210_fused_bsz_fp4fp8.py:182-294
 *   ffa-nf4fp8/attn_kernel/attn_kernel_v1210_fused_bsz_nf4fp8.py:212-330
 *   ffa-nvfp4fp8/attn_kernel/attn_kernel_v1210_fused_bsz_nvfp4fp8.py:225-367 */
int ffa_decode(const FfaDecodeArgs* args, ffa_stream_t stream);

/* Scratch needed by ffa_decode for these dimensions (the reference allocates m_buf, l_buf,
 * o_buf and mask_buf per call: ...q2fp8.py:269-273). */
size_t ffa_decode_workspace_bytes(int32_t B, int32_t T, int32_t HQ, int32_t HKV, int32_t pages_per_chunk);

/* Chunking ffa_decode will use: pages per CTA and CTAs per (b, kv-head). */
int ffa_decode_plan(int32_t B, int32_t T, int32_t HKV, int32_t pages_per_chunk_in,
                    int32_t* pages_per_chunk, int32_t* n_chunks);

/* Size of the scratch array built into the library for ffa_decode_static_scratch (4 MiB). */
#define FFA_STATIC_SCRATCH_BYTES (4u << 20)
size_t ffa_static_scratch_bytes(void);

/* The same decode step as ffa_decode for callers that cannot allocate device memory (a plug-in in a
 * host that owns and has already partitioned all of it, a loop where cudaMalloc is forbidden because
 * it stalls the device).  No counterpart in the reference, which allocates its scratch tensors on
 * every call.  args->workspace and args->workspace_bytes are ignored: the partial results go to an
 * array of FFA_STATIC_SCRATCH_BYTES that is part of the library image on every GPU that loads it.
 * Returns FFA_E_LIMIT, launching nothing, when ffa_decode_workspace_bytes(...) for the shape exceeds
 * that size.  The first call on a device resolves the array's device address; make it outside any
 * stream capture.  Calls on one device share the array: do not let two of them overlap on the GPU.
 * Allocates nothing. */
int ffa_decode_static_scratch(const FfaDecodeArgs* args, ffa_stream_t stream);

/* Status block of the last ffa_decode_static_scratch call on the current device: seven ints, [0] = 1
 * when one of the kernel's bounded waits gave up (outputs of the affected heads are NaN), the rest
 * say where.  `out` is device memory or pinned host memory; the copy is enqueued on `stream`, after
 * the decode call whose status it reports.  The next ffa_decode_static_scratch call clears the block.
 * No counterpart in the reference.  Allocates nothing. */
int ffa_static_scratch_status(int32_t* out, ffa_stream_t stream);

/* Merge R partial results (split-KV inside a GPU, or one per rank after an all-gather):
 * parts is [R, rows, 129] fp32 holding a normalised partial output (128) followed by its
 * base-2 LSE (-inf when the part kept nothing).  out is [rows, 128] in out_dtype.
 * The reference has only the intra-GPU form: attn_forward_stage2_masked
 * (ffa-q2fp8/attn_kernel/attn_kernel_v1210_fused_bsz_q2fp8.py:142-171). */
int ffa_merge_partials(const float* parts, int32_t R, int32_t rows, void* out, int32_t out_dtype,
                       ffa_stream_t stream);

/* Standalone quantisers, bit-exact with the reference's torch functions on the same K.
 * k is [B, T, HKV, 128] in k_dtype (FFA_F16 | FFA_BF16); outputs use the reference layouts.
 * scratch must hold ffa_quantize_scratch_bytes(B, HKV) bytes (per-channel min/max). */
size_t ffa_quantize_scratch_bytes(int32_t B, int32_t HKV);
/* ffa-q2fp8/fused_kproj_rope_q2fp8.py:40-68  quantize_k_2bit_fp8_residual */
int ffa_quantize_q2(const void* k, int32_t k_dtype, int32_t B, int32_t T, int32_t HKV, int32_t fp8_format,
                    uint8_t* codes, void* scale, void* zero, uint8_t* residual, void* scratch, ffa_stream_t stream);
/* ffa-fp8fp8/fused_kproj_rope_fp8fp8.py:58-64  quantize_k_fp8_fp8_residual */
int ffa_quantize_fp8fp8(const void* k, int32_t k_dtype, int32_t B, int32_t T, int32_t HKV, int32_t fp8_format,
                        uint8_t* base, uint8_t* residual, ffa_stream_t stream);
/* ffa-fp4fp8/fused_kproj_rope_fp4fp8.py:40-73  encode_k_fp4_fp8_residual */
int ffa_quantize_fp4(const void* k, int32_t k_dtype, int32_t B, int32_t T, int32_t HKV, int32_t fp8_format,
                     uint8_t* codes, uint8_t* residual, ffa_stream_t stream);
/* ffa-nf4fp8/fused_kproj_rope_nf4fp8.py:72-96  encode_k_nf4_fp8_residual */
int ffa_quantize_nf4(const void* k, int32_t k_dtype, int32_t B, int32_t T, int32_t HKV, int32_t fp8_format,
                     uint8_t* codes, void* scale, uint8_t* residual, void* scratch, ffa_stream_t stream);
/* ffa-nvfp4fp8/fused_kproj_rope_nvfp4fp8.py:62-114  encode_k_nvfp4_fp8_residual */
int ffa_quantize_nvfp4(const void* k, int32_t k_dtype, int32_t B, int32_t T, int32_t HKV, int32_t fp8_format,
                       int32_t page_size, uint8_t* codes, void* scale, uint8_t* residual, ffa_stream_t stream);

/*
 * Sequence-split decode across the GPUs of one box, the exchange fused with the merge (no reference
 * counterpart; the reference is single-GPU).  Every rank has produced its partial [rows, 129] of this
 * step (ffa_decode with partial_out pointing at slot [step & 1][rank] of its own gathered buffer).  This
 * call stores the partial into the same slot of every peer's gathered buffer over peer memory, raises
 * this rank's flag on every peer to `step`, then waits (at most one second) until all `world` flags of
 * this rank carry `step` and merges the world partials into out [rows, 128].
 *   peer_gathered[p]: device pointer, valid on this GPU, to rank p's buffer [2, world, rows, 129] fp32
 *                     (p == rank: the local buffer; others mapped through CUDA IPC by the caller)
 *   peer_flags[p]:    likewise rank p's int32 flags [world], zero before the first step
 *   step:             1, 2, 3, ... the same on every rank; buffers alternate by its parity
 * Both pointer arrays are host arrays of `world` (<= 16) entries, read during the call.  A wait that
 * gives up sets status[0] = 3 (if status is given) and writes NaN rows.  Plain peer stores and loads
 * only.  Replaces an all-gather of the partials followed by ffa_merge_partials.
 */
int ffa_peer_exchange_merge(const float* local_partial, int32_t rows, int32_t rank, int32_t world,
                            float* const* peer_gathered, int32_t* const* peer_flags, int32_t step, void* out,
                            int32_t out_dtype, int32_t* status, ffa_stream_t stream);

/*
 * The same exchange fused into the decode kernel.  ffa_decode_peer is ffa_decode (always on the
 * warp-specialised kernel unless `reserved` names another, which is refused; partial_out = slot [step & 1][rank] of this rank's own gathered buffer) whose merge also stores
 * every finished partial row into this rank's slot on each peer the moment the row exists, and whose
 * last CTA raises this rank's flags; the transfer overlaps the rest of the kernel.  ffa_peer_wait_merge
 * is then the second half of ffa_peer_exchange_merge alone: wait for the `world` flags of `step`, merge.
 */
typedef struct FfaPeerArgs {
  int32_t world, rank, step;           /* as for ffa_peer_exchange_merge                            */
  float* const* peer_gathered;         /* host array [world]                                        */
  int32_t* const* peer_flags;          /* host array [world]                                        */
} FfaPeerArgs;
int ffa_decode_peer(const FfaDecodeArgs* args, const FfaPeerArgs* peer, ffa_stream_t stream);
int ffa_peer_wait_merge(const float* gathered_local, const int32_t* flags_local, int32_t world, int32_t rows,
                        int32_t step, void* out, int32_t out_dtype, int32_t* status, ffa_stream_t stream);

/* Set-up for ffa_peer_exchange_merge (these four allocate, map or free; none belongs in a step):
 * ffa_peer_alloc makes a zeroed device buffer on the current device and its 64-byte inter-process
 * handle; another process of the same box maps it on ITS current device with ffa_peer_open (peer access
 * is enabled by the driver on first use) and unmaps it with ffa_peer_close before the owner frees it
 * with ffa_peer_free. */
int ffa_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64);
int ffa_peer_open(const unsigned char* handle64, void** ptr);
int ffa_peer_close(void* ptr);
int ffa_peer_free(void* ptr);

/*
 * Streaming append for the formats whose scales span the sequence (the incremental update the reference
 * lists as future work, ffa-q2fp8/OPTIMIZATION_NOTES.md:23-27).  K [B, T_new, HKV, 128] of the new tokens
 * is encoded against the scales the cache already has - q2: scale and zero, nf4: scale (absmax), each
 * [B, HKV, 128] in K's dtype, read only - and written into the page slots of positions pos0 .. pos0 +
 * T_new - 1.  Codes saturate at the ends of the existing range; the fp8 residual (k - dequantised code)
 * carries what the code cannot, so refined scores stay as accurate as the fp8 residual allows.  As long
 * as the new tokens stay inside the range the scales were made from, the result is bit-identical to
 * quantising the whole lengthened sequence.  running_minmax (optional) is the scratch buffer a previous
 * ffa_quantize_q2 / ffa_quantize_nf4 call left its per-channel min/max in; the new tokens are folded in,
 * so a caller can see how far the range has drifted and decide to requantise.  scratch: nf4 only,
 * ffa_quantize_scratch_bytes(B, HKV) bytes, distinct from running_minmax.  FFA_K_FP8 / FFA_K_FP4 are
 * accepted too (no statistics).  nvfp4 keeps page-local scales: re-encode the open page with
 * ffa_quantize_nvfp4.
 */
int ffa_quantize_append(int32_t variant, const void* k, int32_t k_dtype, int32_t B, int32_t T_new, int32_t HKV,
                        int32_t fp8_format, uint8_t* codes_pool, const void* scale, const void* zero,
                        uint8_t* residual_pool, void* running_minmax, void* scratch, const int32_t* block_table,
                        int32_t bt_stride, int32_t pos0, ffa_stream_t stream);

/*
 * Appends T_new tokens per sequence to a paged cache: K [B, T_new, HKV, 128] (post-RoPE) is quantised
 * (variant FFA_K_FP8 or FFA_K_FP4, the formats without per-sequence statistics) and its codes and fp8
 * residual are written into the page slots that block_table [B, bt_stride] names for positions
 * pos0 .. pos0 + T_new - 1; V [B, T_new, HKV, 128] (fp16 / bf16) is copied into the same slots of
 * v_pool.  Either of k, v may be NULL (only the other is appended).  Replaces the torch.cat append of
 * ffa-fp8fp8/e2e/fp8fp8_cache.py:74-121 (FP8Fp8DynamicLayer.update).
 */
int ffa_cache_append(int32_t variant, const void* k, const void* v, int32_t dtype, int32_t B, int32_t T_new, int32_t HKV,
                     int32_t fp8_format, uint8_t* codes_pool, uint8_t* residual_pool, void* v_pool,
                     const int32_t* block_table, int32_t bt_stride, int32_t pos0, ffa_stream_t stream);

/*
 * Fused K projection + bias + RoPE (+ quantise and scatter into the cache).  Replaces
 *   kproj_rope_quantize_{triton,fused}   ffa-q2fp8/fused_kproj_rope_q2fp8.py:427-566 (two GEMM passes there)
 *   kproj_rope_fp4_{triton,fused}        ffa-fp4fp8/fused_kproj_rope_fp4fp8.py:415-522
 *   kproj_rope_nf4_{triton,fused}        ffa-nf4fp8/fused_kproj_rope_nf4fp8.py:440-580
 * and the fp8fp8 / nvfp4 variants whose "triton" path in the reference is a torch placeholder
 * (ffa-fp8fp8/fused_kproj_rope_fp8fp8.py:92-113, ffa-nvfp4fp8/fused_kproj_rope_nvfp4fp8.py:143-166).
 * K = rope(h . W_k^T + bias) is computed by one tcgen05 GEMM whose epilogue applies the bias, the
 * rounding to the activation dtype and RoPE; the variant's quantiser then encodes K.
 */
typedef struct FfaKprojArgs {
  int32_t variant;        /* FFA_K_* quantiser to run on K, or -1 to stop after RoPE               */
  int32_t B, T, H, HKV;   /* h is [B, T, H]; H a multiple of 64                                    */
  int32_t head_dim;       /* 128                                                                   */
  int32_t io_dtype;       /* FFA_F16 | FFA_BF16: h, w_k, bias                                      */
  int32_t rope_dtype;     /* FFA_F32 or io_dtype: cos / sin tables; K is produced in promote(io, rope) */
  int32_t fp8_format;     /* FFA_E5M2 | FFA_E4M3                                                   */
  int32_t page_size;      /* nvfp4 scale page                                                      */
  const void* h;          /* [B*T, H]                                                              */
  const void* w;          /* [HKV*128, H] (out, in), contiguous                                    */
  const void* bias;       /* [HKV*128] or NULL                                                     */
  const void* cos;        /* [T, 128]                                                              */
  const void* sin;
  const int32_t* slot_table; /* [B, slot_stride] page ids to scatter token rows into a paged cache, or NULL
                                for the reference layout [B, T, HKV, .]                            */
  int32_t slot_stride;
  int32_t slot_pos0;      /* with slot_table: position in its sequence of token 0 of this call (appending
                             new tokens to a cache); only the elementwise formats (fp8fp8, fp4) accept
                             a non-zero value, the others derive scales from the whole sequence / page */
  void* codes;            /* outputs in the reference layouts (or pool layout with slot_table)     */
  void* scale;
  void* zero;
  void* residual;
  void* k_rope_out;       /* optional [B, T, HKV, 128] post-RoPE K in the promoted dtype           */
  void* workspace;        /* >= ffa_kproj_workspace_bytes(...)                                     */
  size_t workspace_bytes;
} FfaKprojArgs;

int ffa_kproj_rope(const FfaKprojArgs* args, ffa_stream_t stream);
size_t ffa_kproj_workspace_bytes(int32_t B, int32_t T, int32_t HKV, int32_t rope_dtype);

/* Text of the last CUDA runtime error seen by this library on the calling thread ("" if none). */
const char* ffa_last_cuda_error(void);
/* Library version, bumped when the ABI changes (2: FfaDecodeArgs ends in v_mean; FfaKprojArgs.slot_pos0;
 * 3: ffa_static_scratch_status, every SBS in one launch; 4: ffa_cache_append, ffa_quantize_append;
 * 5: SBS 16 / 32, the ffa_peer_* entry points, ffa_decode_peer). */
int ffa_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FFA_B200_H_ */
