// Sequence-split decode across the GPUs of one box: exchange of the ranks' (O, LSE) partials over
// peer memory, fused with the merge.
//
// Every rank owns a page range of every sequence and produces one partial [rows, 129] (normalised
// output + base-2 LSE per q head).  The library-only way to finish the step is an NCCL all-gather of
// the partials followed by the merge kernel (two launches, about 20 us + 8 us for 66 KB per rank).
// Here each rank instead STORES its partial straight into its slot of every peer's gathered buffer
// (plain peer stores over NVLink; the peers' buffers are mapped through CUDA IPC) and then raises its
// flag on that peer; the merge kernel of a rank waits until all flags carry the current step number and
// merges from its own local copy.  Only ordinary stores and loads are used.
//
// Protocol.  The gathered buffer is double-buffered by step parity and the flags carry the step number,
// so nothing is ever reset: rank r can be at most one step ahead of a peer (its merge of step k + 1
// needs that peer's push of step k + 1, which the peer's stream issues after its own merge of step k),
// hence slot (k mod 2) is rewritten no earlier than step k + 2, after every reader of step k is done.
// Every wait is bounded in wall-clock time (one second); a merge kernel that gives up writes NaN rows and
// sets the status word instead of hanging.
#include <cstring>

#include "ffa_common.cuh"
#include "ffa_decode_shared.cuh"

namespace ffa {
namespace {

constexpr int kMaxPeers = 16;
constexpr unsigned long long kPeerWaitNs = 1000000000ull;   // 1 s

struct PeerPtrs {
  float* gathered[kMaxPeers];   // peer p's buffer [2][world][rows * 129]
  int* flags[kMaxPeers];        // peer p's flags [world]
};

// One CTA per peer: copy this rank's partial into its slot on the peer, then publish the step number.
__global__ void __launch_bounds__(1024) peer_push_kernel(const float* __restrict__ local, int n_floats, int rank, int world,
                                                         int step, PeerPtrs pp) {
  const int peer = blockIdx.x;
  if (peer == rank) {
    // own slot: the decode kernel wrote it in place; only the flag is raised
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      *reinterpret_cast<volatile int*>(pp.flags[peer] + rank) = step;
    }
    return;
  }
  float* dst = pp.gathered[peer] + (static_cast<int64_t>(step & 1) * world + rank) * n_floats;
  const int n4 = n_floats / 4;
  const float4* s4 = reinterpret_cast<const float4*>(local);
  float4* d4 = reinterpret_cast<float4*>(dst);
  for (int i = threadIdx.x; i < n4; i += blockDim.x) d4[i] = s4[i];
  for (int i = 4 * n4 + threadIdx.x; i < n_floats; i += blockDim.x) dst[i] = local[i];
  __threadfence_system();                      // this thread's stores are visible to the peer ...
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    *reinterpret_cast<volatile int*>(pp.flags[peer] + rank) = step;    // ... before the flag is
  }
}

// One CTA per q head row: wait for every rank's flag, then merge the world partials of this step
// (same arithmetic as merge_partials_kernel).
__global__ void __launch_bounds__(kHeadDim) peer_wait_merge_kernel(const float* __restrict__ gathered,
                                                                   const int* __restrict__ flags, int world, int rows,
                                                                   int step, void* out, int out_dtype, int* status) {
  __shared__ int s_ok;
  const int64_t row = blockIdx.x;
  const int c = threadIdx.x;
  if (c == 0) s_ok = 1;
  __syncthreads();
  if (c < world) {
    unsigned long long t0 = 0;
    const volatile int* f = flags + c;
    for (int spin = 0; *f != step; ++spin) {
      if ((spin & 255) == 255) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > kPeerWaitNs) { s_ok = 0; break; }
      }
    }
    __threadfence_system();                    // the partial behind the flag is read after the flag
  }
  __syncthreads();
  if (!s_ok) {
    if (c == 0 && status) atomicCAS(status, 0, 3);
    store_from_float(out, row * kHeadDim + c, out_dtype, __int_as_float(0x7fc00000));
    return;
  }
  const float* parts = gathered + static_cast<int64_t>(step & 1) * world * rows * 129;
  float top = -INFINITY;
  for (int r = 0; r < world; ++r) top = fmaxf(top, __ldcv(parts + (static_cast<int64_t>(r) * rows + row) * 129 + 128));
  float den = 0.f, num = 0.f;
  if (top != -INFINITY) {
    for (int r = 0; r < world; ++r) {
      const float* pr = parts + (static_cast<int64_t>(r) * rows + row) * 129;
      const float lse = __ldcv(pr + 128);
      if (lse == -INFINITY) continue;
      const float w = exp2f(lse - top);
      den += w;
      num += w * __ldcv(pr + c);
    }
  }
  store_from_float(out, row * kHeadDim + c, out_dtype, den == 0.f ? 0.f : num / den);
}

}  // namespace
}  // namespace ffa

using namespace ffa;

extern "C" int ffa_peer_exchange_merge(const float* local_partial, int32_t rows, int32_t rank, int32_t world,
                                       float* const* peer_gathered, int32_t* const* peer_flags, int32_t step, void* out,
                                       int32_t out_dtype, int32_t* status, ffa_stream_t stream_) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  if (!local_partial || !peer_gathered || !peer_flags || !out) return FFA_E_NULL;
  if (rows <= 0 || world <= 0 || world > kMaxPeers || rank < 0 || rank >= world || step <= 0) return FFA_E_SHAPE;
  if (out_dtype < FFA_F16 || out_dtype > FFA_F32) return FFA_E_DTYPE;
  PeerPtrs pp{};
  for (int p = 0; p < world; ++p) {
    if (!peer_gathered[p] || !peer_flags[p]) return FFA_E_NULL;
    pp.gathered[p] = peer_gathered[p];
    pp.flags[p] = peer_flags[p];
  }
  const int n_floats = rows * 129;
  peer_push_kernel<<<world, 1024, 0, st>>>(local_partial, n_floats, rank, world, step, pp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return note_cuda_error(e, "peer_push launch");
  peer_wait_merge_kernel<<<static_cast<unsigned>(rows), kHeadDim, 0, st>>>(pp.gathered[rank], pp.flags[rank], world, rows,
                                                                          step, out, out_dtype, status);
  e = cudaGetLastError();
  return e == cudaSuccess ? FFA_OK : note_cuda_error(e, "peer_wait_merge launch");
}

extern "C" int ffa_peer_wait_merge(const float* gathered_local, const int32_t* flags_local, int32_t world, int32_t rows,
                                   int32_t step, void* out, int32_t out_dtype, int32_t* status, ffa_stream_t stream_) {
  if (!gathered_local || !flags_local || !out) return FFA_E_NULL;
  if (rows <= 0 || world <= 0 || world > kMaxPeers || step <= 0) return FFA_E_SHAPE;
  if (out_dtype < FFA_F16 || out_dtype > FFA_F32) return FFA_E_DTYPE;
  peer_wait_merge_kernel<<<static_cast<unsigned>(rows), kHeadDim, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      gathered_local, flags_local, world, rows, step, out, out_dtype, status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? FFA_OK : note_cuda_error(e, "peer_wait_merge launch");
}

// ---- set-up: a buffer other processes of the box can map ---------------------------------------------
extern "C" int ffa_peer_alloc(size_t bytes, void** ptr, unsigned char* handle64) {
  if (!ptr || !handle64 || bytes == 0) return FFA_E_NULL;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e != cudaSuccess) return note_cuda_error(e, "cudaMalloc(peer buffer)");
  e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return note_cuda_error(e, "cudaIpcGetMemHandle");
  }
  memcpy(handle64, &h, 64);
  *ptr = p;
  return FFA_OK;
}

extern "C" int ffa_peer_open(const unsigned char* handle64, void** ptr) {
  if (!ptr || !handle64) return FFA_E_NULL;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? FFA_OK : note_cuda_error(e, "cudaIpcOpenMemHandle");
}

extern "C" int ffa_peer_close(void* ptr) {
  if (!ptr) return FFA_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? FFA_OK : note_cuda_error(e, "cudaIpcCloseMemHandle");
}

extern "C" int ffa_peer_free(void* ptr) {
  if (!ptr) return FFA_OK;
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? FFA_OK : note_cuda_error(e, "cudaFree(peer buffer)");
}
