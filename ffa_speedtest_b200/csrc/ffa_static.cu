// ffa_decode_static_scratch: the decode step for callers that cannot hand over scratch memory.
//
// Some hosts of this library have no way to allocate device memory at the point where they call a
// decode step: a plug-in inside a serving process whose device memory is owned and fully
// pre-partitioned by the host application, a latency-critical loop in which cudaMalloc is banned
// because it synchronises the whole device and can fail under fragmentation, or a binding from a
// language runtime that only passes through the tensors it was given.  ffa_decode() needs a
// workspace for its per-range partial results; this variant keeps that workspace in a fixed array
// that is part of the library image, so the caller passes inputs and outputs only.
//
// What that costs and what to watch for:
//   * every GPU on which the library is loaded carries the array (FFA_STATIC_SCRATCH_BYTES) until
//     the process exits, whether or not this entry point is ever used;
//   * decode shapes whose workspace does not fit are refused with FFA_E_LIMIT, nothing is launched;
//   * the first call on each device looks up the device address of the array (one
//     cudaGetSymbolAddress with that device current).  Make that first call outside any stream
//     capture; later calls do no set-up;
//   * all calls on a device share the one array and each call leaves its partial results behind.
//     The parts that must start from zero - the status word the kernels can set and the arrival
//     counters at the head of the workspace - are cleared on the stream at the start of every call;
//     everything else is overwritten before it is read.
//     Two calls whose kernels overlap on the GPU (different streams without an ordering between
//     them, or concurrent host threads on one device) would race on the array: serialise them.
//   * the status word a kernel sets when one of its bounded waits gave up (the outputs of the heads it
//     touched are then NaN) lives in that array too and is cleared by the next call: a caller that
//     wants to see it enqueues ffa_static_scratch_status() right after the decode call;
//   * no cudaMalloc, cudaFree or other allocating routine is called, here or in ffa_decode().
#include <mutex>

#include "ffa_common.cuh"

namespace {

// In host code the name of a __device__ array is only a handle for the runtime; its device address
// has to be asked for (cudaGetSymbolAddress) and is different on every device.
static __device__ __align__(256) unsigned char g_static_scratch[FFA_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// Device address of the array on the current device; resolved once per device.
int static_scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return ffa::note_cuda_error(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return FFA_E_LIMIT;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return ffa::note_cuda_error(e, "cudaGetSymbolAddress(static scratch)");
    if (!ptr) return FFA_E_NULL;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return FFA_OK;
}

}  // namespace

extern "C" size_t ffa_static_scratch_bytes(void) { return FFA_STATIC_SCRATCH_BYTES; }

extern "C" int ffa_decode_static_scratch(const FfaDecodeArgs* args, ffa_stream_t stream) {
  if (!args) return FFA_E_NULL;
  const size_t need = ffa_decode_workspace_bytes(args->B, args->T, args->HQ, args->HKV, args->pages_per_chunk);
  if (need == 0) return FFA_E_SHAPE;
  if (need > FFA_STATIC_SCRATCH_BYTES) return FFA_E_LIMIT;     // too large for the built-in array
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != FFA_OK) return rc;
  // the first 64 KiB of the workspace hold the arrival counters (one int per batch x kv-head) and,
  // in their last 256 bytes, the status word: all of it has to read zero when the kernel starts
  cudaError_t e = cudaMemsetAsync(scratch, 0, 64 * 1024, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return ffa::note_cuda_error(e, "cudaMemsetAsync(static scratch)");
  FfaDecodeArgs local = *args;
  local.workspace = scratch;
  local.workspace_bytes = need;
  return ffa_decode(&local, stream);
}


// Copies the status block of the last ffa_decode_static_scratch() call on the current device (seven
// ints: [0] = 1 if a bounded wait gave up, then where) to `out`, which may be device memory or pinned
// host memory; enqueued on `stream`, so it reads what the decode call before it on that stream left.
extern "C" int ffa_static_scratch_status(int32_t* out, ffa_stream_t stream) {
  if (!out) return FFA_E_NULL;
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != FFA_OK) return rc;
  cudaError_t e = cudaMemcpyAsync(out, static_cast<unsigned char*>(scratch) + 64 * 1024 - 256, 7 * sizeof(int32_t),
                                  cudaMemcpyDefault, reinterpret_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? FFA_OK : ffa::note_cuda_error(e, "cudaMemcpyAsync(static scratch status)");
}
