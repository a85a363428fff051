// Library-wide state of libffa_b200.so: last CUDA error text and ABI version.
#include <stdio.h>

#include "ffa_common.cuh"

namespace ffa {

static thread_local char g_last_error[256] = "";

int note_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_last_error, sizeof(g_last_error), "%s: %s", where, cudaGetErrorString(e));
  return FFA_E_LAUNCH;
}

}  // namespace ffa

extern "C" const char* ffa_last_cuda_error(void) { return ffa::g_last_error; }
extern "C" int ffa_abi_version(void) { return 5; }   // 5: sub-page prune blocks, peer-memory exchange, ffa_decode_peer
