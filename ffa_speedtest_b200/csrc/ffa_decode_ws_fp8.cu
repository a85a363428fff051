// Warp-specialised decode kernel, instantiated for the FFA_K_FP8 coarse format.
#include "ffa_decode_ws.cuh"
#include "ffa_decode_ws_launch.h"

namespace ffa {

int launch_ws_fp8(const DecodeParams& p, int f8, const CUtensorMap* maps, cudaStream_t stream) {
  return launch_ws_fmt_impl<FFA_K_FP8>(p, f8, maps, stream);
}

}  // namespace ffa
