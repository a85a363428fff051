// Per-format launchers of the warp-specialised decode kernel; each lives in its own translation unit
// (ffa_decode_ws_<format>.cu) so that the formats compile in parallel.
// maps: coarse tile (64 rows), coarse sample (16 rows), residual, V.
#pragma once

#include <cuda.h>

#include "ffa_decode_shared.cuh"

namespace ffa {

int launch_ws_fp8(const DecodeParams& p, int f8, const CUtensorMap* maps, cudaStream_t stream);
int launch_ws_q2(const DecodeParams& p, int f8, const CUtensorMap* maps, cudaStream_t stream);
int launch_ws_fp4(const DecodeParams& p, int f8, const CUtensorMap* maps, cudaStream_t stream);
int launch_ws_nf4(const DecodeParams& p, int f8, const CUtensorMap* maps, cudaStream_t stream);
int launch_ws_nvfp4(const DecodeParams& p, int f8, const CUtensorMap* maps, cudaStream_t stream);

}  // namespace ffa
