// Launch description of the CTA-pair NVFP4 prefill GEMM (gemm_pair.cu):
// Y[rows, n] = bf16(alpha * Xq . Wq^T), tokens on the lanes (256 per pair tile),
// weights on the columns (256 per tile, 128 staged by each CTA of the pair).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace gw {

struct PairGemmParams {
  CUtensorMap map_tokens;          // packed activations [rows, k/2], box 128 rows x 128 bytes, 128-byte swizzle
  CUtensorMap map_weights;         // packed weights [n, k/2], same box
  CUtensorMap map_weight_scales;   // tiled weight scales as [row blocks][k/64 atoms] of 8-byte words, box 4 atoms x 2
  const uint8_t* sf_tokens;        // tiled activation scales
  int32_t token_row_blocks;        // 128-row blocks the activation scale storage holds
  int32_t k, rows, n;
  int32_t l_tiles, c_tiles;        // 256-token tiles, 256-channel tiles
  void* out;                       // BF16 [rows, ld_out]
  int64_t ld_out;
  float alpha;
  uint32_t* error;                 // device error word (0 = fine)
  long long* profile;              // optional [grid][8] cycle counters (debug aid)
};

// Debug aid: later launches write per-CTA cycle counters into this device buffer, eight per CTA:
// [0] producer waiting for an empty stage, [2] MMA lane waiting for the scale-ready barrier, [3] MMA lane
// issuing (blocked while the tensor pipe is busy), [4] MMA lane waiting for the accumulator, [5] scale
// loader copying, [6] total, [7] scale loader between its copy and its arrival (operand wait).
void set_pair_profile_buffer(long long* device_buffer);

cudaError_t launch_gemm_pair(const PairGemmParams& params, int sm_count, cudaStream_t stream);

}  // namespace gw
