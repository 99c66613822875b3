// Launch description of the two grouped CTA-pair NVFP4 GEMMs of the MoE layer
// (gemm_pair_moe.cu), used for large batches whose experts quantise the gate
// and up inputs with one scale:
//   gate/up  tokens on the lanes (256 per pair tile: 128 per CTA), the gate rows of a
//            128-channel tile staged by the pair's first CTA and the up rows by its
//            second; GeGLU + FP4 quantisation of the down input in the epilogue
//   down     tokens on the lanes, the quantised activations of a pair tile resident in
//            shared memory while the pair sweeps the 2816 output channels in
//            128-channel tiles with two accumulator stages; BF16 rows out
// Both kernels find their work from the expert offsets themselves (no separate
// descriptor kernel) and clamp offsets that exceed the declared capacity.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "moe_kernels.h"

namespace gw {

struct PairMoeParams {
  CUtensorMap map_tokens;          // quantised token rows [capacity, K/2] (row pitch may exceed K/2), box 128 rows
  const CUtensorMap* map_table;    // kMoeMapsPerExpert maps per expert, in global memory (host written)
  const MoeExpertInfo* experts;    // [128]
  const int32_t* offsets;          // [129] first sorted row of every expert
  const uint8_t* sf_tokens;        // tiled scales of the token rows, expert e's region at row (first/128 + e) * 128
  uint32_t capacity;               // rows the token buffers hold
  // gate/up: packed E2M1 [capacity, 352] + tiled scales (same regions, K = 704), optional BF16 captures
  uint8_t* packed_out;
  uint8_t* scales_out;
  uint8_t* records_out;            // optional: instead of packed_out / scales_out, one 416-byte record per row (352 B of
                                   // E2M1, then the 44 scale bytes in K order) -- what a row's home rank fetches
  void* capture_gate_up;           // optional BF16 [capacity, 1408]
  void* capture_activated;         // optional BF16 [capacity, 704]
  // down: BF16 [capacity, 2816] or per-row destinations
  void* out;
  const uint64_t* row_dest;        // optional: byte address of the home of every sorted row (0 = none)
  uint32_t* error;                 // device error word (0 = fine)
  long long* profile;              // optional [grid][8] cycle counters (tuning aid), normally nullptr
};

// Tuning aid: later launches write per-CTA cycle counters into this device buffer ([2][148][8] int64: the
// gate/up kernel into the first half, the down kernel into the second): [0] producer waiting for a free
// stage, [1] MMA lane waiting for a stage's data, [2] MMA lane issuing, [3] MMA lane waiting for the
// accumulator, [4] an epilogue warp waiting for the accumulator, [5] that warp working, [6] total,
// [7] down: MMA lane waiting for a unit's resident rows.  nullptr switches it off.
void set_pair_moe_profile_buffer(long long* device_buffer);

cudaError_t launch_pair_moe_gate_up(const PairMoeParams& params, int sm_count, cudaStream_t stream);
cudaError_t launch_pair_moe_down(const PairMoeParams& params, int sm_count, cudaStream_t stream);

}  // namespace gw
