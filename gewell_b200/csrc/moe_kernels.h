// Internal launch functions of the MoE routing / permutation / quantise /
// combine kernels (moe_kernels.cu).
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

#include "gemm_tc.cuh"

namespace gw {

// Static per-expert data the device kernels need; built once when the expert
// table is bound.  Index 0 gate, 1 up, 2 down.
struct MoeExpertInfo {
  const uint8_t* scales[3];        // tiled E4M3 weight scales
  float alpha[3];                  // fmul_rn(input_scale, weight_scale)
  float inverse_input_scale[3];    // 1 / input_scale (IEEE division)
  int32_t pad_;
};

enum { kMoeFormSwap = 0, kMoeFormDirect = 1, kMoeFormFused = 2 };

// Everything the group-descriptor kernel needs (all pointers on the device).
struct MoeGroupPlan {
  const int32_t* offsets;          // [129]
  const MoeExpertInfo* experts;    // [128]
  const uint8_t* scales_in;        // scale storage of the packed gate/up input
  const uint8_t* scales_act;       // scale storage of the packed down input
  uint32_t n;                      // sorted rows (8 * tokens)
  uint32_t scale_rows;             // rows of one part of the scale storage
  int form;                        // kMoeForm*
  int block_n_first;               // column tile of the gate/up GEMM
  int block_n_down;                // column tile of the down GEMM
  int shared_gate_up;              // gate and up read one quantised copy of the input
  uint32_t* error;                 // device error word: offsets beyond n are clamped and reported here
};

uint32_t moe_chunks(uint32_t rows);

cudaError_t launch_moe_dispatch(const void* scores, const void* expert_scales, uint32_t rows, int32_t* keys,
                                float* weights, uint32_t* bitmaps, int32_t* chunk_counts, int32_t* offsets,
                                int32_t* sorted_assignments, int32_t* sorted_keys, int32_t* inverse,
                                cudaStream_t stream);
cudaError_t launch_moe_keys_from_offsets(const int32_t* offsets, uint32_t first_expert, uint32_t expert_count,
                                         uint32_t rows, int32_t* sorted_keys, int32_t* full_offsets,
                                         cudaStream_t stream);
cudaError_t launch_moe_prepare_groups(const MoeGroupPlan& plan, GemmGroup* first_groups, GemmGroup* down_groups,
                                      cudaStream_t stream);
// gather_index != nullptr: sorted row i reads input row gather_index[i] / gather_divisor.
cudaError_t launch_moe_quantize_input(const void* input, const int32_t* gather_index, uint32_t gather_divisor,
                                      const int32_t* sorted_keys, const int32_t* offsets,
                                      const MoeExpertInfo* experts, uint32_t n, uint32_t scale_rows, int parts,
                                      uint8_t* packed, uint8_t* scales, cudaStream_t stream);
// Token-major form of the same quantisation for the whole-layer path: reads each token once and
// writes its eight copies at inverse[8 t + slot].
cudaError_t launch_moe_quantize_tokens(const void* input, const int32_t* keys, const int32_t* inverse,
                                       const int32_t* offsets, const MoeExpertInfo* experts, uint32_t tokens,
                                       uint32_t scale_rows, int parts, uint8_t* packed, uint8_t* scales,
                                       cudaStream_t stream);
cudaError_t launch_moe_activate_quantize(const void* gate_up, const int32_t* sorted_keys, const int32_t* offsets,
                                         const MoeExpertInfo* experts, uint32_t n, uint32_t scale_rows, uint8_t* packed,
                                         uint8_t* scales, void* activated, cudaStream_t stream);
cudaError_t launch_moe_combine(const void* down, const int32_t* inverse, const float* weights, uint32_t rows,
                               uint32_t width, void* output, cudaStream_t stream);
cudaError_t launch_gather_rows(const void* input, const int32_t* index, uint32_t divisor, uint32_t rows,
                               uint32_t width, void* output, cudaStream_t stream);


// Expert parallelism over peer memory: 1584-byte records (1408 B packed E2M1 + 176 scale bytes).
constexpr uint32_t kEpRecordBytes = 1584;
cudaError_t launch_ep_dispatch(const void* input, const int32_t* keys, const int32_t* inverse, const int32_t* offsets,
                               const float* inverse_input_scale, const int32_t* dest_rank, const int32_t* dest_row0,
                               void* const* peer_records, uint32_t tokens, uint32_t capacity_rows, uint32_t* error,
                               cudaStream_t stream);
cudaError_t launch_ep_tables(const int32_t* counts, const int32_t* physical, uint32_t rank, uint32_t world,
                             int32_t* dest_row0, int32_t* local_offsets, int32_t* segment_start, int32_t* home_base,
                             cudaStream_t stream);
cudaError_t launch_ep_row_home(const int32_t* sorted_keys, const int32_t* offsets, const int32_t* segment_start,
                               const int32_t* home_base, void* const* peer_returned, uint32_t first_expert,
                               uint32_t per_rank, uint32_t world, uint32_t n, uint32_t home_capacity_rows,
                               uint32_t* error, uint64_t* row_home, cudaStream_t stream);
cudaError_t launch_ep_retile_scales(const void* records, const int32_t* sorted_keys, const int32_t* offsets,
                                    uint32_t n, uint8_t* scales, cudaStream_t stream);
cudaError_t launch_ep_combine(const int32_t* keys, const int32_t* inverse, const float* weights,
                              const int32_t* offsets, const int32_t* dest_rank, const int32_t* dest_row0,
                              void* const* peer_down, uint32_t rows, uint32_t capacity_rows, uint32_t* error,
                              void* output, cudaStream_t stream);

}  // namespace gw
