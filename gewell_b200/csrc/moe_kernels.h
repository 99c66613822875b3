// Internal launch functions of the MoE routing / permutation / quantise /
// combine kernels (moe_kernels.cu).
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

#include "../../include/gewell_b200.h"
#include "gemm_tc.cuh"

namespace gw {

// Tensor maps per expert in the table: [0..2] gate, up, down as NVFP4 (128-row boxes), [3] down as NVFP4
// with 64-row boxes, [4..6] gate, up, down in their 8/16-bit form: the FP8 matrix, the BF16 matrix, or
// the BF16 copy of an NVFP4 matrix (W4A16).
constexpr int kMoeMapsPerExpert = 7;

// How a projection's GEMM runs: which tcgen05 kind, which operand preparation.
enum { kMoeKindNvfp4 = 0, kMoeKindBf16 = 1, kMoeKindFp8 = 2, kMoeKindNone = 3 };

// Static per-expert data the device kernels need; built once when the expert
// table is bound.  Index 0 gate, 1 up, 2 down.
struct MoeExpertInfo {
  const uint8_t* scales[3];        // NVFP4: tiled E4M3 weight scales
  const float* channel_alpha[3];   // FP8: optional per-output-channel multipliers (input * weight scale)
  float alpha[3];                  // fmul_rn(input_scale, weight_scale); 1 for BF16
  float inverse_input_scale[3];    // 1 / input_scale (IEEE division); 1 for BF16
  int32_t storage[3];              // GW_STORAGE_* of the projection (GW_STORAGE_ABSENT: lives on another rank)
  int32_t bf16_copy;               // NVFP4 projections also have BF16 copies behind maps [4..6]
};

// The kind a projection runs as: NVFP4 weights take FP4 activations (W4A4) or, with fp4 == 0, their
// BF16 copies take BF16 activations (W4A16); BF16 and FP8 weights run as what they are.
__host__ __device__ inline int moe_effective_kind(int storage, int fp4) {
  if (storage == GW_STORAGE_NVFP4_W4A4) return fp4 ? kMoeKindNvfp4 : kMoeKindBf16;
  if (storage == GW_STORAGE_BF16) return kMoeKindBf16;
  if (storage == GW_STORAGE_FP8_W8A8) return kMoeKindFp8;
  return kMoeKindNone;
}

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
  int kind;                        // kMoeKind*: only projections that run as this kind get work
  int fp4;                         // NVFP4 weights run with FP4 activations (else as BF16 copies)
};

uint32_t moe_chunks(uint32_t rows);

cudaError_t launch_moe_dispatch(const void* scores, const void* expert_scales, uint32_t rows, int32_t* keys,
                                float* weights, uint32_t* bitmaps, int32_t* chunk_counts, int32_t* offsets,
                                int32_t* sorted_assignments, int32_t* sorted_keys, int32_t* inverse,
                                uint32_t* barrier_state, uint32_t* error, int sm_count, bool one_launch,
                                cudaStream_t stream);
// barrier_state: two zero-initialised uint32 in device memory owned by the workspace (counter, generation)
// for the grid-wide barrier of the one-launch form; one_launch == false keeps the three-launch form.
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
// FP8 expert inputs: row r (sorted) of part p is e4m3_sat(x * 1 / input_scale of expert(r)'s projection
// first_projection + p); source rows through gather_index / gather_divisor like the NVFP4 quantiser.
cudaError_t launch_moe_quantize_fp8(const void* input, const int32_t* gather_index, uint32_t gather_divisor,
                                    const int32_t* sorted_keys, const int32_t* offsets, const MoeExpertInfo* experts,
                                    uint32_t n, uint32_t width, int first_projection, int parts, uint8_t* packed,
                                    cudaStream_t stream);
// GeGLU alone: gate_up BF16 [n, 1408] -> activated BF16 [n, 704] (moe.cu:439-445).
cudaError_t launch_moe_activate(const void* gate_up, const int32_t* offsets, uint32_t n, void* activated,
                                cudaStream_t stream);
cudaError_t launch_moe_combine(const void* down, const int32_t* inverse, const float* weights, uint32_t rows,
                               uint32_t width, void* output, cudaStream_t stream);
cudaError_t launch_gather_rows(const void* input, const int32_t* index, uint32_t divisor, uint32_t rows,
                               uint32_t width, void* output, cudaStream_t stream);


// Expert parallelism over peer memory: 1584-byte records (1408 B packed E2M1 + 176 scale bytes).
constexpr uint32_t kEpRecordBytes = 1584;
// activation record of the down-at-home exchange: 352 B of E2M1, 44 scale bytes in K order, padded to 16 bytes
constexpr uint32_t kEpActivationRecordBytes = 416;
cudaError_t launch_ep_dispatch(const void* input, const int32_t* keys, const int32_t* inverse, const int32_t* offsets,
                               const float* inverse_input_scale, const int32_t* dest_rank, const int32_t* dest_row0,
                               void* const* peer_records, uint32_t tokens, uint32_t capacity_rows, uint32_t* error,
                               cudaStream_t stream);
cudaError_t launch_ep_export_activations(const void* packed, const uint8_t* scales, const int32_t* sorted_keys,
                                         const int32_t* offsets, uint32_t rows, void* records, cudaStream_t stream);
cudaError_t launch_ep_import_activations(const int32_t* keys, const int32_t* inverse, const int32_t* offsets,
                                         const int32_t* dest_rank, const int32_t* dest_row0, void* const* peer_records,
                                         uint32_t assignments, uint32_t capacity_rows, uint32_t* error, void* packed,
                                         uint8_t* scales, cudaStream_t stream);
// Small all-to-all exchange + barrier over peer memory (see ep_exchange_kernel).
constexpr size_t kEpMailboxBytes = 2 * 8 * 1024;
constexpr uint32_t kEpMailboxMaxInts = (1024 - 16) / 4;
cudaError_t launch_ep_exchange(const int32_t* payload, uint32_t count, void* const* mailboxes, uint32_t rank,
                               uint32_t world, uint32_t* epoch_counter, int32_t* gathered, uint32_t* error,
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
