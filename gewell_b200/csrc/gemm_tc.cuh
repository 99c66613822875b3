// Host-visible description of one launch of the tcgen05 GEMM kernel.
//
// The kernel computes, for every group g,
//     D_g[a_row, b_row] = sum_k A_g[a_row, k] * B[b_row0_g + b_row, k]
// with A on the 128-lane side of the tensor core (TMEM lanes = rows of A) and
// B on the column side (TMEM columns = rows of B), and writes
//     out[(out_row0_g + b_row) * ld_out + out_col0_g + a_row] = bf16(D * alpha).
// Used with A = weights [N_out, K] and B = activations [tokens, K] this is the
// "swap-AB" form Y = X W^T: the token count only has to be a multiple of 16
// per tile (ragged expert groups and 1..64-row decode batches cost no padding
// to 128) while weight rows stream through the 128-lane operand.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <string>

namespace gw {

struct GemmGroup {
  const uint8_t* sf_a;         // tiled E4M3 scales of this group's A matrix (NVFP4 only)
  const float* channel_alpha;  // optional multiplier per A row (FP8 joined projections)
  float alpha;                 // scalar multiplier (used when channel_alpha == nullptr)
  int32_t map_a;               // index into GemmParams::map_a_table, or -1 for GemmParams::map_a
  int32_t a_tiles;             // number of 128-row tiles of A
  int32_t a_rows;              // valid rows of A (output channels)
  int32_t b_row0;              // first row of the group inside the B tensor map
  int32_t b_rows;              // valid rows of B (tokens) in the group
  int32_t sfb_row0;            // first row of the group's region in B's scale storage (multiple of 128)
  int32_t out_row0;            // first output row of the group
  int32_t out_col0;            // first output column of the group
  int32_t work_begin;          // index of the group's first work item (prefix sum)
  int32_t pad_;
};

struct GemmParams {
  CUtensorMap map_a;               // A operand when the group says map_a == -1
  CUtensorMap map_b;               // B operand (box height = BLOCK_N rows)
  const CUtensorMap* map_a_table;  // per-group A operands in global memory (host written)
  const GemmGroup* groups;         // num_groups + 1 entries in global memory, or nullptr
  GemmGroup single;                // the only group when groups == nullptr
  int32_t num_groups;
  int32_t total_work;              // work items when groups == nullptr
  const uint8_t* sf_b;             // tiled E4M3 scales of B (NVFP4 only)
  int32_t k;                       // reduction length in elements
  void* out;                       // BF16
  int64_t ld_out;                  // elements between output rows
  uint32_t* error;                 // device error word (0 = fine)
};

enum class GemmKind { nvfp4, fp8 };

// block_n in {32, 64, 128, 256}.  Returns cudaErrorInvalidValue for others.
cudaError_t launch_gemm_tc(GemmKind kind, int block_n, const GemmParams& params, int grid,
                           cudaStream_t stream);
// Dynamic shared memory the launch will request (for occupancy reasoning/tests).
size_t gemm_tc_smem_bytes(GemmKind kind, int block_n);

// Host helper: 2-D byte tensor map {inner = row_bytes, outer = rows} with a
// 128-byte x box_rows box and the 128-byte swizzle.
bool encode_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows,
                          uint32_t box_rows, std::string* error);

}  // namespace gw
