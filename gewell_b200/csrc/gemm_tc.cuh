// Host-visible description of one launch of the tcgen05 GEMM kernel.
//
// The tensor core sees two K-major operands:
//   L  the "lane" operand: 128 rows per tile, one row per TMEM lane
//   C  the "column" operand: BLOCK_N rows per tile, one row per TMEM column
//      (loaded as 1 or 2 boxes of <=128 rows, which may come from two
//      different matrices: the gate and up weights of an expert)
// and accumulates D[l, c] = sum_k L[l, k] * C[c, k] in TMEM.  Which of weights /
// activations plays which role is the caller's choice:
//   * "swap" form (decode, small batches): L = weights, C = tokens.  The token
//     tile only needs a multiple of 16 valid rows, so 1..64-row batches and
//     ragged expert groups cost no padding to 128.
//   * "direct" form (prefill): L = tokens, C = weights.  Every epilogue thread
//     owns one token row and sees consecutive output channels, so stores are
//     16-byte vectors and GeGLU + FP4 quantisation fuse into the epilogue.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <string>

namespace gw {

struct GemmGroup {
  // lane operand
  const uint8_t* sf_l;        // tiled E4M3 scales of L (NVFP4), row 0 = the group's first 128-row block
  int32_t map_l;              // index into GemmParams::map_table, or -1 for GemmParams::map_l
  int32_t l_row0;             // first row of the group inside the L tensor map
  int32_t l_rows;             // valid rows (lanes beyond are masked in the epilogue)
  int32_t l_tiles;            // number of 128-row tiles
  // column operand: `halves` boxes of (BLOCK_N / halves) rows each
  const uint8_t* sf_c[2];     // tiled scales of each half's matrix, row 0 = the group's first 128-row block
  int32_t map_c[2];           // tensor maps of the halves (-1 = GemmParams::map_c)
  int32_t c_row0;             // first row of the group inside the C tensor map(s)
  int32_t c_rows;             // valid rows per matrix (columns beyond are masked)
  int32_t c_tiles;            // number of column tiles
  int32_t c_half_stride;      // row offset of half 1 relative to half 0 inside one matrix (0: separate matrices)
  int32_t sf_c_sub;           // swap form, BLOCK_N < 128: the group's first C row modulo 128 (multiple of 32)
  // epilogue
  float alpha[2];             // multiplier of the accumulator (per half)
  const float* channel_alpha; // optional per-output-channel multipliers (FP8 joined projections)
  float quant_inverse_scale;  // GeGLU+quantise epilogue: 1 / input_scale of the consumer
  int32_t out_row0;           // first output row
  int32_t out_col0;           // first output column
  int32_t sf_out_row0;        // GeGLU+quantise epilogue: first row of the group's output scale region
  int32_t work_begin;         // index of the group's first work item (prefix sum)
};

struct GemmParams {
  CUtensorMap map_l;              // used when a group says map_l == -1
  CUtensorMap map_c;              // used when a group says map_c[h] == -1
  CUtensorMap map_sfc;            // c_single_box: scale atoms of the C operand's matrix (NVFP4)
  int32_t c_single_box;           // BLOCK_N 256, groups == nullptr: map_c has a 256-row box over one matrix
  const CUtensorMap* map_table;   // per-group operands in global memory (host written)
  const GemmGroup* groups;        // num_groups + 1 entries in global memory, or nullptr
  GemmGroup single;               // the only group when groups == nullptr
  int32_t num_groups;
  int32_t total_work;             // work items when groups == nullptr
  int32_t k;                      // reduction length in elements
  int32_t c_rows_per_tile;        // rows of one matrix covered by one column tile
  void* out;                      // BF16 output (swap/direct), packed E2M1 output (GeGLU+quantise)
  int64_t ld_out;                 // elements (bytes for the packed output) between output rows
  const uint64_t* row_dest;       // direct store, optional: byte address of the start of every output row
                                  // (indexed like rows of `out`); rows may live in other GPUs' memory
  uint8_t* out_scales;            // GeGLU+quantise: tiled scale storage of the output
  int32_t out_width;              // GeGLU+quantise: logical width (K of the consumer)
  void* capture_gate_up;          // GeGLU+quantise: optional BF16 [rows, 2*out_width]
  void* capture_activated;        // GeGLU+quantise: optional BF16 [rows, out_width]
  // Split mode (swap form, groups == nullptr): work is divided into equal ranges of
  // (tile, K stage) units; partial tiles are summed through these buffers.
  float* split_partials;          // [2 * grid][128 * BLOCK_N] FP32, or nullptr (whole tiles per CTA)
  int32_t* split_counters;        // [work items], zero at launch; left zero by the kernel
  int32_t work_chunk;             // consecutive work items a CTA takes before it strides on (0 or 1: one)
  int32_t early_weights;          // swap form, groups == nullptr: the L operand (weights, weight scales) does not
                                  // depend on the previous kernel in the stream, so its first copies may be
                                  // issued before that kernel has finished (programmatic dependent launch)
  uint32_t* error;                // device error word (0 = fine)
  long long* profile;             // optional [grid][8] cycle counters (debug aid), normally nullptr
};

// nvfp4: E2M1 with E4M3 K16 block scales (kind::mxf4nvf4); fp8: E4M3 (kind::f8f6f4); bf16: BF16 (kind::f16).
// All accumulate in FP32 in tensor memory.
enum class GemmKind { nvfp4, fp8, bf16 };
enum class GemmEpilogue { swap_store, direct_store, geglu_quant };

// swap_store: block_n in {32, 64, 128}; direct_store: {128, 256}; geglu_quant: 256 (NVFP4).
cudaError_t launch_gemm_tc(GemmKind kind, GemmEpilogue epilogue, int block_n, const GemmParams& params, int grid,
                           cudaStream_t stream);

// Ring stages of one work item's K loop (row_bytes = bytes of K per operand row): the unit in which the
// split mode divides a launch over the CTAs.
int gemm_tc_k_stages(GemmKind kind, GemmEpilogue epilogue, uint64_t row_bytes);

// Debug aid: subsequent launches write per-CTA cycle counters ([2][148][8] int64:
// producer wait, MMA wait for data, MMA issue, MMA wait for accumulator, epilogue
// wait, epilogue work, total, epilogue TMEM-load time) into this device buffer; nullptr turns it off.
void set_gemm_profile_buffer(long long* device_buffer);

// Host helper: 2-D byte tensor map {inner = row_bytes, outer = rows} with a
// 128-byte x box_rows box and the 128-byte swizzle.  pitch_bytes (0 = row_bytes)
// is the distance between rows in memory.
bool encode_tensor_map_2d(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows,
                          uint32_t box_rows, std::string* error, uint64_t pitch_bytes = 0);

// Host helper: tiled NVFP4 scale storage ([row blocks][K/64 atoms of 512 bytes]) as a 2-D map of
// 8-byte words with a box of 4 atoms x box_row_blocks.
bool encode_tensor_map_scales(CUtensorMap* map, const void* base, uint64_t k_atoms, uint64_t row_blocks,
                              uint32_t box_row_blocks, std::string* error);

}  // namespace gw
