// One dense projection Y[rows, n] = bf16(alpha * Xq . Wq^T) on the tcgen05
// kernel: picks the operand roles and tile for the row count, builds the TMA
// descriptors (cached per plan) and launches.
#pragma once

#include "common.cuh"
#include "gemm_tc.cuh"

namespace gw {

// Tuning overrides of the dense projections, read from the environment once per plan (when its
// descriptors are first used), not at every call:
//   GW_DENSE_FORM=swap|direct, GW_DENSE_BLOCK_N=128|256   operand roles / column tile
//   GW_DENSE_NO_PAIR=1    NVFP4 projections with >= 256 rows stay on the single-CTA kernel
//   GW_DENSE_NO_SPLIT=1   decode-shaped plans run whole tiles per CTA
struct DenseTuning {
  char form = 0;            // 's', 'd' or 0
  int block_n = 0;
  bool no_pair = false, no_split = false;
  static DenseTuning from_environment();
};

struct DenseDescriptors {          // re-encoded only when a pointer changes
  DenseTuning tuning = DenseTuning::from_environment();
  const void* weight = nullptr;
  const void* activations = nullptr;
  const void* weight_scales = nullptr;
  CUtensorMap weight_map{}, activation_map{}, weight_scale_map{};
  const void* weight_half = nullptr;
  CUtensorMap weight_half_map{};     // 128-row box over the weights (CTA-pair kernel: each CTA stages half a tile)
  // Split mode: one arrival counter per weight tile, owned by the plan (device memory,
  // zeroed at creation; the kernel leaves every counter at zero again).
  int32_t* split_counters = nullptr;
  cudaError_t allocate_split_counters(uint32_t rows, uint32_t n);
  ~DenseDescriptors();
};

struct DenseProblem {
  GemmKind kind;
  uint32_t rows, k, n;
  const void* weight;              // [n, k] E4M3, [n, k/2] packed E2M1 or [n, k] BF16
  const uint8_t* weight_scales;    // NVFP4 only
  const void* activations;         // quantised [rows, k(/2)], or the BF16 input itself for the BF16 kind
  const uint8_t* activation_scales;
  float alpha;
  const float* channel_alpha;
  void* output;
  uint32_t* error;
  // Optional, decode shapes only: dense_split_bytes() bytes, 256-byte aligned, for FP32
  // partial tiles.  With it (and the plan's counters) the K loop of the weight tiles is
  // divided evenly over the SMs (see GemmParams).
  void* split_workspace = nullptr;
};

// true: weights on the 128-lane operand and tokens on the column operand.
bool dense_uses_swap_form(const DenseTuning& tuning, uint32_t rows);
int dense_block_n(const DenseTuning& tuning, uint32_t rows);

// Bytes of split workspace a projection of this shape can use (0: none).
size_t dense_split_bytes(const DenseTuning& tuning, uint32_t rows, uint32_t n);

gw_status launch_dense(const DenseProblem& problem, DenseDescriptors* cache, cudaStream_t stream);

}  // namespace gw
