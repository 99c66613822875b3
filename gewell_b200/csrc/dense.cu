#include "dense.h"
#include "gemm_pair.h"

#include <cstdlib>
#include <string>

namespace gw {

DenseTuning DenseTuning::from_environment() {
  DenseTuning tuning;
  if (const char* forced = std::getenv("GW_DENSE_FORM")) tuning.form = forced[0];
  if (const char* forced = std::getenv("GW_DENSE_BLOCK_N")) tuning.block_n = std::atoi(forced);
  tuning.no_pair = std::getenv("GW_DENSE_NO_PAIR") != nullptr;
  tuning.no_split = std::getenv("GW_DENSE_NO_SPLIT") != nullptr;
  return tuning;
}

bool dense_uses_swap_form(const DenseTuning& tuning, uint32_t rows) {
  if (tuning.form == 's' && rows <= 128) return true;
  if (tuning.form == 'd') return false;
  return rows <= 128;
}

int dense_block_n(const DenseTuning& tuning, uint32_t rows) {
  if (dense_uses_swap_form(tuning, rows)) return rows <= 32 ? 32 : rows <= 64 ? 64 : 128;
  if (tuning.block_n == 128 || tuning.block_n == 256) return tuning.block_n;
  return 256;
}

namespace {
size_t split_counter_bytes(const DenseTuning& tuning, uint32_t rows, uint32_t n) {
  const int block_n = dense_block_n(tuning, rows);
  const size_t tiles = size_t((n + 127) / 128) * ((rows + block_n - 1) / block_n);
  return align_up(tiles * sizeof(int32_t), 256);
}
}  // namespace

size_t dense_split_bytes(const DenseTuning& tuning, uint32_t rows, uint32_t n) {
  (void)n;
  if (!dense_uses_swap_form(tuning, rows) || tuning.no_split) return 0;
  return size_t(2) * sm_count() * 128 * dense_block_n(tuning, rows) * sizeof(float);
}

cudaError_t DenseDescriptors::allocate_split_counters(uint32_t rows, uint32_t n) {
  if (dense_split_bytes(tuning, rows, n) == 0) return cudaSuccess;
  const size_t bytes = split_counter_bytes(tuning, rows, n);
  cudaError_t status = cudaMalloc(&split_counters, bytes);
  if (status == cudaSuccess) status = cudaMemset(split_counters, 0, bytes);
  return status;
}

DenseDescriptors::~DenseDescriptors() {
  if (split_counters != nullptr) cudaFree(split_counters);
}

gw_status launch_dense(const DenseProblem& q, DenseDescriptors* cache, cudaStream_t stream) {
  const DenseTuning& tuning = cache->tuning;
  const bool swap = dense_uses_swap_form(tuning, q.rows);
  const int block_n = dense_block_n(tuning, q.rows);
  const bool fp4 = q.kind == GemmKind::nvfp4;
  const uint64_t row_bytes = fp4 ? q.k / 2 : (q.kind == GemmKind::bf16 ? uint64_t(2) * q.k : q.k);
  std::string error;
  const bool single_box = !swap && block_n == 256;   // both column halves come from the one weight matrix
  if (cache->weight != q.weight) {
    if (!encode_tensor_map_2d(&cache->weight_map, q.weight, row_bytes, q.n, single_box ? 256 : 128, &error))
      return fail(GW_CUDA_ERROR, "weight descriptor: " + error);
    cache->weight = q.weight;
  }
  if (single_box && fp4 && cache->weight_scales != q.weight_scales) {
    if (!encode_tensor_map_scales(&cache->weight_scale_map, q.weight_scales, q.k / 64, (q.n + 127) / 128, 2, &error))
      return fail(GW_CUDA_ERROR, "weight scale descriptor: " + error);
    cache->weight_scales = q.weight_scales;
  }
  if (cache->activations != q.activations) {
    if (!encode_tensor_map_2d(&cache->activation_map, q.activations, row_bytes, q.rows, swap ? block_n : 128, &error))
      return fail(GW_CUDA_ERROR, "activation descriptor: " + error);
    cache->activations = q.activations;
  }
  // NVFP4 prefill: the CTA-pair kernel (each CTA stages half of the weight tile) unless disabled
  if (fp4 && single_box && q.rows >= 256 && !tuning.no_pair) {
    if (cache->weight_half != q.weight) {
      if (!encode_tensor_map_2d(&cache->weight_half_map, q.weight, row_bytes, q.n, 128, &error))
        return fail(GW_CUDA_ERROR, "weight descriptor: " + error);
      cache->weight_half = q.weight;
    }
    PairGemmParams pair{};
    pair.map_tokens = cache->activation_map;
    pair.map_weights = cache->weight_half_map;
    pair.map_weight_scales = cache->weight_scale_map;
    pair.sf_tokens = q.activation_scales;
    pair.token_row_blocks = int32_t((q.rows + 127) / 128);
    pair.k = int32_t(q.k);
    pair.rows = int32_t(q.rows);
    pair.n = int32_t(q.n);
    pair.l_tiles = int32_t((q.rows + 255) / 256);
    pair.c_tiles = int32_t((q.n + 255) / 256);
    pair.out = q.output;
    pair.ld_out = q.n;
    pair.alpha = q.alpha;
    pair.error = q.error;
    GW_CUDA_CHECK(launch_gemm_pair(pair, sm_count(), stream), "NVFP4 CTA-pair tensor-core GEMM");
    return GW_OK;
  }
  GemmParams params{};
  GemmGroup& g = params.single;
  params.groups = nullptr;
  params.num_groups = 1;
  params.k = int32_t(q.k);
  params.out = q.output;
  params.ld_out = q.n;
  params.error = q.error;
  g.alpha[0] = g.alpha[1] = q.alpha;
  g.channel_alpha = q.channel_alpha;
  g.map_l = -1;
  g.map_c[0] = g.map_c[1] = -1;
  if (swap) {
    params.early_weights = 1;   // weights are never written by the activation-quantise kernel before this launch
    params.map_l = cache->weight_map;
    params.map_c = cache->activation_map;
    params.c_rows_per_tile = block_n;
    g.sf_l = q.weight_scales;
    g.l_rows = int32_t(q.n);
    g.l_tiles = int32_t((q.n + 127) / 128);
    g.sf_c[0] = g.sf_c[1] = q.activation_scales;
    g.c_rows = int32_t(q.rows);
    g.c_tiles = int32_t((q.rows + block_n - 1) / block_n);
    g.c_half_stride = 0;
  } else {
    params.map_l = cache->activation_map;
    params.map_c = cache->weight_map;
    params.c_rows_per_tile = block_n;
    g.sf_l = q.activation_scales;
    g.l_rows = int32_t(q.rows);
    g.l_tiles = int32_t((q.rows + 127) / 128);
    g.sf_c[0] = g.sf_c[1] = q.weight_scales;
    g.c_rows = int32_t(q.n);
    g.c_tiles = int32_t((q.n + block_n - 1) / block_n);
    g.c_half_stride = block_n > 128 ? 128 : 0;
    if (single_box) {
      params.c_single_box = 1;
      if (fp4) params.map_sfc = cache->weight_scale_map;
    }
  }
  params.total_work = g.l_tiles * g.c_tiles;
  int grid = params.total_work < sm_count() ? params.total_work : sm_count();
  if (swap && q.split_workspace != nullptr && cache->split_counters != nullptr) {
    params.split_counters = cache->split_counters;
    params.split_partials = static_cast<float*>(q.split_workspace);
    const long long stages = (long long)gemm_tc_k_stages(q.kind, GemmEpilogue::swap_store, row_bytes) * params.total_work;
    grid = stages < sm_count() ? int(stages) : sm_count();
  }
  GW_CUDA_CHECK(launch_gemm_tc(q.kind, swap ? GemmEpilogue::swap_store : GemmEpilogue::direct_store, block_n, params,
                               grid, stream),
                fp4 ? "NVFP4 tensor-core GEMM" : (q.kind == GemmKind::bf16 ? "BF16 tensor-core GEMM" : "FP8 tensor-core GEMM"));
  return GW_OK;
}

}  // namespace gw
