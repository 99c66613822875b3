// Projection binding and the shared-scratch projection workspace of the 26B
// model behind the C ABI: bind_projection and ProjectionWorkspace of the
// reference (models/gemma4/26b_a4b/sm120/projection.cuh:11-41,
// projection.cu:31-145), on this library's plans.
//
// A bound projection is run by storage type, activation policy and phase:
//   FP8                         -> fp8 plan (W8A8)
//   NVFP4, FP4 activations      -> nvfp4 plan (W4A4)
//   NVFP4, BF16 activations     -> dequantise the whole weight to BF16 scratch, BF16 GEMM (W4A16)
//   BF16                        -> BF16 GEMM
// and, when the NVFP4 output dimension was padded to 128 rows, the padded
// result is compacted to the logical width.  Plans are (re)built in prepare(),
// outside the layer loop; run() allocates nothing.
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <new>
#include <string>
#include <tuple>
#include <vector>

#include "common.cuh"
#include "dense.h"

using namespace gw;

namespace {

__global__ void __launch_bounds__(256)
compact_rows_kernel(const bf16* __restrict__ input, bf16* __restrict__ output, uint32_t rows, uint32_t logical,
                    uint32_t physical) {
  // strip the padding columns: output[r, c] = input[r, c] for c < logical   (projection.cu:25-28)
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i < size_t(rows) * logical) output[i] = input[(i / logical) * physical + i % logical];
}

struct Buffer {
  void* data = nullptr;
  size_t bytes = 0;
  cudaError_t allocate(size_t n) {
    bytes = n;
    return n ? cudaMalloc(&data, n) : cudaSuccess;
  }
  ~Buffer() { if (data) cudaFree(data); }
};

enum PlanKind { kPlanNvfp4 = 0, kPlanFp8 = 1, kPlanBf16 = 2 };
using Shape = std::tuple<int, uint32_t, uint32_t>;   // plan kind, K, physical N

struct Plans {
  gw_nvfp4_plan* nvfp4 = nullptr;
  gw_fp8_plan* fp8 = nullptr;
  gw_bf16_plan* bf16 = nullptr;
  void reset() {
    if (nvfp4) gw_nvfp4_plan_destroy(nvfp4);
    if (fp8) gw_fp8_plan_destroy(fp8);
    if (bf16) gw_bf16_plan_destroy(bf16);
    nvfp4 = nullptr; fp8 = nullptr; bf16 = nullptr;
  }
};

bool finite_positive(float v) { return v > 0.0F && std::isfinite(v); }

}  // namespace

struct gw_projection_workspace {
  std::map<Shape, Plans> plans;
  Buffer scratch, padded, dequantized;
  uint32_t capacity = 0, rows = 0;
  int policy = GW_POLICY_ALWAYS;
  bool fp4 = false;
  cudaStream_t stream = nullptr;
  ~gw_projection_workspace() { for (auto& entry : plans) entry.second.reset(); }
};

extern "C" {

int gw_nvfp4_fp4_activations(int policy, int phase) {
  return policy == GW_POLICY_ALWAYS || phase == GW_PHASE_PREFILL;   // include/gewell/nvfp4_policy.h:9-11
}

gw_status gw_bind_projection(uint32_t storage, uint32_t rows, uint32_t columns, const uint8_t* host_payload,
                             const void* device_payload, size_t entry_bytes, gw_projection* projection) {
  clear_error();
  if (!host_payload || !device_payload || !projection || rows == 0 || columns == 0)
    return fail(GW_INVALID_ARGUMENT, "invalid 26B projection binding");
  gw_projection result{};
  result.storage = storage;
  result.input = columns;
  result.output = rows;
  result.physical_output = storage == GW_STORAGE_NVFP4_W4A4 ? (rows + 127) / 128 * 128 : rows;
  result.bf16 = device_payload;
  if (storage == GW_STORAGE_BF16) {
    if (entry_bytes < size_t(rows) * columns * 2) return fail(GW_INVALID_ARGUMENT, "26B projection entry is shorter than its BF16 matrix");
    *projection = result;
    return GW_OK;
  }
  if (storage != GW_STORAGE_NVFP4_W4A4 && storage != GW_STORAGE_FP8_W8A8)
    return fail(GW_INVALID_ARGUMENT, "invalid 26B projection storage");
  const size_t weights = storage == GW_STORAGE_NVFP4_W4A4 ? size_t(result.physical_output) * columns / 2
                                                          : size_t(rows) * columns;
  const size_t scales = storage == GW_STORAGE_NVFP4_W4A4 ? scale_storage_bytes(result.physical_output, columns) : 0;
  if (entry_bytes < weights + scales + 8)
    return fail(GW_INVALID_ARGUMENT, "26B projection entry is shorter than its packed weights, scales and globals");
  // the two FP32 globals close the entry: <weight_scale><input_scale>, little endian
  float weight_scale, input_scale;
  std::memcpy(&weight_scale, host_payload + entry_bytes - 8, 4);
  std::memcpy(&input_scale, host_payload + entry_bytes - 4, 4);
  const auto* packed = static_cast<const uint8_t*>(device_payload);
  if (storage == GW_STORAGE_NVFP4_W4A4) {
    result.nvfp4_data = packed;
    result.nvfp4_scales = packed + weights;
    result.nvfp4_input_scale = input_scale;
    result.nvfp4_weight_scale = weight_scale;
  } else {
    result.fp8_data = packed;
    result.fp8_input_scale = input_scale;
    result.fp8_weight_scale = weight_scale;
    result.fp8_channel_scales = nullptr;
  }
  *projection = result;
  return GW_OK;
}

size_t gw_projection_entry_bytes(uint32_t storage, uint32_t rows, uint32_t columns) {
  // tensor_bytes (models/gemma4/26b_a4b/artifact.cc:64-71)
  if (storage == GW_STORAGE_BF16) return size_t(rows) * columns * 2;
  if (storage == GW_STORAGE_FP8_W8A8) return size_t(rows) * columns + 8;
  if (storage != GW_STORAGE_NVFP4_W4A4) return 0;
  const size_t padded_rows = (size_t(rows) + 127) / 128 * 128;
  const size_t scale_columns = (size_t(columns) / 16 + 3) / 4 * 4;
  return padded_rows * columns / 2 + padded_rows * scale_columns + 8;
}

gw_status gw_validate_projection_entry(uint32_t storage, uint32_t rows, uint32_t columns, const uint8_t* host_payload,
                                       size_t entry_bytes) {
  clear_error();
  if (!host_payload || rows == 0 || columns == 0) return fail(GW_INVALID_ARGUMENT, "invalid 26B projection entry");
  const size_t expected = gw_projection_entry_bytes(storage, rows, columns);
  if (expected == 0) return fail(GW_INVALID_ARGUMENT, "invalid 26B storage type");
  if (entry_bytes != expected) return fail(GW_INVALID_ARGUMENT, "26B entry size does not match its shape and storage type");
  if (storage == GW_STORAGE_BF16) return GW_OK;
  // validate_globals (artifact.cc:72-80)
  float weight, input;
  std::memcpy(&weight, host_payload + entry_bytes - 8, 4);
  std::memcpy(&input, host_payload + entry_bytes - 4, 4);
  if (!(std::isfinite(weight) && weight > 0 && std::isfinite(input) && input > 0 && std::isfinite(1.0F / input) &&
        std::isfinite(weight * input) && weight * input > 0))
    return fail(GW_INVALID_ARGUMENT, "invalid 26B global scales");
  // validate_quantized_payload (artifact.cc:81-104)
  if (storage == GW_STORAGE_FP8_W8A8) {
    const size_t elements = size_t(rows) * columns;
    for (size_t i = 0; i < elements; ++i)
      if ((host_payload[i] & 0x7F) == 0x7F) return fail(GW_INVALID_ARGUMENT, "nonfinite 26B FP8 payload");
    return GW_OK;
  }
  if (columns % 16) return fail(GW_INVALID_ARGUMENT, "NVFP4 entry needs a column count divisible by 16");
  const size_t padded_rows = (size_t(rows) + 127) / 128 * 128;
  const size_t logical_bytes = size_t(rows) * columns / 2, packed_bytes = padded_rows * columns / 2;
  for (size_t i = logical_bytes; i < packed_bytes; ++i)
    if (host_payload[i] != 0) return fail(GW_INVALID_ARGUMENT, "nonzero 26B NVFP4 weight padding");
  const size_t blocks = columns / 16, scale_columns = (blocks + 3) / 4 * 4;
  const uint8_t* scales = host_payload + packed_bytes;
  // every 128-row tile stores its scales as [K tile][row % 32][row / 32][block % 4]
  for (size_t row = 0; row < padded_rows; ++row)
    for (size_t column = 0; column < scale_columns; ++column) {
      const size_t local = row % 128;
      const size_t offset = (row / 128) * 128 * scale_columns + (((column / 4) * 32 + local % 32) * 4 + local / 32) * 4 + column % 4;
      const uint8_t value = scales[offset];
      if (row >= rows || column >= blocks) {
        if (value != 0) return fail(GW_INVALID_ARGUMENT, "nonzero 26B NVFP4 scale padding");
      } else if (value >= 0x7F) {
        return fail(GW_INVALID_ARGUMENT, "invalid 26B NVFP4 block scale");
      }
    }
  return GW_OK;
}

gw_status gw_projection_workspace_create(const gw_projection* projections, uint32_t count, uint32_t max_rows,
                                         int policy, void* stream, gw_projection_workspace** workspace) {
  clear_error();
  if (!workspace || (!projections && count != 0) || max_rows == 0 || max_rows > 65536 ||
      (policy != GW_POLICY_ALWAYS && policy != GW_POLICY_PREFILL))
    return fail(GW_INVALID_ARGUMENT, "invalid 26B projection capacity/policy");
  auto w = std::unique_ptr<gw_projection_workspace>(new (std::nothrow) gw_projection_workspace());
  if (!w) return fail(GW_CUDA_ERROR, "out of host memory");
  w->capacity = max_rows;
  w->policy = policy;
  w->stream = as_stream(stream);
  size_t scratch_bytes = 0, padded_bytes = 0, dequantized_bytes = 0;
  // FP32 partial tiles of the K split that decode-shaped BF16 plans use (<= 128 rows, 128-wide tiles)
  const size_t bf16_scratch = size_t(2) * size_t(sm_count()) * 128 * 128 * sizeof(float) + 256;
  for (uint32_t i = 0; i < count; ++i) {
    const gw_projection& p = projections[i];
    if (p.input == 0 || p.output == 0 || p.physical_output < p.output)
      return fail(GW_INVALID_ARGUMENT, "invalid 26B projection shape");
    if (p.storage == GW_STORAGE_BF16) {
      if (!p.bf16 || p.input % 8 || p.output % 8) return fail(GW_INVALID_ARGUMENT, "BF16 projection needs K and N divisible by 8");
      // no scratch on account of BF16 weights (the reference's BF16 projections need none either); when
      // other bindings bring scratch along, small batches use it for the K split
      w->plans.emplace(Shape{kPlanBf16, p.input, p.physical_output}, Plans{});
    } else if (p.storage == GW_STORAGE_NVFP4_W4A4) {
      if (!p.nvfp4_data || !p.nvfp4_scales || p.input % 64 || p.physical_output % 128 ||
          !finite_positive(p.nvfp4_input_scale) || !finite_positive(p.nvfp4_weight_scale))
        return fail(GW_INVALID_ARGUMENT, "invalid NVFP4 projection binding");
      w->plans.emplace(Shape{kPlanNvfp4, p.input, p.physical_output}, Plans{});
      scratch_bytes = std::max(scratch_bytes, gw_nvfp4_scratch_upper_bound_bytes(max_rows, p.input, p.physical_output));
      if (p.output != p.physical_output)
        padded_bytes = std::max(padded_bytes, size_t(max_rows) * p.physical_output * sizeof(bf16));
      if (policy == GW_POLICY_PREFILL) {     // decode keeps BF16 activations: whole-weight dequantisation + BF16 GEMM
        dequantized_bytes = std::max(dequantized_bytes, size_t(p.physical_output) * p.input * sizeof(bf16));
        w->plans.emplace(Shape{kPlanBf16, p.input, p.physical_output}, Plans{});
        scratch_bytes = std::max(scratch_bytes, bf16_scratch);
      }
    } else if (p.storage == GW_STORAGE_FP8_W8A8) {
      if (!p.fp8_data || p.input % 16 || p.output % 16 || !finite_positive(p.fp8_input_scale) ||
          !finite_positive(p.fp8_weight_scale))
        return fail(GW_INVALID_ARGUMENT, "invalid FP8 projection binding");
      w->plans.emplace(Shape{kPlanFp8, p.input, p.physical_output}, Plans{});
      scratch_bytes = std::max(scratch_bytes, gw_fp8_scratch_upper_bound_bytes(max_rows, p.input));
    } else {
      return fail(GW_INVALID_ARGUMENT, "invalid 26B projection storage");
    }
  }
  cudaError_t status = w->scratch.allocate(scratch_bytes);
  if (status == cudaSuccess) status = w->padded.allocate(padded_bytes);
  if (status == cudaSuccess) status = w->dequantized.allocate(dequantized_bytes);
  if (status != cudaSuccess)
    return fail(GW_CUDA_ERROR, std::string("projection workspace allocation: ") + cudaGetErrorString(status));
  *workspace = w.release();
  return GW_OK;
}

void gw_projection_workspace_destroy(gw_projection_workspace* workspace) { delete workspace; }

size_t gw_projection_workspace_bytes(const gw_projection_workspace* w) {
  return w ? w->scratch.bytes + w->padded.bytes + w->dequantized.bytes : 0;
}

gw_status gw_projection_workspace_prepare(gw_projection_workspace* w, uint32_t rows, int phase) {
  clear_error();
  if (!w || rows == 0 || rows > w->capacity || (phase != GW_PHASE_PREFILL && phase != GW_PHASE_DECODE))
    return fail(GW_INVALID_ARGUMENT, "invalid 26B projection rows/phase");
  const bool fp4 = gw_nvfp4_fp4_activations(w->policy, phase) != 0;
  if (w->rows == rows && w->fp4 == fp4) return GW_OK;
  // Keep a plan when only the phase changes; rebuild on a new row count, outside the layer loop.
  // Every requested plan is built first and published only when all of them exist.
  std::map<Shape, Plans> replacements;
  gw_status status = GW_OK;
  for (const auto& entry : w->plans) {
    const auto [kind, k, n] = entry.first;
    Plans& next = replacements[entry.first];
    const bool stale = w->rows != rows;
    if (kind == kPlanFp8 && (stale || !entry.second.fp8)) status = gw_fp8_plan_create(rows, k, n, 0, &next.fp8);
    if (kind == kPlanNvfp4 && fp4 && (stale || !entry.second.nvfp4)) status = gw_nvfp4_plan_create(rows, k, n, &next.nvfp4);
    if (kind == kPlanBf16 && (stale || !entry.second.bf16)) status = gw_bf16_plan_create(rows, k, n, &next.bf16);
    if (status != GW_OK) break;
  }
  if (status != GW_OK) {
    for (auto& entry : replacements) entry.second.reset();
    return status;
  }
  for (auto& entry : replacements) {
    Plans& current = w->plans.at(entry.first);
    Plans& next = entry.second;
    if (next.fp8) { if (current.fp8) gw_fp8_plan_destroy(current.fp8); current.fp8 = next.fp8; }
    if (next.bf16) { if (current.bf16) gw_bf16_plan_destroy(current.bf16); current.bf16 = next.bf16; }
    if (next.nvfp4) {
      if (current.nvfp4) gw_nvfp4_plan_destroy(current.nvfp4);
      current.nvfp4 = next.nvfp4;
    } else if (w->rows != rows && current.nvfp4) {
      gw_nvfp4_plan_destroy(current.nvfp4);       // built for another row count
      current.nvfp4 = nullptr;
    }
  }
  w->rows = rows;
  w->fp4 = fp4;
  return GW_OK;
}

gw_status gw_projection_workspace_run(gw_projection_workspace* w, const gw_projection* projection,
                                      const void* input_bf16, void* output_bf16) {
  clear_error();
  if (!w || !projection || w->rows == 0 || !input_bf16 || !output_bf16)
    return fail(GW_INVALID_ARGUMENT, "prepare 26B projections before run");
  const gw_projection& p = *projection;
  const bool padded = p.output != p.physical_output;
  if (padded && (!w->padded.data || size_t(w->rows) * p.physical_output * sizeof(bf16) > w->padded.bytes))
    return fail(GW_INVALID_ARGUMENT, "projection was not among the workspace's bindings");
  void* destination = padded ? w->padded.data : output_bf16;
  const int kind = p.storage == GW_STORAGE_FP8_W8A8 ? kPlanFp8
                   : (p.storage == GW_STORAGE_NVFP4_W4A4 && w->fp4) ? kPlanNvfp4 : kPlanBf16;
  const auto found = w->plans.find(Shape{kind, p.input, p.physical_output});
  if (found == w->plans.end()) return fail(GW_INVALID_ARGUMENT, "projection was not among the workspace's bindings");
  const Plans& plans = found->second;
  gw_status status = GW_OK;
  if (kind == kPlanFp8) {
    if (!plans.fp8) return fail(GW_INVALID_ARGUMENT, "prepare 26B projections before run");
    status = gw_fp8_plan_run(plans.fp8, input_bf16, p.fp8_data, p.fp8_input_scale, p.fp8_weight_scale, nullptr,
                             destination, w->scratch.data, w->scratch.bytes, w->stream, GW_TRANSFORM_IDENTITY);
  } else if (kind == kPlanNvfp4) {
    if (!plans.nvfp4) return fail(GW_INVALID_ARGUMENT, "prepare 26B projections before run");
    status = gw_nvfp4_plan_run(plans.nvfp4, input_bf16, p.nvfp4_data, p.nvfp4_scales, p.nvfp4_input_scale,
                               p.nvfp4_weight_scale, destination, w->scratch.data, w->scratch.bytes, w->stream,
                               GW_TRANSFORM_IDENTITY);
  } else {
    if (!plans.bf16) return fail(GW_INVALID_ARGUMENT, "prepare 26B projections before run");
    const void* weights = p.bf16;
    if (p.storage == GW_STORAGE_NVFP4_W4A4) {
      if (!w->dequantized.data || size_t(p.physical_output) * p.input * sizeof(bf16) > w->dequantized.bytes)
        return fail(GW_INVALID_ARGUMENT, "projection was not among the workspace's bindings");
      status = gw_nvfp4_dequantize(p.nvfp4_data, p.nvfp4_scales, p.nvfp4_weight_scale, p.input, p.physical_output,
                                   w->dequantized.data, w->stream);
      if (status != GW_OK) return status;
      weights = w->dequantized.data;
    }
    const bool split = w->scratch.data && w->scratch.bytes >= gw_bf16_plan_scratch_bytes(plans.bf16);
    status = gw_bf16_plan_run(plans.bf16, input_bf16, weights, destination, split ? w->scratch.data : nullptr,
                              split ? w->scratch.bytes : 0, w->stream);
  }
  if (status != GW_OK) return status;
  if (padded) {
    const size_t count = size_t(w->rows) * p.output;
    compact_rows_kernel<<<unsigned((count + 255) / 256), 256, 0, w->stream>>>(
        static_cast<const bf16*>(destination), static_cast<bf16*>(output_bf16), w->rows, p.output, p.physical_output);
    note_launch();
    GW_CUDA_CHECK(cudaGetLastError(), "compact 26B projection output");
  }
  return GW_OK;
}

}  // extern "C"
