// C ABI of gewell_b200: argument validation (same contract as the reference
// classes), plan objects and the element-wise entry points.
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <mutex>
#include <new>
#include <string>

#include "common.cuh"
#include "dense.h"
#include "gemm_pair.h"
#include "gemm_pair_moe.h"
#include "gemm_tc.cuh"
#include "kernels.h"

namespace gw {

namespace {
thread_local std::string g_last_error;
}

gw_status fail(gw_status code, const std::string& message) {
  g_last_error = message;
  return code;
}
void clear_error() { g_last_error.clear(); }

namespace {
std::atomic<unsigned long long> g_launches{0};
}
void note_launch(unsigned kernels) { g_launches.fetch_add(kernels, std::memory_order_relaxed); }

// Per-GPU state is keyed by the device ordinal that is current at the call, so one
// process may drive several GPUs.
int current_device_slot() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0) device = 0;
  return device % kMaxDeviceSlots;
}

uint32_t* device_error_word() {
  static uint32_t* words[kMaxDeviceSlots] = {};
  static std::mutex mutex;
  const int slot = current_device_slot();
  std::lock_guard<std::mutex> lock(mutex);
  if (words[slot] == nullptr) {
    uint32_t* word = nullptr;
    if (cudaMalloc(&word, sizeof(uint32_t)) == cudaSuccess && cudaMemset(word, 0, sizeof(uint32_t)) == cudaSuccess)
      words[slot] = word;
    else
      (void)cudaGetLastError();
  }
  return words[slot];
}

int sm_count() {
  static int counts[kMaxDeviceSlots] = {};
  const int slot = current_device_slot();
  if (counts[slot] == 0) {
    int device = 0, count = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || count <= 0)
      count = 148;
    counts[slot] = count;
  }
  return counts[slot];
}

namespace {

bool finite_positive(float v) { return v > 0.0F && std::isfinite(v); }

bool aligned(const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; }

}  // namespace
}  // namespace gw

using namespace gw;

extern "C" {

const char* gw_last_error(void) { return g_last_error.c_str(); }
int gw_abi_version(void) { return 2; }

size_t gw_nvfp4_scale_storage_bytes(size_t rows, size_t input_width) { return scale_storage_bytes(rows, input_width); }
size_t gw_nvfp4_scale_offset(size_t row, size_t block, size_t input_width) { return scale_offset(row, block, input_width); }

size_t gw_nvfp4_scratch_upper_bound_bytes(size_t max_rows, size_t input_width, size_t output_width) {
  // include/gewell/nvfp4_linear.h:42-49 (kept identical so callers size the same buffer)
  const size_t padded_rows = (max_rows + 31) / 32 * 32;
  return padded_rows * (input_width / 2 + output_width * 2) + scale_storage_bytes(max_rows, input_width) +
         size_t(36) * 1024 * 1024 + 3 * 255;
}
size_t gw_fp8_scratch_upper_bound_bytes(size_t max_rows, size_t input_width) {
  return max_rows * input_width + size_t(32) * 1024 * 1024 + 255;   // include/gewell/fp8_linear.h:30-33
}

uint32_t gw_debug_kernel_error(void) {
  uint32_t value = 0;
  uint32_t* word = device_error_word();
  if (word == nullptr) return 0xFFFFFFFFu;
  if (cudaDeviceSynchronize() != cudaSuccess) return 0xFFFFFFFEu;
  cudaMemcpy(&value, word, sizeof(value), cudaMemcpyDeviceToHost);
  if (value != 0) cudaMemset(word, 0, sizeof(value));
  // the allocation-free linear reports into a word of its own (it may not use the allocated one)
  const uint32_t built_in = take_static_scratch_error();
  return value != 0 ? value : built_in;
}

uint64_t gw_debug_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

gw_status gw_debug_gemm_profile(void* device_buffer) {
  clear_error();
  set_gemm_profile_buffer(static_cast<long long*>(device_buffer));
  set_pair_profile_buffer(static_cast<long long*>(device_buffer));
  set_pair_moe_profile_buffer(static_cast<long long*>(device_buffer));
  return GW_OK;
}

gw_status gw_debug_rcp_approx(const float* input, float* output, uint64_t count, void* stream) {
  clear_error();
  if (!input || !output) return fail(GW_INVALID_ARGUMENT, "rcp probe requires input and output buffers");
  if (!count) return GW_OK;
  GW_CUDA_CHECK(launch_rcp_approx(input, output, count, as_stream(stream)), "approximate reciprocal probe");
  return GW_OK;
}

gw_status gw_debug_geglu_bf16(const void* gate_bf16, const void* up_bf16, void* output_bf16, uint64_t count,
                              void* stream) {
  clear_error();
  if (!gate_bf16 || !up_bf16 || !output_bf16) return fail(GW_INVALID_ARGUMENT, "GeGLU probe requires three buffers");
  if (!count) return GW_OK;
  GW_CUDA_CHECK(launch_geglu(gate_bf16, up_bf16, output_bf16, count, as_stream(stream)), "GeGLU probe");
  return GW_OK;
}

// --------------------------------------------------------------------------- NVFP4 element-wise

gw_status gw_nvfp4_dequantize(const uint8_t* data, const uint8_t* scales, float weight_scale, uint32_t input_width,
                              uint32_t output_width, void* output_bf16, void* stream) {
  clear_error();
  if (!data || !scales || !output_bf16 || !input_width || input_width % 64 || !output_width ||
      output_width % 128 || !finite_positive(weight_scale))
    return fail(GW_INVALID_ARGUMENT,
                "NVFP4 dequantize requires valid buffers, K divisible by 64, N divisible by 128, and a finite "
                "positive weight scale");
  if (!aligned(data, 8) || !aligned(output_bf16, 16))
    return fail(GW_INVALID_ARGUMENT, "NVFP4 dequantize requires 8-byte aligned weights and 16-byte aligned output");
  GW_CUDA_CHECK(launch_nvfp4_dequantize(data, scales, weight_scale, input_width, output_width, output_bf16,
                                        as_stream(stream)),
                "NVFP4 dequantize weights");
  return GW_OK;
}

gw_status gw_nvfp4_pack_weights(const void* weights_bf16, uint32_t output_width, uint32_t input_width,
                                float weight_scale, uint8_t* data, uint8_t* scales, void* stream) {
  clear_error();
  if (!weights_bf16 || !data || !scales || !output_width || !input_width || input_width % 64 ||
      !finite_positive(weight_scale) || !aligned(weights_bf16, 16) || !aligned(data, 8))
    return fail(GW_INVALID_ARGUMENT,
                "NVFP4 weight packing requires aligned buffers, K divisible by 64 and a finite positive global scale");
  GW_CUDA_CHECK(launch_nvfp4_pack_weights(weights_bf16, output_width, input_width, weight_scale, data, scales,
                                          as_stream(stream)),
                "NVFP4 pack weights");
  return GW_OK;
}

gw_status gw_nvfp4_quantize_activations(const void* input_bf16, uint32_t rows, uint32_t input_width,
                                        float input_scale, int transform, uint8_t* packed, uint8_t* scales,
                                        void* stream) {
  clear_error();
  if (!input_bf16 || !packed || !scales || !rows || !input_width || input_width % 64 ||
      !finite_positive(input_scale) || !std::isfinite(1.0F / input_scale) ||
      (transform != GW_TRANSFORM_IDENTITY && transform != GW_TRANSFORM_GELU_TANH_MULTIPLY) ||
      !aligned(input_bf16, 16) || !aligned(packed, 8))
    return fail(GW_INVALID_ARGUMENT,
                "NVFP4 activation quantisation requires 16-byte aligned input, K divisible by 64 and a finite "
                "positive input scale with a finite reciprocal");
  GW_CUDA_CHECK(launch_nvfp4_quantize(input_bf16, rows, input_width, 1.0F / input_scale,
                                      transform == GW_TRANSFORM_GELU_TANH_MULTIPLY, packed, scales, as_stream(stream)),
                "NVFP4 quantize activations");
  return GW_OK;
}

gw_status gw_nvfp4_gemv_w4a16(const void* input_bf16, uint32_t rows, const uint8_t* weight_data,
                              const uint8_t* weight_scales, float weight_scale, uint32_t input_width,
                              uint32_t output_width, void* output_bf16, void* stream) {
  clear_error();
  if (!input_bf16 || !weight_data || !weight_scales || !output_bf16 || rows == 0 || rows > 8 || !input_width ||
      input_width % 64 || !output_width || output_width % 128 || !finite_positive(weight_scale) ||
      !aligned(input_bf16, 16) || !aligned(weight_data, 16))
    return fail(GW_INVALID_ARGUMENT,
                "W4A16 projection requires 1..8 rows, K divisible by 64, N divisible by 128, 16-byte aligned "
                "input and weights and a finite positive weight scale");
  GW_CUDA_CHECK(launch_gemv_w4a16(input_bf16, rows, weight_data, weight_scales, weight_scale, input_width,
                                  output_width, output_bf16, as_stream(stream)),
                "W4A16 projection");
  return GW_OK;
}

// --------------------------------------------------------------------------- NVFP4 plan

struct gw_nvfp4_plan {
  uint32_t rows, input_width, output_width;
  size_t scale_offset, split_offset, total_bytes;
  DenseDescriptors descriptors;
};

gw_status gw_nvfp4_plan_create(uint32_t rows, uint32_t input_width, uint32_t output_width, gw_nvfp4_plan** plan) {
  clear_error();
  if (!plan || rows == 0 || rows > uint32_t(std::numeric_limits<int>::max() - 127) || input_width == 0 ||
      input_width % 64 || output_width == 0 || output_width % 128)
    return fail(GW_INVALID_ARGUMENT, "NVFP4 plan requires positive rows, K divisible by 64 and N divisible by 128");
  auto* p = new (std::nothrow) gw_nvfp4_plan();
  if (!p) return fail(GW_CUDA_ERROR, "out of host memory");
  p->rows = rows;
  p->input_width = input_width;
  p->output_width = output_width;
  // scratch = packed activations | tiled activation scales   (each 256-byte aligned)
  p->scale_offset = align_up(size_t(rows) * input_width / 2, 256);
  p->split_offset = p->scale_offset + align_up(scale_storage_bytes(rows, input_width), 256);
  // Decode shapes split the K loop evenly over the SMs; that needs per-tile counters owned
  // by the plan and room for FP32 partial tiles in the scratch.  Without a usable device
  // (or memory for the counters) the plan falls back to whole tiles per CTA.
  p->total_bytes = p->split_offset;
  const cudaError_t counters = p->descriptors.allocate_split_counters(rows, output_width);
  if (counters != cudaSuccess) {
    (void)cudaGetLastError();
    // Without any device the plan is only a shape record (it cannot run); every other failure is an error,
    // not a silent fall-back to whole tiles per CTA, which would be a performance cliff.
    if (counters != cudaErrorNoDevice && counters != cudaErrorInsufficientDriver) {
      delete p;
      return fail(GW_CUDA_ERROR, std::string("plan: tile counters of the K split: ") + cudaGetErrorString(counters));
    }
  }
  if (p->descriptors.split_counters) p->total_bytes += align_up(dense_split_bytes(p->descriptors.tuning, rows, output_width), 256);
  *plan = p;
  return GW_OK;
}

size_t gw_nvfp4_plan_scratch_bytes(const gw_nvfp4_plan* plan) { return plan ? plan->total_bytes : 0; }
void gw_nvfp4_plan_destroy(gw_nvfp4_plan* plan) { delete plan; }

gw_status gw_nvfp4_plan_run(gw_nvfp4_plan* plan, const void* input_bf16, const uint8_t* weight_data,
                            const uint8_t* weight_scales, float input_scale, float weight_scale, void* output_bf16,
                            void* scratch, size_t scratch_capacity, void* stream, int transform) {
  clear_error();
  if (!plan) return fail(GW_INVALID_ARGUMENT, "NVFP4 run requires a plan");
  const float alpha = input_scale * weight_scale;
  if (!input_bf16 || !weight_data || !weight_scales || !output_bf16 || !scratch || !aligned(scratch, 256) ||
      scratch_capacity < plan->total_bytes || !finite_positive(input_scale) || !finite_positive(weight_scale) ||
      !finite_positive(alpha) || !std::isfinite(1.0F / input_scale) ||
      (transform != GW_TRANSFORM_IDENTITY && transform != GW_TRANSFORM_GELU_TANH_MULTIPLY))
    return fail(GW_INVALID_ARGUMENT,
                "NVFP4 run requires valid device buffers, aligned sufficient scratch, and finite positive global "
                "scales");
  if (!aligned(input_bf16, 16) || !aligned(weight_data, 16) || !aligned(weight_scales, 16) || !aligned(output_bf16, 2))
    return fail(GW_INVALID_ARGUMENT, "NVFP4 run requires 16-byte aligned input, weights and weight scales");
  cudaStream_t s = as_stream(stream);
  auto* packed = static_cast<uint8_t*>(scratch);
  uint8_t* scales = packed + plan->scale_offset;
  GW_CUDA_CHECK(launch_nvfp4_quantize(input_bf16, plan->rows, plan->input_width, 1.0F / input_scale,
                                      transform == GW_TRANSFORM_GELU_TANH_MULTIPLY, packed, scales, s),
                "NVFP4 quantize activations");
  DenseProblem problem{GemmKind::nvfp4, plan->rows, plan->input_width, plan->output_width, weight_data, weight_scales,
                       packed, scales, alpha, nullptr, output_bf16, device_error_word()};
  if (plan->total_bytes != plan->split_offset) problem.split_workspace = packed + plan->split_offset;
  return launch_dense(problem, &plan->descriptors, s);
}

// --------------------------------------------------------------------------- FP8

gw_status gw_fp8_quantize_activations(const void* input_bf16, uint32_t rows, uint32_t input_width, float input_scale,
                                      int transform, uint8_t* packed, void* stream) {
  clear_error();
  if (!input_bf16 || !packed || !rows || !input_width || input_width % 16 || !finite_positive(input_scale) ||
      !std::isfinite(1.0F / input_scale) || !aligned(input_bf16, 2) || !aligned(packed, 8) ||
      (transform != GW_TRANSFORM_IDENTITY && transform != GW_TRANSFORM_GELU_TANH_MULTIPLY))
    return fail(GW_INVALID_ARGUMENT, "FP8 activation quantisation requires K divisible by 16 and a finite positive input scale");
  GW_CUDA_CHECK(launch_fp8_quantize(input_bf16, rows, input_width, 1.0F / input_scale,
                                    transform == GW_TRANSFORM_GELU_TANH_MULTIPLY, packed, as_stream(stream)),
                "FP8 quantize activations");
  return GW_OK;
}

gw_status gw_fp8_pack_weights(const void* weights_bf16, uint32_t output_width, uint32_t input_width, float weight_scale,
                              const float* row_scales, uint8_t* data, void* stream) {
  clear_error();
  if (!weights_bf16 || !data || !output_width || !input_width || input_width % 16 ||
      (!row_scales && !finite_positive(weight_scale)) || !aligned(weights_bf16, 16) || !aligned(data, 8))
    return fail(GW_INVALID_ARGUMENT, "FP8 weight packing requires aligned buffers, K divisible by 16 and a finite positive scale");
  GW_CUDA_CHECK(launch_fp8_pack_weights(weights_bf16, output_width, input_width, weight_scale, row_scales, data,
                                        as_stream(stream)),
                "FP8 pack weights");
  return GW_OK;
}

struct gw_fp8_plan {
  uint32_t rows, input_width, output_width;
  bool channel_scales;
  int gemv_rows = 0;      // GW_FP8_GEMV_ROWS, read when the plan is created
  size_t split_offset, total_bytes;
  DenseDescriptors descriptors;
};

gw_status gw_fp8_plan_create(uint32_t rows, uint32_t input_width, uint32_t output_width, int channel_scales,
                             gw_fp8_plan** plan) {
  clear_error();
  const uint32_t int_max = uint32_t(std::numeric_limits<int>::max());
  if (!plan || rows == 0 || rows > int_max || input_width == 0 || input_width % 16 || input_width > int_max ||
      output_width == 0 || output_width % 16 || output_width > int_max)
    return fail(GW_INVALID_ARGUMENT,
                "FP8 plan requires positive rows, K and N divisible by 16, and dimensions within int range");
  auto* p = new (std::nothrow) gw_fp8_plan();
  if (!p) return fail(GW_CUDA_ERROR, "out of host memory");
  p->rows = rows;
  p->input_width = input_width;
  p->output_width = output_width;
  p->channel_scales = channel_scales != 0;
  if (const char* gemv_env = std::getenv("GW_FP8_GEMV_ROWS")) p->gemv_rows = std::atoi(gemv_env);
  p->split_offset = align_up(size_t(rows) * input_width, 256);
  // Decode shapes split the K loop evenly over the SMs; that needs per-tile counters owned
  // by the plan and room for FP32 partial tiles in the scratch.  Without a usable device
  // (or memory for the counters) the plan falls back to whole tiles per CTA.
  p->total_bytes = p->split_offset;
  const cudaError_t counters = p->descriptors.allocate_split_counters(rows, output_width);
  if (counters != cudaSuccess) {
    (void)cudaGetLastError();
    // Without any device the plan is only a shape record (it cannot run); every other failure is an error,
    // not a silent fall-back to whole tiles per CTA, which would be a performance cliff.
    if (counters != cudaErrorNoDevice && counters != cudaErrorInsufficientDriver) {
      delete p;
      return fail(GW_CUDA_ERROR, std::string("plan: tile counters of the K split: ") + cudaGetErrorString(counters));
    }
  }
  if (p->descriptors.split_counters) p->total_bytes += align_up(dense_split_bytes(p->descriptors.tuning, rows, output_width), 256);
  *plan = p;
  return GW_OK;
}

size_t gw_fp8_plan_scratch_bytes(const gw_fp8_plan* plan) { return plan ? plan->total_bytes : 0; }
void gw_fp8_plan_destroy(gw_fp8_plan* plan) { delete plan; }

gw_status gw_fp8_plan_run(gw_fp8_plan* plan, const void* input_bf16, const uint8_t* weight_data, float input_scale,
                          float weight_scale, const float* channel_scales, void* output_bf16, void* scratch,
                          size_t scratch_capacity, void* stream, int transform) {
  clear_error();
  if (!plan) return fail(GW_INVALID_ARGUMENT, "FP8 run requires a plan");
  const float alpha = input_scale * weight_scale;
  if (!input_bf16 || !weight_data || !output_bf16 || !scratch || !aligned(input_bf16, 2) ||
      !aligned(weight_data, 16) || !aligned(output_bf16, 16) || !aligned(scratch, 256) ||
      scratch_capacity < plan->total_bytes || !finite_positive(input_scale) || !finite_positive(weight_scale) ||
      !finite_positive(alpha) || !std::isfinite(1.0F / input_scale) ||
      (plan->channel_scales && (!channel_scales || !aligned(channel_scales, 16))) ||
      (transform != GW_TRANSFORM_IDENTITY && transform != GW_TRANSFORM_GELU_TANH_MULTIPLY))
    return fail(GW_INVALID_ARGUMENT,
                "FP8 run requires valid aligned device buffers, sufficient scratch, and finite positive global "
                "scales with a finite positive product and finite input-scale reciprocal");
  cudaStream_t s = as_stream(stream);
  auto* packed = static_cast<uint8_t*>(scratch);
  // Optional CUDA-core path for 1..4 rows (weight streaming with warp reductions, activations
  // quantised inside the kernel).  Measured on B200 it is slower than the tensor-core path
  // (55 us against 50 us for one row of the 43008 x 5376 projection, 82 us for two), so it is
  // off unless GW_FP8_GEMV_ROWS names a row limit.
  if (transform == GW_TRANSFORM_IDENTITY && int(plan->rows) <= plan->gemv_rows && gemv_fp8_supports(plan->rows, plan->input_width) &&
      aligned(input_bf16, 2)) {
    GW_CUDA_CHECK(launch_gemv_fp8(input_bf16, plan->rows, weight_data, 1.0F / input_scale, alpha,
                                  plan->channel_scales ? channel_scales : nullptr, plan->input_width, plan->output_width,
                                  output_bf16, sm_count(), s),
                  "FP8 weight-streaming projection");
    return GW_OK;
  }
  GW_CUDA_CHECK(launch_fp8_quantize(input_bf16, plan->rows, plan->input_width, 1.0F / input_scale,
                                    transform == GW_TRANSFORM_GELU_TANH_MULTIPLY, packed, s),
                "FP8 quantize activations");
  DenseProblem problem{GemmKind::fp8, plan->rows, plan->input_width, plan->output_width, weight_data, nullptr,
                       packed, nullptr, alpha, plan->channel_scales ? channel_scales : nullptr, output_bf16,
                       device_error_word()};
  if (plan->total_bytes != plan->split_offset) problem.split_workspace = packed + plan->split_offset;
  return launch_dense(problem, &plan->descriptors, s);
}

// --------------------------------------------------------------------------- BF16

struct gw_bf16_plan {
  uint32_t rows, input_width, output_width;
  size_t total_bytes;
  DenseDescriptors descriptors;
};

gw_status gw_bf16_plan_create(uint32_t rows, uint32_t input_width, uint32_t output_width, gw_bf16_plan** plan) {
  clear_error();
  const uint32_t int_max = uint32_t(std::numeric_limits<int>::max());
  if (!plan || rows == 0 || rows > int_max - 127 || input_width == 0 || input_width % 8 || input_width > int_max / 2 ||
      output_width == 0 || output_width % 8 || output_width > int_max)
    return fail(GW_INVALID_ARGUMENT, "BF16 plan requires positive rows and K and N divisible by 8");
  auto* p = new (std::nothrow) gw_bf16_plan();
  if (!p) return fail(GW_CUDA_ERROR, "out of host memory");
  p->rows = rows;
  p->input_width = input_width;
  p->output_width = output_width;
  // Decode shapes split the K loop evenly over the SMs (FP32 partial tiles in the scratch).
  p->total_bytes = 0;
  const cudaError_t status = p->descriptors.allocate_split_counters(rows, output_width);
  if (status == cudaSuccess && p->descriptors.split_counters) {
    p->total_bytes = align_up(dense_split_bytes(p->descriptors.tuning, rows, output_width), 256);
  } else if (status != cudaSuccess) {
    (void)cudaGetLastError();
    if (status != cudaErrorNoDevice && status != cudaErrorInsufficientDriver) {
      delete p;
      return fail(GW_CUDA_ERROR, std::string("BF16 plan: tile counters of the K split: ") + cudaGetErrorString(status));
    }
  }
  *plan = p;
  return GW_OK;
}

size_t gw_bf16_plan_scratch_bytes(const gw_bf16_plan* plan) { return plan ? plan->total_bytes : 0; }
void gw_bf16_plan_destroy(gw_bf16_plan* plan) { delete plan; }

gw_status gw_bf16_plan_run(gw_bf16_plan* plan, const void* input_bf16, const void* weight_bf16, void* output_bf16,
                           void* scratch, size_t scratch_capacity, void* stream) {
  clear_error();
  if (!plan) return fail(GW_INVALID_ARGUMENT, "BF16 run requires a plan");
  // scratch == NULL is allowed: decode-shaped plans then keep whole tiles per CTA instead of the K split
  if (!input_bf16 || !weight_bf16 || !output_bf16 || !aligned(input_bf16, 16) || !aligned(weight_bf16, 16) ||
      !aligned(output_bf16, 16) || (scratch && plan->total_bytes != 0 && (!aligned(scratch, 256) ||
                                                                           scratch_capacity < plan->total_bytes)))
    return fail(GW_INVALID_ARGUMENT, "BF16 run requires 16-byte aligned device buffers and aligned sufficient scratch");
  DenseProblem problem{GemmKind::bf16, plan->rows, plan->input_width, plan->output_width, weight_bf16, nullptr,
                       input_bf16, nullptr, 1.0F, nullptr, output_bf16, device_error_word()};
  if (plan->total_bytes != 0 && scratch) problem.split_workspace = scratch;
  return launch_dense(problem, &plan->descriptors, as_stream(stream));
}

// --------------------------------------------------------------------------- weight QDQ

gw_status gw_absmax_bf16(const void* values_bf16, uint64_t elements, uint32_t* state, void* stream) {
  clear_error();
  if (!values_bf16 || !state || !aligned(values_bf16, 2) || !aligned(state, 4))
    return fail(GW_INVALID_ARGUMENT, "absmax requires a tensor and a device state word pair");
  GW_CUDA_CHECK(launch_absmax(values_bf16, elements, state, as_stream(stream)), "launch QDQ absmax kernel");
  return GW_OK;
}

gw_status gw_weight_qdq_apply(int type, void* values_bf16, uint64_t elements, uint32_t* state, void* stream) {
  clear_error();
  if (type != GW_QDQ_BF16 && type != GW_QDQ_FP8 && type != GW_QDQ_NVFP4)
    return fail(GW_INVALID_ARGUMENT, "unknown QDQ type");
  if (type == GW_QDQ_BF16 || elements == 0) return GW_OK;
  if (!values_bf16 || !state) return fail(GW_INVALID_ARGUMENT, "QDQ requires a tensor and a device state word pair");
  cudaStream_t s = as_stream(stream);
  GW_CUDA_CHECK(launch_absmax(values_bf16, elements, state, s), "launch QDQ absmax kernel");
  uint32_t host[2] = {0, 0};
  GW_CUDA_CHECK(cudaMemcpyAsync(host, state, sizeof(host), cudaMemcpyDeviceToHost, s), "copy QDQ reduction state");
  GW_CUDA_CHECK(cudaStreamSynchronize(s), "synchronize QDQ reduction");
  if (host[1] != 0) return fail(GW_INVALID_ARGUMENT, "selected QDQ weight contains a non-finite BF16 value");
  float amax;
  std::memcpy(&amax, &host[0], sizeof(amax));
  if (amax == 0.0F) return GW_OK;
  if (type == GW_QDQ_FP8) {
    GW_CUDA_CHECK(launch_fp8_qdq(values_bf16, elements, amax / 448.0F, s), "launch static FP8 QDQ kernel");
  } else {
    if (elements % 16 != 0 || !aligned(values_bf16, 16))
      return fail(GW_INVALID_ARGUMENT, "NVFP4 QDQ tensor element count is not divisible by 16");
    GW_CUDA_CHECK(launch_nvfp4_qdq(values_bf16, elements, amax / (6.0F * 448.0F), s), "launch NVFP4 QDQ kernel");
  }
  return GW_OK;
}

}  // extern "C"
