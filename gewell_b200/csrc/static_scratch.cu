// NVFP4 linear layer that borrows nothing from the caller except inputs and
// outputs and allocates nothing: its activation scratch (packed E2M1 rows and
// their scale tiles) lives in a fixed array inside this library's device image.
//
// Who needs this: an engine that hands every free byte of HBM to its KV cache
// when it starts has nothing left to cudaMalloc later, and a decode loop cannot
// afford the device-wide stall a cudaMalloc/cudaFree causes.  Such callers can
// still run a projection through this entry point without carving a scratch
// region out of their own arena.
//
// Cost and limits: the array (kStaticScratchBytes) is part of the module, so
// every GPU that loads the library keeps it resident until the process exits.
// Problems whose scratch need is larger are refused.  All calls share the one
// array per GPU: it still holds the previous call's bytes (every byte a call
// later reads is rewritten by that call first, so nothing has to be cleared),
// and two calls that overlap on the GPU -- different streams, or different
// host threads -- race on it.  Issue them on one stream.
#include <cmath>
#include <mutex>
#include <string>

#include "common.cuh"
#include "dense.h"
#include "gemm_tc.cuh"
#include "kernels.h"

namespace {

constexpr size_t kStaticScratchBytes = size_t(2) * 1024 * 1024;
constexpr int kMaxDevices = 64;

// In host code these two names are only handles for cudaGetSymbolAddress; the
// device addresses are looked up once per GPU below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ uint32_t g_static_error_word = 0;

struct DeviceSlot {
  unsigned char* scratch = nullptr;
  uint32_t* error = nullptr;
  bool ready = false;
};
DeviceSlot g_slots[kMaxDevices];
std::mutex g_slots_mutex;

// Resolve the device addresses of the static arrays for the current GPU.
gw_status resolve_slot(DeviceSlot** out) {
  int device = -1;
  cudaError_t status = cudaGetDevice(&device);
  if (status != cudaSuccess)
    return gw::fail(GW_CUDA_ERROR, std::string("static-scratch set-up, cudaGetDevice: ") + cudaGetErrorString(status));
  if (device < 0 || device >= kMaxDevices)
    return gw::fail(GW_INVALID_ARGUMENT, "static-scratch linear supports device ordinals below 64");
  std::lock_guard<std::mutex> lock(g_slots_mutex);
  DeviceSlot& slot = g_slots[device];
  if (!slot.ready) {
    void* scratch = nullptr;
    void* error = nullptr;
    status = cudaGetSymbolAddress(&scratch, g_static_scratch);
    if (status != cudaSuccess)
      return gw::fail(GW_CUDA_ERROR, std::string("static-scratch set-up, scratch address: ") + cudaGetErrorString(status));
    status = cudaGetSymbolAddress(&error, g_static_error_word);
    if (status != cudaSuccess)
      return gw::fail(GW_CUDA_ERROR, std::string("static-scratch set-up, error word address: ") + cudaGetErrorString(status));
    slot.scratch = static_cast<unsigned char*>(scratch);
    slot.error = static_cast<uint32_t*>(error);
    slot.ready = true;
  }
  *out = &slot;
  return GW_OK;
}

bool finite_positive(float v) { return v > 0.0F && std::isfinite(v); }
bool aligned(const void* p, size_t a) { return reinterpret_cast<uintptr_t>(p) % a == 0; }

}  // namespace

// The kernels launched from here record bounded-wait failures in g_static_error_word (they must not
// touch allocated memory).  gw_debug_kernel_error() collects it through this function; the caller has
// synchronised the device.
uint32_t gw::take_static_scratch_error() {
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return 0;
  uint32_t* word = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_slots_mutex);
    if (!g_slots[device].ready) return 0;      // the entry point never ran on this GPU
    word = g_slots[device].error;
  }
  uint32_t value = 0;
  if (cudaMemcpy(&value, word, sizeof(value), cudaMemcpyDeviceToHost) != cudaSuccess) return 0xFFFFFFFDu;
  if (value != 0) cudaMemset(word, 0, sizeof(value));
  return value;
}

extern "C" {

size_t gw_nvfp4_linear_static_scratch_limit(void) { return kStaticScratchBytes; }

gw_status gw_nvfp4_linear_static_scratch(const void* input_bf16, uint32_t rows, uint32_t input_width,
                                         uint32_t output_width, const uint8_t* weight_data,
                                         const uint8_t* weight_scales, float input_scale, float weight_scale,
                                         void* output_bf16, void* stream, int transform) {
  using namespace gw;
  clear_error();
  const float alpha = input_scale * weight_scale;
  if (!input_bf16 || !weight_data || !weight_scales || !output_bf16 || rows == 0 || input_width == 0 ||
      input_width % 64 || output_width == 0 || output_width % 128 || !finite_positive(input_scale) ||
      !finite_positive(weight_scale) || !finite_positive(alpha) || !std::isfinite(1.0F / input_scale) ||
      !aligned(input_bf16, 16) || !aligned(weight_data, 16) || !aligned(weight_scales, 16) ||
      !aligned(output_bf16, 2) ||
      (transform != GW_TRANSFORM_IDENTITY && transform != GW_TRANSFORM_GELU_TANH_MULTIPLY))
    return fail(GW_INVALID_ARGUMENT,
                "static-scratch NVFP4 linear requires valid 16-byte aligned device buffers, rows > 0, K divisible by "
                "64, N divisible by 128 and finite positive global scales");
  const size_t scale_offset_bytes = align_up(size_t(rows) * input_width / 2, 256);
  const size_t need = scale_offset_bytes + scale_storage_bytes(rows, input_width);
  if (need > kStaticScratchBytes)
    return fail(GW_INVALID_ARGUMENT,
                "static-scratch NVFP4 linear: rows*K/2 + scale tiles = " + std::to_string(need) +
                    " bytes exceed the built-in scratch of " + std::to_string(kStaticScratchBytes) +
                    " bytes; use gw_nvfp4_plan_run with caller scratch for this size");
  DeviceSlot* slot = nullptr;
  if (gw_status status = resolve_slot(&slot); status != GW_OK) return status;
  cudaStream_t s = as_stream(stream);
  unsigned char* packed = slot->scratch;
  unsigned char* scales = slot->scratch + scale_offset_bytes;
  GW_CUDA_CHECK(launch_nvfp4_quantize(input_bf16, rows, input_width, 1.0F / input_scale,
                                      transform == GW_TRANSFORM_GELU_TANH_MULTIPLY, packed, scales, s),
                "static-scratch NVFP4 quantize activations");
  // descriptors live on this call's stack: nothing is cached, nothing allocated
  DenseDescriptors descriptors;
  DenseProblem problem{GemmKind::nvfp4, rows, input_width, output_width, weight_data, weight_scales, packed, scales,
                       alpha, nullptr, output_bf16, slot->error};
  return launch_dense(problem, &descriptors, s);
}

}  // extern "C"
