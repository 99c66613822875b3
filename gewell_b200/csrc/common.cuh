// Shared host/device helpers of the gewell_b200 kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

#include "../../include/gewell_b200.h"
#include "../../include/gewell_b200_test.h"

namespace gw {

// ---------------------------------------------------------------------------
// host: status + error message plumbing
// ---------------------------------------------------------------------------
gw_status fail(gw_status code, const std::string& message);
void clear_error();

#define GW_CUDA_CHECK(expr, what)                                                          \
  do {                                                                                     \
    cudaError_t gw_cuda_status_ = (expr);                                                  \
    if (gw_cuda_status_ != cudaSuccess)                                                    \
      return ::gw::fail(GW_CUDA_ERROR, std::string(what) + ": " + cudaGetErrorString(gw_cuda_status_)); \
  } while (0)

inline size_t align_up(size_t value, size_t alignment) {
  return (value + alignment - 1) / alignment * alignment;
}

inline cudaStream_t as_stream(void* stream) { return static_cast<cudaStream_t>(stream); }

// Per-GPU state (keyed by the device that is current at the call).
constexpr int kMaxDeviceSlots = 64;
int current_device_slot();
// Error word written by bounded waits (0 = no error): lazily allocated, one per GPU.
uint32_t* device_error_word();
int sm_count();
// Counts the kernels this library launches (read by gw_debug_launch_count); every launch site calls it.
void note_launch(unsigned kernels = 1);
// Error word of the allocation-free linear (static_scratch.cu) on the current GPU, cleared on read;
// 0 when that entry point has not run on this GPU.
uint32_t take_static_scratch_error();

constexpr size_t scale_storage_bytes(size_t rows, size_t width) {
  return ((rows + 127) / 128) * ((width + 63) / 64) * 512;
}

// ---------------------------------------------------------------------------
// device: number formats
// ---------------------------------------------------------------------------
using bf16 = __nv_bfloat16;

__host__ __device__ __forceinline__ size_t scale_offset(size_t row, size_t block, size_t width) {
  return ((row / 128) * (width / 64) + block / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 +
         block % 4;
}

#ifdef __CUDACC__
// Programmatic dependent launch.  A kernel launched with the programmatic-
// serialisation attribute may start while its predecessor in the stream still
// runs; griddep_wait() blocks until that predecessor has completed and its
// writes are visible (no-op for a normal launch).  griddep_launch() lets the
// successor start being scheduled.  Every kernel that can be launched that way
// calls griddep_wait() in all threads before touching global memory, so the
// usual stream order still holds transitively.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#endif  // __CUDACC__

// Launch with the programmatic-serialisation attribute: the kernel may be scheduled while
// its predecessor in the stream drains; it must call griddep_wait() before it touches global
// memory (every kernel launched through this helper does so first thing).
template <typename... Params, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(Params...), dim3 grid, dim3 block, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  note_launch();
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

#ifdef __CUDACC__
__device__ __forceinline__ float rcp_approx_ftz(float value) {
  float result;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(result) : "f"(value));
  return result;
}

__device__ __forceinline__ float e4m3_to_float(uint8_t code) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(code, __NV_E4M3)));
}

__device__ __forceinline__ uint8_t float_to_e4m3(float value) {
  return __nv_cvt_float_to_fp8(value, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ float2 e2m1x2_to_float2(uint8_t packed) {
  return __half22float2(__half2(__nv_cvt_fp4x2_to_halfraw2(packed, __NV_E2M1)));
}

__device__ __forceinline__ uint8_t float2_to_e2m1x2(float lo, float hi) {
  return __nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest);
}

// GeGLU with both BF16 rounding boundaries kept: FP32 operation order of the
// reference's gelu_tanh_multiply_bf16 (src/bf16_activation.cuh:10-16).
__device__ __forceinline__ float gelu_tanh_multiply_bf16(float gate, float up) {
  const float cube = gate * gate * gate;
  const float inner = 0.7978845608028654F * (gate + 0.044715F * cube);
  const float activated = 0.5F * gate * (1.0F + tanhf(inner));
  const bf16 rounded = __float2bfloat16_rn(activated);
  return __bfloat162float(__float2bfloat16_rn(__bfloat162float(rounded) * up));
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}
#endif  // __CUDACC__

}  // namespace gw
