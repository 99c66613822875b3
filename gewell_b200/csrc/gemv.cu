// CUDA-core weight-streaming projections for very small row counts: the
// W4A16 path (BF16 activations, NVFP4 weights decoded in registers, FP32
// accumulation).  One warp per output channel; lanes stride over K in
// 32-element pieces (one 16-byte load of packed weights each), partial sums are
// combined with warp shuffles.  HBM-bound: every weight byte is read once.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace gw {
namespace {

constexpr int kMaxRows = 8;
constexpr int kWarpsPerBlock = 8;

template <int ROWS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
gemv_w4a16_kernel(const bf16* __restrict__ input, const uint8_t* __restrict__ data,
                  const uint8_t* __restrict__ scales, float weight_scale, uint32_t width, uint32_t out_width,
                  bf16* __restrict__ output) {
  const uint32_t channel = blockIdx.x * kWarpsPerBlock + threadIdx.x / 32;
  const uint32_t lane = threadIdx.x % 32;
  if (channel >= out_width) return;
  float acc[ROWS];
#pragma unroll
  for (int m = 0; m < ROWS; ++m) acc[m] = 0.0F;
  const uint4* row_data = reinterpret_cast<const uint4*>(data + size_t(channel) * (width / 2));
  for (uint32_t piece = lane; piece < width / 32; piece += 32) {
    const uint4 packed = row_data[piece];
    const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
    // two K16 blocks per piece; their scale bytes are adjacent in the tile
    const uint32_t kb = piece * 2;
    const size_t so = scale_offset(channel, kb, width);
    const float s0 = __fmul_rn(e4m3_to_float(scales[so]), weight_scale);
    const float s1 = __fmul_rn(e4m3_to_float(scales[so + 1]), weight_scale);
    float w[32];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float2 pair = e2m1x2_to_float2((words[i / 4] >> (8 * (i % 4))) & 0xFF);
      const float s = i < 8 ? s0 : s1;
      // the reference's W4A16 path multiplies BF16-rounded weights
      w[2 * i] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(pair.x, s)));
      w[2 * i + 1] = __bfloat162float(__float2bfloat16_rn(__fmul_rn(pair.y, s)));
    }
#pragma unroll
    for (int m = 0; m < ROWS; ++m) {
      const uint4* x = reinterpret_cast<const uint4*>(input + size_t(m) * width + piece * 32);
#pragma unroll
      for (int v = 0; v < 4; ++v) {
        const uint4 raw = x[v];
        const uint32_t xs[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[m] = fmaf(__uint_as_float(xs[i] << 16), w[v * 8 + 2 * i], acc[m]);
          acc[m] = fmaf(__uint_as_float(xs[i] & 0xFFFF0000u), w[v * 8 + 2 * i + 1], acc[m]);
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < ROWS; ++m) {
    for (int offset = 16; offset; offset /= 2) acc[m] += __shfl_xor_sync(0xffffffffu, acc[m], offset);
    if (lane == 0) output[size_t(m) * out_width + channel] = __float2bfloat16_rn(acc[m]);
  }
}

}  // namespace

cudaError_t launch_gemv_w4a16(const void* input, uint32_t rows, const uint8_t* data, const uint8_t* scales,
                              float weight_scale, uint32_t width, uint32_t out_width, void* output,
                              cudaStream_t stream) {
  const unsigned grid = (out_width + kWarpsPerBlock - 1) / kWarpsPerBlock;
  auto* in = static_cast<const bf16*>(input);
  auto* out = static_cast<bf16*>(output);
#define GW_GEMV_CASE(R)                                                                                   \
  case R:                                                                                                 \
    gemv_w4a16_kernel<R><<<grid, kWarpsPerBlock * 32, 0, stream>>>(in, data, scales, weight_scale, width, \
                                                                   out_width, out);                       \
    break;
  switch (rows) {
    GW_GEMV_CASE(1) GW_GEMV_CASE(2) GW_GEMV_CASE(3) GW_GEMV_CASE(4)
    GW_GEMV_CASE(5) GW_GEMV_CASE(6) GW_GEMV_CASE(7) GW_GEMV_CASE(8)
    default: return cudaErrorInvalidValue;
  }
#undef GW_GEMV_CASE
  (void)kMaxRows;
  note_launch();
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// FP8 W8A8 decode projection for one to four rows on the CUDA cores: vectorised,
// coalesced weight streaming with warp-level reductions.  Every block first
// quantises the activations itself (e4m3_sat(x * 1/input_scale), the recipe of
// src/fp8_linear.cu:33-52) into shared memory as FP16, which holds every E4M3
// value exactly, so no separate quantise kernel and no dependency between two
// launches remain.  A warp owns an output channel at a time: its lanes read the
// channel's K bytes in 16-byte pieces (512 contiguous bytes per warp
// instruction, streamed past L1), convert E4M3 -> FP16 -> FP32 and accumulate
// in FP32; the partial sums are folded with shuffles and lane 0 stores
// bf16(sum * alpha_n).  Weight bytes are read exactly once.
// ---------------------------------------------------------------------------
namespace {

constexpr int kGemvFp8MaxRows = 4;
constexpr int kGemvFp8Warps = 8;

__device__ __forceinline__ uint4 load_streaming(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

template <int ROWS>
__global__ void __launch_bounds__(kGemvFp8Warps * 32)
gemv_fp8_kernel(const bf16* __restrict__ input, const uint8_t* __restrict__ weights, float inverse_input_scale,
                float alpha, const float* __restrict__ channel_alpha, uint32_t width, uint32_t out_width,
                bf16* __restrict__ output) {
  extern __shared__ __half x_shared[];          // [ROWS][width] quantised activations as FP16
  for (uint32_t i = threadIdx.x; i < ROWS * width; i += blockDim.x) {
    const float scaled = __fmul_rn(__bfloat162float(input[i]), inverse_input_scale);
    const uint8_t code = float_to_e4m3(scaled);
    x_shared[i] = __half(__nv_cvt_fp8_to_halfraw(code, __NV_E4M3));
  }
  __syncthreads();
  const uint32_t lane = threadIdx.x % 32;
  const uint32_t warps = gridDim.x * kGemvFp8Warps;
  const uint32_t pieces = width / 16;            // 16-byte pieces per channel
  for (uint32_t channel = blockIdx.x * kGemvFp8Warps + threadIdx.x / 32; channel < out_width; channel += warps) {
    const uint4* row = reinterpret_cast<const uint4*>(weights + size_t(channel) * width);
    float acc[ROWS];
#pragma unroll
    for (int m = 0; m < ROWS; ++m) acc[m] = 0.0F;
#pragma unroll 4
    for (uint32_t piece = lane; piece < pieces; piece += 32) {
      const uint4 packed = load_streaming(row + piece);
      const uint32_t words[4] = {packed.x, packed.y, packed.z, packed.w};
      float w[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const __half2 pair = __half2(__nv_cvt_fp8x2_to_halfraw2(uint16_t(words[i / 2] >> (16 * (i % 2))), __NV_E4M3));
        const float2 f = __half22float2(pair);
        w[2 * i] = f.x;
        w[2 * i + 1] = f.y;
      }
#pragma unroll
      for (int m = 0; m < ROWS; ++m) {
        const uint4* xs = reinterpret_cast<const uint4*>(x_shared + size_t(m) * width + piece * 16);
#pragma unroll
        for (int v = 0; v < 2; ++v) {
          const uint4 raw = xs[v];
          const uint32_t xw[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 x2 = __half22float2(*reinterpret_cast<const __half2*>(&xw[i]));
            acc[m] = fmaf(x2.x, w[8 * v + 2 * i], acc[m]);
            acc[m] = fmaf(x2.y, w[8 * v + 2 * i + 1], acc[m]);
          }
        }
      }
    }
    const float scale = channel_alpha != nullptr ? channel_alpha[channel] : alpha;
#pragma unroll
    for (int m = 0; m < ROWS; ++m) {
      float sum = acc[m];
      for (int offset = 16; offset; offset /= 2) sum += __shfl_xor_sync(0xffffffffu, sum, offset);
      if (lane == 0) output[size_t(m) * out_width + channel] = __float2bfloat16_rn(__fmul_rn(sum, scale));
    }
  }
}

template <int ROWS>
cudaError_t launch_gemv_fp8_rows(const void* input, const uint8_t* weights, float inverse_input_scale, float alpha,
                                 const float* channel_alpha, uint32_t width, uint32_t out_width, void* output,
                                 int blocks, cudaStream_t stream) {
  const size_t smem = size_t(ROWS) * width * sizeof(__half);
  static bool configured_on[kMaxDeviceSlots] = {};   // the attribute is per GPU
  bool& configured = configured_on[current_device_slot()];
  if (!configured && smem > 48 * 1024) {
    cudaError_t status = cudaFuncSetAttribute(gemv_fp8_kernel<ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (status != cudaSuccess) return status;
    configured = true;
  }
  gemv_fp8_kernel<ROWS><<<blocks, kGemvFp8Warps * 32, smem, stream>>>(
      static_cast<const bf16*>(input), weights, inverse_input_scale, alpha, channel_alpha, width, out_width,
      static_cast<bf16*>(output));
  note_launch();
  return cudaGetLastError();
}

}  // namespace

bool gemv_fp8_supports(uint32_t rows, uint32_t width) {
  return rows >= 1 && rows <= uint32_t(kGemvFp8MaxRows) && width % 16 == 0 && size_t(rows) * width * 2 <= 96 * 1024;
}

cudaError_t launch_gemv_fp8(const void* input, uint32_t rows, const uint8_t* weights, float inverse_input_scale,
                            float alpha, const float* channel_alpha, uint32_t width, uint32_t out_width, void* output,
                            int sm_count, cudaStream_t stream) {
  // enough resident warps per SM to keep the memory system busy: 4 blocks of 8 warps per SM
  const int blocks = sm_count * 4;
  switch (rows) {
    case 1: return launch_gemv_fp8_rows<1>(input, weights, inverse_input_scale, alpha, channel_alpha, width, out_width, output, blocks, stream);
    case 2: return launch_gemv_fp8_rows<2>(input, weights, inverse_input_scale, alpha, channel_alpha, width, out_width, output, blocks, stream);
    case 3: return launch_gemv_fp8_rows<3>(input, weights, inverse_input_scale, alpha, channel_alpha, width, out_width, output, blocks, stream);
    case 4: return launch_gemv_fp8_rows<4>(input, weights, inverse_input_scale, alpha, channel_alpha, width, out_width, output, blocks, stream);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace gw
