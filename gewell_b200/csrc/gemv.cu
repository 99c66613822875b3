// CUDA-core weight-streaming projections for very small row counts: the
// W4A16 path (BF16 activations, NVFP4 weights decoded in registers, FP32
// accumulation).  One warp per output channel; lanes stride over K in
// 32-element pieces (one 16-byte load of packed weights each), partial sums are
// combined with warp shuffles.  HBM-bound: every weight byte is read once.
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
  return cudaGetLastError();
}

}  // namespace gw
