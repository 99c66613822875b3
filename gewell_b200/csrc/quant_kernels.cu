// HBM-bound element-wise kernels of the quantised-projection path: weight
// dequantise / pack / fake-quant and activation quantisation (NVFP4 and FP8,
// with optional fused GeGLU).  All are pure streaming kernels: 16- or 32-byte
// vector accesses, one K16 block (or eight FP8 values) per thread.
#include "common.cuh"
#include "kernels.h"

#include <cmath>

namespace gw {
namespace {

constexpr int kThreads = 256;

struct alignas(16) Bf16x8 { uint4 v; };

__device__ __forceinline__ void unpack8(const uint4& raw, float* out) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&pair);
}

// ---------------------------------------------------------------------------
// NVFP4 weight dequantise: one thread per K16 block (8 packed bytes in,
// 32 bytes of BF16 out).  Reference: src/nvfp4_linear.cu:39-56.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
nvfp4_dequantize_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ scales,
                        float weight_scale, uint32_t width, size_t blocks, uint4* __restrict__ output) {
  const size_t block = size_t(blockIdx.x) * kThreads + threadIdx.x;
  if (block >= blocks) return;
  const uint32_t blocks_per_row = width / 16;
  const size_t row = block / blocks_per_row;
  const uint32_t kb = block % blocks_per_row;
  const float scale = __fmul_rn(e4m3_to_float(scales[scale_offset(row, kb, width)]), weight_scale);
  const uint2 packed = reinterpret_cast<const uint2*>(data)[block];
  const uint32_t words[2] = {packed.x, packed.y};
  uint32_t out[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 pair = e2m1x2_to_float2((words[i / 4] >> (8 * (i % 4))) & 0xFF);
    out[i] = pack_bf16x2(__fmul_rn(pair.x, scale), __fmul_rn(pair.y, scale));
  }
  output[2 * block] = make_uint4(out[0], out[1], out[2], out[3]);
  output[2 * block + 1] = make_uint4(out[4], out[5], out[6], out[7]);
}

// ---------------------------------------------------------------------------
// NVFP4 weight pack: tools/convert.py:111-137 / src/weight_qdq_detail.cuh:73-82.
// One thread per (row in the 128-padded grid, K16 block in the 4-padded grid)
// so that every byte of the scale storage is written (padding = 0).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
nvfp4_pack_weights_kernel(const uint4* __restrict__ weights, uint32_t rows, uint32_t width,
                          float global_scale, uint2* __restrict__ data, uint8_t* __restrict__ scales,
                          size_t padded_blocks, uint32_t padded_blocks_per_row) {
  const size_t index = size_t(blockIdx.x) * kThreads + threadIdx.x;
  if (index >= padded_blocks) return;
  const size_t row = index / padded_blocks_per_row;
  const uint32_t kb = index % padded_blocks_per_row;
  const uint32_t blocks_per_row = width / 16;
  uint8_t scale_code = 0;
  if (row < rows && kb < blocks_per_row) {
    const size_t block = row * blocks_per_row + kb;
    float values[16];
    unpack8(weights[2 * block], values);
    unpack8(weights[2 * block + 1], values + 8);
    float amax = 0.0F;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(values[i]));
    float unrounded = 1.0F;
    if (amax != 0.0F)
      unrounded = fminf(448.0F, fmaxf(0x1p-9F, __fdiv_rn(amax, __fmul_rn(6.0F, global_scale))));
    scale_code = float_to_e4m3(unrounded);
    const float decoded = __fmul_rn(e4m3_to_float(scale_code), global_scale);
    uint32_t words[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t byte = float2_to_e2m1x2(__fdiv_rn(values[2 * i], decoded),
                                             __fdiv_rn(values[2 * i + 1], decoded));
      words[i / 4] |= byte << (8 * (i % 4));
    }
    data[block] = make_uint2(words[0], words[1]);
  }
  scales[scale_offset(row, kb, width)] = scale_code;
}

// ---------------------------------------------------------------------------
// NVFP4 activation quantise (+GeGLU): src/nvfp4_linear.cu:61-116.  The three
// approximate reciprocals and the FP32 multiply order are the reference's.
// One thread per scale-storage entry; entries outside [rows, K/16] are the
// zero padding of the scale tiles.
// ---------------------------------------------------------------------------
template <bool Gelu>
__global__ void __launch_bounds__(kThreads)
nvfp4_quantize_kernel(const uint4* __restrict__ input, uint32_t rows, uint32_t width,
                      float inverse_global_scale, uint2* __restrict__ packed,
                      uint8_t* __restrict__ scales, size_t padded_blocks,
                      uint32_t padded_blocks_per_row) {
  griddep_launch();   // the GEMM that follows may set itself up while this kernel runs
  const size_t index = size_t(blockIdx.x) * kThreads + threadIdx.x;
  if (index >= padded_blocks) return;
  const size_t row = index / padded_blocks_per_row;
  const uint32_t kb = index % padded_blocks_per_row;
  const uint32_t blocks_per_row = width / 16;
  uint8_t scale_code = 0;
  if (row < rows && kb < blocks_per_row) {
    float values[16];
    if constexpr (Gelu) {
      // input is [rows, 2K]: gate slice then up slice
      const size_t gate = row * (2 * blocks_per_row) + kb;
      float g[16], u[16];
      unpack8(input[2 * gate], g);
      unpack8(input[2 * gate + 1], g + 8);
      unpack8(input[2 * (gate + blocks_per_row)], u);
      unpack8(input[2 * (gate + blocks_per_row) + 1], u + 8);
#pragma unroll
      for (int i = 0; i < 16; ++i) values[i] = gelu_tanh_multiply_bf16(g[i], u[i]);
    } else {
      const size_t block = row * blocks_per_row + kb;
      unpack8(input[2 * block], values);
      unpack8(input[2 * block + 1], values + 8);
    }
    float amax = 0.0F;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(values[i]));
    scale_code = float_to_e4m3(inverse_global_scale * (amax * rcp_approx_ftz(6.0F)));
    const float block_scale = e4m3_to_float(scale_code);
    const float factor = block_scale == 0.0F
                             ? 0.0F
                             : rcp_approx_ftz(block_scale * rcp_approx_ftz(inverse_global_scale));
    uint32_t words[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t byte = float2_to_e2m1x2(values[2 * i] * factor, values[2 * i + 1] * factor);
      words[i / 4] |= byte << (8 * (i % 4));
    }
    packed[row * blocks_per_row + kb] = make_uint2(words[0], words[1]);
  }
  scales[scale_offset(row, kb, width)] = scale_code;
}

// ---------------------------------------------------------------------------
// FP8 activation quantise (+GeGLU): src/fp8_linear.cu:33-52.  Eight values per
// thread (16-byte load, 8-byte store).  width % 16 == 0 keeps rows 16B aligned
// when the input pointer is; a 2-byte-aligned input takes the scalar kernel.
// ---------------------------------------------------------------------------
template <bool Gelu, bool Vector>
__global__ void __launch_bounds__(kThreads)
fp8_quantize_kernel(const bf16* __restrict__ input, size_t groups, uint32_t width, float inverse_scale,
                    uint2* __restrict__ packed) {
  griddep_launch();   // the GEMM that follows may set itself up while this kernel runs
  for (size_t group = size_t(blockIdx.x) * kThreads + threadIdx.x; group < groups;
       group += size_t(gridDim.x) * kThreads) {
    const size_t row = group / (width / 8);
    const uint32_t col = (group % (width / 8)) * 8;
    float values[8];
    auto load8 = [&](const bf16* src, float* dst) {
      if constexpr (Vector) {
        unpack8(*reinterpret_cast<const uint4*>(src), dst);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) dst[i] = __bfloat162float(src[i]);
      }
    };
    if constexpr (Gelu) {
      float g[8], u[8];
      load8(input + row * 2 * width + col, g);
      load8(input + row * 2 * width + width + col, u);
#pragma unroll
      for (int i = 0; i < 8; ++i) values[i] = gelu_tanh_multiply_bf16(g[i], u[i]);
    } else {
      load8(input + row * width + col, values);
    }
    uint32_t words[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t pair = __nv_cvt_float2_to_fp8x2(
          make_float2(__fmul_rn(values[2 * i], inverse_scale), __fmul_rn(values[2 * i + 1], inverse_scale)),
          __NV_SATFINITE, __NV_E4M3);
      words[i / 2] |= pair << (16 * (i % 2));
    }
    packed[group] = make_uint2(words[0], words[1]);
  }
}

// FP8 weight pack: tools/convert.py:49-62 (code = e4m3(x / scale)).
__global__ void __launch_bounds__(kThreads)
fp8_pack_weights_kernel(const uint4* __restrict__ weights, size_t groups, uint32_t width, float scale,
                        const float* __restrict__ row_scales, uint2* __restrict__ data) {
  for (size_t group = size_t(blockIdx.x) * kThreads + threadIdx.x; group < groups;
       group += size_t(gridDim.x) * kThreads) {
    const float s = row_scales ? row_scales[group / (width / 8)] : scale;
    float values[8];
    unpack8(weights[group], values);
    uint32_t words[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t pair = __nv_cvt_float2_to_fp8x2(
          make_float2(__fdiv_rn(values[2 * i], s), __fdiv_rn(values[2 * i + 1], s)), __NV_SATFINITE,
          __NV_E4M3);
      words[i / 2] |= pair << (16 * (i % 2));
    }
    data[group] = make_uint2(words[0], words[1]);
  }
}

// ---------------------------------------------------------------------------
// Weight QDQ: src/weight_qdq.cu:105-189.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
absmax_kernel(const bf16* __restrict__ values, uint64_t elements, uint32_t* __restrict__ state) {
  float local = 0.0F;
  bool bad = false;
  for (uint64_t i = uint64_t(blockIdx.x) * kThreads + threadIdx.x; i < elements;
       i += uint64_t(gridDim.x) * kThreads) {
    const float v = __bfloat162float(values[i]);
    if (!isfinite(v)) bad = true; else local = fmaxf(local, fabsf(v));
  }
  for (int offset = 16; offset; offset /= 2)
    local = fmaxf(local, __shfl_xor_sync(0xffffffffu, local, offset));
  bad = __any_sync(0xffffffffu, bad);
  __shared__ float warp_max[kThreads / 32];
  __shared__ int warp_bad[kThreads / 32];
  if (threadIdx.x % 32 == 0) { warp_max[threadIdx.x / 32] = local; warp_bad[threadIdx.x / 32] = bad; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 0; w < kThreads / 32; ++w) { local = fmaxf(local, warp_max[w]); bad |= warp_bad[w] != 0; }
    atomicMax(state, __float_as_uint(local));   // non-negative floats order like their bits
    if (bad) atomicExch(state + 1, 1u);
  }
}

__global__ void __launch_bounds__(kThreads)
fp8_qdq_kernel(bf16* __restrict__ values, uint64_t elements, float scale) {
  for (uint64_t i = uint64_t(blockIdx.x) * kThreads + threadIdx.x; i < elements;
       i += uint64_t(gridDim.x) * kThreads) {
    const float normalized = __fdiv_rn(__bfloat162float(values[i]), scale);
    values[i] = __float2bfloat16_rn(__fmul_rn(e4m3_to_float(float_to_e4m3(normalized)), scale));
  }
}

// One thread per K16 block of the flat tensor (32-byte load and store).
__global__ void __launch_bounds__(kThreads)
nvfp4_qdq_kernel(uint4* __restrict__ values, uint64_t blocks, float global_scale) {
  for (uint64_t block = uint64_t(blockIdx.x) * kThreads + threadIdx.x; block < blocks;
       block += uint64_t(gridDim.x) * kThreads) {
    float v[16];
    unpack8(values[2 * block], v);
    unpack8(values[2 * block + 1], v + 8);
    float amax = 0.0F;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    float block_scale = 1.0F;
    if (amax != 0.0F) {
      const float clamped =
          fminf(448.0F, fmaxf(0x1p-9F, __fdiv_rn(amax, __fmul_rn(6.0F, global_scale))));
      block_scale = e4m3_to_float(float_to_e4m3(clamped));
    }
    const float combined = __fmul_rn(block_scale, global_scale);
    uint32_t out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 q = e2m1x2_to_float2(
          float2_to_e2m1x2(__fdiv_rn(v[2 * i], combined), __fdiv_rn(v[2 * i + 1], combined)));
      out[i] = pack_bf16x2(__fmul_rn(q.x, combined), __fmul_rn(q.y, combined));
    }
    values[2 * block] = make_uint4(out[0], out[1], out[2], out[3]);
    values[2 * block + 1] = make_uint4(out[4], out[5], out[6], out[7]);
  }
}

__global__ void rcp_approx_kernel(const float* __restrict__ in, float* __restrict__ out, size_t n) {
  const size_t i = size_t(blockIdx.x) * kThreads + threadIdx.x;
  if (i < n) out[i] = rcp_approx_ftz(in[i]);
}

__global__ void geglu_kernel(const bf16* __restrict__ gate, const bf16* __restrict__ up, bf16* __restrict__ out, size_t n) {
  const size_t i = size_t(blockIdx.x) * kThreads + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16_rn(gelu_tanh_multiply_bf16(__bfloat162float(gate[i]), __bfloat162float(up[i])));
}

// [rows, gate | up] -> [rows, width]: eight channels per thread, 16-byte loads and stores
__global__ void geglu_interleaved_kernel(const uint4* __restrict__ gate_up, uint4* __restrict__ out, size_t vectors,
                                         uint32_t row_vectors) {
  const size_t i = size_t(blockIdx.x) * kThreads + threadIdx.x;
  if (i >= vectors) return;
  const size_t row = i / row_vectors, v = i % row_vectors;
  const uint4 g = gate_up[row * 2 * row_vectors + v], u = gate_up[row * 2 * row_vectors + row_vectors + v];
  const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
  uint32_t words[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float a = gelu_tanh_multiply_bf16(__uint_as_float(gw[k] << 16), __uint_as_float(uw[k] << 16));
    const float b = gelu_tanh_multiply_bf16(__uint_as_float(gw[k] & 0xFFFF0000u), __uint_as_float(uw[k] & 0xFFFF0000u));
    words[k] = (__float_as_uint(a) >> 16) | (__float_as_uint(b) & 0xFFFF0000u);
  }
  out[i] = make_uint4(words[0], words[1], words[2], words[3]);
}

unsigned grid_for(size_t items, size_t cap = 1u << 20) {
  size_t blocks = (items + kThreads - 1) / kThreads;
  if (blocks < 1) blocks = 1;
  if (blocks > cap) blocks = cap;
  return static_cast<unsigned>(blocks);
}

}  // namespace

cudaError_t launch_nvfp4_dequantize(const uint8_t* data, const uint8_t* scales, float weight_scale,
                                    uint32_t width, uint32_t rows, void* output, cudaStream_t stream) {
  const size_t blocks = size_t(rows) * (width / 16);
  nvfp4_dequantize_kernel<<<grid_for(blocks, ~0u), kThreads, 0, stream>>>(
      data, scales, weight_scale, width, blocks, static_cast<uint4*>(output));
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_nvfp4_pack_weights(const void* weights, uint32_t rows, uint32_t width,
                                      float weight_scale, uint8_t* data, uint8_t* scales,
                                      cudaStream_t stream) {
  const uint32_t padded_bpr = (width + 63) / 64 * 4;
  const size_t padded = size_t((rows + 127) / 128 * 128) * padded_bpr;
  nvfp4_pack_weights_kernel<<<grid_for(padded, ~0u), kThreads, 0, stream>>>(
      static_cast<const uint4*>(weights), rows, width, weight_scale, reinterpret_cast<uint2*>(data),
      scales, padded, padded_bpr);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_nvfp4_quantize(const void* input, uint32_t rows, uint32_t width,
                                  float inverse_global_scale, bool gelu, uint8_t* packed,
                                  uint8_t* scales, cudaStream_t stream) {
  const uint32_t padded_bpr = (width + 63) / 64 * 4;
  const size_t padded = size_t((rows + 127) / 128 * 128) * padded_bpr;
  auto* in = static_cast<const uint4*>(input);
  auto* out = reinterpret_cast<uint2*>(packed);
  if (gelu)
    nvfp4_quantize_kernel<true><<<grid_for(padded, ~0u), kThreads, 0, stream>>>(
        in, rows, width, inverse_global_scale, out, scales, padded, padded_bpr);
  else
    nvfp4_quantize_kernel<false><<<grid_for(padded, ~0u), kThreads, 0, stream>>>(
        in, rows, width, inverse_global_scale, out, scales, padded, padded_bpr);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_fp8_quantize(const void* input, uint32_t rows, uint32_t width, float inverse_scale,
                                bool gelu, uint8_t* packed, cudaStream_t stream) {
  const size_t groups = size_t(rows) * (width / 8);
  const bool vector = reinterpret_cast<uintptr_t>(input) % 16 == 0;
  auto* in = static_cast<const bf16*>(input);
  auto* out = reinterpret_cast<uint2*>(packed);
  const unsigned grid = grid_for(groups, 148 * 32);
  if (gelu && vector) fp8_quantize_kernel<true, true><<<grid, kThreads, 0, stream>>>(in, groups, width, inverse_scale, out);
  else if (gelu) fp8_quantize_kernel<true, false><<<grid, kThreads, 0, stream>>>(in, groups, width, inverse_scale, out);
  else if (vector) fp8_quantize_kernel<false, true><<<grid, kThreads, 0, stream>>>(in, groups, width, inverse_scale, out);
  else fp8_quantize_kernel<false, false><<<grid, kThreads, 0, stream>>>(in, groups, width, inverse_scale, out);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_fp8_pack_weights(const void* weights, uint32_t rows, uint32_t width, float scale,
                                    const float* row_scales, uint8_t* data, cudaStream_t stream) {
  const size_t groups = size_t(rows) * (width / 8);
  fp8_pack_weights_kernel<<<grid_for(groups, 148 * 32), kThreads, 0, stream>>>(
      static_cast<const uint4*>(weights), groups, width, scale, row_scales, reinterpret_cast<uint2*>(data));
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_rcp_approx(const float* in, float* out, size_t n, cudaStream_t stream) {
  rcp_approx_kernel<<<grid_for(n, ~0u), kThreads, 0, stream>>>(in, out, n);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_geglu(const void* gate, const void* up, void* out, size_t n, cudaStream_t stream) {
  geglu_kernel<<<grid_for(n, ~0u), kThreads, 0, stream>>>(static_cast<const bf16*>(gate), static_cast<const bf16*>(up),
                                                          static_cast<bf16*>(out), n);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_geglu_interleaved(const void* gate_up, void* out, uint32_t rows, uint32_t width, cudaStream_t stream) {
  const size_t vectors = size_t(rows) * (width / 8);
  geglu_interleaved_kernel<<<grid_for(vectors, ~0u), kThreads, 0, stream>>>(static_cast<const uint4*>(gate_up),
                                                                            static_cast<uint4*>(out), vectors, width / 8);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_absmax(const void* values, uint64_t elements, uint32_t* state, cudaStream_t stream) {
  cudaError_t status = cudaMemsetAsync(state, 0, 2 * sizeof(uint32_t), stream);
  if (status != cudaSuccess) return status;
  absmax_kernel<<<grid_for(elements, 148 * 16), kThreads, 0, stream>>>(
      static_cast<const bf16*>(values), elements, state);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_fp8_qdq(void* values, uint64_t elements, float scale, cudaStream_t stream) {
  fp8_qdq_kernel<<<grid_for(elements, 148 * 16), kThreads, 0, stream>>>(static_cast<bf16*>(values), elements, scale);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_nvfp4_qdq(void* values, uint64_t elements, float global_scale, cudaStream_t stream) {
  nvfp4_qdq_kernel<<<grid_for(elements / 16, 148 * 16), kThreads, 0, stream>>>(
      static_cast<uint4*>(values), elements / 16, global_scale);
  note_launch();
  return cudaGetLastError();
}

}  // namespace gw
