// Internal launch functions of the element-wise and MoE kernels.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>

namespace gw {

// quant_kernels.cu
cudaError_t launch_nvfp4_dequantize(const uint8_t* data, const uint8_t* scales, float weight_scale,
                                    uint32_t width, uint32_t rows, void* output, cudaStream_t stream);
cudaError_t launch_nvfp4_pack_weights(const void* weights, uint32_t rows, uint32_t width,
                                      float weight_scale, uint8_t* data, uint8_t* scales, cudaStream_t stream);
cudaError_t launch_nvfp4_quantize(const void* input, uint32_t rows, uint32_t width,
                                  float inverse_global_scale, bool gelu, uint8_t* packed, uint8_t* scales,
                                  cudaStream_t stream);
cudaError_t launch_fp8_quantize(const void* input, uint32_t rows, uint32_t width, float inverse_scale,
                                bool gelu, uint8_t* packed, cudaStream_t stream);
cudaError_t launch_fp8_pack_weights(const void* weights, uint32_t rows, uint32_t width, float scale,
                                    const float* row_scales, uint8_t* data, cudaStream_t stream);
cudaError_t launch_rcp_approx(const float* in, float* out, size_t n, cudaStream_t stream);
cudaError_t launch_geglu(const void* gate, const void* up, void* out, size_t n, cudaStream_t stream);
// [rows, gate | up] (2 * width columns) -> [rows, width]
cudaError_t launch_geglu_interleaved(const void* gate_up, void* out, uint32_t rows, uint32_t width, cudaStream_t stream);
cudaError_t launch_absmax(const void* values, uint64_t elements, uint32_t* state, cudaStream_t stream);
cudaError_t launch_fp8_qdq(void* values, uint64_t elements, float scale, cudaStream_t stream);
cudaError_t launch_nvfp4_qdq(void* values, uint64_t elements, float global_scale, cudaStream_t stream);

// gemv.cu
cudaError_t launch_gemv_w4a16(const void* input, uint32_t rows, const uint8_t* data, const uint8_t* scales,
                              float weight_scale, uint32_t width, uint32_t out_width, void* output,
                              cudaStream_t stream);

// FP8 W8A8 projection for 1..4 rows on the CUDA cores (quantises the activations itself).
bool gemv_fp8_supports(uint32_t rows, uint32_t width);
cudaError_t launch_gemv_fp8(const void* input, uint32_t rows, const uint8_t* weights, float inverse_input_scale,
                            float alpha, const float* channel_alpha, uint32_t width, uint32_t out_width, void* output,
                            int sm_count, cudaStream_t stream);

}  // namespace gw
