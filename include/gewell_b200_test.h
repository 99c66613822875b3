/*
 * gewell_b200 -- entry points that exist for the test-suite and for tuning only.
 *
 * They are exported by the same library as include/gewell_b200.h but are not
 * part of the drop-in surface: nothing a caller of the projection / MoE path
 * needs is declared here, and none of them has a counterpart in the reference.
 */
#ifndef GEWELL_B200_TEST_H_
#define GEWELL_B200_TEST_H_

#include "gewell_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Tuning aid: when `device_buffer` (2 x 148 x 8 int64 on the device; consecutive launches alternate between the halves) is not NULL,
 * every later tensor-core GEMM launch writes per-CTA cycle counters into it
 * (producer wait, MMA wait for data, MMA issue, MMA wait for the accumulator,
 * epilogue wait, epilogue work, total, time the direct-store epilogue spends in
 * tensor-memory loads); NULL switches it off again. */
gw_status gw_debug_gemm_profile(void* device_buffer);

/* Test aid: output[i] = rcp.approx.ftz.f32(input[i]) evaluated on the device.
 * The activation recipe (src/nvfp4_linear.cu:92-114) is defined in terms of
 * this instruction, whose last bit a CPU cannot predict; the parity tests feed
 * the hardware's values into the CPU oracle so that the comparison is exact. */
gw_status gw_debug_rcp_approx(const float* input, float* output, uint64_t count, void* stream);

/* Test aid: element-wise GeGLU with both BF16 roundings
 * (src/bf16_activation.cuh:10-16) on the device, so that the CPU oracle can use
 * the device's tanhf bits where a one-ulp difference would flip an FP4 code. */
gw_status gw_debug_geglu_bf16(const void* gate_bf16, const void* up_bf16, void* output_bf16, uint64_t count,
                              void* stream);

/* Number of kernels this library has launched in this process so far (every launch site counts
 * itself).  A benchmark reads it before and after its timed region. */
uint64_t gw_debug_launch_count(void);

/* Test aid: the quantised gate/up input the last gw_moe_run / gw_moe_run_sorted left in the
 * workspace (the output of the reference's quantize_fp4 step, moe.cu:254-304): packed E2M1
 * [parts * 8 * max_rows, 1408] (part 0 = quantised with the gate input scale, part 1 = with the up
 * input scale, present only when those differ) and the tiled E4M3 scales, `scale_rows` rows per
 * part, expert e's region starting at row (offsets[e] / 128 + e) * 128.  Device pointers. */
gw_status gw_debug_moe_quantized_input(const gw_moe_workspace* workspace, const uint8_t** packed,
                                       const uint8_t** scales, uint32_t* scale_rows, uint32_t* part_rows);

/* Test aids of the RMS norms: rsqrtf evaluated on the device for `count` host values (the norm is
 * defined in terms of this approximate instruction), and the number of logical lanes the row
 * reduction uses for a launch of `rows` rows of `width` values. */
gw_status gw_debug_rsqrt(const float* host_input, float* host_output, uint32_t count);
uint32_t gw_rms_norm_reduction_lanes(uint32_t rows, uint32_t width);

#ifdef __cplusplus
}
#endif
#endif /* GEWELL_B200_TEST_H_ */
