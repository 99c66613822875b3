// The feed-forward block of one Gemma-4-26B-A4B layer around the MoE, behind
// the C ABI: the three-output RMS norm that feeds the shared MLP, the router
// and the experts, the shared MLP, the router projection, the MoE layer, the
// three post norms with their residual adds and the layer scalar -- the second
// half of BatchedExecutor's layer loop in the reference
// (models/gemma4/26b_a4b/sm120/batched_executor.cu:250-286) with the element-wise
// math of bf16_math.cuh:17-117.
//
// Every BF16 rounding of the reference is kept, and so is the order of its
// FP32 row reduction (the reference builds without fused multiply-add and
// fixes the order to match a pinned FP32 mean): element i of a row belongs to
// logical lane (i / 4) % lanes and accumulator i % 4, an accumulator adds its
// squares by ascending i, a lane's total is ((a0 + a1) + a2) + a3, and lanes
// fold in a halving tree.  `lanes` depends on the row count and the width.
//
// Here a row is read from HBM once (it stays in shared memory between the
// reduction and the output), and the block's tail -- two post norms, add, the
// third norm, residual add, layer scalar: seven launches in the reference --
// is one kernel with one block per row.
#include <algorithm>
#include <cmath>
#include <memory>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.h"

using namespace gw;

namespace {

constexpr int kNormThreads = 256;
constexpr float kRmsEpsilon = 1e-6F;   // include/gewell/models/gemma4/26b_a4b/model.h:26

uint32_t floor_power_of_two(uint32_t value) {
  uint32_t result = 1;
  while (result * 2 <= value) result *= 2;
  return result;
}

// Logical lanes of the row reduction for a launch of `rows` rows of `width` values: the rule of
// normalize_to (bf16_math.cuh:86-95) -- as many lanes as the width feeds with whole 4-vectors, at most
// 512, shared among up to 16 rows.
uint32_t reduction_lanes(uint32_t rows, uint32_t width) {
  const uint32_t by_width = floor_power_of_two(std::min<uint32_t>(512, std::max<uint32_t>(1, width / 4)));
  const uint32_t by_rows = 512 / floor_power_of_two(std::min<uint32_t>(16, std::max<uint32_t>(1, rows)));
  return std::min(by_width, by_rows);
}

__device__ __forceinline__ float as_float(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 rounded(float v) { return __float2bfloat16_rn(v); }

// Copies one row of `width` BF16 values (width % 8 == 0, 16-byte aligned) into shared memory.
__device__ __forceinline__ void stage_row(const bf16* __restrict__ source, bf16* row, uint32_t width) {
  const uint4* in = reinterpret_cast<const uint4*>(source);
  uint4* out = reinterpret_cast<uint4*>(row);
  for (uint32_t i = threadIdx.x; i < width / 8; i += blockDim.x) out[i] = __ldg(in + i);
}

// 1 / sqrt(mean(row^2) + eps) of the row in shared memory, in the reference's order (see the head of
// this file).  `partial` holds 5 * lanes floats.  Every thread returns the same value.  No fused
// multiply-add anywhere: the reference's translation unit is built with --fmad=false.
__device__ float inverse_rms(const bf16* row, uint32_t width, uint32_t lanes, float inverse_width, float* partial) {
  __syncthreads();                                     // the row is complete; `partial` is free
  const uint32_t accumulators = 4 * lanes;
  for (uint32_t p = threadIdx.x; p < accumulators; p += blockDim.x) {
    float sum = 0.F;
    for (uint32_t i = p; i < width; i += accumulators) {
      const float v = as_float(row[i]);
      sum = __fadd_rn(sum, __fmul_rn(v, v));
    }
    partial[p] = sum;
  }
  __syncthreads();
  float* totals = partial + accumulators;            // lane totals live beside the accumulators
  for (uint32_t lane = threadIdx.x; lane < lanes; lane += blockDim.x) {
    const float4 a = reinterpret_cast<const float4*>(partial)[lane];
    totals[lane] = __fadd_rn(__fadd_rn(__fadd_rn(a.x, a.y), a.z), a.w);
  }
  __syncthreads();
  for (uint32_t stride = lanes / 2; stride; stride /= 2) {
    for (uint32_t lane = threadIdx.x; lane < stride; lane += blockDim.x)
      totals[lane] = __fadd_rn(totals[lane], totals[lane + stride]);
    __syncthreads();
  }
  const float mean = __fadd_rn(__fmul_rn(totals[0], inverse_width), kRmsEpsilon);
  return rsqrtf(mean);
}

struct NormArgs {
  const bf16* input;
  uint32_t width, lanes;
  float inverse_width;
};

// y = bf16(x * inv * w)   (w == nullptr: no weight)       -- NormOutput, bf16_math.cuh:18-24
__global__ void __launch_bounds__(kNormThreads) rms_norm_kernel(NormArgs a, const bf16* __restrict__ weight,
                                                               bf16* __restrict__ output) {
  extern __shared__ __align__(16) unsigned char norm_smem[];
  bf16* row = reinterpret_cast<bf16*>(norm_smem);
  float* partial = reinterpret_cast<float*>(norm_smem + size_t(a.width) * sizeof(bf16));
  stage_row(a.input + size_t(blockIdx.x) * a.width, row, a.width);
  const float inv = inverse_rms(row, a.width, a.lanes, a.inverse_width, partial);
  bf16* out = output + size_t(blockIdx.x) * a.width;
  for (uint32_t i = threadIdx.x; i < a.width; i += blockDim.x) {
    const float x = __fmul_rn(as_float(row[i]), inv);
    out[i] = rounded(weight ? __fmul_rn(x, as_float(weight[i])) : x);
  }
}

struct FeedForwardNormArgs {
  const bf16 *shared_weight, *router_weight, *expert_weight;
  bf16 *shared, *router, *expert;
  float router_scale;                    // 1 / sqrt(width), formed on the host
};

// FeedForwardNormOutput (bf16_math.cuh:25-37): one RMS, three outputs; the router input keeps its three
// separate roundings (unweighted norm, weighted product, final scale).
__global__ void __launch_bounds__(kNormThreads) rms_norm_feedforward_kernel(NormArgs a, FeedForwardNormArgs f) {
  extern __shared__ __align__(16) unsigned char norm_smem[];
  bf16* row = reinterpret_cast<bf16*>(norm_smem);
  float* partial = reinterpret_cast<float*>(norm_smem + size_t(a.width) * sizeof(bf16));
  stage_row(a.input + size_t(blockIdx.x) * a.width, row, a.width);
  const float inv = inverse_rms(row, a.width, a.lanes, a.inverse_width, partial);
  const size_t base = size_t(blockIdx.x) * a.width;
  for (uint32_t i = threadIdx.x; i < a.width; i += blockDim.x) {
    const float x = __fmul_rn(as_float(row[i]), inv);
    f.shared[base + i] = rounded(__fmul_rn(x, as_float(f.shared_weight[i])));
    f.expert[base + i] = rounded(__fmul_rn(x, as_float(f.expert_weight[i])));
    const bf16 weighted = rounded(__fmul_rn(as_float(rounded(x)), as_float(f.router_weight[i])));
    f.router[base + i] = rounded(__fmul_rn(as_float(weighted), f.router_scale));
  }
}

struct TailArgs {
  const bf16 *shared_mlp, *routed;                    // [rows, width]: shared MLP output, MoE output
  const bf16 *norm_shared, *norm_routed, *norm_sum;   // post_feedforward_norm_1, _2, post_feedforward_norm
  const bf16* layer_scalar;                           // [1]
  bf16* hidden;                                       // [rows, width], updated in place
};

// shared = norm1(shared_mlp); branch = norm2(routed); sum = bf16(shared + branch); branch = norm3(sum);
// hidden = bf16(hidden + branch); hidden = bf16(hidden * scalar)        (batched_executor.cu:260,278-285)
__global__ void __launch_bounds__(kNormThreads) ffn_tail_kernel(NormArgs a, TailArgs t) {
  extern __shared__ __align__(16) unsigned char norm_smem[];
  bf16* first = reinterpret_cast<bf16*>(norm_smem);
  bf16* second = first + a.width;
  float* partial = reinterpret_cast<float*>(norm_smem + size_t(2) * a.width * sizeof(bf16));
  const size_t base = size_t(blockIdx.x) * a.width;
  stage_row(t.shared_mlp + base, first, a.width);
  stage_row(t.routed + base, second, a.width);
  const float inv_shared = inverse_rms(first, a.width, a.lanes, a.inverse_width, partial);
  const float inv_routed = inverse_rms(second, a.width, a.lanes, a.inverse_width, partial);
  for (uint32_t i = threadIdx.x; i < a.width; i += blockDim.x) {
    const bf16 shared = rounded(__fmul_rn(__fmul_rn(as_float(first[i]), inv_shared), as_float(t.norm_shared[i])));
    const bf16 branch = rounded(__fmul_rn(__fmul_rn(as_float(second[i]), inv_routed), as_float(t.norm_routed[i])));
    first[i] = rounded(__fadd_rn(as_float(shared), as_float(branch)));
  }
  const float inv_sum = inverse_rms(first, a.width, a.lanes, a.inverse_width, partial);
  const float scalar = as_float(*t.layer_scalar);
  for (uint32_t i = threadIdx.x; i < a.width; i += blockDim.x) {
    const bf16 branch = rounded(__fmul_rn(__fmul_rn(as_float(first[i]), inv_sum), as_float(t.norm_sum[i])));
    const bf16 updated = rounded(__fadd_rn(as_float(t.hidden[base + i]), as_float(branch)));
    t.hidden[base + i] = rounded(__fmul_rn(as_float(updated), scalar));
  }
}

// y = bf16(a + b)                                                       (bf16_math.cuh:109-112)
__global__ void add_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, bf16* __restrict__ y, size_t n) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) y[i] = rounded(__fadd_rn(as_float(a[i]), as_float(b[i])));
}

// x = bf16(x * scalar[0])                                               (batched_executor.cu:30-33)
__global__ void scale_kernel(bf16* __restrict__ x, const bf16* __restrict__ scalar, size_t n) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) x[i] = rounded(__fmul_rn(as_float(x[i]), as_float(*scalar)));
}

__global__ void rsqrt_kernel(const float* in, float* out, uint32_t n) {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = rsqrtf(in[i]);
}

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

gw_status check_norm_shape(uint32_t rows, uint32_t width) {
  if (rows == 0 || width == 0 || width % 8 || width > 16384)
    return fail(GW_INVALID_ARGUMENT, "RMS norm requires rows > 0 and a width divisible by 8, at most 16384");
  return GW_OK;
}

NormArgs norm_args(const void* input, uint32_t rows, uint32_t width) {
  return NormArgs{static_cast<const bf16*>(input), width, reduction_lanes(rows, width), 1.F / float(width)};
}

size_t norm_shared_bytes(uint32_t width, uint32_t lanes, int staged_rows) {
  return size_t(staged_rows) * width * sizeof(bf16) + size_t(5) * lanes * sizeof(float);
}

struct DeviceBuffer {
  void* data = nullptr;
  size_t bytes = 0;
  cudaError_t allocate(size_t n) {
    bytes = n;
    return n ? cudaMalloc(&data, n) : cudaSuccess;
  }
  ~DeviceBuffer() { if (data) cudaFree(data); }
};

constexpr uint32_t kHidden = 2816, kSharedMlp = 2112, kExperts = 128;   // model.h:12-13

}  // namespace

struct gw_ffn_block {
  uint32_t capacity = 0, rows = 0;
  int policy = GW_POLICY_ALWAYS, phase = GW_PHASE_PREFILL;
  cudaStream_t stream = nullptr;
  gw_projection_workspace* projections = nullptr;
  gw_moe_workspace* moe = nullptr;
  DeviceBuffer buffers;                  // one allocation, carved below
  bf16 *normalized = nullptr, *router_input = nullptr, *expert_input = nullptr, *gate = nullptr, *up = nullptr,
       *product = nullptr, *shared_mlp = nullptr, *logits = nullptr, *routed = nullptr;
  ~gw_ffn_block() {
    if (projections) gw_projection_workspace_destroy(projections);
    if (moe) gw_moe_destroy(moe);
  }
};

extern "C" {

gw_status gw_rms_norm_bf16(const void* input_bf16, const void* weight_bf16, void* output_bf16, uint32_t rows,
                           uint32_t width, void* stream) {
  clear_error();
  if (rows == 0) return GW_OK;
  if (gw_status s = check_norm_shape(rows, width); s != GW_OK) return s;
  if (!input_bf16 || !output_bf16 || !aligned16(input_bf16))
    return fail(GW_INVALID_ARGUMENT, "RMS norm requires a 16-byte aligned input and an output");
  const NormArgs a = norm_args(input_bf16, rows, width);
  rms_norm_kernel<<<rows, kNormThreads, norm_shared_bytes(width, a.lanes, 1), as_stream(stream)>>>(
      a, static_cast<const bf16*>(weight_bf16), static_cast<bf16*>(output_bf16));
  note_launch();
  GW_CUDA_CHECK(cudaGetLastError(), "RMS norm");
  return GW_OK;
}

gw_status gw_rms_norm_feedforward_bf16(const void* input_bf16, const void* shared_weight, const void* router_weight,
                                       const void* expert_weight, void* shared_bf16, void* router_bf16,
                                       void* expert_bf16, uint32_t rows, uint32_t width, void* stream) {
  clear_error();
  if (rows == 0) return GW_OK;
  if (gw_status s = check_norm_shape(rows, width); s != GW_OK) return s;
  if (!input_bf16 || !aligned16(input_bf16) || !shared_weight || !router_weight || !expert_weight || !shared_bf16 ||
      !router_bf16 || !expert_bf16)
    return fail(GW_INVALID_ARGUMENT, "feed-forward norm requires its input, three weights and three outputs");
  const NormArgs a = norm_args(input_bf16, rows, width);
  const FeedForwardNormArgs f{static_cast<const bf16*>(shared_weight), static_cast<const bf16*>(router_weight),
                              static_cast<const bf16*>(expert_weight), static_cast<bf16*>(shared_bf16),
                              static_cast<bf16*>(router_bf16), static_cast<bf16*>(expert_bf16),
                              1.F / std::sqrt(float(width))};
  rms_norm_feedforward_kernel<<<rows, kNormThreads, norm_shared_bytes(width, a.lanes, 1), as_stream(stream)>>>(a, f);
  note_launch();
  GW_CUDA_CHECK(cudaGetLastError(), "feed-forward norm");
  return GW_OK;
}

gw_status gw_ffn_tail_bf16(const void* shared_mlp_bf16, const void* routed_bf16, const void* norm_shared_weight,
                           const void* norm_routed_weight, const void* norm_sum_weight, const void* layer_scalar_bf16,
                           void* hidden_bf16, uint32_t rows, uint32_t width, void* stream) {
  clear_error();
  if (rows == 0) return GW_OK;
  if (gw_status s = check_norm_shape(rows, width); s != GW_OK) return s;
  if (!shared_mlp_bf16 || !routed_bf16 || !aligned16(shared_mlp_bf16) || !aligned16(routed_bf16) || !norm_shared_weight ||
      !norm_routed_weight || !norm_sum_weight || !layer_scalar_bf16 || !hidden_bf16)
    return fail(GW_INVALID_ARGUMENT, "feed-forward tail requires two 16-byte aligned inputs, three norm weights, "
                                     "the layer scalar and the hidden state");
  const NormArgs a = norm_args(shared_mlp_bf16, rows, width);
  const TailArgs t{static_cast<const bf16*>(shared_mlp_bf16), static_cast<const bf16*>(routed_bf16),
                   static_cast<const bf16*>(norm_shared_weight), static_cast<const bf16*>(norm_routed_weight),
                   static_cast<const bf16*>(norm_sum_weight), static_cast<const bf16*>(layer_scalar_bf16),
                   static_cast<bf16*>(hidden_bf16)};
  const size_t shared_bytes = norm_shared_bytes(width, a.lanes, 2);
  static bool raised[kMaxDeviceSlots] = {};
  if (shared_bytes > 48 * 1024 && !raised[current_device_slot()]) {
    GW_CUDA_CHECK(cudaFuncSetAttribute(ffn_tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024),
                  "feed-forward tail shared memory");
    raised[current_device_slot()] = true;
  }
  ffn_tail_kernel<<<rows, kNormThreads, shared_bytes, as_stream(stream)>>>(a, t);
  note_launch();
  GW_CUDA_CHECK(cudaGetLastError(), "feed-forward tail");
  return GW_OK;
}

gw_status gw_add_bf16(const void* a_bf16, const void* b_bf16, void* output_bf16, uint64_t count, void* stream) {
  clear_error();
  if (count == 0) return GW_OK;
  if (!a_bf16 || !b_bf16 || !output_bf16) return fail(GW_INVALID_ARGUMENT, "add requires three buffers");
  add_kernel<<<unsigned((count + 255) / 256), 256, 0, as_stream(stream)>>>(
      static_cast<const bf16*>(a_bf16), static_cast<const bf16*>(b_bf16), static_cast<bf16*>(output_bf16), count);
  note_launch();
  GW_CUDA_CHECK(cudaGetLastError(), "add");
  return GW_OK;
}

gw_status gw_scale_bf16(void* values_bf16, const void* scalar_bf16, uint64_t count, void* stream) {
  clear_error();
  if (count == 0) return GW_OK;
  if (!values_bf16 || !scalar_bf16) return fail(GW_INVALID_ARGUMENT, "scale requires values and a device scalar");
  scale_kernel<<<unsigned((count + 255) / 256), 256, 0, as_stream(stream)>>>(static_cast<bf16*>(values_bf16),
                                                                            static_cast<const bf16*>(scalar_bf16), count);
  note_launch();
  GW_CUDA_CHECK(cudaGetLastError(), "scale");
  return GW_OK;
}

gw_status gw_debug_rsqrt(const float* host_in, float* host_out, uint32_t count) {
  clear_error();
  if (count == 0) return GW_OK;
  if (!host_in || !host_out) return fail(GW_INVALID_ARGUMENT, "rsqrt probe requires two host arrays");
  DeviceBuffer in, out;
  GW_CUDA_CHECK(in.allocate(size_t(count) * 4), "rsqrt probe");
  GW_CUDA_CHECK(out.allocate(size_t(count) * 4), "rsqrt probe");
  GW_CUDA_CHECK(cudaMemcpy(in.data, host_in, size_t(count) * 4, cudaMemcpyHostToDevice), "rsqrt probe");
  rsqrt_kernel<<<(count + 255) / 256, 256>>>(static_cast<const float*>(in.data), static_cast<float*>(out.data), count);
  GW_CUDA_CHECK(cudaGetLastError(), "rsqrt probe");
  GW_CUDA_CHECK(cudaMemcpy(host_out, out.data, size_t(count) * 4, cudaMemcpyDeviceToHost), "rsqrt probe");
  return GW_OK;
}

uint32_t gw_rms_norm_reduction_lanes(uint32_t rows, uint32_t width) { return reduction_lanes(rows, width); }

// ---------------------------------------------------------------------------------------------------

gw_status gw_ffn_block_create(const gw_ffn_block_weights* layers, uint32_t count, uint32_t max_rows, int policy,
                              uint32_t moe_flags, void* stream, gw_ffn_block** block) {
  clear_error();
  if (!block || !layers || count == 0 || max_rows == 0 || max_rows > 65536)
    return fail(GW_INVALID_ARGUMENT, "feed-forward block requires layers and 1..65536 rows");
  std::vector<gw_projection> bindings;
  for (uint32_t l = 0; l < count; ++l) {
    const gw_ffn_block_weights& w = layers[l];
    if (w.gate.input != kHidden || w.gate.output != kSharedMlp || w.up.input != kHidden || w.up.output != kSharedMlp ||
        w.down.input != kSharedMlp || w.down.output != kHidden)
      return fail(GW_INVALID_ARGUMENT, "shared MLP projections must be 2816 -> 2112 -> 2816");
    if (!w.router_proj) return fail(GW_INVALID_ARGUMENT, "router projection is required");
    bindings.push_back(w.gate);
    bindings.push_back(w.up);
    bindings.push_back(w.down);
    gw_projection router{};
    router.storage = GW_STORAGE_BF16;
    router.input = kHidden;
    router.output = router.physical_output = kExperts;
    router.bf16 = w.router_proj;
    bindings.push_back(router);
  }
  auto b = std::unique_ptr<gw_ffn_block>(new (std::nothrow) gw_ffn_block());
  if (!b) return fail(GW_CUDA_ERROR, "out of host memory");
  b->capacity = max_rows;
  b->policy = policy;
  b->stream = as_stream(stream);
  gw_status status = gw_projection_workspace_create(bindings.data(), uint32_t(bindings.size()), max_rows, policy, stream,
                                                    &b->projections);
  if (status != GW_OK) return status;
  status = gw_moe_create_ex(max_rows, moe_flags, &b->moe);
  if (status != GW_OK) return status;
  const size_t wide = align_up(size_t(max_rows) * kHidden * sizeof(bf16), 256);
  const size_t narrow = align_up(size_t(max_rows) * kSharedMlp * sizeof(bf16), 256);
  const size_t scores = align_up(size_t(max_rows) * kExperts * sizeof(bf16), 256);
  GW_CUDA_CHECK(b->buffers.allocate(5 * wide + 3 * narrow + scores), "feed-forward block buffers");
  auto* cursor = static_cast<unsigned char*>(b->buffers.data);
  auto carve = [&cursor](size_t bytes) {
    bf16* p = reinterpret_cast<bf16*>(cursor);
    cursor += bytes;
    return p;
  };
  b->normalized = carve(wide);
  b->router_input = carve(wide);
  b->expert_input = carve(wide);
  b->shared_mlp = carve(wide);
  b->routed = carve(wide);
  b->gate = carve(narrow);
  b->up = carve(narrow);
  b->product = carve(narrow);
  b->logits = carve(scores);
  *block = b.release();
  return GW_OK;
}

void gw_ffn_block_destroy(gw_ffn_block* block) { delete block; }

size_t gw_ffn_block_bytes(const gw_ffn_block* b) {
  return b ? b->buffers.bytes + gw_projection_workspace_bytes(b->projections) + gw_moe_bytes(b->moe) : 0;
}

gw_status gw_ffn_block_prepare(gw_ffn_block* b, uint32_t rows, int phase) {
  clear_error();
  if (!b || rows == 0 || rows > b->capacity) return fail(GW_INVALID_ARGUMENT, "feed-forward block: invalid rows");
  const gw_status status = gw_projection_workspace_prepare(b->projections, rows, phase);
  if (status != GW_OK) return status;
  b->rows = rows;
  b->phase = phase;
  return GW_OK;
}

gw_status gw_ffn_block_run(gw_ffn_block* b, const gw_ffn_block_weights* weights, void* hidden_bf16) {
  clear_error();
  if (!b || !weights || !hidden_bf16 || b->rows == 0)
    return fail(GW_INVALID_ARGUMENT, "prepare the feed-forward block before run");
  const gw_ffn_block_weights& w = *weights;
  if (!w.pre_feedforward_norm || !w.router_scale || !w.pre_feedforward_norm_2 || !w.post_feedforward_norm_1 ||
      !w.post_feedforward_norm_2 || !w.post_feedforward_norm || !w.layer_scalar || !w.router_proj ||
      !w.router_per_expert_scale || !w.experts)
    return fail(GW_INVALID_ARGUMENT, "feed-forward block: a weight is missing");
  const uint32_t rows = b->rows;
  void* s = b->stream;
  gw_status status = gw_rms_norm_feedforward_bf16(hidden_bf16, w.pre_feedforward_norm, w.router_scale,
                                                  w.pre_feedforward_norm_2, b->normalized, b->router_input,
                                                  b->expert_input, rows, kHidden, s);
  if (status != GW_OK) return status;
  // shared MLP (batched_executor.cu:256-259)
  if ((status = gw_projection_workspace_run(b->projections, &w.gate, b->normalized, b->gate)) != GW_OK) return status;
  if ((status = gw_projection_workspace_run(b->projections, &w.up, b->normalized, b->up)) != GW_OK) return status;
  if ((status = gw_gelu_tanh_multiply_bf16(b->gate, b->up, b->product, uint64_t(rows) * kSharedMlp, s)) != GW_OK) return status;
  if ((status = gw_projection_workspace_run(b->projections, &w.down, b->product, b->shared_mlp)) != GW_OK) return status;
  // router logits and the experts (batched_executor.cu:262-266)
  gw_projection router{};
  router.storage = GW_STORAGE_BF16;
  router.input = kHidden;
  router.output = router.physical_output = kExperts;
  router.bf16 = w.router_proj;
  if ((status = gw_projection_workspace_run(b->projections, &router, b->router_input, b->logits)) != GW_OK) return status;
  status = gw_moe_run(b->moe, b->expert_input, b->logits, w.router_per_expert_scale, w.experts, b->routed, rows,
                      w.has_bf16, w.has_fp8, w.has_nvfp4, gw_nvfp4_fp4_activations(b->policy, b->phase), s);
  if (status != GW_OK) return status;
  return gw_ffn_tail_bf16(b->shared_mlp, b->routed, w.post_feedforward_norm_1, w.post_feedforward_norm_2,
                          w.post_feedforward_norm, w.layer_scalar, hidden_bf16, rows, kHidden, s);
}

const void* gw_ffn_block_buffer(const gw_ffn_block* b, int which) {
  if (!b) return nullptr;
  switch (which) {
    case GW_FFN_NORMALIZED: return b->normalized;
    case GW_FFN_ROUTER_INPUT: return b->router_input;
    case GW_FFN_EXPERT_INPUT: return b->expert_input;
    case GW_FFN_SHARED_MLP: return b->shared_mlp;
    case GW_FFN_ROUTER_LOGITS: return b->logits;
    case GW_FFN_ROUTED: return b->routed;
    default: return nullptr;
  }
}

gw_moe_workspace* gw_ffn_block_moe(gw_ffn_block* b) { return b ? b->moe : nullptr; }

}  // extern "C"
