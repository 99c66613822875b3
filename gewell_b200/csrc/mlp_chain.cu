// The dense MLP of the 31B model as one unit behind the C ABI: gate + up
// projection, GeGLU, down projection, picking for every step the fastest form
// the layer's weights allow -- Executor::project_mlp and projection_linear of
// the reference (models/gemma4/31b/sm120/executor.cuh:1187-1215,1248-1291) on
// this library's plans:
//
//   gate + up   one joined GEMM over [gate | up] when the loader laid the two matrices out back to
//               back: NVFP4 with FP4 activations (contiguous rows and scale tiles, equal globals),
//               FP8 with per-channel scales, or BF16; otherwise two separate projections
//   GeGLU       fused into the activation quantiser of the down projection when that one runs
//               quantised on a joined [rows, gate | up] tensor; an element-wise kernel otherwise
//   down        FP8, NVFP4 (W4A4) or BF16 GEMM; NVFP4 weights with BF16 activations are
//               dequantised into the chain's scratch first (W4A16)
//
// prepare(rows) builds the plans outside the layer loop; run() allocates nothing.
#include <algorithm>
#include <cmath>
#include <map>
#include <memory>
#include <new>
#include <string>
#include <tuple>

#include "common.cuh"
#include "kernels.h"

using namespace gw;

namespace {

struct Buffer {
  void* data = nullptr;
  size_t bytes = 0;
  cudaError_t allocate(size_t n) {
    bytes = n;
    return n ? cudaMalloc(&data, n) : cudaSuccess;
  }
  ~Buffer() { if (data) cudaFree(data); }
};

enum Kind { kNvfp4 = 0, kFp8 = 1, kFp8Channel = 2, kBf16 = 3 };
using Key = std::tuple<int, uint32_t, uint32_t>;   // kind, K, N

struct PlanSet {
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

uintptr_t address(const void* p) { return reinterpret_cast<uintptr_t>(p); }

// 31b/sm120/nvfp4_projections.h:21-33
bool nvfp4_joined(const gw_projection& gate, const gw_projection& up) {
  return gate.storage == GW_STORAGE_NVFP4_W4A4 && up.storage == GW_STORAGE_NVFP4_W4A4 && gate.nvfp4_data &&
         up.nvfp4_data && gate.nvfp4_scales && up.nvfp4_scales && gate.output % 128 == 0 &&
         gate.nvfp4_input_scale == up.nvfp4_input_scale && gate.nvfp4_weight_scale == up.nvfp4_weight_scale &&
         address(up.nvfp4_data) == address(gate.nvfp4_data) + size_t(gate.output) * gate.input / 2 &&
         address(up.nvfp4_scales) == address(gate.nvfp4_scales) + scale_storage_bytes(gate.output, gate.input);
}
// 31b/sm120/fp8_projections.h:20-50: adjacent matrices, one input scale, per-channel scales for both parts
bool fp8_joined(const gw_projection& gate, const gw_projection& up) {
  return gate.storage == GW_STORAGE_FP8_W8A8 && up.storage == GW_STORAGE_FP8_W8A8 && gate.fp8_data && up.fp8_data &&
         gate.fp8_channel_scales && up.fp8_channel_scales == gate.fp8_channel_scales + gate.output &&
         gate.fp8_input_scale == up.fp8_input_scale &&
         address(up.fp8_data) == address(gate.fp8_data) + size_t(gate.output) * gate.input;
}
// 31b/sm120/projection_fusion.h: BF16 gate and up stored back to back
bool bf16_joined(const gw_projection& gate, const gw_projection& up) {
  return gate.storage == GW_STORAGE_BF16 && up.storage == GW_STORAGE_BF16 && gate.bf16 && up.bf16 &&
         address(up.bf16) == address(gate.bf16) + size_t(gate.output) * gate.input * sizeof(bf16);
}

}  // namespace

struct gw_mlp_chain {
  uint32_t hidden = 0, mlp = 0, max_rows = 0, rows = 0;
  int policy = GW_POLICY_ALWAYS;
  std::map<Key, PlanSet> plans;
  Buffer scratch, dequantized;
  ~gw_mlp_chain() { for (auto& entry : plans) entry.second.reset(); }
};

extern "C" {

gw_status gw_gelu_tanh_multiply_bf16(const void* gate_bf16, const void* up_bf16, void* output_bf16, uint64_t count,
                                     void* stream) {
  clear_error();
  if (!count) return GW_OK;
  if (!gate_bf16 || !up_bf16 || !output_bf16) return fail(GW_INVALID_ARGUMENT, "GeGLU requires three buffers");
  GW_CUDA_CHECK(launch_geglu(gate_bf16, up_bf16, output_bf16, count, as_stream(stream)), "GeGLU");
  return GW_OK;
}

gw_status gw_gelu_tanh_multiply_interleaved_bf16(const void* gate_up_bf16, void* output_bf16, uint32_t rows,
                                                 uint32_t width, void* stream) {
  clear_error();
  if (!rows) return GW_OK;
  if (!gate_up_bf16 || !output_bf16 || !width || width % 8 || address(gate_up_bf16) % 16 || address(output_bf16) % 16)
    return fail(GW_INVALID_ARGUMENT, "interleaved GeGLU requires 16-byte aligned buffers and a width divisible by 8");
  GW_CUDA_CHECK(launch_geglu_interleaved(gate_up_bf16, output_bf16, rows, width, as_stream(stream)), "GeGLU");
  return GW_OK;
}

gw_status gw_mlp_chain_create(uint32_t hidden, uint32_t mlp, uint32_t max_rows, int policy, gw_mlp_chain** chain) {
  clear_error();
  if (!chain || hidden == 0 || mlp == 0 || hidden % 128 || mlp % 128 || max_rows == 0 ||
      (policy != GW_POLICY_ALWAYS && policy != GW_POLICY_PREFILL))
    return fail(GW_INVALID_ARGUMENT, "MLP chain requires hidden and mlp divisible by 128, rows > 0 and a policy");
  auto c = std::unique_ptr<gw_mlp_chain>(new (std::nothrow) gw_mlp_chain());
  if (!c) return fail(GW_CUDA_ERROR, "out of host memory");
  c->hidden = hidden;
  c->mlp = mlp;
  c->max_rows = max_rows;
  c->policy = policy;
  // one scratch for every plan of the chain (they run one after another on one stream)
  const size_t need = std::max({gw_nvfp4_scratch_upper_bound_bytes(max_rows, hidden, 2 * size_t(mlp)),
                                gw_nvfp4_scratch_upper_bound_bytes(max_rows, mlp, hidden),
                                gw_fp8_scratch_upper_bound_bytes(max_rows, std::max(hidden, mlp))});
  cudaError_t status = c->scratch.allocate(need);
  // the widest matrix bounds every dequantised weight: [2 * mlp, hidden] when gate and up are joined
  if (status == cudaSuccess && policy == GW_POLICY_PREFILL)
    status = c->dequantized.allocate(size_t(2) * mlp * hidden * sizeof(bf16));
  if (status != cudaSuccess) return fail(GW_CUDA_ERROR, std::string("MLP chain scratch: ") + cudaGetErrorString(status));
  *chain = c.release();
  return GW_OK;
}

void gw_mlp_chain_destroy(gw_mlp_chain* chain) { delete chain; }

size_t gw_mlp_chain_bytes(const gw_mlp_chain* chain) { return chain ? chain->scratch.bytes + chain->dequantized.bytes : 0; }

gw_status gw_mlp_chain_prepare(gw_mlp_chain* c, uint32_t rows) {
  clear_error();
  if (!c || rows == 0 || rows > c->max_rows)
    return fail(GW_INVALID_ARGUMENT, "MLP chain prepare requires 0 < rows <= the chain's max_rows");
  if (c->rows == rows) return GW_OK;
  std::map<Key, PlanSet> next;
  const uint32_t h = c->hidden, m = c->mlp;
  gw_status status = GW_OK;
  auto add = [&](int kind, uint32_t k, uint32_t n) {
    if (status != GW_OK) return;
    PlanSet& set = next[Key{kind, k, n}];
    if (kind == kNvfp4) status = gw_nvfp4_plan_create(rows, k, n, &set.nvfp4);
    else if (kind == kBf16) status = gw_bf16_plan_create(rows, k, n, &set.bf16);
    else status = gw_fp8_plan_create(rows, k, n, kind == kFp8Channel ? 1 : 0, &set.fp8);
  };
  for (int kind : {kNvfp4, kFp8, kFp8Channel, kBf16}) {
    add(kind, h, m);        // gate or up alone
    add(kind, h, 2 * m);    // joined gate + up
    add(kind, m, h);        // down
  }
  if (status != GW_OK) {
    for (auto& entry : next) entry.second.reset();
    return status;
  }
  for (auto& entry : c->plans) entry.second.reset();
  c->plans = std::move(next);
  c->rows = rows;
  return GW_OK;
}

}  // extern "C"

namespace {

// projection_linear (executor.cuh:1187-1215): FP8 -> NVFP4 with FP4 activations -> BF16 GEMM (on the
// BF16 weight, or on the NVFP4 weight dequantised into the chain's scratch)
gw_status run_linear(gw_mlp_chain* c, const gw_projection& p, const void* input, void* output, bool fp4, int transform,
                     cudaStream_t s) {
  const uint32_t n = p.storage == GW_STORAGE_NVFP4_W4A4 ? p.physical_output : p.output;
  if (p.storage == GW_STORAGE_FP8_W8A8) {
    const int kind = p.fp8_channel_scales ? kFp8Channel : kFp8;
    return gw_fp8_plan_run(c->plans.at(Key{kind, p.input, n}).fp8, input, p.fp8_data, p.fp8_input_scale, p.fp8_weight_scale,
                           p.fp8_channel_scales, output, c->scratch.data, c->scratch.bytes, s, transform);
  }
  if (p.storage == GW_STORAGE_NVFP4_W4A4 && fp4)
    return gw_nvfp4_plan_run(c->plans.at(Key{kNvfp4, p.input, n}).nvfp4, input, p.nvfp4_data, p.nvfp4_scales,
                             p.nvfp4_input_scale, p.nvfp4_weight_scale, output, c->scratch.data, c->scratch.bytes, s,
                             transform);
  if (transform != GW_TRANSFORM_IDENTITY) return fail(GW_INVALID_ARGUMENT, "the BF16 path has no fused input transform");
  const void* weights = p.bf16;
  if (p.storage == GW_STORAGE_NVFP4_W4A4) {
    if (!c->dequantized.data || size_t(n) * p.input * sizeof(bf16) > c->dequantized.bytes)
      return fail(GW_INVALID_ARGUMENT, "NVFP4 BF16 decode workspace is disabled (policy always)");
    const gw_status status = gw_nvfp4_dequantize(p.nvfp4_data, p.nvfp4_scales, p.nvfp4_weight_scale, p.input, n,
                                                 c->dequantized.data, s);
    if (status != GW_OK) return status;
    weights = c->dequantized.data;
  }
  return gw_bf16_plan_run(c->plans.at(Key{kBf16, p.input, n}).bf16, input, weights, output, c->scratch.data,
                          c->scratch.bytes, s);
}

}  // namespace

extern "C" {

gw_status gw_mlp_chain_run(gw_mlp_chain* c, const gw_projection* gate, const gw_projection* up,
                           const gw_projection* down, const void* input_bf16, void* gate_up_bf16, void* product_bf16,
                           void* output_bf16, int phase, void* stream) {
  clear_error();
  if (!c || !gate || !up || !down || !input_bf16 || !gate_up_bf16 || !product_bf16 || !output_bf16 || c->rows == 0 ||
      (phase != GW_PHASE_PREFILL && phase != GW_PHASE_DECODE))
    return fail(GW_INVALID_ARGUMENT, "prepare the MLP chain before run; all buffers are required");
  const uint32_t h = c->hidden, m = c->mlp, rows = c->rows;
  for (const gw_projection* p : {gate, up})
    if (p->input != h || p->output != m || p->physical_output != m)
      return fail(GW_INVALID_ARGUMENT, "gate / up projection does not have the chain's shape");
  if (down->input != m || down->output != h || down->physical_output != h)
    return fail(GW_INVALID_ARGUMENT, "down projection does not have the chain's shape");
  cudaStream_t s = as_stream(stream);
  const bool fp4 = gw_nvfp4_fp4_activations(c->policy, phase) != 0;
  auto* gate_out = static_cast<bf16*>(gate_up_bf16);
  gw_status status = GW_OK;
  bool interleaved = true;       // gate_up holds [rows, gate | up]; otherwise gate rows, then up rows
  if (nvfp4_joined(*gate, *up) && fp4) {
    gw_projection both = *gate;
    both.output = both.physical_output = 2 * m;
    status = run_linear(c, both, input_bf16, gate_out, true, GW_TRANSFORM_IDENTITY, s);
  } else if (fp8_joined(*gate, *up)) {
    gw_projection both = *gate;
    both.output = both.physical_output = 2 * m;
    status = run_linear(c, both, input_bf16, gate_out, fp4, GW_TRANSFORM_IDENTITY, s);
  } else if (bf16_joined(*gate, *up)) {
    gw_projection both = *gate;
    both.output = both.physical_output = 2 * m;
    status = run_linear(c, both, input_bf16, gate_out, fp4, GW_TRANSFORM_IDENTITY, s);
  } else {
    status = run_linear(c, *gate, input_bf16, gate_out, fp4, GW_TRANSFORM_IDENTITY, s);
    if (status == GW_OK) status = run_linear(c, *up, input_bf16, gate_out + size_t(rows) * m, fp4, GW_TRANSFORM_IDENTITY, s);
    interleaved = false;
  }
  if (status != GW_OK) return status;
  const bool down_quantised = down->storage == GW_STORAGE_FP8_W8A8 || (down->storage == GW_STORAGE_NVFP4_W4A4 && fp4);
  if (interleaved && down_quantised)      // GeGLU inside the down projection's activation quantiser
    return run_linear(c, *down, gate_out, output_bf16, fp4, GW_TRANSFORM_GELU_TANH_MULTIPLY, s);
  if (interleaved)
    status = gw_gelu_tanh_multiply_interleaved_bf16(gate_out, product_bf16, rows, m, s);
  else
    status = gw_gelu_tanh_multiply_bf16(gate_out, gate_out + size_t(rows) * m, product_bf16, uint64_t(rows) * m, s);
  if (status != GW_OK) return status;
  return run_linear(c, *down, product_bf16, output_bf16, fp4, GW_TRANSFORM_IDENTITY, s);
}

}  // extern "C"
