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
//
// The attention input projections of a layer follow the same rules
// (Executor::project_qkv, executor.cuh:1218-1247): one joined GEMM over
// [Q | K | V] for adjacent BF16 matrices or adjacent FP8 matrices with
// per-channel scales, three projections otherwise.  The joins the loader makes
// in place (Weights, weights.cuh:146-223) are gw_join_nvfp4_pair and
// gw_join_fp8_group.
#include <algorithm>
#include <cmath>
#include <map>
#include <memory>
#include <new>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

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

// Plans of one object (all for the same row count), its scratch and the buffer NVFP4 weights are
// dequantised into when they run with BF16 activations.
struct PlanBook {
  uint32_t max_rows = 0, rows = 0;
  int policy = GW_POLICY_ALWAYS;
  std::map<Key, PlanSet> plans;
  Buffer scratch, dequantized;
  ~PlanBook() { for (auto& entry : plans) entry.second.reset(); }

  // shapes: (K, N) pairs; scratch for the widest of them, the dequantised buffer for the largest
  cudaError_t allocate(uint32_t rows_limit, int activation_policy, const std::vector<std::pair<uint32_t, uint32_t>>& shapes) {
    max_rows = rows_limit;
    policy = activation_policy;
    size_t need = 0, largest = 0;
    for (const auto& [k, n] : shapes) {
      need = std::max({need, size_t(gw_nvfp4_scratch_upper_bound_bytes(max_rows, k, n)),
                       size_t(gw_fp8_scratch_upper_bound_bytes(max_rows, k))});
      largest = std::max(largest, size_t(k) * n);
    }
    cudaError_t status = scratch.allocate(need);
    if (status == cudaSuccess && policy == GW_POLICY_PREFILL) status = dequantized.allocate(largest * sizeof(bf16));
    return status;
  }

  gw_status prepare(uint32_t new_rows, const std::vector<std::pair<uint32_t, uint32_t>>& shapes) {
    if (new_rows == 0 || new_rows > max_rows)
      return fail(GW_INVALID_ARGUMENT, "prepare requires 0 < rows <= the object's max_rows");
    if (rows == new_rows) return GW_OK;
    std::map<Key, PlanSet> next;
    gw_status status = GW_OK;
    for (int kind : {kNvfp4, kFp8, kFp8Channel, kBf16})
      for (const auto& [k, n] : shapes) {
        if (status != GW_OK) break;
        PlanSet& set = next[Key{kind, k, n}];
        if (set.nvfp4 || set.fp8 || set.bf16) continue;        // the same shape listed twice
        if (kind == kNvfp4) status = gw_nvfp4_plan_create(new_rows, k, n, &set.nvfp4);
        else if (kind == kBf16) status = gw_bf16_plan_create(new_rows, k, n, &set.bf16);
        else status = gw_fp8_plan_create(new_rows, k, n, kind == kFp8Channel ? 1 : 0, &set.fp8);
      }
    if (status != GW_OK) {
      for (auto& entry : next) entry.second.reset();
      return status;
    }
    for (auto& entry : plans) entry.second.reset();
    plans = std::move(next);
    rows = new_rows;
    return GW_OK;
  }
};

}  // namespace

struct gw_mlp_chain {
  uint32_t hidden = 0, mlp = 0;
  PlanBook book;
  std::vector<std::pair<uint32_t, uint32_t>> shapes() const { return {{hidden, mlp}, {hidden, 2 * mlp}, {mlp, hidden}}; }
};

struct gw_qkv_projector {
  uint32_t hidden = 0, q = 0, kv = 0;
  PlanBook book;
  std::vector<std::pair<uint32_t, uint32_t>> shapes() const {
    return {{hidden, q}, {hidden, kv}, {hidden, q + kv}, {hidden, q + 2 * kv}};
  }
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
  // one scratch for every plan of the chain (they run one after another on one stream); the widest
  // matrix bounds every dequantised weight: [2 * mlp, hidden] when gate and up are joined
  const cudaError_t status = c->book.allocate(max_rows, policy, c->shapes());
  if (status != cudaSuccess) return fail(GW_CUDA_ERROR, std::string("MLP chain scratch: ") + cudaGetErrorString(status));
  *chain = c.release();
  return GW_OK;
}

void gw_mlp_chain_destroy(gw_mlp_chain* chain) { delete chain; }

size_t gw_mlp_chain_bytes(const gw_mlp_chain* chain) {
  return chain ? chain->book.scratch.bytes + chain->book.dequantized.bytes : 0;
}

gw_status gw_mlp_chain_prepare(gw_mlp_chain* c, uint32_t rows) {
  clear_error();
  if (!c) return fail(GW_INVALID_ARGUMENT, "MLP chain prepare requires a chain");
  return c->book.prepare(rows, c->shapes());
}

gw_status gw_qkv_projector_create(uint32_t hidden, uint32_t q_width, uint32_t kv_width, uint32_t max_rows, int policy,
                                  gw_qkv_projector** projector) {
  clear_error();
  if (!projector || hidden == 0 || hidden % 128 || q_width == 0 || q_width % 128 || kv_width == 0 || kv_width % 128 ||
      max_rows == 0 || (policy != GW_POLICY_ALWAYS && policy != GW_POLICY_PREFILL))
    return fail(GW_INVALID_ARGUMENT, "QKV projector requires widths divisible by 128, rows > 0 and a policy");
  auto q = std::unique_ptr<gw_qkv_projector>(new (std::nothrow) gw_qkv_projector());
  if (!q) return fail(GW_CUDA_ERROR, "out of host memory");
  q->hidden = hidden;
  q->q = q_width;
  q->kv = kv_width;
  const cudaError_t status = q->book.allocate(max_rows, policy, q->shapes());
  if (status != cudaSuccess) return fail(GW_CUDA_ERROR, std::string("QKV projector scratch: ") + cudaGetErrorString(status));
  *projector = q.release();
  return GW_OK;
}

void gw_qkv_projector_destroy(gw_qkv_projector* projector) { delete projector; }

size_t gw_qkv_projector_bytes(const gw_qkv_projector* q) { return q ? q->book.scratch.bytes + q->book.dequantized.bytes : 0; }

gw_status gw_qkv_projector_prepare(gw_qkv_projector* q, uint32_t rows) {
  clear_error();
  if (!q) return fail(GW_INVALID_ARGUMENT, "QKV projector prepare requires a projector");
  return q->book.prepare(rows, q->shapes());
}

}  // extern "C"

namespace {

// projection_linear (executor.cuh:1187-1215): FP8 -> NVFP4 with FP4 activations -> BF16 GEMM (on the
// BF16 weight, or on the NVFP4 weight dequantised into the book's buffer)
gw_status run_linear(PlanBook& book, const gw_projection& p, const void* input, void* output, bool fp4, int transform,
                     cudaStream_t s) {
  const uint32_t n = p.storage == GW_STORAGE_NVFP4_W4A4 ? p.physical_output : p.output;
  const auto plan = [&](int kind) -> const PlanSet* {
    const auto found = book.plans.find(Key{kind, p.input, n});
    return found == book.plans.end() ? nullptr : &found->second;
  };
  if (p.storage == GW_STORAGE_FP8_W8A8) {
    const PlanSet* set = plan(p.fp8_channel_scales ? kFp8Channel : kFp8);
    if (!set) return fail(GW_INVALID_ARGUMENT, "projection shape is not one of the object's shapes");
    return gw_fp8_plan_run(set->fp8, input, p.fp8_data, p.fp8_input_scale, p.fp8_weight_scale, p.fp8_channel_scales, output,
                           book.scratch.data, book.scratch.bytes, s, transform);
  }
  if (p.storage == GW_STORAGE_NVFP4_W4A4 && fp4) {
    const PlanSet* set = plan(kNvfp4);
    if (!set) return fail(GW_INVALID_ARGUMENT, "projection shape is not one of the object's shapes");
    return gw_nvfp4_plan_run(set->nvfp4, input, p.nvfp4_data, p.nvfp4_scales, p.nvfp4_input_scale, p.nvfp4_weight_scale,
                             output, book.scratch.data, book.scratch.bytes, s, transform);
  }
  if (transform != GW_TRANSFORM_IDENTITY) return fail(GW_INVALID_ARGUMENT, "the BF16 path has no fused input transform");
  const PlanSet* set = plan(kBf16);
  if (!set) return fail(GW_INVALID_ARGUMENT, "projection shape is not one of the object's shapes");
  const void* weights = p.bf16;
  if (p.storage == GW_STORAGE_NVFP4_W4A4) {
    if (!book.dequantized.data || size_t(n) * p.input * sizeof(bf16) > book.dequantized.bytes)
      return fail(GW_INVALID_ARGUMENT, "NVFP4 BF16 decode workspace is disabled (policy always)");
    const gw_status status = gw_nvfp4_dequantize(p.nvfp4_data, p.nvfp4_scales, p.nvfp4_weight_scale, p.input, n,
                                                 book.dequantized.data, s);
    if (status != GW_OK) return status;
    weights = book.dequantized.data;
  }
  return gw_bf16_plan_run(set->bf16, input, weights, output, book.scratch.data, book.scratch.bytes, s);
}

gw_projection widened(const gw_projection& first, uint32_t output) {
  gw_projection joined = first;
  joined.output = joined.physical_output = output;
  return joined;
}

}  // namespace

extern "C" {

gw_status gw_mlp_chain_run(gw_mlp_chain* c, const gw_projection* gate, const gw_projection* up,
                           const gw_projection* down, const void* input_bf16, void* gate_up_bf16, void* product_bf16,
                           void* output_bf16, int phase, void* stream) {
  clear_error();
  if (!c || !gate || !up || !down || !input_bf16 || !gate_up_bf16 || !product_bf16 || !output_bf16 || c->book.rows == 0 ||
      (phase != GW_PHASE_PREFILL && phase != GW_PHASE_DECODE))
    return fail(GW_INVALID_ARGUMENT, "prepare the MLP chain before run; all buffers are required");
  const uint32_t h = c->hidden, m = c->mlp, rows = c->book.rows;
  for (const gw_projection* p : {gate, up})
    if (p->input != h || p->output != m || p->physical_output != m)
      return fail(GW_INVALID_ARGUMENT, "gate / up projection does not have the chain's shape");
  if (down->input != m || down->output != h || down->physical_output != h)
    return fail(GW_INVALID_ARGUMENT, "down projection does not have the chain's shape");
  cudaStream_t s = as_stream(stream);
  const bool fp4 = gw_nvfp4_fp4_activations(c->book.policy, phase) != 0;
  auto* gate_out = static_cast<bf16*>(gate_up_bf16);
  gw_status status = GW_OK;
  bool interleaved = true;       // gate_up holds [rows, gate | up]; otherwise gate rows, then up rows
  if ((nvfp4_joined(*gate, *up) && fp4) || fp8_joined(*gate, *up) || bf16_joined(*gate, *up)) {
    status = run_linear(c->book, widened(*gate, 2 * m), input_bf16, gate_out, fp4, GW_TRANSFORM_IDENTITY, s);
  } else {
    status = run_linear(c->book, *gate, input_bf16, gate_out, fp4, GW_TRANSFORM_IDENTITY, s);
    if (status == GW_OK)
      status = run_linear(c->book, *up, input_bf16, gate_out + size_t(rows) * m, fp4, GW_TRANSFORM_IDENTITY, s);
    interleaved = false;
  }
  if (status != GW_OK) return status;
  const bool down_quantised = down->storage == GW_STORAGE_FP8_W8A8 || (down->storage == GW_STORAGE_NVFP4_W4A4 && fp4);
  if (interleaved && down_quantised)      // GeGLU inside the down projection's activation quantiser
    return run_linear(c->book, *down, gate_out, output_bf16, fp4, GW_TRANSFORM_GELU_TANH_MULTIPLY, s);
  if (interleaved)
    status = gw_gelu_tanh_multiply_interleaved_bf16(gate_out, product_bf16, rows, m, s);
  else
    status = gw_gelu_tanh_multiply_bf16(gate_out, gate_out + size_t(rows) * m, product_bf16, uint64_t(rows) * m, s);
  if (status != GW_OK) return status;
  return run_linear(c->book, *down, product_bf16, output_bf16, fp4, GW_TRANSFORM_IDENTITY, s);
}

gw_status gw_qkv_projector_run(gw_qkv_projector* q, const gw_projection* query, const gw_projection* key,
                               const gw_projection* value, const void* input_bf16, void* q_bf16, void* k_bf16,
                               void* v_bf16, int phase, void* stream, int* joined) {
  clear_error();
  if (!q || !query || !key || !input_bf16 || !q_bf16 || !k_bf16 || (value && !v_bf16) || q->book.rows == 0 ||
      (phase != GW_PHASE_PREFILL && phase != GW_PHASE_DECODE))
    return fail(GW_INVALID_ARGUMENT, "prepare the QKV projector before run; every projection needs its output");
  const auto shaped = [&](const gw_projection* p, uint32_t n) {
    return p->input == q->hidden && p->output == n && p->physical_output == n;
  };
  if (!shaped(query, q->q) || !shaped(key, q->kv) || (value && !shaped(value, q->kv)))
    return fail(GW_INVALID_ARGUMENT, "Q / K / V projection does not have the projector's shape");
  cudaStream_t s = as_stream(stream);
  const bool fp4 = gw_nvfp4_fp4_activations(q->book.policy, phase) != 0;
  const uint32_t width = q->q + q->kv * (value ? 2 : 1);
  // fusion::qkv_weight (projection_fusion.h:23-33) and fp8::qkv_weight (fp8_projections.h:26-35)
  const bool bf16_run = bf16_joined(*query, *key) && (!value || bf16_joined(*key, *value));
  const bool fp8_run = fp8_joined(*query, *key) && (!value || fp8_joined(*key, *value));
  if (joined) *joined = (bf16_run || fp8_run) ? 1 : 0;
  if (bf16_run || fp8_run)      // one GEMM; the caller reads [rows, Q | K | V] from q_bf16
    return run_linear(q->book, widened(*query, width), input_bf16, q_bf16, fp4, GW_TRANSFORM_IDENTITY, s);
  gw_status status = run_linear(q->book, *query, input_bf16, q_bf16, fp4, GW_TRANSFORM_IDENTITY, s);
  if (status == GW_OK) status = run_linear(q->book, *key, input_bf16, k_bf16, fp4, GW_TRANSFORM_IDENTITY, s);
  if (status == GW_OK && value) status = run_linear(q->book, *value, input_bf16, v_bf16, fp4, GW_TRANSFORM_IDENTITY, s);
  return status;
}

// weights.cuh:146-168: [first packed | second packed | first scales | second scales] written over the
// region that starts at first's packed rows (which must reach to the end of second's scale tiles)
gw_status gw_join_nvfp4_pair(gw_projection* first, gw_projection* second, void* temp, size_t temp_bytes, void* stream,
                             int* joined) {
  clear_error();
  if (!first || !second || !joined) return fail(GW_INVALID_ARGUMENT, "join requires two projections");
  *joined = 0;
  if (first->storage != GW_STORAGE_NVFP4_W4A4 || second->storage != GW_STORAGE_NVFP4_W4A4 || !first->nvfp4_data ||
      !second->nvfp4_data || first->input != second->input || first->physical_output != second->physical_output ||
      first->physical_output % 128 || first->nvfp4_input_scale != second->nvfp4_input_scale ||
      first->nvfp4_weight_scale != second->nvfp4_weight_scale)
    return GW_OK;                       // left apart, as the reference leaves pairs whose scales differ
  const size_t packed = size_t(first->physical_output) * first->input / 2;
  const size_t scales = scale_storage_bytes(first->physical_output, first->input);
  const size_t total = 2 * (packed + scales);
  auto* base = const_cast<uint8_t*>(first->nvfp4_data);
  // the joined form may only overwrite what the two payloads occupy today
  if (address(second->nvfp4_data) < address(first->nvfp4_scales) + scales || address(second->nvfp4_scales) < address(second->nvfp4_data) + packed ||
      address(first->nvfp4_scales) < address(base) + packed || address(second->nvfp4_scales) + scales < address(base) + total)
    return fail(GW_INVALID_ARGUMENT, "the second matrix must follow the first one inside one payload region");
  if (!temp || temp_bytes < total) return fail(GW_INVALID_ARGUMENT, "join needs 2 * (packed + scale) bytes of temporary memory");
  cudaStream_t s = as_stream(stream);
  auto* t = static_cast<uint8_t*>(temp);
  GW_CUDA_CHECK(cudaMemcpyAsync(t, first->nvfp4_data, packed, cudaMemcpyDeviceToDevice, s), "join first weights");
  GW_CUDA_CHECK(cudaMemcpyAsync(t + packed, second->nvfp4_data, packed, cudaMemcpyDeviceToDevice, s), "join second weights");
  GW_CUDA_CHECK(cudaMemcpyAsync(t + 2 * packed, first->nvfp4_scales, scales, cudaMemcpyDeviceToDevice, s), "join first scales");
  GW_CUDA_CHECK(cudaMemcpyAsync(t + 2 * packed + scales, second->nvfp4_scales, scales, cudaMemcpyDeviceToDevice, s),
                "join second scales");
  GW_CUDA_CHECK(cudaMemcpyAsync(base, t, total, cudaMemcpyDeviceToDevice, s), "store joined pair");
  first->nvfp4_scales = base + 2 * packed;
  second->nvfp4_data = base + packed;
  second->nvfp4_scales = first->nvfp4_scales + scales;
  *joined = 1;
  return GW_OK;
}

// weights.cuh:169-223: the group's rows packed back to back from the first matrix's address on, and one
// FP32 scale per output channel (input_scale * weight_scale of the channel's own matrix)
gw_status gw_join_fp8_group(gw_projection* group, uint32_t count, float* channel_scales, void* temp, size_t temp_bytes,
                            void* stream, int* joined) {
  clear_error();
  if (!group || count < 2 || !joined) return fail(GW_INVALID_ARGUMENT, "join requires at least two projections");
  *joined = 0;
  size_t bytes = 0, channels = 0;
  for (uint32_t i = 0; i < count; ++i) {
    const gw_projection& p = group[i];
    if (p.storage != GW_STORAGE_FP8_W8A8 || !p.fp8_data || p.input != group[0].input ||
        p.fp8_input_scale != group[0].fp8_input_scale)
      return GW_OK;                     // mixed storage or different input scales: left apart
    if (i && address(p.fp8_data) < address(group[i - 1].fp8_data) + size_t(group[i - 1].output) * p.input)
      return fail(GW_INVALID_ARGUMENT, "the group's matrices must follow one another in memory");
    bytes += size_t(p.output) * p.input;
    channels += p.output;
  }
  if (!channel_scales || !temp || temp_bytes < bytes)
    return fail(GW_INVALID_ARGUMENT, "join needs the channel-scale array and the group's bytes of temporary memory");
  cudaStream_t s = as_stream(stream);
  std::vector<float> host(channels);
  size_t offset = 0, channel = 0;
  auto* t = static_cast<uint8_t*>(temp);
  for (uint32_t i = 0; i < count; ++i) {
    const gw_projection& p = group[i];
    const size_t n = size_t(p.output) * p.input;
    GW_CUDA_CHECK(cudaMemcpyAsync(t + offset, p.fp8_data, n, cudaMemcpyDeviceToDevice, s), "join FP8 rows");
    offset += n;
    for (uint32_t c = 0; c < p.output; ++c) host[channel++] = p.fp8_input_scale * p.fp8_weight_scale;
  }
  auto* base = const_cast<uint8_t*>(group[0].fp8_data);
  GW_CUDA_CHECK(cudaMemcpyAsync(base, t, bytes, cudaMemcpyDeviceToDevice, s), "store joined FP8 rows");
  GW_CUDA_CHECK(cudaMemcpyAsync(channel_scales, host.data(), channels * sizeof(float), cudaMemcpyHostToDevice, s),
                "FP8 channel scales");
  GW_CUDA_CHECK(cudaStreamSynchronize(s), "FP8 join");      // `host` leaves scope
  offset = 0;
  channel = 0;
  for (uint32_t i = 0; i < count; ++i) {
    group[i].fp8_data = base + offset;
    group[i].fp8_channel_scales = channel_scales + channel;
    offset += size_t(group[i].output) * group[i].input;
    channel += group[i].output;
  }
  *joined = 1;
  return GW_OK;
}

}  // extern "C"
