// C++ host-side shim over the C ABI (gewell_b200.h) with the reference's class
// names, argument order and exception behaviour, so that a call site written
// against gewell::nvfp4::Plan / gewell::fp8::Plan / sm120::MoeWorkspace only has
// to switch namespaces.  Header only; link against libgewell_b200.so.
//
//   reference                                              here
//   gewell::nvfp4::{Weight,Plan,dequantize,...}            gewell_b200::nvfp4::...
//     (include/gewell/nvfp4_linear.h:13-91)
//   gewell::fp8::{Weight,Plan}                             gewell_b200::fp8::...
//     (include/gewell/fp8_linear.h:13-69)
//   gemma4_26b_a4b::sm120::{Projection,ExpertWeights,      gewell_b200::sm120::...
//     MoeWorkspace} (projection.cuh:11-17, moe.cuh:11-48)
//
// Contract violations throw std::invalid_argument, CUDA / kernel failures
// std::runtime_error, exactly as the reference does.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime_api.h>

#include <cstddef>
#include <cstdint>
#include <map>
#include <memory>
#include <set>
#include <stdexcept>
#include <string>
#include <tuple>
#include <type_traits>
#include <vector>

#include "gewell_b200.h"

namespace gewell_b200 {

namespace detail {
inline void check(gw_status status) {
  if (status == GW_OK) return;
  const std::string message = gw_last_error();
  if (status == GW_INVALID_ARGUMENT) throw std::invalid_argument(message);
  throw std::runtime_error(message);
}
}  // namespace detail

namespace nvfp4 {

inline constexpr std::size_t kMaxWorkspaceBytes = 36 * 1024 * 1024;

struct Weight {
  const std::uint8_t* data{};
  const std::uint8_t* scales{};
  float input_scale{};
  float weight_scale{};
};

enum class InputTransform { identity, gelu_tanh_multiply };

inline void dequantize(Weight weight, std::uint32_t input_width, std::uint32_t output_width,
                       __nv_bfloat16* output, cudaStream_t stream = nullptr) {
  detail::check(gw_nvfp4_dequantize(weight.data, weight.scales, weight.weight_scale, input_width, output_width,
                                    output, stream));
}

constexpr std::size_t scale_storage_bytes(std::size_t rows, std::size_t input_width) {
  return ((rows + 127) / 128) * ((input_width + 63) / 64) * 512;
}

constexpr std::size_t scratch_upper_bound_bytes(std::size_t max_rows, std::size_t input_width,
                                                std::size_t output_width) {
  const auto padded_rows = ((max_rows + 31) / 32) * 32;
  return padded_rows * (input_width / 2 + output_width * 2) + scale_storage_bytes(max_rows, input_width) +
         kMaxWorkspaceBytes + 3 * 255;
}

constexpr std::size_t scale_offset(std::size_t row, std::size_t block, std::size_t input_width) {
  return ((row / 128) * (input_width / 64) + block / 4) * 512 + (row % 32) * 16 + ((row % 128) / 32) * 4 +
         block % 4;
}

enum class ActivationPolicy : std::uint8_t { always = GW_POLICY_ALWAYS, prefill = GW_POLICY_PREFILL };
enum class Phase : std::uint8_t { prefill = GW_PHASE_PREFILL, decode = GW_PHASE_DECODE };
// include/gewell/nvfp4_policy.h:9-16
constexpr bool fp4_activations(ActivationPolicy policy, Phase phase) {
  return policy == ActivationPolicy::always || phase == Phase::prefill;
}
constexpr const char* activation_policy_name(ActivationPolicy policy) {
  return policy == ActivationPolicy::prefill ? "prefill" : "always";
}

class Plan {
 public:
  Plan(std::uint32_t rows, std::uint32_t input_width, std::uint32_t output_width) {
    detail::check(gw_nvfp4_plan_create(rows, input_width, output_width, &plan_));
  }
  // The reference constructor takes a cublasLtHandle_t first.  No library GEMM is used here, so the
  // handle is ignored; call sites compile unchanged (any pointer converts), and a null handle is still
  // rejected as the reference rejects it.
  Plan(const void* handle, std::uint32_t rows, std::uint32_t input_width, std::uint32_t output_width) {
    if (handle == nullptr) throw std::invalid_argument("NVFP4 plan requires a handle");
    detail::check(gw_nvfp4_plan_create(rows, input_width, output_width, &plan_));
  }
  ~Plan() { gw_nvfp4_plan_destroy(plan_); }
  Plan(Plan&& other) noexcept : plan_(other.plan_) { other.plan_ = nullptr; }
  Plan& operator=(Plan&& other) noexcept {
    if (this != &other) { gw_nvfp4_plan_destroy(plan_); plan_ = other.plan_; other.plan_ = nullptr; }
    return *this;
  }
  Plan(const Plan&) = delete;
  Plan& operator=(const Plan&) = delete;

  std::size_t scratch_bytes() const { return gw_nvfp4_plan_scratch_bytes(plan_); }

  void run(const __nv_bfloat16* input, Weight weight, __nv_bfloat16* output, void* scratch,
           std::size_t scratch_capacity, cudaStream_t stream = nullptr,
           InputTransform transform = InputTransform::identity) {
    detail::check(gw_nvfp4_plan_run(plan_, input, weight.data, weight.scales, weight.input_scale,
                                    weight.weight_scale, output, scratch, scratch_capacity, stream,
                                    static_cast<int>(transform)));
  }

 private:
  gw_nvfp4_plan* plan_{};
};

// Join rule of the reference loader (31b/sm120/nvfp4_projections.h:21-33, there
// fixed to the gate/up pair): two projections with the same input can run as
// one GEMM when the second one's packed rows and scale tiles follow the first
// one's in memory (first_rows a multiple of 128) and their global scales are
// equal.  Returns `first` (now covering both) or an empty Weight.
inline Weight joined(Weight first, Weight second, std::size_t first_rows, std::size_t input_width) {
  const auto address = [](const void* p) { return reinterpret_cast<std::uintptr_t>(p); };
  if (!first.data || !second.data || !first.scales || !second.scales || first_rows % 128 != 0 ||
      first.input_scale != second.input_scale || first.weight_scale != second.weight_scale ||
      address(second.data) != address(first.data) + first_rows * input_width / 2 ||
      address(second.scales) != address(first.scales) + scale_storage_bytes(first_rows, input_width))
    return {};
  return first;
}

}  // namespace nvfp4

namespace detail {
// Plans per (rows, K, N, flag) sharing one scratch buffer, as the reference's
// ProjectionPlans classes do (31b/sm120/nvfp4_projections.h:35-120,
// fp8_projections.h:53-113): prepare() creates the plans of every registered
// shape for a row count and grows the scratch (allocates: call it outside
// capture); run() only enqueues work.
template <typename PlanT, typename WeightT, typename TransformT>
class PlanCache {
 public:
  PlanCache() = default;
  ~PlanCache() { if (scratch_) cudaFree(scratch_); }
  PlanCache(const PlanCache&) = delete;
  PlanCache& operator=(const PlanCache&) = delete;

  void add_shape(std::uint32_t input_width, std::uint32_t output_width, bool flag = false) {
    shapes_.emplace(input_width, output_width, flag);
  }
  void prepare(std::uint32_t rows) {
    for (const auto& [input_width, output_width, flag] : shapes_) {
      const auto key = std::make_tuple(rows, input_width, output_width, flag);
      if (plans_.count(key)) continue;
      auto plan = make(rows, input_width, output_width, flag);
      const std::size_t needed = plan->scratch_bytes();
      if (needed > scratch_bytes_) {
        void* replacement = nullptr;
        const cudaError_t status = cudaMalloc(&replacement, needed);
        if (status != cudaSuccess)
          throw std::runtime_error(std::string("projection workspace: ") + cudaGetErrorString(status));
        if (scratch_) cudaFree(scratch_);
        scratch_ = replacement;
        scratch_bytes_ = needed;
      }
      plans_.emplace(key, std::move(plan));
    }
  }
  std::size_t scratch_bytes() const { return scratch_bytes_; }
  void run(std::uint32_t rows, std::uint32_t input_width, std::uint32_t output_width, const __nv_bfloat16* input,
           WeightT weight, __nv_bfloat16* output, cudaStream_t stream, TransformT transform = TransformT::identity,
           bool flag = false) {
    plans_.at(std::make_tuple(rows, input_width, output_width, flag))
        ->run(input, weight, output, scratch_, scratch_bytes_, stream, transform);
  }

 private:
  static std::unique_ptr<PlanT> make(std::uint32_t rows, std::uint32_t k, std::uint32_t n, bool flag) {
    if constexpr (std::is_constructible_v<PlanT, std::uint32_t, std::uint32_t, std::uint32_t, bool>)
      return std::make_unique<PlanT>(rows, k, n, flag);
    else
      return std::make_unique<PlanT>(rows, k, n);
  }
  std::set<std::tuple<std::uint32_t, std::uint32_t, bool>> shapes_;
  std::map<std::tuple<std::uint32_t, std::uint32_t, std::uint32_t, bool>, std::unique_ptr<PlanT>> plans_;
  void* scratch_{};
  std::size_t scratch_bytes_{};
};
}  // namespace detail

namespace nvfp4 {
using ProjectionPlans = detail::PlanCache<Plan, Weight, InputTransform>;
}  // namespace nvfp4

namespace fp8 {

inline constexpr std::size_t kMaxWorkspaceBytes = 32 * 1024 * 1024;

struct Weight {
  const std::uint8_t* data{};
  float input_scale{};
  float weight_scale{};
  const float* channel_scales{};
};

enum class InputTransform { identity, gelu_tanh_multiply };

constexpr std::size_t scratch_upper_bound_bytes(std::size_t max_rows, std::size_t input_width) {
  return max_rows * input_width + kMaxWorkspaceBytes + 255;
}

class Plan {
 public:
  Plan(std::uint32_t rows, std::uint32_t input_width, std::uint32_t output_width, bool channel_scales = false) {
    detail::check(gw_fp8_plan_create(rows, input_width, output_width, channel_scales ? 1 : 0, &plan_));
  }
  // reference signature with its (ignored, but non-null) cublasLtHandle_t first
  Plan(const void* handle, std::uint32_t rows, std::uint32_t input_width, std::uint32_t output_width,
       bool channel_scales = false) {
    if (handle == nullptr) throw std::invalid_argument("FP8 plan requires a handle");
    detail::check(gw_fp8_plan_create(rows, input_width, output_width, channel_scales ? 1 : 0, &plan_));
  }
  ~Plan() { gw_fp8_plan_destroy(plan_); }
  Plan(Plan&& other) noexcept : plan_(other.plan_) { other.plan_ = nullptr; }
  Plan& operator=(Plan&& other) noexcept {
    if (this != &other) { gw_fp8_plan_destroy(plan_); plan_ = other.plan_; other.plan_ = nullptr; }
    return *this;
  }
  Plan(const Plan&) = delete;
  Plan& operator=(const Plan&) = delete;

  std::size_t scratch_bytes() const { return gw_fp8_plan_scratch_bytes(plan_); }

  void run(const __nv_bfloat16* input, Weight weight, __nv_bfloat16* output, void* scratch,
           std::size_t scratch_capacity, cudaStream_t stream = nullptr,
           InputTransform transform = InputTransform::identity) {
    detail::check(gw_fp8_plan_run(plan_, input, weight.data, weight.input_scale, weight.weight_scale,
                                  weight.channel_scales, output, scratch, scratch_capacity, stream,
                                  static_cast<int>(transform)));
  }

 private:
  gw_fp8_plan* plan_{};
};

// Join rules of the reference loader (31b/sm120/fp8_projections.h:20-50): the
// second matrix starts `elements` bytes after the first and quantises its
// input with the same scale; a joined projection needs per-channel scales
// (they carry each part's own weight scale).
inline bool adjacent(Weight first, Weight second, std::size_t elements) {
  return first.data && second.data && first.input_scale == second.input_scale &&
         reinterpret_cast<std::uintptr_t>(second.data) == reinterpret_cast<std::uintptr_t>(first.data) + elements;
}
inline Weight joined(Weight first, Weight second, std::size_t first_rows, std::size_t input_width) {
  return first.channel_scales && adjacent(first, second, first_rows * input_width) ? first : Weight{};
}

// flag = the plan uses per-channel scales (joined projections)
using ProjectionPlans = detail::PlanCache<Plan, Weight, InputTransform>;

}  // namespace fp8

namespace bf16 {
// The reference's BF16 LinearPlan (models/gemma4/31b/sm120/resources.cuh:118-190): Y = X . W^T.
class LinearPlan {
 public:
  LinearPlan(std::uint32_t rows, std::uint32_t input_width, std::uint32_t output_width) {
    detail::check(gw_bf16_plan_create(rows, input_width, output_width, &plan_));
  }
  ~LinearPlan() { gw_bf16_plan_destroy(plan_); }
  LinearPlan(const LinearPlan&) = delete;
  LinearPlan& operator=(const LinearPlan&) = delete;
  std::size_t scratch_bytes() const { return gw_bf16_plan_scratch_bytes(plan_); }
  // scratch may be null (decode-shaped plans then run without the K split)
  void run(const __nv_bfloat16* input, const __nv_bfloat16* weight, __nv_bfloat16* output, void* scratch = nullptr,
           std::size_t scratch_capacity = 0, cudaStream_t stream = nullptr) {
    detail::check(gw_bf16_plan_run(plan_, input, weight, output, scratch, scratch_capacity, stream));
  }

 private:
  gw_bf16_plan* plan_{};
};
}  // namespace bf16

namespace sm120 {

using Projection = gw_projection;
using ExpertWeights = gw_expert_weights;

// bind_projection (projection.cu:31-50).  `storage` is a GW_STORAGE_* tag; rows x columns is the logical
// (output x input) shape of the entry whose payload starts at host_payload / device_payload.
inline Projection bind_projection(std::uint32_t storage, std::uint32_t rows, std::uint32_t columns,
                                  const std::uint8_t* host_payload, const void* device_payload,
                                  std::size_t entry_bytes) {
  Projection projection{};
  detail::check(gw_bind_projection(storage, rows, columns, host_payload, device_payload, entry_bytes, &projection));
  return projection;
}

// ProjectionWorkspace (projection.cuh:19-41).  run() keeps the reference's handle parameter (ignored).
class ProjectionWorkspace {
 public:
  ProjectionWorkspace(const std::vector<Projection>& projections, unsigned max_rows, nvfp4::ActivationPolicy policy,
                      cudaStream_t stream) {
    detail::check(gw_projection_workspace_create(projections.data(), static_cast<std::uint32_t>(projections.size()),
                                                 max_rows, static_cast<int>(policy), stream, &workspace_));
  }
  ~ProjectionWorkspace() { gw_projection_workspace_destroy(workspace_); }
  ProjectionWorkspace(const ProjectionWorkspace&) = delete;
  ProjectionWorkspace& operator=(const ProjectionWorkspace&) = delete;
  void prepare(unsigned rows, nvfp4::Phase phase) {
    detail::check(gw_projection_workspace_prepare(workspace_, rows, static_cast<int>(phase)));
  }
  void run(const void* /*cublas handle, unused*/, const Projection& projection, const __nv_bfloat16* input,
           __nv_bfloat16* output) {
    detail::check(gw_projection_workspace_run(workspace_, &projection, input, output));
  }
  std::size_t bytes() const { return gw_projection_workspace_bytes(workspace_); }

 private:
  gw_projection_workspace* workspace_{};
};

// Host-bound expert table (see gw_moe_expert_table_create).
class ExpertTable {
 public:
  explicit ExpertTable(const std::vector<ExpertWeights>& experts) {
    detail::check(gw_moe_expert_table_create(experts.data(), static_cast<std::uint32_t>(experts.size()), &table_));
  }
  ~ExpertTable() { gw_moe_expert_table_destroy(table_); }
  ExpertTable(const ExpertTable&) = delete;
  ExpertTable& operator=(const ExpertTable&) = delete;
  const gw_expert_table* get() const { return table_; }

 private:
  gw_expert_table* table_{};
};

class MoeWorkspace {
 public:
  explicit MoeWorkspace(unsigned max_rows) { detail::check(gw_moe_create(max_rows, &workspace_)); }
  ~MoeWorkspace() { gw_moe_destroy(workspace_); }
  MoeWorkspace(const MoeWorkspace&) = delete;
  MoeWorkspace& operator=(const MoeWorkspace&) = delete;

  void run(const __nv_bfloat16* input, const __nv_bfloat16* scores, const __nv_bfloat16* expert_scales,
           const ExpertTable& weights, __nv_bfloat16* output, unsigned rows, bool has_bf16, bool has_fp8,
           bool has_nvfp4, bool fp4, cudaStream_t stream = nullptr) {
    detail::check(gw_moe_run(workspace_, input, scores, expert_scales, weights.get(), output, rows, has_bf16,
                             has_fp8, has_nvfp4, fp4, stream));
  }
  void dispatch(const __nv_bfloat16* scores, const __nv_bfloat16* expert_scales, unsigned rows,
                cudaStream_t stream = nullptr) {
    detail::check(gw_moe_dispatch(workspace_, scores, expert_scales, rows, stream));
  }
  std::size_t bytes() const { return gw_moe_bytes(workspace_); }
  std::size_t routing_bytes() const { return gw_moe_routing_bytes(workspace_); }
  std::size_t projection_bytes() const { return gw_moe_projection_bytes(workspace_); }
  std::size_t reduction_bytes() const { return gw_moe_reduction_bytes(workspace_); }
  const int* selected_experts() const { return gw_moe_selected_experts(workspace_); }
  const float* routing_weights() const { return gw_moe_routing_weights(workspace_); }
  const int* offsets() const { return gw_moe_offsets(workspace_); }
  const int* sorted_assignments() const { return gw_moe_sorted_assignments(workspace_); }
  const __nv_bfloat16* gate_up_capture() const {
    return static_cast<const __nv_bfloat16*>(gw_moe_gate_up_capture(workspace_));
  }
  const __nv_bfloat16* activated_capture() const {
    return static_cast<const __nv_bfloat16*>(gw_moe_activated_capture(workspace_));
  }
  const __nv_bfloat16* down_capture() const {
    return static_cast<const __nv_bfloat16*>(gw_moe_down_capture(workspace_));
  }

 private:
  gw_moe_workspace* workspace_{};
};

}  // namespace sm120

namespace weight_qdq {
enum class Type : std::uint8_t { bf16 = GW_QDQ_BF16, fp8 = GW_QDQ_FP8, nvfp4 = GW_QDQ_NVFP4 };

// weight_qdq::detail::apply_tensor (src/weight_qdq.cu:222-258); `state` is two
// device uint32 (the reference's DeviceReductionState).
inline void apply_tensor(std::uint32_t* state, Type type, __nv_bfloat16* values, std::uint64_t elements,
                         cudaStream_t stream = nullptr) {
  const gw_status status = gw_weight_qdq_apply(static_cast<int>(type), values, elements, state, stream);
  if (status == GW_INVALID_ARGUMENT) throw std::runtime_error(gw_last_error());   // the reference fail()s with runtime_error
  detail::check(status);
}
}  // namespace weight_qdq

}  // namespace gewell_b200
