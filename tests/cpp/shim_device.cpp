// Device test of the C++ shim (include/gewell_b200.hpp): the join rules of the
// 31B projection plans on real device memory.  A joined gate+up projection (one
// GEMM over the concatenated matrix) must give, bit for bit, what the two
// separate GEMMs give (tests/nvfp4_linear_test.cu:298-376); pairs that violate
// a rule are rejected; the fused GeGLU input of the down projection equals
// GeGLU followed by a plain run; and the shape-keyed plan cache runs plans with
// one shared scratch.  Same for the FP8 join with per-channel scales
// (tests/fp8_linear_test.cu:120-185).  Exit code 0 and "PASS" on success.
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "gewell_b200.hpp"
#include "gewell_b200_test.h"

namespace {
int failures = 0;
void expect(bool ok, const char* what) {
  if (!ok) { std::printf("FAIL %s\n", what); ++failures; }
}
void cuda(cudaError_t status, const char* what) {
  if (status != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(status));
}
template <typename T> T* device(std::size_t count) {
  void* p = nullptr;
  cuda(cudaMalloc(&p, count * sizeof(T)), "cudaMalloc");
  return static_cast<T*>(p);
}
// BF16 bits of a deterministic pseudo-random value in [-scale, scale)
std::vector<std::uint16_t> random_bf16(std::size_t count, std::uint32_t seed, float scale) {
  std::vector<std::uint16_t> out(count);
  std::uint32_t state = seed * 2654435761u + 12345u;
  for (auto& v : out) {
    state = state * 1664525u + 1013904223u;
    const float f = (float((state >> 8) & 0xFFFF) / 32768.0F - 1.0F) * scale;
    std::uint32_t bits;
    std::memcpy(&bits, &f, 4);
    v = std::uint16_t((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16);
  }
  return out;
}
std::vector<std::uint16_t> download(const __nv_bfloat16* p, std::size_t count) {
  std::vector<std::uint16_t> out(count);
  cuda(cudaMemcpy(out.data(), p, count * 2, cudaMemcpyDeviceToHost), "download");
  return out;
}
}  // namespace

int main() {
  using namespace gewell_b200;
  try {
    constexpr std::uint32_t K = 512, N1 = 256, N2 = 384, rows = 40;
    // ---------------------------------------------------------------- NVFP4: joined gate/up
    const auto host_w = random_bf16(std::size_t(N1 + N2) * K, 1, 0.05F);
    const auto host_x = random_bf16(std::size_t(rows) * K, 2, 1.0F);
    auto* w = device<__nv_bfloat16>(host_w.size());
    auto* x = device<__nv_bfloat16>(host_x.size());
    cuda(cudaMemcpy(w, host_w.data(), host_w.size() * 2, cudaMemcpyHostToDevice), "upload");
    cuda(cudaMemcpy(x, host_x.data(), host_x.size() * 2, cudaMemcpyHostToDevice), "upload");
    auto* data = device<std::uint8_t>(std::size_t(N1 + N2) * K / 2);
    auto* scales = device<std::uint8_t>(nvfp4::scale_storage_bytes(N1 + N2, K));
    // one packing call with one global scale: gate rows first, up rows right behind them
    detail::check(gw_nvfp4_pack_weights(w, N1 + N2, K, 0.05F / (6 * 448), data, scales, nullptr));
    const nvfp4::Weight gate{data, scales, 1.0F / 2688, 0.05F / (6 * 448)};
    const nvfp4::Weight up{data + std::size_t(N1) * K / 2, scales + nvfp4::scale_storage_bytes(N1, K), gate.input_scale,
                           gate.weight_scale};
    const nvfp4::Weight both = nvfp4::joined(gate, up, N1, K);
    expect(both.data == data, "contiguous gate/up with equal globals join");
    nvfp4::Weight wrong = up;
    wrong.input_scale *= 2;
    expect(nvfp4::joined(gate, wrong, N1, K).data == nullptr, "different input scales do not join");
    wrong = up;
    wrong.scales += 512;
    expect(nvfp4::joined(gate, wrong, N1, K).data == nullptr, "scale tiles that do not follow do not join");
    expect(nvfp4::joined(gate, up, 192, K).data == nullptr, "a first part that ends inside a scale tile does not join");

    nvfp4::ProjectionPlans plans;               // shape-keyed cache, one shared scratch
    plans.add_shape(K, N1);
    plans.add_shape(K, N2);
    plans.add_shape(K, N1 + N2);
    plans.prepare(rows);
    auto* y_gate = device<__nv_bfloat16>(std::size_t(rows) * N1);
    auto* y_up = device<__nv_bfloat16>(std::size_t(rows) * N2);
    auto* y_both = device<__nv_bfloat16>(std::size_t(rows) * (N1 + N2));
    plans.run(rows, K, N1, x, gate, y_gate, nullptr);
    plans.run(rows, K, N2, x, up, y_up, nullptr);
    plans.run(rows, K, N1 + N2, x, both, y_both, nullptr);
    cuda(cudaDeviceSynchronize(), "joined projections");
    expect(gw_debug_kernel_error() == 0, "no kernel error");
    const auto g = download(y_gate, std::size_t(rows) * N1), u = download(y_up, std::size_t(rows) * N2),
               b = download(y_both, std::size_t(rows) * (N1 + N2));
    bool equal = true, nonzero = false;
    for (std::uint32_t r = 0; r < rows; ++r) {
      for (std::uint32_t c = 0; c < N1; ++c) equal = equal && b[std::size_t(r) * (N1 + N2) + c] == g[std::size_t(r) * N1 + c];
      for (std::uint32_t c = 0; c < N2; ++c) equal = equal && b[std::size_t(r) * (N1 + N2) + N1 + c] == u[std::size_t(r) * N2 + c];
      nonzero = nonzero || (g[std::size_t(r) * N1] & 0x7FFF) != 0;
    }
    expect(equal, "joined gate/up GEMM equals the separate GEMMs bit for bit");
    expect(nonzero, "outputs are not all zero");

    // fused GeGLU input of a down projection == GeGLU, then the same projection.  The joined output above is
    // [rows, gate | up] only when N1 == N2, so use a [rows, 2K] tensor of its own.
    const auto host_gu = random_bf16(std::size_t(rows) * 2 * K, 3, 1.5F);
    auto* gu = device<__nv_bfloat16>(host_gu.size());
    cuda(cudaMemcpy(gu, host_gu.data(), host_gu.size() * 2, cudaMemcpyHostToDevice), "upload");
    auto* act = device<__nv_bfloat16>(std::size_t(rows) * K);
    std::vector<std::uint16_t> gate_half(std::size_t(rows) * K), up_half(std::size_t(rows) * K);
    for (std::uint32_t r = 0; r < rows; ++r) {
      std::memcpy(&gate_half[std::size_t(r) * K], &host_gu[std::size_t(r) * 2 * K], K * 2);
      std::memcpy(&up_half[std::size_t(r) * K], &host_gu[std::size_t(r) * 2 * K + K], K * 2);
    }
    auto* dg = device<__nv_bfloat16>(gate_half.size());
    auto* du = device<__nv_bfloat16>(up_half.size());
    cuda(cudaMemcpy(dg, gate_half.data(), gate_half.size() * 2, cudaMemcpyHostToDevice), "upload");
    cuda(cudaMemcpy(du, up_half.data(), up_half.size() * 2, cudaMemcpyHostToDevice), "upload");
    detail::check(gw_debug_geglu_bf16(dg, du, act, std::size_t(rows) * K, nullptr));
    auto* y_fused = device<__nv_bfloat16>(std::size_t(rows) * N1);
    auto* y_plain = device<__nv_bfloat16>(std::size_t(rows) * N1);
    plans.run(rows, K, N1, gu, gate, y_fused, nullptr, nvfp4::InputTransform::gelu_tanh_multiply);
    plans.run(rows, K, N1, act, gate, y_plain, nullptr);
    cuda(cudaDeviceSynchronize(), "fused GeGLU input");
    expect(download(y_fused, std::size_t(rows) * N1) == download(y_plain, std::size_t(rows) * N1),
           "fused GeGLU input equals GeGLU followed by the projection, bit for bit");

    // ---------------------------------------------------------------- FP8: joined with per-channel scales
    auto* f8 = device<std::uint8_t>(std::size_t(N1 + N2) * K);
    std::vector<float> row_scale(N1 + N2);
    for (std::uint32_t n = 0; n < N1 + N2; ++n) row_scale[n] = (n < N1 ? 0.05F : 0.1F) / 448;   // each part its own weight scale
    auto* d_row_scale = device<float>(N1 + N2);
    cuda(cudaMemcpy(d_row_scale, row_scale.data(), row_scale.size() * 4, cudaMemcpyHostToDevice), "upload");
    detail::check(gw_fp8_pack_weights(w, N1 + N2, K, 0.0F, d_row_scale, f8, nullptr));
    const float input_scale = 1.0F / 448;
    std::vector<float> channel(N1 + N2);
    for (std::uint32_t n = 0; n < N1 + N2; ++n) channel[n] = input_scale * row_scale[n];
    auto* d_channel = device<float>(N1 + N2);
    cuda(cudaMemcpy(d_channel, channel.data(), channel.size() * 4, cudaMemcpyHostToDevice), "upload");
    const fp8::Weight q{f8, input_scale, row_scale[0], d_channel};
    const fp8::Weight k{f8 + std::size_t(N1) * K, input_scale, row_scale[N1], d_channel + N1};
    expect(fp8::joined(q, k, N1, K).data == f8, "adjacent FP8 matrices with one input scale join");
    expect(fp8::joined(q, fp8::Weight{k.data, input_scale * 2, k.weight_scale, k.channel_scales}, N1, K).data == nullptr,
           "FP8 join needs one input scale");
    fp8::ProjectionPlans fplans;
    fplans.add_shape(K, N1, false);
    fplans.add_shape(K, N2, false);
    fplans.add_shape(K, N1 + N2, true);
    fplans.prepare(rows);
    fplans.run(rows, K, N1, x, fp8::Weight{q.data, q.input_scale, q.weight_scale, nullptr}, y_gate, nullptr);
    fplans.run(rows, K, N2, x, fp8::Weight{k.data, k.input_scale, k.weight_scale, nullptr}, y_up, nullptr);
    fplans.run(rows, K, N1 + N2, x, fp8::joined(q, k, N1, K), y_both, nullptr, fp8::InputTransform::identity, true);
    cuda(cudaDeviceSynchronize(), "joined FP8 projections");
    expect(gw_debug_kernel_error() == 0, "no kernel error (FP8)");
    const auto fg = download(y_gate, std::size_t(rows) * N1), fu = download(y_up, std::size_t(rows) * N2),
               fb = download(y_both, std::size_t(rows) * (N1 + N2));
    equal = true;
    for (std::uint32_t r = 0; r < rows; ++r) {
      for (std::uint32_t c = 0; c < N1; ++c) equal = equal && fb[std::size_t(r) * (N1 + N2) + c] == fg[std::size_t(r) * N1 + c];
      for (std::uint32_t c = 0; c < N2; ++c) equal = equal && fb[std::size_t(r) * (N1 + N2) + N1 + c] == fu[std::size_t(r) * N2 + c];
    }
    expect(equal, "joined FP8 GEMM with per-channel scales equals the separate GEMMs bit for bit");
  } catch (const std::exception& error) {
    std::printf("FAIL exception: %s\n", error.what());
    ++failures;
  }
  std::printf(failures ? "shim device test: %d failure(s)\n" : "shim device test: PASS\n", failures);
  return failures != 0;
}
