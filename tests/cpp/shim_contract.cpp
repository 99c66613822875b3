// Host-only contract test of the C++ shim (include/gewell_b200.hpp): the
// validation matrix of the reference's plans (tests/nvfp4_linear_test.cu:421-423,
// tests/fp8_linear_test.cu:306-335) must throw std::invalid_argument before any
// CUDA work happens, and constexpr layout helpers must match the C ABI.
#include <cstdio>
#include <stdexcept>

#include "gewell_b200.hpp"

template <typename F> static bool rejects(F&& f) {
  try { f(); } catch (const std::invalid_argument&) { return true; } catch (...) { return false; }
  return false;
}

int main() {
  using namespace gewell_b200;
  int failures = 0;
  auto expect = [&](bool ok, const char* what) { if (!ok) { std::printf("FAIL %s\n", what); ++failures; } };
  expect(rejects([] { nvfp4::Plan(0, 256, 256); }), "nvfp4 rows=0");
  expect(rejects([] { nvfp4::Plan(1, 250, 256); }), "nvfp4 K%64");
  expect(rejects([] { nvfp4::Plan(1, 256, 200); }), "nvfp4 N%128");
  expect(rejects([] { fp8::Plan(1, 24, 16); }), "fp8 K%16");
  expect(rejects([] { fp8::Plan(1, 16, 24); }), "fp8 N%16");
  expect(rejects([] { fp8::Plan(0, 16, 16); }), "fp8 rows=0");
  expect(rejects([] { sm120::MoeWorkspace(0); }), "moe capacity 0");
  {
    nvfp4::Plan plan(4, 256, 256);
    expect(plan.scratch_bytes() <= nvfp4::scratch_upper_bound_bytes(4, 256, 256), "scratch bound");
    expect(rejects([&] { plan.run(nullptr, {}, nullptr, nullptr, 0); }), "nvfp4 run null buffers");
    nvfp4::Plan moved(std::move(plan));
    expect(moved.scratch_bytes() == 512 + 2048, "moved plan keeps its state");
  }
  {
    // join rules: contiguous data and scale tiles with equal global scales join, anything else does not
    alignas(16) static std::uint8_t data[2 * 128 * 128], scales[2 * 1024];
    const nvfp4::Weight gate{data, scales, 0.5F, 0.25F}, up{data + 128 * 256 / 2, scales + nvfp4::scale_storage_bytes(128, 256), 0.5F, 0.25F};
    expect(nvfp4::joined(gate, up, 128, 256).data == data, "nvfp4 gate/up join");
    nvfp4::Weight other = up; other.weight_scale = 0.5F;
    expect(nvfp4::joined(gate, other, 128, 256).data == nullptr, "nvfp4 join needs equal scales");
    other = up; other.data += 16;
    expect(nvfp4::joined(gate, other, 128, 256).data == nullptr, "nvfp4 join needs contiguous rows");
    static float channel[4];
    const fp8::Weight q{data, 0.5F, 1.0F, channel}, k{data + 64 * 128, 0.5F, 2.0F, channel};
    expect(fp8::joined(q, k, 64, 128).data == data, "fp8 join");
    expect(fp8::joined(fp8::Weight{data, 0.5F, 1.0F, nullptr}, k, 64, 128).data == nullptr, "fp8 join needs channel scales");
    expect(!fp8::adjacent(q, fp8::Weight{data + 64 * 128, 0.25F, 2.0F, channel}, 64 * 128), "fp8 adjacency needs one input scale");
    nvfp4::ProjectionPlans plans;
    plans.add_shape(256, 256);
    expect(plans.scratch_bytes() == 0, "no scratch before prepare");
    expect(rejects([&] { plans.add_shape(250, 256); plans.prepare(4); }), "plan cache forwards validation");
  }
  expect(nvfp4::scale_offset(130, 5, 256) == gw_nvfp4_scale_offset(130, 5, 256), "scale_offset");
  expect(nvfp4::scale_storage_bytes(768, 2816) == gw_nvfp4_scale_storage_bytes(768, 2816), "scale_storage_bytes");
  expect(fp8::scratch_upper_bound_bytes(33, 256) == gw_fp8_scratch_upper_bound_bytes(33, 256), "fp8 bound");
  std::printf(failures ? "shim contract: %d failure(s)\n" : "shim contract: PASS\n", failures);
  return failures != 0;
}
