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
  expect(nvfp4::scale_offset(130, 5, 256) == gw_nvfp4_scale_offset(130, 5, 256), "scale_offset");
  expect(nvfp4::scale_storage_bytes(768, 2816) == gw_nvfp4_scale_storage_bytes(768, 2816), "scale_storage_bytes");
  expect(fp8::scratch_upper_bound_bytes(33, 256) == gw_fp8_scratch_upper_bound_bytes(33, 256), "fp8 bound");
  std::printf(failures ? "shim contract: %d failure(s)\n" : "shim contract: PASS\n", failures);
  return failures != 0;
}
