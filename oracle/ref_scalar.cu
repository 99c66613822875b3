// Thin C-ABI wrapper that compiles the reference's OWN scalar quantisation
// helpers (src/weight_qdq_detail.cuh:61-82: round_e4m3, round_e2m1, round_bf16,
// nvfp4_block_scale) as host code, from the reference sources where they lie.
// TEST INFRASTRUCTURE ONLY: used to cross-check the NumPy restatement in
// oracle/codecs.py and oracle/nvfp4.py.  Built by oracle/Makefile into
// oracle/_ref/, never shipped.
#include "weight_qdq_detail.cuh"

#include <cstdint>
#include <cstring>

namespace ref = gewell::weight_qdq::detail;

extern "C" {

void ref_round_e4m3(const float* in, float* out, long n) {
  for (long i = 0; i < n; ++i) out[i] = ref::round_e4m3(in[i]);
}

void ref_round_e2m1(const float* in, float* out, long n) {
  for (long i = 0; i < n; ++i) out[i] = ref::round_e2m1(in[i]);
}

void ref_round_bf16(const float* in, std::uint16_t* out, long n) {
  for (long i = 0; i < n; ++i) {
    const auto value = ref::round_bf16(in[i]);
    std::memcpy(out + i, &value, 2);
  }
}

void ref_nvfp4_block_scale(const float* amax, float global_scale, float* out, long n) {
  for (long i = 0; i < n; ++i) out[i] = ref::nvfp4_block_scale(amax[i], global_scale);
}

}  // extern "C"
