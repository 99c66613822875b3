// Device helpers shared by the CTA-pair (tcgen05 cta_group::2) kernels: cluster
// rank and barrier, addressing the pair leader's shared memory, tensor-memory
// allocation for a pair, the pair MMA and its commit.  The commit is the only
// instruction here that signals both CTAs at once; no load fans out to other CTAs.
#pragma once

#include <cstdint>

#include "ptx.cuh"

namespace gw::pair {

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in the pair's leader (cluster rank 0)
__device__ __forceinline__ uint32_t leader_address(const void* local) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, 0;" : "=r"(remote) : "r"(ptx::smem_u32(local)));
  return remote;
}
// Plain (CTA-scope release) form on purpose: measured on B200, the .release.cluster form of this arrive
// cost the scale-loader warps about 1000 cycles per stage.  What the arrival publishes is tensor memory
// written by tcgen05.st, which tcgen05.wait::st and the tcgen05 fences on both sides order.
__device__ __forceinline__ void arrive_cluster(uint32_t cluster_address) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_address) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* slot, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(ptx::smem_u32(slot)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void mma_pair_nvfp4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t sfa, uint32_t sfb,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
// arrive on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(ptx::smem_u32(bar)), "h"(uint16_t(3)) : "memory");
}
// E2M1 x E2M1 with UE4M3 scales, FP32 accumulate, M = 256 across the pair, K-major operands
__host__ __device__ constexpr uint32_t idesc_pair_nvfp4(uint32_t n) {
  return (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((256u >> 4) << 24);
}
__device__ __forceinline__ void report(uint32_t* error, uint32_t code, volatile int* abort_flag) {
  *abort_flag = 1;
  if (error != nullptr) atomicCAS(error, 0u, code);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 pair = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&pair);
}
__device__ __forceinline__ uint4 shfl_xor_u4(const uint4& v, int mask) {
  return make_uint4(__shfl_xor_sync(0xffffffffu, v.x, mask), __shfl_xor_sync(0xffffffffu, v.y, mask),
                    __shfl_xor_sync(0xffffffffu, v.z, mask), __shfl_xor_sync(0xffffffffu, v.w, mask));
}
// 4x4 transpose of 16-byte units inside every group of four lanes: before, u[q] of lane 4j+k is unit q
// (8 consecutive channels) of row 4j+k; afterwards u[i] of lane 4j+k is unit k of row 4j+i, so four
// neighbouring lanes hold 64 contiguous bytes of one row.
__device__ __forceinline__ void transpose_units(uint4* u, int lane) {
  const bool hi = (lane & 2) != 0, lo = (lane & 1) != 0;
  {
    const uint4 send_a = hi ? u[0] : u[2], send_b = hi ? u[1] : u[3];
    const uint4 got_a = shfl_xor_u4(send_a, 2), got_b = shfl_xor_u4(send_b, 2);
    if (hi) { u[0] = got_a; u[1] = got_b; } else { u[2] = got_a; u[3] = got_b; }
  }
  {
    const uint4 send_a = lo ? u[0] : u[1], send_b = lo ? u[2] : u[3];
    const uint4 got_a = shfl_xor_u4(send_a, 1), got_b = shfl_xor_u4(send_b, 1);
    if (lo) { u[0] = got_a; u[2] = got_b; } else { u[1] = got_a; u[3] = got_b; }
  }
}

}  // namespace gw::pair
