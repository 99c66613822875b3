// NVFP4 prefill GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a.
//
// Two CTAs of a cluster (the two SMs of a TPC) compute one 256-token x
// 256-channel tile: every CTA stages its own 128 token rows and only ITS HALF of
// the 256 weight rows; the pair's tensor cores read both halves.  Per CTA and
// K stage (128 bytes of K) that is 16 KB tokens + 16 KB weights + 2 KB token
// scales + 4 KB weight scales = 38 KB instead of the 54 KB of the single-CTA
// 128x256 tile, which is what limits that kernel (shared-memory port and L2->SM
// fill).  Roles per CTA as in gemm_tc.cu: one producer lane, one MMA lane (only
// in the pair's leader, rank 0), four scale-loader warps, eight epilogue warps.
//
// Cross-CTA protocol (all mbarriers sit at the same shared-memory offsets in both
// CTAs):
//   sf_full[s]   local; the stage's scale atoms (copied first) complete on it
//   full[s]      local; the stage's operand tiles complete on it
//   sf_ready[s]  in the leader, 8 arrivals: the loader warps of BOTH CTAs arrive
//                (the peer's remotely) once their CTA's scales are in tensor
//                memory AND its operand tiles have landed -- the only barrier the
//                MMA lane waits on per stage
//   empty[s], acc_full   local; signalled in both CTAs at once by the leader's
//                tcgen05.commit with the pair mask
//   acc_empty    in the leader, 16 arrivals (epilogue warps of both CTAs)
// Every wait is bounded; the kernel ends with a cluster barrier before the
// tensor memory is released.  No load fans out to other CTAs.
#include <string>

#include "common.cuh"
#include "gemm_pair.h"
#include "pair.cuh"
#include "ptx.cuh"

namespace gw {
namespace {

using namespace pair;

constexpr int kStages = 5;
constexpr int kKBlocks = 4;                       // MMAs (K = 64 each) per stage
constexpr int kTokBytes = 128 * 128;              // 128 token rows x 128 bytes of K
constexpr int kWgtBytes = 128 * 128;              // this CTA's 128 of the tile's 256 weight rows
constexpr int kSfTokBytes = kKBlocks * 512;       // scale atoms of the CTA's token rows
constexpr int kSfWgtBytes = 2 * kKBlocks * 512;   // scale atoms of all 256 weight rows
constexpr int kStageBytes = kTokBytes + kWgtBytes + kSfTokBytes + kSfWgtBytes;   // 38912
constexpr int kScaleWarps = 4, kEpilogueWarps = 8, kFirstEpilogueWarp = 2 + kScaleWarps;
constexpr int kThreads = 32 * (2 + kScaleWarps + kEpilogueWarps);
constexpr int kAccCols = 256;
constexpr int kSfSlotCols = kKBlocks * (4 + 8);   // per stage: token scales 4 columns per K block, weight scales 8
constexpr int kTmemCols = 512;
static_assert(kAccCols + kStages * kSfSlotCols <= kTmemCols, "tensor memory over-subscribed");
constexpr int kBarrierBytes = (4 * kStages + 2) * 8 + 16;
constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;

template <bool kProfile>   // cycle counters of the tuning aid live in an instantiation of their own
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ PairGemmParams p) {
  constexpr bool prof = kProfile;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* sf_ready_bar = empty_bar + kStages;
  uint64_t* sf_full_bar = sf_ready_bar + kStages;
  uint64_t* acc_full_bar = sf_full_bar + kStages;
  uint64_t* acc_empty_bar = acc_full_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = cluster_rank();           // 0 = leader of the pair
  griddep_launch();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar + s, 1);
      ptx::mbar_init(empty_bar + s, 1);
      ptx::mbar_init(sf_ready_bar + s, 2 * kScaleWarps);
      ptx::mbar_init(sf_full_bar + s, 1);
    }
    ptx::mbar_init(acc_full_bar, 1);
    ptx::mbar_init(acc_empty_bar, 2 * kEpilogueWarps);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                               // both CTAs' barriers exist before anybody signals them
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  griddep_wait();

  const int total_kb = p.k / 64;
  const int k_stages = (total_kb + kKBlocks - 1) / kKBlocks;
  const int k_atoms = p.k / 64;
  const int pairs = gridDim.x / 2, pair = blockIdx.x / 2;
  const int total_work = p.l_tiles * p.c_tiles;
  constexpr uint32_t kDescHiSw128 = uint32_t(1024 >> 4) | (1u << 14) | (2u << 29);
  auto make_desc = [](uint32_t hi, uint32_t lo) { return (uint64_t(hi) << 32) | lo; };
  const uint32_t smem_base16 = ptx::smem_u32(smem) >> 4;
  const long long prof_start = prof ? clock64() : 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (one lane)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      long long prof_wait = 0;
      for (int w = pair; w < total_work && !*abort_flag; w += pairs) {
        const int c_tile = w % p.c_tiles, l_tile = w / p.c_tiles;
        const int token_row = (l_tile * 2 + int(rank)) * 128;        // this CTA's 128 token rows
        const int weight_row = c_tile * 256 + int(rank) * 128;       // this CTA's half of the weight rows
        // rows beyond the matrix are zero-filled by the tensor copy and masked in the epilogue; their
        // scale atoms are read from the last block that exists
        const int token_block = min(l_tile * 2 + int(rank), p.token_row_blocks - 1);
        const uint8_t* sf_tokens = p.sf_tokens + size_t(token_block) * k_atoms * 512;
        bool failed = false;
        for (int ks = 0; ks < k_stages; ++ks) {
          const long long t0 = prof ? clock64() : 0;
          if (!ptx::mbar_wait_bounded(empty_bar + stage, phase ^ 1)) {
            report(p.error, 0x11000000u | (blockIdx.x << 8) | stage, abort_flag);
            failed = true;
            break;
          }
          if (prof) prof_wait += clock64() - t0;
          const int nkb = min(kKBlocks, total_kb - ks * kKBlocks);
          uint8_t* base = smem + stage * kStageBytes;
          // the scales go first and complete on their own barrier: the loader warps move them into tensor
          // memory while the operand tiles are still in flight
          uint64_t* sf_bar = sf_full_bar + stage;
          ptx::mbar_expect_tx(sf_bar, nkb * 512 + kSfWgtBytes);
          ptx::bulk_load(base + kTokBytes + kWgtBytes, sf_tokens + size_t(ks) * kKBlocks * 512, nkb * 512, sf_bar);
          // weight scales of both halves: [row blocks][K/64 atoms] of 8-byte words, box = 4 atoms x 2 row blocks
          ptx::tma_load_2d(base + kTokBytes + kWgtBytes + kSfTokBytes, &p.map_weight_scales, ks * 256, c_tile * 2, sf_bar);
          uint64_t* bar = full_bar + stage;
          ptx::mbar_expect_tx(bar, kTokBytes + kWgtBytes);
          ptx::tma_load_2d(base, &p.map_tokens, ks * 128, token_row, bar);
          ptx::tma_load_2d(base + kTokBytes, &p.map_weights, ks * 128, weight_row, bar);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
      }
      if (prof) p.profile[size_t(blockIdx.x) * 8 + 0] = prof_wait;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA, one lane)
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      const uint32_t idesc = idesc_pair_nvfp4(256);
      long long prof_sf = 0, prof_issue = 0, prof_acc = 0;
      for (int w = pair; w < total_work && !*abort_flag; w += pairs) {
        const long long ta = prof ? clock64() : 0;
        if (!ptx::mbar_wait_bounded(acc_empty_bar, acc_phase ^ 1)) {
          report(p.error, 0x21000000u | (blockIdx.x << 8), abort_flag);
          break;
        }
        if (prof) prof_acc += clock64() - ta;
        ptx::tc_fence_after_sync();
        bool failed = false;
        for (int ks = 0; ks < k_stages; ++ks) {
          const long long t0 = prof ? clock64() : 0;
          // sf_ready implies that both CTAs' operands have landed (the loader warps arrive after their
          // CTA's operand barrier), so this is the only wait of the stage
          const bool ok = ptx::mbar_wait_bounded(sf_ready_bar + stage, phase);
          const long long t2 = prof ? clock64() : 0;
          if (!ok) {
            report(p.error, 0x31000000u | (blockIdx.x << 8) | stage, abort_flag);
            failed = true;
            break;
          }
          if (prof) prof_sf += t2 - t0;
          ptx::tc_fence_after_sync();
          const int nkb = min(kKBlocks, total_kb - ks * kKBlocks);
          const uint32_t base16 = smem_base16 + uint32_t(stage) * uint32_t(kStageBytes >> 4);
          const uint32_t sf_tok = tmem_base + kAccCols + uint32_t(stage) * kSfSlotCols;
          const uint32_t sf_wgt = sf_tok + 4 * kKBlocks;
#pragma unroll
          for (int kb = 0; kb < kKBlocks; ++kb)
            if (kb < nkb)
              mma_pair_nvfp4(tmem_base, make_desc(kDescHiSw128, base16 + 2 * kb),
                             make_desc(kDescHiSw128, base16 + (kTokBytes >> 4) + 2 * kb), idesc, sf_tok + 4 * kb,
                             sf_wgt + 8 * kb, (ks | kb) != 0 ? 1u : 0u);
          commit_pair(empty_bar + stage);
          if (prof) prof_issue += clock64() - t2;
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        commit_pair(acc_full_bar);
        acc_phase ^= 1;
      }
      if (prof) {
        long long* row = p.profile + size_t(blockIdx.x) * 8;
        row[2] = prof_sf; row[3] = prof_issue; row[4] = prof_acc;
      }
    }
    if (prof && lane == 0) p.profile[size_t(blockIdx.x) * 8 + 6] = clock64() - prof_start;
    __syncwarp();
  } else if (warp < kFirstEpilogueWarp) {
    // ------------------------------------------------------------------ scale loaders
    const uint32_t quad_lane = uint32_t((warp % 4) * 32) << 16;
    const uint32_t leader_sf_ready = leader_address(sf_ready_bar);
    int stage = 0;
    uint32_t phase = 0;
    long long prof_copy = 0, prof_arrive = 0;
    for (int w = pair; w < total_work && !*abort_flag; w += pairs) {
      bool failed = false;
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(sf_full_bar + stage, phase))) {
          report(p.error, 0x61000000u | (blockIdx.x << 8) | stage, abort_flag);
          failed = true;
          break;
        }
        const long long t1 = prof ? clock64() : 0;
        const uint32_t src = ptx::smem_u32(smem + stage * kStageBytes + kTokBytes + kWgtBytes) + lane * 16;
        const uint32_t slot = tmem_base + kAccCols + uint32_t(stage) * kSfSlotCols + quad_lane;
        uint32_t r[16];
#pragma unroll
        for (int kb = 0; kb < kKBlocks; ++kb) {
          const uint4 v = ptx::lds128(src + kb * 512);
          r[4 * kb] = v.x; r[4 * kb + 1] = v.y; r[4 * kb + 2] = v.z; r[4 * kb + 3] = v.w;
        }
        ptx::tmem_store16(slot, r);
        // weight scales: per K block [rows 0..127: 4 columns][rows 128..255: 4 columns]
#pragma unroll
        for (int half_pair = 0; half_pair < 2; ++half_pair) {
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int kb = 2 * half_pair + i;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint4 v = ptx::lds128(src + kSfTokBytes + (h * kKBlocks + kb) * 512);
              r[8 * i + 4 * h] = v.x; r[8 * i + 4 * h + 1] = v.y; r[8 * i + 4 * h + 2] = v.z; r[8 * i + 4 * h + 3] = v.w;
            }
          }
          ptx::tmem_store16(slot + 4 * kKBlocks + 16 * half_pair, r);
        }
        ptx::tmem_store_wait();
        const long long t2 = prof ? clock64() : 0;
        ptx::tc_fence_before_sync();
        // the arrival also vouches for this CTA's operand tiles
        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(full_bar + stage, phase))) {
          report(p.error, 0x62000000u | (blockIdx.x << 8) | stage, abort_flag);
          failed = true;
          break;
        }
        if (lane == 0) arrive_cluster(leader_sf_ready + stage * 8);
        if (prof) { prof_copy += t2 - t1; prof_arrive += clock64() - t2; }
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (failed) break;
    }
    if (prof && lane == 0 && warp == 2) {
      long long* row = p.profile + size_t(blockIdx.x) * 8;
      row[5] = prof_copy;
      row[7] = prof_arrive;
    }
  } else {
    // ------------------------------------------------------------------ epilogue (own 128 rows x 256 channels)
    const int quad = warp % 4;
    const int col_half = (warp - kFirstEpilogueWarp) / 4;
    const uint32_t leader_acc_empty = leader_address(acc_empty_bar);
    const bool hi = (lane & 2) != 0, lo = (lane & 1) != 0;
    uint32_t acc_phase = 0;
    bf16* out = static_cast<bf16*>(p.out);
    for (int w = pair; w < total_work && !*abort_flag; w += pairs) {
      const int c_tile = w % p.c_tiles, l_tile = w / p.c_tiles;
      if (!ptx::mbar_wait_warp(acc_full_bar, acc_phase)) {
        report(p.error, 0x41000000u | (blockIdx.x << 8), abort_flag);
        break;
      }
      acc_phase ^= 1;
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16);
      const int row0 = (l_tile * 2 + int(rank)) * 128 + quad * 32 + (lane & ~3);     // first row of this lane group
      const int rows_left = p.rows - row0;
      const int c_base = c_tile * 256;
      uint4 unit[4][4];
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        const int c0 = col_half * 128 + 32 * ch;
        uint32_t r[32];
        ptx::tmem_load16(taddr + c0, r);
        ptx::tmem_load16(taddr + c0 + 16, r + 16);
        ptx::tmem_load_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q)
          unit[ch][q] = make_uint4(
              pack_bf16x2(__fmul_rn(__uint_as_float(r[8 * q]), p.alpha), __fmul_rn(__uint_as_float(r[8 * q + 1]), p.alpha)),
              pack_bf16x2(__fmul_rn(__uint_as_float(r[8 * q + 2]), p.alpha), __fmul_rn(__uint_as_float(r[8 * q + 3]), p.alpha)),
              pack_bf16x2(__fmul_rn(__uint_as_float(r[8 * q + 4]), p.alpha), __fmul_rn(__uint_as_float(r[8 * q + 5]), p.alpha)),
              pack_bf16x2(__fmul_rn(__uint_as_float(r[8 * q + 6]), p.alpha), __fmul_rn(__uint_as_float(r[8 * q + 7]), p.alpha)));
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) arrive_cluster(leader_acc_empty);             // the next tile's MMAs may start
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        const int c0 = col_half * 128 + 32 * ch;
        uint4* u = unit[ch];
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
        const int c = c_base + c0 + 8 * (lane & 3);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (i >= rows_left || c >= p.n) continue;
          bf16* dst = out + size_t(row0 + i) * p.ld_out + c;
          if (c + 8 <= p.n) {
            *reinterpret_cast<uint4*>(dst) = u[i];
          } else {
            const uint32_t words[4] = {u[i].x, u[i].y, u[i].z, u[i].w};
            for (int e = 0; e < 8; ++e)
              if (c + e < p.n) reinterpret_cast<uint16_t*>(dst)[e] = uint16_t(words[e / 2] >> (16 * (e % 2)));
          }
        }
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                               // the peer no longer reads this CTA's shared or tensor memory
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

long long* g_pair_profile = nullptr;

}  // namespace

void set_pair_profile_buffer(long long* device_buffer) { g_pair_profile = device_buffer; }

namespace {
template <bool kProfile>
cudaError_t launch_pair_instance(const PairGemmParams& params, int sm_count, cudaStream_t stream) {
  static bool configured_on[kMaxDeviceSlots] = {};   // the attribute is per GPU
  bool& configured = configured_on[current_device_slot()];
  if (!configured) {
    cudaError_t status =
        cudaFuncSetAttribute(gemm_pair_kernel<kProfile>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (status != cudaSuccess) return status;
    configured = true;
  }
  const int work = params.l_tiles * params.c_tiles;
  int pairs = sm_count / 2;
  if (work < pairs) pairs = work;
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(2 * pairs);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attributes[2]{};
  attributes[0].id = cudaLaunchAttributeClusterDimension;
  attributes[0].val.clusterDim.x = 2;
  attributes[0].val.clusterDim.y = 1;
  attributes[0].val.clusterDim.z = 1;
  attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attributes;
  config.numAttrs = 2;
  note_launch();
  return cudaLaunchKernelEx(&config, gemm_pair_kernel<kProfile>, params);
}
}  // namespace

cudaError_t launch_gemm_pair(const PairGemmParams& params_in, int sm_count, cudaStream_t stream) {
  PairGemmParams params = params_in;
  params.profile = g_pair_profile;
  if (params.profile != nullptr) return launch_pair_instance<true>(params, sm_count, stream);
  return launch_pair_instance<false>(params, sm_count, stream);
}

}  // namespace gw
