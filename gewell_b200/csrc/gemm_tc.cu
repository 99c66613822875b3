// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   warp 0      TMA producer: operand tiles (cp.async.bulk.tensor, 128B swizzle)
//               and scale-factor atoms (cp.async.bulk) into a ring of smem stages
//   warp 1      MMA issuer: scale atoms smem->TMEM (tcgen05.cp), block-scaled
//               tcgen05.mma (kind::mxf4nvf4, or kind::f8f6f4 for FP8) into a
//               TMEM accumulator, tcgen05.commit to free stages / publish tiles
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one TMEM lane quadrant
//               per warp), scale, round to BF16, store
//
// A (128 rows per tile) sits on the TMEM-lane side, B (BLOCK_N rows per tile,
// any multiple of 16 valid) on the TMEM-column side; see gemm_tc.cuh.
// Every wait is bounded: on a timeout the role records an error word, raises
// the CTA's abort flag and all roles unwind to the common exit, where TMEM is
// released.
#include <string>

#include "common.cuh"
#include "gemm_tc.cuh"
#include "ptx.cuh"

namespace gw {
namespace {

constexpr int kThreads = 192;
constexpr int kTileA = 128;
constexpr int kStageRowBytes = 128;   // bytes of K per stage row (= swizzle span)
constexpr int kAtomBytes = 512;       // one scale atom: 128 rows x 4 K16 blocks
constexpr int kKBlocksPerStage = 4;   // MMAs per stage (K=64 FP4 / K=32 FP8 each: 32 bytes)

template <bool kNvfp4, int BLOCK_N>
struct Config {
  static constexpr int kAccStages = BLOCK_N >= 256 ? 1 : 2;
  static constexpr int kBAtomRows = BLOCK_N > 128 ? BLOCK_N / 128 : 1;
  static constexpr int kABytes = kTileA * kStageRowBytes;
  static constexpr int kBBytes = BLOCK_N * kStageRowBytes;
  static constexpr int kSfaBytes = kNvfp4 ? kKBlocksPerStage * kAtomBytes : 0;
  static constexpr int kSfbBytes = kNvfp4 ? kBAtomRows * kKBlocksPerStage * kAtomBytes : 0;
  static constexpr int kStageBytes = kABytes + kBBytes + kSfaBytes + kSfbBytes;
  static constexpr int kMaxSmem = 227 * 1024 - 2048;   // leave room for barriers + alignment slack
  static constexpr int kStagesRaw = kMaxSmem / kStageBytes;
  static constexpr int kStages = kStagesRaw > 8 ? 8 : kStagesRaw;
  static constexpr int kSfbColsPerKb = 4 * kBAtomRows;
  static constexpr int kAccCols = kAccStages * BLOCK_N;
  static constexpr int kSfaCol = kAccCols;
  static constexpr int kSfbCol = kSfaCol + (kNvfp4 ? 4 * kKBlocksPerStage : 0);
  static constexpr int kUsedCols = kSfbCol + (kNvfp4 ? kSfbColsPerKb * kKBlocksPerStage : 0);
  static constexpr int kTmemCols = kUsedCols <= 32 ? 32 : kUsedCols <= 64 ? 64 : kUsedCols <= 128 ? 128
                                   : kUsedCols <= 256 ? 256 : 512;
  static constexpr int kBarrierBytes = (2 * kStages + 2 * kAccStages) * 8 + 16;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;  // +1024 alignment slack
  static_assert(kUsedCols <= 512, "TMEM over-subscribed");
  static_assert(kStages >= 2, "need at least two stages");
  // More than half of the SM's shared memory: at most one CTA per SM, so a
  // 512-column TMEM allocation can never wait on a co-resident CTA.
  static_assert(kSmemBytes > 116 * 1024, "one CTA per SM is assumed by the TMEM allocation");
};

struct WorkItem {
  GemmGroup group;
  int a_tile, b_tile;
  int n_valid;   // valid B rows in this tile
  int mma_n;     // n_valid rounded up to 16
};

template <int BLOCK_N>
__device__ __forceinline__ bool decode_work(const GemmParams& p, int w, WorkItem& item) {
  int gi = 0;
  if (p.groups != nullptr) {
    // largest gi with groups[gi].work_begin <= w  (groups[num_groups] is the sentinel)
    int lo = 0, hi = p.num_groups;
    while (lo + 1 < hi) {
      const int mid = (lo + hi) / 2;
      if (p.groups[mid].work_begin <= w) lo = mid; else hi = mid;
    }
    gi = lo;
    item.group = p.groups[gi];
  } else {
    item.group = p.single;
  }
  const int local = w - item.group.work_begin;
  item.a_tile = local % item.group.a_tiles;
  item.b_tile = local / item.group.a_tiles;
  const int remaining = item.group.b_rows - item.b_tile * BLOCK_N;
  item.n_valid = remaining < BLOCK_N ? remaining : BLOCK_N;
  item.mma_n = (item.n_valid + 15) & ~15;
  return item.n_valid > 0;
}

__device__ __forceinline__ void report(uint32_t* error, uint32_t code, volatile int* abort_flag) {
  *abort_flag = 1;
  if (error != nullptr) atomicCAS(error, 0u, code);
}

template <bool kNvfp4, int BLOCK_N>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ GemmParams p) {
  using C = Config<kNvfp4, BLOCK_N>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* acc_full_bar = empty_bar + C::kStages;
  uint64_t* acc_empty_bar = acc_full_bar + C::kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + C::kAccStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) { ptx::mbar_init(full_bar + s, 1); ptx::mbar_init(empty_bar + s, 1); }
    for (int a = 0; a < C::kAccStages; ++a) { ptx::mbar_init(acc_full_bar + a, 1); ptx::mbar_init(acc_empty_bar + a, 4); }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::fence_proxy_async_smem();
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, C::kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total_work = p.groups != nullptr ? p.groups[p.num_groups].work_begin : p.total_work;
  const int k_bytes = kNvfp4 ? p.k / 2 : p.k;
  const int total_kb = (k_bytes + 31) / 32;                 // MMA K-blocks (32 bytes of K each)
  const int k_stages = (total_kb + kKBlocksPerStage - 1) / kKBlocksPerStage;
  const int k_atoms = p.k / 64;                             // scale atoms per 128-row block (NVFP4)

  auto stage_a = [&](int s) { return smem + s * C::kStageBytes; };
  auto stage_b = [&](int s) { return smem + s * C::kStageBytes + C::kABytes; };
  auto stage_sfa = [&](int s) { return smem + s * C::kStageBytes + C::kABytes + C::kBBytes; };
  auto stage_sfb = [&](int s) { return smem + s * C::kStageBytes + C::kABytes + C::kBBytes + C::kSfaBytes; };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x) {
      WorkItem item;
      if (!decode_work<BLOCK_N>(p, w, item)) continue;
      const CUtensorMap* map_a = item.group.map_a >= 0 ? p.map_a_table + item.group.map_a : &p.map_a;
      if (item.group.map_a >= 0 && lane == 0) ptx::tensormap_acquire(map_a);
      const int b_row = item.group.b_row0 + item.b_tile * BLOCK_N;
      const int sfb_row = item.group.sfb_row0 + item.b_tile * BLOCK_N;
      const int b_atom_rows = (item.n_valid + 127) / 128;
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!ptx::mbar_wait_bounded(empty_bar + stage, phase ^ 1)) {
          report(p.error, 0x10000000u | (blockIdx.x << 8) | stage, abort_flag);
          break;
        }
        if (*abort_flag) break;
        if (lane == 0) {
          const int nkb = min(kKBlocksPerStage, total_kb - ks * kKBlocksPerStage);
          uint32_t bytes = C::kABytes + C::kBBytes;
          if constexpr (kNvfp4) bytes += nkb * kAtomBytes * (1 + b_atom_rows);
          ptx::mbar_expect_tx(full_bar + stage, bytes);
          ptx::tma_load_2d(stage_a(stage), map_a, ks * kStageRowBytes, item.a_tile * kTileA, full_bar + stage);
          ptx::tma_load_2d(stage_b(stage), &p.map_b, ks * kStageRowBytes, b_row, full_bar + stage);
          if constexpr (kNvfp4) {
            const size_t atom0 = size_t(ks) * kKBlocksPerStage;
            ptx::bulk_load(stage_sfa(stage),
                           item.group.sf_a + (size_t(item.a_tile) * k_atoms + atom0) * kAtomBytes,
                           nkb * kAtomBytes, full_bar + stage);
            for (int j = 0; j < b_atom_rows; ++j)
              ptx::bulk_load(stage_sfb(stage) + j * kKBlocksPerStage * kAtomBytes,
                             p.sf_b + (size_t(sfb_row / 128 + j) * k_atoms + atom0) * kAtomBytes,
                             nkb * kAtomBytes, full_bar + stage);
          }
        }
        __syncwarp();
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x) {
      WorkItem item;
      if (!decode_work<BLOCK_N>(p, w, item)) continue;
      if (!ptx::mbar_wait_bounded(acc_empty_bar + acc, acc_phase ^ 1)) {
        report(p.error, 0x20000000u | (blockIdx.x << 8) | acc, abort_flag);
        break;
      }
      ptx::tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
      const uint32_t idesc = kNvfp4 ? ptx::idesc_nvfp4(item.mma_n) : ptx::idesc_fp8(item.mma_n);
      const int sfb_row = item.group.sfb_row0 + item.b_tile * BLOCK_N;
      const uint32_t sfb_sub = BLOCK_N < 128 ? (sfb_row % 128) / 32 : 0;
      const int b_atom_rows = (item.n_valid + 127) / 128;
      bool failed = false;
      for (int ks = 0; ks < k_stages; ++ks) {
        if (!ptx::mbar_wait_bounded(full_bar + stage, phase)) {
          report(p.error, 0x30000000u | (blockIdx.x << 8) | stage, abort_flag);
          failed = true;
          break;
        }
        if (*abort_flag) { failed = true; break; }
        ptx::tc_fence_after_sync();
        if (lane == 0) {
          const int nkb = min(kKBlocksPerStage, total_kb - ks * kKBlocksPerStage);
          if constexpr (kNvfp4) {
            const uint32_t sfa_smem = ptx::smem_u32(stage_sfa(stage));
            const uint32_t sfb_smem = ptx::smem_u32(stage_sfb(stage));
            for (int kb = 0; kb < nkb; ++kb) {
              ptx::tc_copy_sf_atom(tmem_base + C::kSfaCol + 4 * kb, ptx::smem_desc_sf_atom(sfa_smem + kb * kAtomBytes));
              for (int j = 0; j < b_atom_rows; ++j)
                ptx::tc_copy_sf_atom(tmem_base + C::kSfbCol + kb * C::kSfbColsPerKb + 4 * j,
                                     ptx::smem_desc_sf_atom(sfb_smem + (j * kKBlocksPerStage + kb) * kAtomBytes));
            }
          }
          const uint64_t a_desc = ptx::smem_desc_sw128(ptx::smem_u32(stage_a(stage)));
          const uint64_t b_desc = ptx::smem_desc_sw128(ptx::smem_u32(stage_b(stage)));
          for (int kb = 0; kb < nkb; ++kb) {
            const uint32_t accumulate = (ks | kb) != 0;
            if constexpr (kNvfp4)
              ptx::tc_mma_nvfp4(d_tmem, a_desc + 2 * kb, b_desc + 2 * kb, idesc,
                                tmem_base + C::kSfaCol + 4 * kb,
                                tmem_base + C::kSfbCol + kb * C::kSfbColsPerKb + sfb_sub, accumulate);
            else
              ptx::tc_mma_fp8(d_tmem, a_desc + 2 * kb, b_desc + 2 * kb, idesc, accumulate);
          }
          ptx::tc_commit(empty_bar + stage);
        }
        __syncwarp();
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
      if (failed) break;
      if (lane == 0) ptx::tc_commit(acc_full_bar + acc);
      __syncwarp();
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp % 4;   // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    bf16* out = static_cast<bf16*>(p.out);
    for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x) {
      WorkItem item;
      if (!decode_work<BLOCK_N>(p, w, item)) continue;
      if (!ptx::mbar_wait_bounded(acc_full_bar + acc, acc_phase)) {
        report(p.error, 0x40000000u | (blockIdx.x << 8) | acc, abort_flag);
        break;
      }
      ptx::tc_fence_after_sync();
      const int channel = item.a_tile * kTileA + quad * 32 + lane;
      const bool channel_ok = channel < item.group.a_rows;
      float alpha = item.group.alpha;
      if (item.group.channel_alpha != nullptr && channel_ok) alpha = item.group.channel_alpha[channel];
      bf16* dst = out + (size_t(item.group.out_row0) + size_t(item.b_tile) * BLOCK_N) * p.ld_out +
                  item.group.out_col0 + channel;
      const uint32_t taddr = tmem_base + acc * BLOCK_N + (uint32_t(quad * 32) << 16);
      for (int c0 = 0; c0 < item.mma_n; c0 += 16) {
        uint32_t r[16];
        ptx::tmem_load16(taddr + c0, r);
        ptx::tmem_load_wait();
        if (channel_ok) {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (c0 + i < item.n_valid)
              dst[size_t(c0 + i) * p.ld_out] = __float2bfloat16_rn(__fmul_rn(__uint_as_float(r[i]), alpha));
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(acc_empty_bar + acc);
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <bool kNvfp4, int BLOCK_N>
cudaError_t launch(const GemmParams& params, int grid, cudaStream_t stream) {
  using C = Config<kNvfp4, BLOCK_N>;
  static bool configured = false;
  if (!configured) {
    cudaError_t status = cudaFuncSetAttribute(gemm_tc_kernel<kNvfp4, BLOCK_N>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (status != cudaSuccess) return status;
    configured = true;
  }
  gemm_tc_kernel<kNvfp4, BLOCK_N><<<grid, kThreads, C::kSmemBytes, stream>>>(params);
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_gemm_tc(GemmKind kind, int block_n, const GemmParams& params, int grid, cudaStream_t stream) {
  const bool fp4 = kind == GemmKind::nvfp4;
  switch (block_n) {
    case 32: return fp4 ? launch<true, 32>(params, grid, stream) : launch<false, 32>(params, grid, stream);
    case 64: return fp4 ? launch<true, 64>(params, grid, stream) : launch<false, 64>(params, grid, stream);
    case 128: return fp4 ? launch<true, 128>(params, grid, stream) : launch<false, 128>(params, grid, stream);
    case 256: return fp4 ? launch<true, 256>(params, grid, stream) : launch<false, 256>(params, grid, stream);
    default: return cudaErrorInvalidValue;
  }
}

size_t gemm_tc_smem_bytes(GemmKind kind, int block_n) {
  const bool fp4 = kind == GemmKind::nvfp4;
  switch (block_n) {
    case 32: return fp4 ? Config<true, 32>::kSmemBytes : Config<false, 32>::kSmemBytes;
    case 64: return fp4 ? Config<true, 64>::kSmemBytes : Config<false, 64>::kSmemBytes;
    case 128: return fp4 ? Config<true, 128>::kSmemBytes : Config<false, 128>::kSmemBytes;
    case 256: return fp4 ? Config<true, 256>::kSmemBytes : Config<false, 256>::kSmemBytes;
    default: return 0;
  }
}

}  // namespace gw
