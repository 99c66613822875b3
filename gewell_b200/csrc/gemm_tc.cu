// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   warp 0       TMA producer: operand tiles (cp.async.bulk.tensor, 128B swizzle)
//                and scale-factor atoms (cp.async.bulk) into a ring of smem stages
//   warp 1       MMA issuer: block-scaled tcgen05.mma (kind::mxf4nvf4, or
//                kind::f8f6f4 for FP8); tcgen05.commit frees stages / publishes
//                accumulators.  Nothing else runs in the tensor pipe.
//   warps 2..5   scale loaders (NVFP4): one warp per TMEM lane quadrant moves the
//                stage's scale atoms smem -> registers -> TMEM (tcgen05.st) into a
//                per-stage TMEM slot.  Measured on B200, a tcgen05.cp scale copy
//                occupies the tensor pipe for ~40 cycles and never overlaps an MMA
//                (12 copies per stage = 490 cycles next to 630 cycles of MMA);
//                going through registers takes the copies out of that pipe.
//   warps 6..13  epilogue: two warps per TMEM lane quadrant, each draining half of
//                the accumulator columns with tcgen05.ld
//
// Operand roles and the three epilogues are described in gemm_tc.cuh.  Every
// wait is bounded: on a timeout the role records an error word, raises the
// CTA's abort flag and all roles unwind to the common exit, where TMEM is
// released.  No load in this file fans out to other CTAs.
#include <string>

#include "common.cuh"
#include "gemm_tc.cuh"
#include "ptx.cuh"
#include "work_walk.h"

namespace gw {
namespace {

constexpr int kScaleWarps = 4;
constexpr int kEpilogueWarps = 8;
constexpr int kFirstEpilogueWarp = 2 + kScaleWarps;
constexpr int kThreads = 32 * (2 + kScaleWarps + kEpilogueWarps);
constexpr int kTileL = 128;
constexpr int kStageRowBytes = 128;   // bytes of K per stage row (= swizzle span)
constexpr int kAtomBytes = 512;       // one scale atom: 128 rows x 4 K16 blocks
constexpr int kKBlocksPerStage = 4;   // MMAs per 128-byte slab of K (K=64 FP4 / K=32 FP8 each: 32 bytes)

// Slabs (128 bytes of K each) per ring stage.  The FP8 swap form -- the decode shapes, which stream
// the weights once -- takes two: a stage's barrier round (wait, commit, release, refill) costs about
// as much as two of its MMAs, and with 256 bytes of K per round it is paid half as often.
__host__ __device__ constexpr int slabs_per_stage(GemmKind kind, GemmEpilogue epilogue) {
  return kind == GemmKind::fp8 && epilogue == GemmEpilogue::swap_store ? 2 : 1;
}

template <bool kNvfp4, int BLOCK_N, int SLABS = 1>
struct Config {
  static_assert(SLABS == 1 || !kNvfp4, "the scale slots are laid out for one slab per stage");
  static constexpr int kSlabs = SLABS;
  static constexpr int kLSlabBytes = kTileL * kStageRowBytes;
  static constexpr int kCSlabBytes = BLOCK_N * kStageRowBytes;
  static constexpr int kAccStages = BLOCK_N >= 256 ? 1 : 2;
  static constexpr int kHalves = BLOCK_N > 128 ? BLOCK_N / 128 : 1;
  static constexpr int kHalfRows = BLOCK_N / kHalves;
  static constexpr int kLBytes = SLABS * kLSlabBytes;
  static constexpr int kCBytes = SLABS * kCSlabBytes;
  static constexpr int kSflBytes = kNvfp4 ? kKBlocksPerStage * kAtomBytes : 0;
  static constexpr int kSfcBytes = kNvfp4 ? kHalves * kKBlocksPerStage * kAtomBytes : 0;
  static constexpr int kStageBytes = kLBytes + kCBytes + kSflBytes + kSfcBytes;
  static constexpr int kMaxSmem = 227 * 1024 - 2048;   // leave room for barriers + alignment slack
  static constexpr int kStagesRaw = kMaxSmem / kStageBytes;
  static constexpr int kStages = kStagesRaw > 12 ? 12 : kStagesRaw;
  static constexpr int kSfcColsPerKb = 4 * kHalves;
  static constexpr int kAccCols = kAccStages * BLOCK_N;
  // one scale slot per smem stage: [L scales: 4 columns per K-block][C scales]
  static constexpr int kSfSlotCols = kNvfp4 ? kKBlocksPerStage * (4 + kSfcColsPerKb) : 0;
  static constexpr int kSflCol = kAccCols;                               // + stage * kSfSlotCols
  static constexpr int kSfcCol = kSflCol + 4 * kKBlocksPerStage;         // + stage * kSfSlotCols
  static constexpr int kUsedCols = kAccCols + kStages * kSfSlotCols;
  static constexpr int kTmemCols = kUsedCols <= 32 ? 32 : kUsedCols <= 64 ? 64 : kUsedCols <= 128 ? 128
                                   : kUsedCols <= 256 ? 256 : 512;
  static constexpr int kMaxGroups = 256;
  static constexpr int kBarrierBytes = (3 * kStages + 2 * kAccStages) * 8 + 16 + (kMaxGroups + 4) * 4;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;  // +1024 alignment slack
  static_assert(kUsedCols <= 512, "TMEM over-subscribed");
  static_assert(kStages >= 2, "need at least two stages");
  // More than half of the SM's shared memory: at most one CTA per SM, so a
  // 512-column TMEM allocation can never wait on a co-resident CTA.
  static_assert(kSmemBytes > 116 * 1024, "one CTA per SM is assumed by the TMEM allocation");
};

struct WorkItem {
  GemmGroup g;
  int l_tile, c_tile;
  int l_valid;   // valid lanes (rows of L) in this tile
  int c_valid;   // swap form: valid columns (tokens) in this tile
  int halves;    // boxes of the C operand that hold valid rows in this tile
  int mma_n;     // MMA N for this tile
  int group = -1;   // index of g in the launch's group table (grouped launches)
};

template <int BLOCK_N, GemmEpilogue EPI>
__device__ __forceinline__ void decode_work(const GemmParams& p, const int32_t* prefix, int w, WorkItem& item) {
  using C = Config<true, BLOCK_N>;
  if (p.groups != nullptr) {
    // The item decoded into this slot before is usually of the same group: keep its descriptor then
    // (no search, no global load).  prefix[] holds work_begin of every group plus the total.
    if (item.group < 0 || w < prefix[item.group] || w >= prefix[item.group + 1]) {
      // largest gi with work_begin[gi] <= w; the prefix sums were staged in shared memory
      int lo = 0, hi = p.num_groups;
      while (lo + 1 < hi) {
        const int mid = (lo + hi) / 2;
        if (prefix[mid] <= w) lo = mid; else hi = mid;
      }
      item.g = p.groups[lo];
      item.group = lo;
    }
  } else {
    item.g = p.single;
  }
  const int local = w - item.g.work_begin;
  if constexpr (EPI == GemmEpilogue::swap_store) {
    // consecutive work items share the token tile and sweep the weight tiles
    item.l_tile = local % item.g.l_tiles;
    item.c_tile = local / item.g.l_tiles;
  } else {
    // consecutive work items share the token tile (L) and sweep the weight tiles (C)
    item.c_tile = local % item.g.c_tiles;
    item.l_tile = local / item.g.c_tiles;
  }
  const int l_left = item.g.l_rows - item.l_tile * kTileL;
  item.l_valid = l_left < kTileL ? l_left : kTileL;
  const int c_left = item.g.c_rows - item.c_tile * p.c_rows_per_tile;
  item.c_valid = c_left < C::kHalfRows ? c_left : C::kHalfRows;
  // a dense projection whose row count is not a multiple of BLOCK_N leaves the
  // second half of its last column tile empty
  item.halves = C::kHalves;
  if (C::kHalves == 2 && item.g.c_half_stride != 0 && c_left <= C::kHalfRows) item.halves = 1;
  if constexpr (EPI == GemmEpilogue::swap_store) item.mma_n = (item.c_valid + 15) & ~15;   // kHalves == 1
  else item.mma_n = item.halves * C::kHalfRows;
}

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
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

// kProfile: the cycle counters of the tuning aid are compiled into an instantiation of their own,
// so the production kernel carries none of their registers.
template <GemmKind KIND, int BLOCK_N, GemmEpilogue EPI, bool kProfile>
// 14 warps are allocated as 16: 128 registers per thread is the most one CTA can have.
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ GemmParams p) {
  constexpr bool kNvfp4 = KIND == GemmKind::nvfp4;
  using C = Config<kNvfp4, BLOCK_N, slabs_per_stage(KIND, EPI)>;
  constexpr int kSlabs = C::kSlabs;
  constexpr int kKbPerStage = kKBlocksPerStage * kSlabs;    // MMAs per stage
  constexpr bool prof = kProfile;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
  uint64_t* empty_bar = full_bar + C::kStages;
  uint64_t* sf_ready_bar = empty_bar + C::kStages;
  uint64_t* acc_full_bar = sf_ready_bar + C::kStages;
  uint64_t* acc_empty_bar = acc_full_bar + C::kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + C::kAccStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* split_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
  int32_t* prefix = reinterpret_cast<int32_t*>(tmem_slot + 4);   // work_begin of every group (+ sentinel)
  griddep_launch();

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      ptx::mbar_init(full_bar + s, 1);
      ptx::mbar_init(empty_bar + s, 1);
      ptx::mbar_init(sf_ready_bar + s, kScaleWarps);
    }
    for (int a = 0; a < C::kAccStages; ++a) {
      ptx::mbar_init(acc_full_bar + a, 1);
      ptx::mbar_init(acc_empty_bar + a, kEpilogueWarps);
    }
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
  // Everything above is independent of earlier kernels in the stream and may overlap
  // them (programmatic dependent launch); from here on their results are read.
  const bool early_weights = EPI == GemmEpilogue::swap_store && p.groups == nullptr && p.early_weights != 0;
  if (!(early_weights && warp == 0)) griddep_wait();
  if (p.groups != nullptr) {
    for (int i = threadIdx.x; i <= p.num_groups; i += kThreads) prefix[i] = p.groups[i].work_begin;
    __syncthreads();
  }

  const int total_work = p.groups != nullptr ? prefix[p.num_groups] : p.total_work;
  // bytes of K per row: two E2M1 values, one E4M3 value or half a BF16 value per byte
  const int k_bytes = kNvfp4 ? p.k / 2 : (KIND == GemmKind::bf16 ? 2 * p.k : p.k);
  const int total_kb = (k_bytes + 31) / 32;                 // MMA K-blocks (32 bytes of K each)
  const int k_stages = (total_kb + kKbPerStage - 1) / kKbPerStage;
  const int k_atoms = p.k / 64;                             // scale atoms per 128-row block (NVFP4)
  const bool split = p.split_partials != nullptr;

  // shared-memory descriptors: high words are constants, low word = address >> 4
  constexpr uint32_t kDescHiSw128 = uint32_t(1024 >> 4) | (1u << 14) | (2u << 29);   // SBO 1024 B, version 1, SWIZZLE_128B
  constexpr uint32_t kCOff16 = C::kLBytes >> 4;
  constexpr uint32_t kSflOff16 = (C::kLBytes + C::kCBytes) >> 4;
  constexpr uint32_t kSfcOff16 = (C::kLBytes + C::kCBytes + C::kSflBytes) >> 4;
  auto make_desc = [](uint32_t hi, uint32_t lo) { return (uint64_t(hi) << 32) | lo; };
  const uint32_t smem_base16 = ptx::smem_u32(smem) >> 4;
  const uint32_t sfl_tmem = tmem_base + C::kSflCol;
  const uint32_t sfc_tmem = tmem_base + C::kSfcCol;

  auto stage_l = [&](int s) { return smem + s * C::kStageBytes; };
  auto stage_c = [&](int s) { return smem + s * C::kStageBytes + C::kLBytes; };
  auto stage_sfl = [&](int s) { return smem + s * C::kStageBytes + C::kLBytes + C::kCBytes; };
  auto stage_sfc = [&](int s) { return smem + s * C::kStageBytes + C::kLBytes + C::kCBytes + C::kSflBytes; };

  // optional cycle counters (debug aid): [cta][8] = producer wait, mma wait for data, mma issue,
  // mma wait for accumulator, epilogue wait, epilogue work, role total, items
  long long prof_wait = 0, prof_work = 0, prof_wait2 = 0;
  const long long prof_start = prof ? clock64() : 0;
  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    // One thread runs the whole role (no per-stage warp votes or shuffles); the other lanes
    // wait at the end of the branch.
    if (lane == 0) {
    int stage = 0;
    uint32_t phase = 0;
    bool waited = !early_weights;        // this warp defers its wait for the previous kernel (see below)
    WorkItem item, next;
    SegmentWalk walk(int(blockIdx.x), int(gridDim.x), split, total_work, k_stages, p.work_chunk);
    int tile, ks0, ks1, next_tile, next_ks0, next_ks1;
    bool at_start, next_at_start;
    bool more = walk.next(next_tile, next_ks0, next_ks1, next_at_start);
    if (more) decode_work<BLOCK_N, EPI>(p, prefix, next_tile, next);
    while (more && !*abort_flag) {
      item = next; tile = next_tile; ks0 = next_ks0; ks1 = next_ks1; at_start = next_at_start;
      // the next item's descriptor is fetched while this one is processed
      more = walk.next(next_tile, next_ks0, next_ks1, next_at_start);
      if (more) decode_work<BLOCK_N, EPI>(p, prefix, next_tile, next);
      (void)tile; (void)at_start;
      const CUtensorMap* map_l = item.g.map_l >= 0 ? p.map_table + item.g.map_l : &p.map_l;
      const CUtensorMap* map_c[2];
#pragma unroll
      for (int h = 0; h < C::kHalves; ++h) map_c[h] = item.g.map_c[h] >= 0 ? p.map_table + item.g.map_c[h] : &p.map_c;
      // The descriptors in map_table were written by the host before any launch that uses
      // them (expert table creation), so ordinary launch ordering makes them visible to the
      // copy engine; no proxy fence is needed per use (one system-scope fence per work item
      // cost more than the item's copies).
      const int l_row = item.g.l_row0 + item.l_tile * kTileL;
      const int c_local = item.c_tile * p.c_rows_per_tile;   // row inside each matrix of the C operand
      const int halves = item.halves;
      // per-item source addresses; per stage they advance by a constant
      const uint8_t* sfl_src = nullptr;
      const uint8_t* sfc_src[2] = {nullptr, nullptr};
      int c_row[2] = {0, 0};
      if constexpr (kNvfp4) sfl_src = item.g.sf_l + size_t(item.l_tile) * k_atoms * kAtomBytes;
#pragma unroll
      for (int h = 0; h < C::kHalves; ++h) {
        c_row[h] = item.g.c_row0 + c_local + h * item.g.c_half_stride;
        if constexpr (kNvfp4)
          sfc_src[h] = item.g.sf_c[h] + size_t((c_local + h * item.g.c_half_stride) / 128) * k_atoms * kAtomBytes;
      }
      // dense direct form: both column halves are consecutive rows of one matrix, so one
      // 256-row box and one two-row box of scale atoms replace four copies (the copy
      // engine's cost per operation, not per byte, is what limits the fill rate)
      const bool single_box = C::kHalves == 2 && p.c_single_box != 0;
      const uint32_t c_bytes = single_box ? uint32_t(C::kCBytes) : uint32_t(kSlabs * halves * C::kHalfRows * kStageRowBytes);
      // one stage's copies; `weights` / `tokens` select the L-side and the C-side copies
      auto issue = [&](int ks, int st, bool l_side, bool c_side) {
        const int nkb = min(kKbPerStage, total_kb - ks * kKbPerStage);
        uint8_t* base = smem + st * C::kStageBytes;
        uint64_t* bar = full_bar + st;
        if (l_side) {                      // the stage's byte count is announced with its first copies
          uint32_t bytes = C::kLBytes + c_bytes;
          if constexpr (kNvfp4)
            bytes += nkb * kAtomBytes + (single_box ? uint32_t(C::kSfcBytes) : uint32_t(nkb * kAtomBytes * halves));
          ptx::mbar_expect_tx(bar, bytes);
          // a slab past the end of K is filled with zeros by the copy engine (and skipped by the MMAs)
#pragma unroll
          for (int slab = 0; slab < kSlabs; ++slab)
            ptx::tma_load_2d(base + slab * C::kLSlabBytes, map_l, (ks * kSlabs + slab) * kStageRowBytes, l_row, bar);
          if constexpr (kNvfp4)
            ptx::bulk_load(base + C::kLBytes + C::kCBytes, sfl_src + size_t(ks) * kKBlocksPerStage * kAtomBytes,
                           nkb * kAtomBytes, bar);
        }
        if (c_side) {
          if (single_box) {
            ptx::tma_load_2d(base + C::kLBytes, &p.map_c, ks * kStageRowBytes, c_row[0], bar);
          } else {
#pragma unroll
            for (int h = 0; h < C::kHalves; ++h)     // compile-time bound: map_c / c_row stay in registers
              if (h < halves) {
#pragma unroll
                for (int slab = 0; slab < kSlabs; ++slab)
                  ptx::tma_load_2d(base + C::kLBytes + slab * C::kCSlabBytes + h * C::kHalfRows * kStageRowBytes, map_c[h],
                                   (ks * kSlabs + slab) * kStageRowBytes, c_row[h], bar);
              }
          }
          if constexpr (kNvfp4) {
            const size_t atom_offset = size_t(ks) * kKBlocksPerStage * kAtomBytes;
            if (single_box) {
              // scale storage seen as [row blocks][K/64 atoms] of 8-byte words: 256 words = 4 atoms
              ptx::tma_load_2d(base + C::kLBytes + C::kCBytes + C::kSflBytes, &p.map_sfc, ks * 256, c_local / 128, bar);
            } else {
#pragma unroll
              for (int h = 0; h < C::kHalves; ++h)
                if (h < halves)
                  ptx::bulk_load(base + C::kLBytes + C::kCBytes + C::kSflBytes + h * kKBlocksPerStage * kAtomBytes,
                                 sfc_src[h] + atom_offset, nkb * kAtomBytes, bar);
            }
          }
        }
      };
      int ks_begin = ks0;
      if (early_weights && !waited) {
        // Decode shapes: the weights (L side) do not depend on the kernel that quantises the
        // activations, so the first ring of weight copies is issued before waiting for it;
        // the token-side copies of those stages follow once it has finished.
        const int ahead = min(C::kStages, ks1 - ks0);
        if (lane == 0)
          for (int i = 0; i < ahead; ++i) issue(ks0 + i, i, true, false);
        griddep_wait();
        waited = true;
        if (lane == 0)
          for (int i = 0; i < ahead; ++i) issue(ks0 + i, i, false, true);
        stage = ahead == C::kStages ? 0 : ahead;
        phase = ahead == C::kStages ? 1 : 0;
        ks_begin = ks0 + ahead;
      }
      for (int ks = ks_begin; ks < ks1; ++ks) {
        const long long t0 = prof ? clock64() : 0;
        if (!ptx::mbar_wait_bounded(empty_bar + stage, phase ^ 1)) {
          report(p.error, 0x10000000u | (blockIdx.x << 8) | stage, abort_flag);
          break;
        }
        if (prof) prof_wait += clock64() - t0;
        if (lane == 0) issue(ks, stage, true, true);
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
    }
    if (!waited) griddep_wait();
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (one thread, as above)
    if (lane == 0) {
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    WorkItem item, next;
    SegmentWalk walk(int(blockIdx.x), int(gridDim.x), split, total_work, k_stages, p.work_chunk);
    int tile, ks0, ks1, next_tile, next_ks0, next_ks1;
    bool at_start, next_at_start;
    bool more = walk.next(next_tile, next_ks0, next_ks1, next_at_start);
    if (more) decode_work<BLOCK_N, EPI>(p, prefix, next_tile, next);
    while (more && !*abort_flag) {
      item = next; tile = next_tile; ks0 = next_ks0; ks1 = next_ks1; at_start = next_at_start;
      more = walk.next(next_tile, next_ks0, next_ks1, next_at_start);
      if (more) decode_work<BLOCK_N, EPI>(p, prefix, next_tile, next);
      (void)tile; (void)at_start;
      const long long ta = prof ? clock64() : 0;
      if (!ptx::mbar_wait_bounded(acc_empty_bar + acc, acc_phase ^ 1)) {
        report(p.error, 0x20000000u | (blockIdx.x << 8) | acc, abort_flag);
        break;
      }
      if (prof) prof_wait2 += clock64() - ta;
      ptx::tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
      const uint32_t idesc = kNvfp4 ? ptx::idesc_nvfp4(item.mma_n)
                             : (KIND == GemmKind::bf16 ? ptx::idesc_bf16(item.mma_n) : ptx::idesc_fp8(item.mma_n));
      bool failed = false;
      for (int ks = ks0; ks < ks1; ++ks) {
        const long long t0 = prof ? clock64() : 0;
        if constexpr (kNvfp4) {
          // The stage's scales are in its TMEM slot once the four loader warps have arrived; they
          // arrive after the stage's copies have landed, so this wait covers the operands too.
          if (!ptx::mbar_wait_bounded(sf_ready_bar + stage, phase)) {
            report(p.error, 0x50000000u | (blockIdx.x << 8) | stage, abort_flag);
            failed = true;
            break;
          }
        } else {
          if (!ptx::mbar_wait_bounded(full_bar + stage, phase)) {
            report(p.error, 0x30000000u | (blockIdx.x << 8) | stage, abort_flag);
            failed = true;
            break;
          }
        }
        const long long t1 = prof ? clock64() : 0;
        if (prof) prof_wait += t1 - t0;
        ptx::tc_fence_after_sync();
        if (lane == 0) {
          // Single in-order instruction stream: descriptors are a constant plus
          // stage * (kStageBytes >> 4) in their low word, the loop is unrolled.
          const int nkb = min(kKbPerStage, total_kb - ks * kKbPerStage);
          const uint32_t base16 = smem_base16 + uint32_t(stage) * uint32_t(C::kStageBytes >> 4);
          const uint32_t sfl_t = sfl_tmem + uint32_t(stage) * C::kSfSlotCols;
          const uint32_t sfc_t = sfc_tmem + uint32_t(stage) * C::kSfSlotCols;
          const uint32_t first = ks == ks0 ? 0u : 1u;
#pragma unroll
          for (int kb = 0; kb < kKbPerStage; ++kb) {
            if (kb < nkb) {
              // operand addresses of K-block kb: its slab, then 32 bytes per K-block inside the slab's swizzle span
              const uint32_t l16 = base16 + uint32_t(kb / kKBlocksPerStage) * uint32_t(C::kLSlabBytes >> 4) +
                                   2 * uint32_t(kb % kKBlocksPerStage);
              const uint32_t c16 = base16 + kCOff16 + uint32_t(kb / kKBlocksPerStage) * uint32_t(C::kCSlabBytes >> 4) +
                                   2 * uint32_t(kb % kKBlocksPerStage);
              if constexpr (kNvfp4)
                ptx::tc_mma_nvfp4(d_tmem, make_desc(kDescHiSw128, l16), make_desc(kDescHiSw128, c16), idesc, sfl_t + 4 * kb,
                                  sfc_t + kb * C::kSfcColsPerKb, kb == 0 ? first : 1u);
              else if constexpr (KIND == GemmKind::bf16)
                ptx::tc_mma_bf16(d_tmem, make_desc(kDescHiSw128, l16), make_desc(kDescHiSw128, c16), idesc, kb == 0 ? first : 1u);
              else
                ptx::tc_mma_fp8(d_tmem, make_desc(kDescHiSw128, l16), make_desc(kDescHiSw128, c16), idesc, kb == 0 ? first : 1u);
            }
          }
          ptx::tc_commit(empty_bar + stage);
        }
        if (prof) prof_work += clock64() - t1;
        if (++stage == C::kStages) { stage = 0; phase ^= 1; }
      }
      if (failed) break;
      if (lane == 0) ptx::tc_commit(acc_full_bar + acc);
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
    }
    }
    __syncwarp();
  } else if (warp < kFirstEpilogueWarp) {
    // ------------------------------------------------------------------ scale loaders
    // TMEM layout the MMA expects for a K-block: lane (row % 32) of every lane quadrant,
    // 32-bit column (row / 32), byte (K16 block % 4) -- i.e. the 16 bytes of row (lane) of a
    // 512-byte atom are four consecutive columns, identical in all four quadrants.  Each of
    // the four warps writes its own quadrant: one 16-byte shared-memory load per atom and
    // lane, then tcgen05.st of 16 columns at a time.
    if constexpr (kNvfp4) {
      const uint32_t quad_lane = uint32_t((warp % 4) * 32) << 16;
      int stage = 0;
      uint32_t phase = 0;
      WorkItem item, next;
      SegmentWalk walk(int(blockIdx.x), int(gridDim.x), split, total_work, k_stages, p.work_chunk);
      int tile, ks0, ks1, next_tile, next_ks0, next_ks1;
      bool at_start, next_at_start;
      bool more = walk.next(next_tile, next_ks0, next_ks1, next_at_start);
      if (more) decode_work<BLOCK_N, EPI>(p, prefix, next_tile, next);
      while (more && !*abort_flag) {
        item = next; tile = next_tile; ks0 = next_ks0; ks1 = next_ks1; at_start = next_at_start;
        more = walk.next(next_tile, next_ks0, next_ks1, next_at_start);
        if (more) decode_work<BLOCK_N, EPI>(p, prefix, next_tile, next);
        (void)tile; (void)at_start;
        const int halves = item.halves;
        const uint32_t sfc_sub = BLOCK_N < 128 ? uint32_t((item.c_tile * p.c_rows_per_tile) % 128) / 32 : 0;
        bool failed = false;
        for (int ks = ks0; ks < ks1; ++ks) {
          // every lane polls the barrier itself: no vote or shuffle between the data's arrival
          // and the first shared-memory load (this latency is in front of every MMA)
          if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(full_bar + stage, phase))) {
            report(p.error, 0x60000000u | (blockIdx.x << 8) | stage, abort_flag);
            failed = true;
            break;
          }
          const uint32_t src = ptx::smem_u32(smem + stage * C::kStageBytes + C::kLBytes + C::kCBytes) + lane * 16;
          const uint32_t slot = tmem_base + C::kSflCol + uint32_t(stage) * C::kSfSlotCols + quad_lane;
          uint32_t r[16];
#pragma unroll
          for (int kb = 0; kb < kKBlocksPerStage; ++kb) {
            const uint4 v = ptx::lds128(src + kb * kAtomBytes);
            r[4 * kb] = v.x; r[4 * kb + 1] = v.y; r[4 * kb + 2] = v.z; r[4 * kb + 3] = v.w;
          }
          ptx::tmem_store16(slot, r);
          // column operand scales: per K-block [half 0: 4 columns][half 1: 4 columns]
          if constexpr (C::kHalves == 1) {
            // A column tile narrower than 128 rows may start part-way into its 128-row scale
            // atom (32-row steps).  The four words of a lane are the atom's four 32-row
            // groups: rotate them so that the tile's first group lands in the slot's first
            // column -- the MMA wants its scale address aligned to the whole four-column group.
#pragma unroll
            for (int kb = 0; kb < kKBlocksPerStage; ++kb) {
              const uint4 v = ptx::lds128(src + C::kSflBytes + kb * kAtomBytes);
              uint32_t a = v.x, b = v.y, c = v.z, d = v.w;
              if (sfc_sub & 1) { const uint32_t t = a; a = b; b = c; c = d; d = t; }
              if (sfc_sub & 2) { uint32_t t = a; a = c; c = t; t = b; b = d; d = t; }
              r[4 * kb] = a; r[4 * kb + 1] = b; r[4 * kb + 2] = c; r[4 * kb + 3] = d;
            }
            ptx::tmem_store16(slot + 4 * kKBlocksPerStage, r);
          } else {
#pragma unroll
            for (int pair = 0; pair < 2; ++pair) {      // two K-blocks (16 columns) per store
#pragma unroll
              for (int i = 0; i < 2; ++i) {
                const int kb = 2 * pair + i;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  uint4 v = make_uint4(0, 0, 0, 0);
                  if (h < halves) v = ptx::lds128(src + C::kSflBytes + (h * kKBlocksPerStage + kb) * kAtomBytes);
                  r[8 * i + 4 * h] = v.x; r[8 * i + 4 * h + 1] = v.y; r[8 * i + 4 * h + 2] = v.z; r[8 * i + 4 * h + 3] = v.w;
                }
              }
              ptx::tmem_store16(slot + 4 * kKBlocksPerStage + 16 * pair, r);
            }
          }
          ptx::tmem_store_wait();
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(sf_ready_bar + stage);
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp % 4;            // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    const int col_half = (warp - kFirstEpilogueWarp) / 4;  // which half of the accumulator columns this warp drains
    int acc = 0;
    uint32_t acc_phase = 0;
    WorkItem item, next;
    SegmentWalk walk(int(blockIdx.x), int(gridDim.x), split, total_work, k_stages, p.work_chunk);
    int tile, ks0, ks1, next_tile, next_ks0, next_ks1;
    bool at_start, next_at_start;
    bool more = walk.next(next_tile, next_ks0, next_ks1, next_at_start);
    if (more) decode_work<BLOCK_N, EPI>(p, prefix, next_tile, next);
    while (more && !*abort_flag) {
      item = next; tile = next_tile; ks0 = next_ks0; ks1 = next_ks1; at_start = next_at_start;
      more = walk.next(next_tile, next_ks0, next_ks1, next_at_start);
      if (more) decode_work<BLOCK_N, EPI>(p, prefix, next_tile, next);
      (void)tile; (void)at_start;
      const long long te0 = prof ? clock64() : 0;
      if (!ptx::mbar_wait_warp(acc_full_bar + acc, acc_phase)) {
        report(p.error, 0x40000000u | (blockIdx.x << 8) | acc, abort_flag);
        break;
      }
      const long long te1 = prof ? clock64() : 0;
      if (prof) prof_wait += te1 - te0;
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + acc * BLOCK_N + (uint32_t(quad * 32) << 16);
      const int l_index = item.l_tile * kTileL + quad * 32 + lane;   // row of L inside the group
      const bool l_ok = quad * 32 + lane < item.l_valid;

      if constexpr (EPI == GemmEpilogue::swap_store) {
        // lanes = output channels, columns = tokens: out[token][channel]
        bf16* out = static_cast<bf16*>(p.out);
        float alpha = item.g.alpha[0];
        if (item.g.channel_alpha != nullptr && l_ok) alpha = item.g.channel_alpha[l_index];
        bf16* dst = out + (size_t(item.g.out_row0) + size_t(item.c_tile) * BLOCK_N) * p.ld_out + item.g.out_col0 + l_index;
        const bool partial = ks1 - ks0 < k_stages;      // only in split mode
        if (!partial) {
          for (int c0 = col_half * 16; c0 < item.mma_n; c0 += 32) {
            uint32_t r[16];
            ptx::tmem_load16(taddr + c0, r);
            ptx::tmem_load_wait();
            if (l_ok) {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (c0 + i < item.c_valid) {
                  bf16* token_dst = dst + size_t(c0 + i) * p.ld_out;
                  if (p.row_dest != nullptr) {   // per-row destinations: the token's row may live on another GPU
                    const uint64_t home = p.row_dest[size_t(item.g.out_row0) + item.c_tile * BLOCK_N + c0 + i];
                    if (home == 0) continue;     // a row without a home (reported when the table was built)
                    token_dst = reinterpret_cast<bf16*>(home) + item.g.out_col0 + l_index;
                  }
                  *token_dst = __float2bfloat16_rn(__fmul_rn(__uint_as_float(r[i]), alpha));
                }
            }
          }
        } else {
          // This CTA covered only K stages [ks0, ks1) of the tile.  Its FP32 partial goes to
          // this CTA's slot ([column][lane], so a warp writes 128 contiguous bytes); the CTA
          // that arrives last at the tile's counter adds the slots in CTA order -- a fixed
          // order, so the result does not depend on which CTA that was -- and stores.
          const int row = quad * 32 + lane;
          float* mine = p.split_partials + (size_t(blockIdx.x) * 2 + (at_start ? 0 : 1)) * size_t(kTileL * BLOCK_N);
          for (int c0 = col_half * 16; c0 < item.mma_n; c0 += 32) {
            uint32_t r[16];
            ptx::tmem_load16(taddr + c0, r);
            ptx::tmem_load_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) __stcg(mine + (c0 + i) * kTileL + row, __uint_as_float(r[i]));
          }
          __threadfence();
          named_barrier_sync(1, kEpilogueWarps * 32);
          const long long tile_first_unit = (long long)tile * k_stages;
          const int cta_first = walk.cta_of(tile_first_unit);
          const int cta_last = walk.cta_of(tile_first_unit + k_stages - 1);
          if (threadIdx.x == kFirstEpilogueWarp * 32) {
            const int arrived = atomicAdd(p.split_counters + tile, 1);
            const int last = arrived == cta_last - cta_first;
            if (last) p.split_counters[tile] = 0;         // ready for the next launch
            *split_flag = last;
          }
          named_barrier_sync(1, kEpilogueWarps * 32);
          if (*split_flag) {
            __threadfence();
            for (int c0 = col_half * 16; c0 < item.mma_n; c0 += 32) {
              float sum[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) sum[i] = 0.0F;
              for (int cta = cta_first; cta <= cta_last; ++cta) {
                // the tile is the first segment of every CTA but (possibly) the first one
                const int which = (cta == cta_first && walk.range_begin(cta) < tile_first_unit) ? 1 : 0;
                const float* theirs = p.split_partials + (size_t(cta) * 2 + which) * size_t(kTileL * BLOCK_N);
#pragma unroll
                for (int i = 0; i < 16; ++i) sum[i] += __ldcg(theirs + (c0 + i) * kTileL + row);
              }
              if (l_ok) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                  if (c0 + i < item.c_valid)
                    dst[size_t(c0 + i) * p.ld_out] = __float2bfloat16_rn(__fmul_rn(sum[i], alpha));
              }
            }
          }
        }
      } else if constexpr (EPI == GemmEpilogue::direct_store) {
        // lanes = tokens, columns = output channels: out[token][channel].  A thread reads
        // 32 consecutive channels of its own row from TMEM; a 4x4 transpose of 16-byte
        // units inside every group of four lanes then lets four neighbouring lanes write
        // 64 contiguous bytes of one row (8 cache lines per store instruction, not 32).
        bf16* out = static_cast<bf16*>(p.out);
        const int c_base = item.c_tile * p.c_rows_per_tile;           // first channel of the tile
        const int c_end = item.g.c_rows;                              // valid channels of the matrix
        const int group_row = item.l_tile * kTileL + quad * 32 + (lane & ~3);   // first row of this lane group
        bf16* dst = out + (size_t(item.g.out_row0) + group_row) * p.ld_out + item.g.out_col0 + c_base + 8 * (lane & 3);
        const int rows_left = item.l_valid - (quad * 32 + (lane & ~3));          // valid rows from group_row on
        // optional per-row destinations (expert parallelism: a row goes straight to its home)
        uint64_t my_row_dest = 0;
        if (p.row_dest != nullptr && l_ok) my_row_dest = p.row_dest[size_t(item.g.out_row0) + l_index];
        uint64_t group_dest[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) group_dest[i] = __shfl_sync(0xffffffffu, my_row_dest, (lane & ~3) + i);
        const float alpha = item.g.alpha[0];
        const bool hi = (lane & 2) != 0, lo = (lane & 1) != 0;
        constexpr int kColsPerWarp = BLOCK_N / 2;
        constexpr int kChunks = kColsPerWarp / 32;
        // With a single accumulator stage (256 columns) the warp drains all of its columns
        // into registers as packed BF16 first and returns the accumulator before it stores,
        // so the stores overlap the next tile's MMAs; with two stages it goes chunk by chunk.
        constexpr bool kEarlyRelease = C::kAccStages == 1;
        uint4 unit[kEarlyRelease ? kChunks : 1][4];                  // unit q of a chunk = channels c0 + 8q .. + 7
        auto drain = [&](int c0, uint4* out_units) {
          uint32_t r[32];
          const long long td0 = prof ? clock64() : 0;
          ptx::tmem_load16(taddr + c0, r);
          ptx::tmem_load16(taddr + c0 + 16, r + 16);
          ptx::tmem_load_wait();
          if (prof) prof_wait2 += clock64() - td0;
          float v[32];
          if (item.g.channel_alpha != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int c = c_base + c0 + i;
              v[i] = __fmul_rn(__uint_as_float(r[i]), c < c_end ? item.g.channel_alpha[c] : 0.0F);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __fmul_rn(__uint_as_float(r[i]), alpha);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q)
            out_units[q] = make_uint4(pack_bf16x2(v[8 * q], v[8 * q + 1]), pack_bf16x2(v[8 * q + 2], v[8 * q + 3]),
                                      pack_bf16x2(v[8 * q + 4], v[8 * q + 5]), pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
        };
        auto store = [&](int c0, uint4* u) {
          // exchange bit 1 of (lane, unit), then bit 0: afterwards u[i] of lane 4j+k is
          // unit k of row 4j+i
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
          const int c = c_base + c0 + 8 * (lane & 3);                 // first channel of this lane's units
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            if (i >= rows_left) continue;
            if (p.row_dest != nullptr && group_dest[i] == 0) continue;   // a row without a home (reported earlier)
            bf16* row_dst = p.row_dest == nullptr
                                ? dst + size_t(i) * p.ld_out + c0
                                : reinterpret_cast<bf16*>(group_dest[i]) + item.g.out_col0 + c_base + 8 * (lane & 3) + c0;
            if (c + 8 <= c_end) {
              *reinterpret_cast<uint4*>(row_dst) = u[i];
            } else {
              const uint32_t words[4] = {u[i].x, u[i].y, u[i].z, u[i].w};
              for (int e = 0; e < 8; ++e)
                if (c + e < c_end)
                  reinterpret_cast<uint16_t*>(row_dst)[e] = uint16_t(words[e / 2] >> (16 * (e % 2)));
            }
          }
        };
        if constexpr (kEarlyRelease) {
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch) {
            const int c0 = col_half * kColsPerWarp + 32 * ch;
            if (c_base + c0 < c_end) drain(c0, unit[ch]);             // warp-uniform
          }
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive(acc_empty_bar + acc);      // the next tile's MMAs may start
#pragma unroll
          for (int ch = 0; ch < kChunks; ++ch) {
            const int c0 = col_half * kColsPerWarp + 32 * ch;
            if (c_base + c0 < c_end) store(c0, unit[ch]);
          }
        } else {
          for (int c0 = col_half * kColsPerWarp; c0 < (col_half + 1) * kColsPerWarp; c0 += 32) {
            if (c_base + c0 >= c_end) break;                          // warp-uniform
            drain(c0, unit[0]);
            store(c0, unit[0]);
          }
        }
      } else {
        // GeGLU + FP4 quantise: columns [0,128) = gate channels, [128,256) = up channels of
        // the same 128 output channels; this warp owns 64 of them (4 K16 blocks).
        //
        // The 256-column accumulator has no second stage (tensor memory is full), so the
        // warp first drains its share into registers -- scaled and rounded to BF16, which is
        // what GeGLU consumes anyway, two values per register -- and hands the accumulator
        // back to the MMA issuer at once; the transcendental math and the stores then
        // overlap the next tile's MMAs.
        const int channel0 = item.c_tile * 128 + col_half * 64;       // first channel of this warp
        const int width = p.out_width;
        const bool active = channel0 < width;
        uint32_t gate_words[32], up_words[32];                        // BF16 pairs: channels channel0 + 2i, + 2i + 1
        if (active) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t g[16], u[16];
            ptx::tmem_load16(taddr + col_half * 64 + 16 * j, g);
            ptx::tmem_load16(taddr + 128 + col_half * 64 + 16 * j, u);
            ptx::tmem_load_wait();
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              gate_words[8 * j + i] = pack_bf16x2(__fmul_rn(__uint_as_float(g[2 * i]), item.g.alpha[0]),
                                                  __fmul_rn(__uint_as_float(g[2 * i + 1]), item.g.alpha[0]));
              up_words[8 * j + i] = pack_bf16x2(__fmul_rn(__uint_as_float(u[2 * i]), item.g.alpha[1]),
                                                __fmul_rn(__uint_as_float(u[2 * i + 1]), item.g.alpha[1]));
            }
          }
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(acc_empty_bar + acc);        // the next tile's MMAs may start
        if (active) {
          const size_t row = size_t(item.g.out_row0) + l_index;
          uint32_t packed_words[8];
          uint32_t scale_word = 0;
          const float inverse_scale = item.g.quant_inverse_scale;
          bf16* cap_gu = static_cast<bf16*>(p.capture_gate_up);
          bf16* cap_act = static_cast<bf16*>(p.capture_activated);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float act[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const uint32_t gw = gate_words[8 * j + i], uw = up_words[8 * j + i];
              act[2 * i] = gelu_tanh_multiply_bf16(__uint_as_float(gw << 16), __uint_as_float(uw << 16));
              act[2 * i + 1] = gelu_tanh_multiply_bf16(__uint_as_float(gw & 0xFFFF0000u), __uint_as_float(uw & 0xFFFF0000u));
            }
            float amax = 0.0F;
#pragma unroll
            for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(act[i]));
            const uint8_t code = float_to_e4m3(inverse_scale * (amax * rcp_approx_ftz(6.0F)));
            const float block_scale = e4m3_to_float(code);
            const float factor =
                block_scale == 0.0F ? 0.0F : rcp_approx_ftz(block_scale * rcp_approx_ftz(inverse_scale));
            scale_word |= uint32_t(code) << (8 * j);
            uint32_t lo = 0, hi = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              lo |= uint32_t(float2_to_e2m1x2(act[2 * i] * factor, act[2 * i + 1] * factor)) << (8 * i);
              hi |= uint32_t(float2_to_e2m1x2(act[8 + 2 * i] * factor, act[8 + 2 * i + 1] * factor)) << (8 * i);
            }
            packed_words[2 * j] = lo;
            packed_words[2 * j + 1] = hi;
            if (cap_gu != nullptr && l_ok) {
              uint32_t aw[8];
#pragma unroll
              for (int i = 0; i < 8; ++i)
                aw[i] = (__float_as_uint(act[2 * i]) >> 16) | (__float_as_uint(act[2 * i + 1]) & 0xFFFF0000u);
              uint4* gdst = reinterpret_cast<uint4*>(cap_gu + row * (2 * size_t(width)) + channel0 + 16 * j);
              uint4* udst = reinterpret_cast<uint4*>(cap_gu + row * (2 * size_t(width)) + width + channel0 + 16 * j);
              uint4* adst = reinterpret_cast<uint4*>(cap_act + row * size_t(width) + channel0 + 16 * j);
              const uint32_t* gw = gate_words + 8 * j;
              const uint32_t* uw = up_words + 8 * j;
              gdst[0] = make_uint4(gw[0], gw[1], gw[2], gw[3]); gdst[1] = make_uint4(gw[4], gw[5], gw[6], gw[7]);
              udst[0] = make_uint4(uw[0], uw[1], uw[2], uw[3]); udst[1] = make_uint4(uw[4], uw[5], uw[6], uw[7]);
              adst[0] = make_uint4(aw[0], aw[1], aw[2], aw[3]); adst[1] = make_uint4(aw[4], aw[5], aw[6], aw[7]);
            }
          }
          if (l_ok) {
            uint8_t* packed_out = static_cast<uint8_t*>(p.out) + row * size_t(p.ld_out) + channel0 / 2;
            uint4* dst = reinterpret_cast<uint4*>(packed_out);
            dst[0] = make_uint4(packed_words[0], packed_words[1], packed_words[2], packed_words[3]);
            dst[1] = make_uint4(packed_words[4], packed_words[5], packed_words[6], packed_words[7]);
            const size_t region = size_t(item.g.sf_out_row0) * (width / 16);
            *reinterpret_cast<uint32_t*>(p.out_scales + region + scale_offset(l_index, channel0 / 16, width)) = scale_word;
          }
        }
      }
      if constexpr (EPI == GemmEpilogue::swap_store || (EPI == GemmEpilogue::direct_store && C::kAccStages > 1)) {
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(acc_empty_bar + acc);
      }
      if (prof) prof_work += clock64() - te1;
      if (++acc == C::kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  }
  if (prof && lane == 0 && (warp <= 1 || warp == kFirstEpilogueWarp)) {
    long long* row = p.profile + size_t(blockIdx.x) * 8;
    const long long total = clock64() - prof_start;
    if (warp == 0) { row[0] = prof_wait; }
    if (warp == 1) { row[1] = prof_wait; row[2] = prof_work; row[3] = prof_wait2; row[6] = total; }
    if (warp == kFirstEpilogueWarp) { row[4] = prof_wait; row[5] = prof_work; row[7] = prof_wait2; }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

long long* g_profile_buffer = nullptr;
unsigned g_profile_launches = 0;

template <GemmKind KIND, int BLOCK_N, GemmEpilogue EPI, bool kProfile>
cudaError_t launch_instance(const GemmParams& params, int grid, cudaStream_t stream) {
  using C = Config<KIND == GemmKind::nvfp4, BLOCK_N, slabs_per_stage(KIND, EPI)>;
  static bool configured_on[kMaxDeviceSlots] = {};   // the attribute is per GPU
  bool& configured = configured_on[current_device_slot()];
  if (!configured) {
    cudaError_t status = cudaFuncSetAttribute(gemm_tc_kernel<KIND, BLOCK_N, EPI, kProfile>,
                                              cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
    if (status != cudaSuccess) return status;
    configured = true;
  }
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(kThreads);
  config.dynamicSmemBytes = C::kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  note_launch();
  return cudaLaunchKernelEx(&config, gemm_tc_kernel<KIND, BLOCK_N, EPI, kProfile>, params);
}

template <GemmKind KIND, int BLOCK_N, GemmEpilogue EPI>
cudaError_t launch(const GemmParams& params_in, int grid, cudaStream_t stream) {
  GemmParams params = params_in;
  // debug aid: consecutive launches alternate between the two halves of the buffer, so the
  // two grouped GEMMs of one MoE pass can be told apart
  params.profile = g_profile_buffer ? g_profile_buffer + size_t(g_profile_launches++ % 2) * 148 * 8 : nullptr;
  if (params.profile != nullptr) return launch_instance<KIND, BLOCK_N, EPI, true>(params, grid, stream);
  return launch_instance<KIND, BLOCK_N, EPI, false>(params, grid, stream);
}

}  // namespace

void set_gemm_profile_buffer(long long* device_buffer) {
  g_profile_buffer = device_buffer;
  g_profile_launches = 0;
}

namespace {
template <GemmKind KIND>
cudaError_t launch_kind(GemmEpilogue epilogue, int block_n, const GemmParams& params, int grid, cudaStream_t stream) {
  if (epilogue == GemmEpilogue::swap_store) {
    switch (block_n) {
      case 32: return launch<KIND, 32, GemmEpilogue::swap_store>(params, grid, stream);
      case 64: return launch<KIND, 64, GemmEpilogue::swap_store>(params, grid, stream);
      case 128: return launch<KIND, 128, GemmEpilogue::swap_store>(params, grid, stream);
      default: return cudaErrorInvalidValue;
    }
  }
  if (epilogue == GemmEpilogue::direct_store) {
    switch (block_n) {
      case 128: return launch<KIND, 128, GemmEpilogue::direct_store>(params, grid, stream);
      case 256: return launch<KIND, 256, GemmEpilogue::direct_store>(params, grid, stream);
      default: return cudaErrorInvalidValue;
    }
  }
  if constexpr (KIND == GemmKind::nvfp4)
    if (block_n == 256) return launch<GemmKind::nvfp4, 256, GemmEpilogue::geglu_quant>(params, grid, stream);
  return cudaErrorInvalidValue;
}
}  // namespace

int gemm_tc_k_stages(GemmKind kind, GemmEpilogue epilogue, uint64_t row_bytes) {
  const uint64_t stage_row_bytes = uint64_t(kStageRowBytes) * uint64_t(slabs_per_stage(kind, epilogue));
  return int((row_bytes + stage_row_bytes - 1) / stage_row_bytes);
}

cudaError_t launch_gemm_tc(GemmKind kind, GemmEpilogue epilogue, int block_n, const GemmParams& params, int grid,
                           cudaStream_t stream) {
  switch (kind) {
    case GemmKind::nvfp4: return launch_kind<GemmKind::nvfp4>(epilogue, block_n, params, grid, stream);
    case GemmKind::fp8: return launch_kind<GemmKind::fp8>(epilogue, block_n, params, grid, stream);
    case GemmKind::bf16: return launch_kind<GemmKind::bf16>(epilogue, block_n, params, grid, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace gw
