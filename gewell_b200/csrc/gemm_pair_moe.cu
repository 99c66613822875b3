// The two grouped NVFP4 GEMMs of the MoE layer on CTA pairs (tcgen05
// cta_group::2) for sm_100a -- the large-batch path of MoeWorkspace::run
// (models/gemma4/26b_a4b/sm120/moe.cu:489-534; the reference runs CUTLASS
// grouped GEMMs there, moe_nvfp4.cuh:15-132).
//
// Why pairs: a single CTA with a 128-token x 256-channel tile has to bring
// 54 KB through L2 -> shared memory for every 633 cycles of MMA, more than an
// SM takes in; two CTAs that share the weight tile (each stages half of it,
// the pair's tensor cores read both halves) need 38 KB each.
//
// Roles per CTA, as in gemm_pair.cu: warp 0 = producer (one lane), warp 1 = MMA
// issuer (one lane, only in the pair's leader), warps 2..5 = scale loaders
// (shared memory -> registers -> tensor memory), warps 6..13 = epilogue.
//
// Work is found on the device: every CTA turns the expert offsets into a table
// of (first row, row count, first work unit) per expert; pair p takes units
// p, p + pairs, ...  A pair tile is 256 token rows of ONE expert: CTA r of the
// pair owns the expert's 128-row block 2 * tile + r (possibly past the expert's
// last row: such lanes compute on whatever follows and are masked in the
// epilogue).  Offsets beyond the declared capacity are clamped and reported.
//
// Every wait is bounded (2 s) and reports through the device error word; the
// kernels end with a cluster barrier before tensor memory is released.  No load
// fans out to other CTAs.
#include <string>

#include "common.cuh"
#include "gemm_pair_moe.h"
#include "pair.cuh"
#include "ptx.cuh"

namespace gw {
namespace {

using namespace pair;

constexpr int kExperts = 128;
constexpr int kHidden = 2816;
constexpr int kInter = 704;
constexpr int kScaleWarps = 4, kFirstEpilogueWarp = 2 + kScaleWarps;
constexpr uint32_t kDescHiSw128 = uint32_t(1024 >> 4) | (1u << 14) | (2u << 29);   // SBO 1024 B, version 1, SWIZZLE_128B

__device__ __forceinline__ uint64_t make_desc(uint32_t lo16) { return (uint64_t(kDescHiSw128) << 32) | lo16; }

// ---------------------------------------------------------------------------
// work table
// ---------------------------------------------------------------------------
struct WorkTable {
  int32_t first[kExperts];        // first sorted row of the expert (clamped to the capacity)
  int32_t count[kExperts];        // its rows
  int32_t prefix[kExperts + 1];   // first work unit of the expert; [128] = all units
};

struct Unit {
  int e, first, count;
  int tile;      // 256-row pair tile inside the expert
  int part;      // channel tile (gate/up) or channel chunk (down)
};

// All threads of the CTA.  units_per_tile work units for every 256-row pair tile of every expert.
__device__ __forceinline__ void build_work_table(const PairMoeParams& p, WorkTable* t, int units_per_tile) {
  __shared__ int32_t warp_totals[4];
  const int e = threadIdx.x;
  int32_t units = 0;
  if (e < kExperts) {
    int32_t first = p.offsets[e], last = p.offsets[e + 1];
    const int32_t capacity = int32_t(p.capacity);
    if (first < 0 || last < first || last > capacity) {
      if (p.error != nullptr) atomicCAS(p.error, 0u, 0x70000100u | uint32_t(e));
      first = min(max(first, 0), capacity);
      last = min(max(last, first), capacity);
    }
    t->first[e] = first;
    t->count[e] = last - first;
    units = ((last - first + 255) / 256) * units_per_tile;
  }
  // exclusive scan over the 128 experts: shuffles inside each of the first four warps, then their totals
  int32_t scan = units;
  const int lane = threadIdx.x % 32;
  if (e < kExperts) {
#pragma unroll
    for (int step = 1; step < 32; step *= 2) {
      const int32_t other = __shfl_up_sync(0xffffffffu, scan, step);
      if (lane >= step) scan += other;
    }
    if (lane == 31) warp_totals[e / 32] = scan;
  }
  __syncthreads();
  if (e < kExperts) {
    int32_t base = 0;
    for (int w = 0; w < e / 32; ++w) base += warp_totals[w];
    t->prefix[e] = base + scan - units;
    if (e == kExperts - 1) t->prefix[kExperts] = base + scan;
  }
  __syncthreads();
}

__device__ __forceinline__ void decode_unit(const WorkTable* t, int w, int units_per_tile, Unit& u) {
  if (u.e < 0 || w < t->prefix[u.e] || w >= t->prefix[u.e + 1]) {
    int lo = 0, hi = kExperts;             // largest e with prefix[e] <= w (it has units, since w < prefix[128])
    while (lo + 1 < hi) {
      const int mid = (lo + hi) / 2;
      if (t->prefix[mid] <= w) lo = mid; else hi = mid;
    }
    u.e = lo;
    u.first = t->first[lo];
    u.count = t->count[lo];
  }
  const int local = w - t->prefix[u.e];
  u.part = local % units_per_tile;
  u.tile = local / units_per_tile;
}

// ===========================================================================
// gate/up: Y = Xq . [Wgate | Wup]^T per expert, GeGLU, FP4 quantisation of the result
// ===========================================================================
namespace gu {
constexpr int kStages = 5;
constexpr int kKBlocks = 4;                       // MMAs (K = 64 each) per stage
constexpr int kKStages = kHidden / 2 / 128;       // 11 stages of 128 bytes of K
constexpr int kKAtoms = kHidden / 64;             // 44 scale atoms per 128-row block
constexpr int kCTiles = (kInter + 127) / 128;     // 6 channel tiles: 128 gate + 128 up columns each
constexpr int kTokBytes = 128 * 128;              // this CTA's 128 token rows x 128 bytes of K
constexpr int kWgtBytes = 128 * 128;              // this CTA's half of the column operand: gate (rank 0) or up (rank 1) rows
constexpr int kSfTokBytes = kKBlocks * 512;
constexpr int kSfWgtBytes = 2 * kKBlocks * 512;   // scale atoms of the gate rows, then of the up rows
constexpr int kStageBytes = kTokBytes + kWgtBytes + kSfTokBytes + kSfWgtBytes;   // 38912
constexpr int kAccCols = 256;
constexpr int kSfSlotCols = kKBlocks * (4 + 8);
constexpr int kTmemCols = 512;
static_assert(kAccCols + kStages * kSfSlotCols <= kTmemCols, "tensor memory over-subscribed");
constexpr int kBarriers = 4 * kStages + 2;
constexpr int kSmemBytes = kStages * kStageBytes + kBarriers * 8 + 16 + int(sizeof(WorkTable)) + 1024;
// GeGLU (tanhf) and the FP4 quantisation cost about as many issue slots per tile as the tile's MMAs
// take cycles; with two epilogue warps per scheduler their dependency chains set the pace of the
// whole kernel, so there are four per scheduler: sixteen warps, each with 32 channels of 32 rows.
constexpr int kEpilogueWarps = 16;
constexpr int kThreads = 32 * (2 + kScaleWarps + kEpilogueWarps);     // 704: at most 88 registers per thread
// A pair takes kChunk consecutive units (same token tile and expert, neighbouring channel tiles: the
// expert's descriptors stay hot and the token tile is re-read from L2) before it strides on.
constexpr int kChunk = 2;
__device__ __forceinline__ int first_unit(int pair_index) { return pair_index * kChunk; }
__device__ __forceinline__ int next_unit(int w, int pairs) {
  return (w + 1) % kChunk != 0 ? w + 1 : w + 1 + (pairs - 1) * kChunk;
}
}  // namespace gu

template <bool kProfile>   // cycle counters of the tuning aid live in an instantiation of their own
__global__ void __launch_bounds__(gu::kThreads, 1)
pair_moe_gate_up_kernel(const __grid_constant__ PairMoeParams p) {
  using namespace gu;
  constexpr bool prof = kProfile;
  const long long prof_start = prof ? clock64() : 0;
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
  WorkTable* table = reinterpret_cast<WorkTable*>(tmem_slot + 4);

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
  griddep_wait();                                   // the offsets and the quantised rows come from earlier kernels
  build_work_table(p, table, kCTiles);

  const int total = table->prefix[kExperts];
  const int pairs = gridDim.x / 2, pair_index = blockIdx.x / 2;
  const uint32_t smem_base16 = ptx::smem_u32(smem) >> 4;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (one lane)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      Unit u{-1, 0, 0, 0, 0};
      const uint8_t* sf_gate = nullptr;
      const uint8_t* sf_up = nullptr;
      int info_of = -1;
      long long prof_wait = 0;
      for (int w = first_unit(pair_index); w < total && !*abort_flag; w = next_unit(w, pairs)) {
        decode_unit(table, w, kCTiles, u);
        if (info_of != u.e) {
          sf_gate = p.experts[u.e].scales[0];
          sf_up = p.experts[u.e].scales[1];
          info_of = u.e;
        }
        const int block = 2 * u.tile + int(rank);                 // this CTA's 128-row block of the expert
        const bool have_rows = block * 128 < u.count;
        const int token_row = u.first + block * 128;
        {
          // the weight descriptor of the unit after this one is fetched while this one streams
          const int next = next_unit(w, pairs);
          if (next < total) {
            Unit v = u;
            decode_unit(table, next, kCTiles, v);
            if (v.e != u.e) ptx::prefetch_tensormap(p.map_table + v.e * kMoeMapsPerExpert + int(rank));
          }
        }
        const uint8_t* sf_tokens = p.sf_tokens + (size_t(u.first / 128 + u.e) + block) * size_t(kKAtoms) * 512;
        const CUtensorMap* map_weights = p.map_table + u.e * kMoeMapsPerExpert + int(rank);   // gate or up
        const int weight_row = u.part * 128;
        const uint8_t* sfw0 = sf_gate + size_t(u.part) * kKAtoms * 512;
        const uint8_t* sfw1 = sf_up + size_t(u.part) * kKAtoms * 512;
        bool failed = false;
        for (int ks = 0; ks < kKStages; ++ks) {
          const long long t0 = prof ? clock64() : 0;
          if (!ptx::mbar_wait_bounded(empty_bar + stage, phase ^ 1)) {
            report(p.error, 0x12000000u | (blockIdx.x << 8) | stage, abort_flag);
            failed = true;
            break;
          }
          if (prof) prof_wait += clock64() - t0;
          uint8_t* base = smem + stage * kStageBytes;
          // the scales go first and complete on their own barrier: the loader warps move them into tensor
          // memory while the operand tiles are still in flight
          uint64_t* sf_bar = sf_full_bar + stage;
          uint64_t* bar = full_bar + stage;
          if (have_rows) {
            ptx::mbar_expect_tx(sf_bar, kSfTokBytes + kSfWgtBytes);
            ptx::bulk_load(base + kTokBytes + kWgtBytes, sf_tokens + size_t(ks) * kSfTokBytes, kSfTokBytes, sf_bar);
          } else {
            // This CTA's block lies past the expert's last row: its lanes are masked in the epilogue, so
            // whatever the stage still holds serves as their operand and scales; only the shared column
            // operand is fetched.
            ptx::mbar_expect_tx(sf_bar, kSfWgtBytes);
          }
          ptx::bulk_load(base + kTokBytes + kWgtBytes + kSfTokBytes, sfw0 + size_t(ks) * kSfTokBytes, kSfTokBytes, sf_bar);
          ptx::bulk_load(base + kTokBytes + kWgtBytes + 2 * kSfTokBytes, sfw1 + size_t(ks) * kSfTokBytes, kSfTokBytes,
                         sf_bar);
          ptx::mbar_expect_tx(bar, (have_rows ? kTokBytes : 0) + kWgtBytes);
          if (have_rows) ptx::tma_load_2d(base, &p.map_tokens, ks * 128, token_row, bar);
          ptx::tma_load_2d(base + kTokBytes, map_weights, ks * 128, weight_row, bar);
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
      long long prof_ready = 0, prof_issue = 0, prof_acc = 0;
      for (int w = first_unit(pair_index); w < total && !*abort_flag; w = next_unit(w, pairs)) {
        const long long ta = prof ? clock64() : 0;
        if (!ptx::mbar_wait_bounded(acc_empty_bar, acc_phase ^ 1)) {
          report(p.error, 0x22000000u | (blockIdx.x << 8), abort_flag);
          break;
        }
        if (prof) prof_acc += clock64() - ta;
        ptx::tc_fence_after_sync();
        bool failed = false;
        for (int ks = 0; ks < kKStages; ++ks) {
          // sf_ready implies that both CTAs' operands have landed (the loader warps arrive after their
          // CTA's operand barrier), so this is the only wait of the stage
          const long long t0 = prof ? clock64() : 0;
          if (!ptx::mbar_wait_bounded(sf_ready_bar + stage, phase)) {
            report(p.error, 0x32000000u | (blockIdx.x << 8) | stage, abort_flag);
            failed = true;
            break;
          }
          const long long t1 = prof ? clock64() : 0;
          if (prof) prof_ready += t1 - t0;
          ptx::tc_fence_after_sync();
          const uint32_t base16 = smem_base16 + uint32_t(stage) * uint32_t(kStageBytes >> 4);
          const uint32_t sf_tok = tmem_base + kAccCols + uint32_t(stage) * kSfSlotCols;
          const uint32_t sf_wgt = sf_tok + 4 * kKBlocks;
#pragma unroll
          for (int kb = 0; kb < kKBlocks; ++kb)
            mma_pair_nvfp4(tmem_base, make_desc(base16 + 2 * kb), make_desc(base16 + (kTokBytes >> 4) + 2 * kb), idesc,
                           sf_tok + 4 * kb, sf_wgt + 8 * kb, (ks | kb) != 0 ? 1u : 0u);
          commit_pair(empty_bar + stage);
          if (prof) prof_issue += clock64() - t1;
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (failed) break;
        commit_pair(acc_full_bar);
        acc_phase ^= 1;
      }
      if (prof) {
        long long* row = p.profile + size_t(blockIdx.x) * 8;
        row[1] = prof_ready; row[2] = prof_issue; row[3] = prof_acc; row[6] = clock64() - prof_start;
      }
    }
    __syncwarp();
  } else if (warp < kFirstEpilogueWarp) {
    // ------------------------------------------------------------------ scale loaders
    const uint32_t quad_lane = uint32_t((warp % 4) * 32) << 16;
    const uint32_t leader_sf_ready = leader_address(sf_ready_bar);
    int stage = 0;
    uint32_t phase = 0;
    for (int w = first_unit(pair_index); w < total && !*abort_flag; w = next_unit(w, pairs)) {
      bool failed = false;
      for (int ks = 0; ks < kKStages; ++ks) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(sf_full_bar + stage, phase))) {
          report(p.error, 0x63000000u | (blockIdx.x << 8) | stage, abort_flag);
          failed = true;
          break;
        }
        const uint32_t src = ptx::smem_u32(smem + stage * kStageBytes + kTokBytes + kWgtBytes) + lane * 16;
        const uint32_t slot = tmem_base + kAccCols + uint32_t(stage) * kSfSlotCols + quad_lane;
        uint32_t r[16];
#pragma unroll
        for (int kb = 0; kb < kKBlocks; ++kb) {
          const uint4 v = ptx::lds128(src + kb * 512);
          r[4 * kb] = v.x; r[4 * kb + 1] = v.y; r[4 * kb + 2] = v.z; r[4 * kb + 3] = v.w;
        }
        ptx::tmem_store16(slot, r);
        // column-operand scales: per K block [gate rows: 4 columns][up rows: 4 columns]
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
        ptx::tc_fence_before_sync();
        // the arrival also vouches for this CTA's operand tiles
        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(full_bar + stage, phase))) {
          report(p.error, 0x64000000u | (blockIdx.x << 8) | stage, abort_flag);
          failed = true;
          break;
        }
        if (lane == 0) arrive_cluster(leader_sf_ready + stage * 8);
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (failed) break;
    }
  } else {
    // ------------------------------------------------------------------ epilogue: GeGLU + FP4 quantise
    // Columns [0,128) of the accumulator are the gate channels of this tile, [128,256) the up channels
    // of the same 128 output channels; this warp owns 32 of them (two K16 blocks of the down input) for
    // the 32 token rows of its lane quadrant.  The accumulator has no second stage (tensor memory is
    // full), so the warp first drains its share into registers -- scaled and rounded to BF16, which is
    // what GeGLU consumes anyway, two values per register -- and hands the accumulator back at once;
    // the transcendental math and the stores then overlap the next tile's MMAs.
    const int quad = warp % 4;
    const int quarter = (warp - kFirstEpilogueWarp) / 4;
    const uint32_t leader_acc_empty = leader_address(acc_empty_bar);
    uint32_t acc_phase = 0;
    Unit u{-1, 0, 0, 0, 0};
    float alpha_gate = 0.0F, alpha_up = 0.0F, inverse_scale = 0.0F;
    int info_of = -1;
    long long prof_wait = 0, prof_work = 0;
    bf16* cap_gu = static_cast<bf16*>(p.capture_gate_up);
    bf16* cap_act = static_cast<bf16*>(p.capture_activated);
    for (int w = first_unit(pair_index); w < total && !*abort_flag; w = next_unit(w, pairs)) {
      decode_unit(table, w, kCTiles, u);
      if (info_of != u.e) {
        alpha_gate = p.experts[u.e].alpha[0];
        alpha_up = p.experts[u.e].alpha[1];
        inverse_scale = p.experts[u.e].inverse_input_scale[2];
        info_of = u.e;
      }
      const long long t0 = prof ? clock64() : 0;
      if (!ptx::mbar_wait_warp(acc_full_bar, acc_phase)) {
        report(p.error, 0x42000000u | (blockIdx.x << 8), abort_flag);
        break;
      }
      const long long t1 = prof ? clock64() : 0;
      if (prof) prof_wait += t1 - t0;
      acc_phase ^= 1;
      ptx::tc_fence_after_sync();
      const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16);
      const int l_index = (2 * u.tile + int(rank)) * 128 + quad * 32 + lane;     // row inside the expert's group
      const bool l_ok = l_index < u.count;
      const int channel0 = u.part * 128 + quarter * 32;                           // first channel of this warp
      const bool active = channel0 < kInter;                                      // warp uniform
      uint32_t gate_words[16], up_words[16];                                      // BF16 pairs
      if (active) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint32_t g[16], v[16];
          ptx::tmem_load16(taddr + quarter * 32 + 16 * j, g);
          ptx::tmem_load16(taddr + 128 + quarter * 32 + 16 * j, v);
          ptx::tmem_load_wait();
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            gate_words[8 * j + i] = pack_bf16x2(__fmul_rn(__uint_as_float(g[2 * i]), alpha_gate),
                                                __fmul_rn(__uint_as_float(g[2 * i + 1]), alpha_gate));
            up_words[8 * j + i] = pack_bf16x2(__fmul_rn(__uint_as_float(v[2 * i]), alpha_up),
                                              __fmul_rn(__uint_as_float(v[2 * i + 1]), alpha_up));
          }
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) arrive_cluster(leader_acc_empty);               // the next tile's MMAs may start
      if (active) {
        const size_t row = size_t(u.first) + l_index;
        uint32_t packed_words[4];
        uint32_t scale_pair = 0;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
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
          const float factor = block_scale == 0.0F ? 0.0F : rcp_approx_ftz(block_scale * rcp_approx_ftz(inverse_scale));
          scale_pair |= uint32_t(code) << (8 * j);
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
            uint4* gdst = reinterpret_cast<uint4*>(cap_gu + row * (2 * size_t(kInter)) + channel0 + 16 * j);
            uint4* udst = reinterpret_cast<uint4*>(cap_gu + row * (2 * size_t(kInter)) + kInter + channel0 + 16 * j);
            uint4* adst = reinterpret_cast<uint4*>(cap_act + row * size_t(kInter) + channel0 + 16 * j);
            const uint32_t* gw = gate_words + 8 * j;
            const uint32_t* uw = up_words + 8 * j;
            gdst[0] = make_uint4(gw[0], gw[1], gw[2], gw[3]); gdst[1] = make_uint4(gw[4], gw[5], gw[6], gw[7]);
            udst[0] = make_uint4(uw[0], uw[1], uw[2], uw[3]); udst[1] = make_uint4(uw[4], uw[5], uw[6], uw[7]);
            adst[0] = make_uint4(aw[0], aw[1], aw[2], aw[3]); adst[1] = make_uint4(aw[4], aw[5], aw[6], aw[7]);
          }
        }
        if (l_ok && p.records_out != nullptr) {
          uint8_t* record = p.records_out + row * size_t(kEpActivationRecordBytes);
          *reinterpret_cast<uint4*>(record + channel0 / 2) =
              make_uint4(packed_words[0], packed_words[1], packed_words[2], packed_words[3]);
          *reinterpret_cast<uint16_t*>(record + kInter / 2 + channel0 / 16) = uint16_t(scale_pair);
        } else if (l_ok) {
          *reinterpret_cast<uint4*>(p.packed_out + row * size_t(kInter / 2) + channel0 / 2) =
              make_uint4(packed_words[0], packed_words[1], packed_words[2], packed_words[3]);
          const size_t region = size_t(u.first / 128 + u.e) * 128 * (kInter / 16);
          // two neighbouring K16 blocks (an even and the following odd one): two adjacent bytes of the tile
          *reinterpret_cast<uint16_t*>(p.scales_out + region + scale_offset(l_index, channel0 / 16, kInter)) =
              uint16_t(scale_pair);
        }
      }
      if (prof) prof_work += clock64() - t1;
    }
    if (prof && lane == 0 && warp == kFirstEpilogueWarp) {
      long long* row = p.profile + size_t(blockIdx.x) * 8;
      row[4] = prof_wait;
      row[5] = prof_work;
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

// ===========================================================================
// down: Y = Aq . Wdown^T per expert, BF16 rows out
// ===========================================================================
// K = 704 is 2.75 stages of 128 bytes: too short for a stage ring per operand (the per-tile work would
// not be amortised) and short enough to keep whole.  A pair tile's quantised activations (128 rows x
// 352 bytes per CTA, three 128-byte slabs, the last one zero-filled past byte 352) stay resident in
// shared memory -- two buffers, so the next unit's rows arrive while this one computes -- and the
// pair sweeps the output channels in 128-channel tiles: each CTA stages 64 of the tile's weight rows
// (whole K, three slabs) per ring stage, 30 KB per 870 cycles of MMA.  Two 128-column accumulator
// stages: the epilogue of one tile overlaps the MMAs of the next.
namespace dn {
constexpr int kSlabs = 3;
constexpr int kKBlocks = kInter / 64;             // 11 MMAs (K = 64) per tile
constexpr int kSfBytes = kKBlocks * 512;          // 5632: the 11 scale atoms of a 128-row block
constexpr int kSfRoom = 12 * 512;                 // copied to tensor memory 16 columns (4 atoms) at a time
constexpr int kASlabBytes = 128 * 128;
constexpr int kABufBytes = kSlabs * kASlabBytes + kSfRoom;     // 55296
constexpr int kBSlabBytes = 64 * 128;
constexpr int kBStageBytes = kSlabs * kBSlabBytes + kSfRoom;   // 30720
constexpr int kBStages = 3;
constexpr int kTileCols = 128;                    // channels per tile (64 weight rows staged by each CTA)
constexpr int kCTiles = kHidden / kTileCols;      // 22
constexpr int kChunks = 2;                        // work units per pair tile
constexpr int kTilesPerUnit = kCTiles / kChunks;  // 11
static_assert(kTilesPerUnit * kChunks == kCTiles, "channel tiles divide evenly over the chunks");
constexpr int kAhead = 3;                         // the next unit's rows are requested after this many tiles of the current one
constexpr int kAccCols = 2 * kTileCols;           // two accumulator stages
constexpr int kSfSlotCols = 48;                   // 12 atoms x 4 columns
constexpr int kSfACol = kAccCols;                 // + buffer * kSfSlotCols
constexpr int kSfBCol = kSfACol + 2 * kSfSlotCols;   // + stage * kSfSlotCols
constexpr int kTmemCols = 512;
static_assert(kSfBCol + kBStages * kSfSlotCols <= kTmemCols, "tensor memory over-subscribed");
constexpr int kBarriers = 3 * 2 + 4 * kBStages + 2 * 2;
constexpr int kSmemBytes = 2 * kABufBytes + kBStages * kBStageBytes + kBarriers * 8 + 16 + int(sizeof(WorkTable)) + 1024;
static_assert(kSmemBytes <= 227 * 1024, "shared memory over-subscribed");
// The epilogue of a tile (drain, scale, transpose, store 32 KB) has to fit into the ~900 cycles of the
// next tile's MMAs; with two warps per scheduler it took ~1500.  Sixteen warps, 32 channels of 32 rows each.
constexpr int kEpilogueWarps = 16;
constexpr int kThreads = 32 * (2 + kScaleWarps + kEpilogueWarps);
}  // namespace dn

template <bool kProfile>
__global__ void __launch_bounds__(dn::kThreads, 1)
pair_moe_down_kernel(const __grid_constant__ PairMoeParams p) {
  using namespace dn;
  constexpr bool prof = kProfile;
  const long long prof_start = prof ? clock64() : 0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* a_buf = smem;                                       // [2][kABufBytes]
  uint8_t* b_ring = smem + 2 * kABufBytes;                     // [kBStages][kBStageBytes]
  uint64_t* a_full_bar = reinterpret_cast<uint64_t*>(b_ring + kBStages * kBStageBytes);
  uint64_t* a_empty_bar = a_full_bar + 2;
  uint64_t* a_ready_bar = a_empty_bar + 2;                     // leader: both CTAs' rows landed, their scales in tensor memory
  uint64_t* b_sf_full_bar = a_ready_bar + 2;
  uint64_t* b_full_bar = b_sf_full_bar + kBStages;
  uint64_t* b_empty_bar = b_full_bar + kBStages;
  uint64_t* b_ready_bar = b_empty_bar + kBStages;              // leader
  uint64_t* acc_full_bar = b_ready_bar + kBStages;
  uint64_t* acc_empty_bar = acc_full_bar + 2;                  // leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  WorkTable* table = reinterpret_cast<WorkTable*>(tmem_slot + 4);

  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const uint32_t rank = cluster_rank();
  griddep_launch();
  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(a_full_bar + b, 1);
      ptx::mbar_init(a_empty_bar + b, 1);
      ptx::mbar_init(a_ready_bar + b, 2 * kScaleWarps);
      ptx::mbar_init(acc_full_bar + b, 1);
      ptx::mbar_init(acc_empty_bar + b, 2 * kEpilogueWarps);
    }
    for (int s = 0; s < kBStages; ++s) {
      ptx::mbar_init(b_sf_full_bar + s, 1);
      ptx::mbar_init(b_full_bar + s, 1);
      ptx::mbar_init(b_empty_bar + s, 1);
      ptx::mbar_init(b_ready_bar + s, 2 * kScaleWarps);
    }
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
  cluster_sync_all();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  griddep_wait();
  build_work_table(p, table, kChunks);

  const int total = table->prefix[kExperts];
  const int pairs = gridDim.x / 2, pair_index = blockIdx.x / 2;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (one lane)
    if (lane == 0) {
      // request the rows (and their scale atoms) of the unit with running number `number`
      auto request_rows = [&](int w, int number) -> bool {
        Unit v{-1, 0, 0, 0, 0};
        decode_unit(table, w, kChunks, v);
        const int buffer = number & 1;
        if (!ptx::mbar_wait_bounded(a_empty_bar + buffer, (uint32_t(number >> 1) & 1u) ^ 1u)) {
          report(p.error, 0x13000000u | (blockIdx.x << 8) | buffer, abort_flag);
          return false;
        }
        const int block = 2 * v.tile + int(rank);
        const int token_row = v.first + block * 128;
        uint8_t* base = a_buf + buffer * kABufBytes;
        uint64_t* bar = a_full_bar + buffer;
        ptx::mbar_expect_tx(bar, kSlabs * kASlabBytes + kSfBytes);
        ptx::bulk_load(base + kSlabs * kASlabBytes,
                       p.sf_tokens + (size_t(v.first / 128 + v.e) + block) * size_t(kSfBytes), kSfBytes, bar);
#pragma unroll
        for (int j = 0; j < kSlabs; ++j) ptx::tma_load_2d(base + j * kASlabBytes, &p.map_tokens, j * 128, token_row, bar);
        return true;
      };
      int stage = 0, number = 0;
      uint32_t phase = 0;
      Unit u{-1, 0, 0, 0, 0};
      const uint8_t* sf_weights = nullptr;
      int info_of = -1;
      long long prof_wait = 0;
      bool failed = pair_index < total ? !request_rows(pair_index, 0) : false;
      for (int w = pair_index; w < total && !failed && !*abort_flag; w += pairs, ++number) {
        decode_unit(table, w, kChunks, u);
        if (info_of != u.e) {
          sf_weights = p.experts[u.e].scales[2];
          info_of = u.e;
        }
        const CUtensorMap* map_weights = p.map_table + u.e * kMoeMapsPerExpert + 3;   // down weights, 64-row boxes
        for (int t = 0; t < kTilesPerUnit; ++t) {
          const int c_tile = u.part * kTilesPerUnit + t;
          const long long t0 = prof ? clock64() : 0;
          if (!ptx::mbar_wait_bounded(b_empty_bar + stage, phase ^ 1)) {
            report(p.error, 0x14000000u | (blockIdx.x << 8) | stage, abort_flag);
            failed = true;
            break;
          }
          if (prof) prof_wait += clock64() - t0;
          uint8_t* base = b_ring + stage * kBStageBytes;
          uint64_t* sf_bar = b_sf_full_bar + stage;
          ptx::mbar_expect_tx(sf_bar, kSfBytes);
          ptx::bulk_load(base + kSlabs * kBSlabBytes, sf_weights + size_t(c_tile) * kSfBytes, kSfBytes, sf_bar);
          uint64_t* bar = b_full_bar + stage;
          ptx::mbar_expect_tx(bar, kSlabs * kBSlabBytes);
#pragma unroll
          for (int j = 0; j < kSlabs; ++j)
            ptx::tma_load_2d(base + j * kBSlabBytes, map_weights, j * 128, c_tile * kTileCols + int(rank) * 64, bar);
          if (++stage == kBStages) { stage = 0; phase ^= 1; }
          // By now the MMAs of the unit before this one are done (this stage was last used by this unit
          // or freed after it), so the other row buffer is free or about to be: ask for the next unit's rows.
          if (t == kAhead - 1 && w + pairs < total && !request_rows(w + pairs, number + 1)) {
            failed = true;
            break;
          }
        }
      }
      if (prof) p.profile[size_t(blockIdx.x) * 8 + 0] = prof_wait;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA, one lane)
    if (lane == 0 && rank == 0) {
      int stage = 0, number = 0, tiles = 0;
      uint32_t phase = 0;
      const uint32_t idesc = idesc_pair_nvfp4(kTileCols);
      const uint32_t a_base16 = ptx::smem_u32(a_buf) >> 4, b_base16 = ptx::smem_u32(b_ring) >> 4;
      bool failed = false;
      long long prof_rows = 0, prof_ready = 0, prof_issue = 0, prof_acc = 0;
      for (int w = pair_index; w < total && !failed && !*abort_flag; w += pairs, ++number) {
        const int buffer = number & 1;
        const long long tr = prof ? clock64() : 0;
        if (!ptx::mbar_wait_bounded(a_ready_bar + buffer, uint32_t(number >> 1) & 1u)) {
          report(p.error, 0x23000000u | (blockIdx.x << 8) | buffer, abort_flag);
          break;
        }
        if (prof) prof_rows += clock64() - tr;
        const uint32_t a16 = a_base16 + uint32_t(buffer) * uint32_t(kABufBytes >> 4);
        const uint32_t sfa = tmem_base + kSfACol + uint32_t(buffer) * kSfSlotCols;
        for (int t = 0; t < kTilesPerUnit; ++t, ++tiles) {
          const int acc = tiles & 1;
          const long long ta = prof ? clock64() : 0;
          if (!ptx::mbar_wait_bounded(acc_empty_bar + acc, (uint32_t(tiles >> 1) & 1u) ^ 1u)) {
            report(p.error, 0x24000000u | (blockIdx.x << 8) | acc, abort_flag);
            failed = true;
            break;
          }
          const long long tb = prof ? clock64() : 0;
          if (!ptx::mbar_wait_bounded(b_ready_bar + stage, phase)) {
            report(p.error, 0x33000000u | (blockIdx.x << 8) | stage, abort_flag);
            failed = true;
            break;
          }
          const long long tc = prof ? clock64() : 0;
          if (prof) { prof_acc += tb - ta; prof_ready += tc - tb; }
          ptx::tc_fence_after_sync();
          const uint32_t b16 = b_base16 + uint32_t(stage) * uint32_t(kBStageBytes >> 4);
          const uint32_t sfb = tmem_base + kSfBCol + uint32_t(stage) * kSfSlotCols;
          const uint32_t d = tmem_base + uint32_t(acc) * kTileCols;
#pragma unroll
          for (int kb = 0; kb < kKBlocks; ++kb)
            mma_pair_nvfp4(d, make_desc(a16 + uint32_t(kb / 4) * (kASlabBytes >> 4) + 2 * (kb % 4)),
                           make_desc(b16 + uint32_t(kb / 4) * (kBSlabBytes >> 4) + 2 * (kb % 4)), idesc, sfa + 4 * kb,
                           sfb + 4 * kb, kb != 0 ? 1u : 0u);
          commit_pair(b_empty_bar + stage);
          commit_pair(acc_full_bar + acc);
          if (prof) prof_issue += clock64() - tc;
          if (++stage == kBStages) { stage = 0; phase ^= 1; }
        }
        commit_pair(a_empty_bar + buffer);
      }
      if (prof) {
        long long* row = p.profile + size_t(blockIdx.x) * 8;
        row[1] = prof_ready; row[2] = prof_issue; row[3] = prof_acc; row[6] = clock64() - prof_start; row[7] = prof_rows;
      }
    }
    __syncwarp();
  } else if (warp < kFirstEpilogueWarp) {
    // ------------------------------------------------------------------ scale loaders
    const uint32_t quad_lane = uint32_t((warp % 4) * 32) << 16;
    const uint32_t leader_a_ready = leader_address(a_ready_bar);
    const uint32_t leader_b_ready = leader_address(b_ready_bar);
    // 12 atoms of 512 bytes (the twelfth is never read by an MMA) -> 48 tensor-memory columns
    auto copy_scales = [&](const uint8_t* atoms, uint32_t column) {
      const uint32_t src = ptx::smem_u32(atoms) + lane * 16;
#pragma unroll
      for (int g = 0; g < 3; ++g) {
        uint32_t r[16];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const uint4 v = ptx::lds128(src + (4 * g + a) * 512);
          r[4 * a] = v.x; r[4 * a + 1] = v.y; r[4 * a + 2] = v.z; r[4 * a + 3] = v.w;
        }
        ptx::tmem_store16(tmem_base + column + 16 * g + quad_lane, r);
      }
      ptx::tmem_store_wait();
      ptx::tc_fence_before_sync();
    };
    int stage = 0, number = 0;
    uint32_t phase = 0;
    bool failed = false;
    for (int w = pair_index; w < total && !failed && !*abort_flag; w += pairs, ++number) {
      const int buffer = number & 1;
      // one barrier covers the unit's rows and their scale atoms
      if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(a_full_bar + buffer, uint32_t(number >> 1) & 1u))) {
        report(p.error, 0x65000000u | (blockIdx.x << 8) | buffer, abort_flag);
        break;
      }
      copy_scales(a_buf + buffer * kABufBytes + kSlabs * kASlabBytes, kSfACol + uint32_t(buffer) * kSfSlotCols);
      __syncwarp();
      if (lane == 0) arrive_cluster(leader_a_ready + buffer * 8);
      for (int t = 0; t < kTilesPerUnit; ++t) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(b_sf_full_bar + stage, phase))) {
          report(p.error, 0x66000000u | (blockIdx.x << 8) | stage, abort_flag);
          failed = true;
          break;
        }
        copy_scales(b_ring + stage * kBStageBytes + kSlabs * kBSlabBytes, kSfBCol + uint32_t(stage) * kSfSlotCols);
        // the arrival also vouches for this CTA's weight rows
        if (!__all_sync(0xffffffffu, ptx::mbar_wait_bounded(b_full_bar + stage, phase))) {
          report(p.error, 0x67000000u | (blockIdx.x << 8) | stage, abort_flag);
          failed = true;
          break;
        }
        if (lane == 0) arrive_cluster(leader_b_ready + stage * 8);
        if (++stage == kBStages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (own 128 rows x 128 channels)
    // A thread reads consecutive channels of its own token row from tensor memory; a 4x4 transpose of
    // 16-byte units inside every group of four lanes then lets four neighbouring lanes write 64
    // contiguous bytes of one row.
    const int quad = warp % 4;
    const int quarter = (warp - kFirstEpilogueWarp) / 4;             // 32 of the tile's 128 channels
    const uint32_t leader_acc_empty = leader_address(acc_empty_bar);
    int tiles = 0;
    Unit u{-1, 0, 0, 0, 0};
    float alpha = 0.0F;
    int info_of = -1;
    bf16* out = static_cast<bf16*>(p.out);
    bool failed = false;
    long long prof_wait = 0, prof_work = 0;
    for (int w = pair_index; w < total && !failed && !*abort_flag; w += pairs) {
      decode_unit(table, w, kChunks, u);
      if (info_of != u.e) {
        alpha = p.experts[u.e].alpha[2];
        info_of = u.e;
      }
      const int row0 = (2 * u.tile + int(rank)) * 128 + quad * 32 + (lane & ~3);   // first row of this lane group in the expert
      const int rows_left = u.count - row0;
      const size_t sorted_row0 = size_t(u.first) + row0;
      uint64_t group_dest[4] = {0, 0, 0, 0};
      if (p.row_dest != nullptr) {
        const int mine = (2 * u.tile + int(rank)) * 128 + quad * 32 + lane;
        const uint64_t home = mine < u.count ? p.row_dest[size_t(u.first) + mine] : 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) group_dest[i] = __shfl_sync(0xffffffffu, home, (lane & ~3) + i);
      }
      for (int t = 0; t < kTilesPerUnit; ++t, ++tiles) {
        const int acc = tiles & 1;
        const long long t0 = prof ? clock64() : 0;
        if (!ptx::mbar_wait_warp(acc_full_bar + acc, uint32_t(tiles >> 1) & 1u)) {
          report(p.error, 0x43000000u | (blockIdx.x << 8) | acc, abort_flag);
          failed = true;
          break;
        }
        const long long t1 = prof ? clock64() : 0;
        if (prof) prof_wait += t1 - t0;
        ptx::tc_fence_after_sync();
        const uint32_t taddr = tmem_base + uint32_t(acc) * kTileCols + (uint32_t(quad * 32) << 16);
        const int c_base = (u.part * kTilesPerUnit + t) * kTileCols + quarter * 32;
        uint4 unit[4];
        {
          uint32_t r[32];
          ptx::tmem_load16(taddr + quarter * 32, r);
          ptx::tmem_load16(taddr + quarter * 32 + 16, r + 16);
          ptx::tmem_load_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q)
            unit[q] = make_uint4(
                pack_bf16x2(__fmul_rn(__uint_as_float(r[8 * q]), alpha), __fmul_rn(__uint_as_float(r[8 * q + 1]), alpha)),
                pack_bf16x2(__fmul_rn(__uint_as_float(r[8 * q + 2]), alpha), __fmul_rn(__uint_as_float(r[8 * q + 3]), alpha)),
                pack_bf16x2(__fmul_rn(__uint_as_float(r[8 * q + 4]), alpha), __fmul_rn(__uint_as_float(r[8 * q + 5]), alpha)),
                pack_bf16x2(__fmul_rn(__uint_as_float(r[8 * q + 6]), alpha), __fmul_rn(__uint_as_float(r[8 * q + 7]), alpha)));
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) arrive_cluster(leader_acc_empty + acc * 8);   // this accumulator stage may be overwritten
        transpose_units(unit, lane);
        const int c = c_base + 8 * (lane & 3);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (i >= rows_left) continue;
          bf16* dst;
          if (p.row_dest != nullptr) {
            if (group_dest[i] == 0) continue;         // a row without a home (reported when the table was built)
            dst = reinterpret_cast<bf16*>(group_dest[i]) + c;
          } else {
            dst = out + (sorted_row0 + i) * size_t(kHidden) + c;
          }
          *reinterpret_cast<uint4*>(dst) = unit[i];
        }
        if (prof) prof_work += clock64() - t1;
      }
    }
    if (prof && lane == 0 && warp == kFirstEpilogueWarp) {
      long long* row = p.profile + size_t(blockIdx.x) * 8;
      row[4] = prof_wait;
      row[5] = prof_work;
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

long long* g_pair_moe_profile = nullptr;

template <typename Kernel>
cudaError_t launch_pair_kernel(Kernel kernel, int threads, int smem_bytes, const PairMoeParams& params, int sm_count,
                               bool* configured, cudaStream_t stream) {
  if (!*configured) {
    cudaError_t status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (status != cudaSuccess) return status;
    *configured = true;
  }
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(2 * (sm_count / 2));
  config.blockDim = dim3(threads);
  config.dynamicSmemBytes = smem_bytes;
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
  return cudaLaunchKernelEx(&config, kernel, params);
}

}  // namespace

void set_pair_moe_profile_buffer(long long* device_buffer) { g_pair_moe_profile = device_buffer; }

cudaError_t launch_pair_moe_gate_up(const PairMoeParams& params_in, int sm_count, cudaStream_t stream) {
  static bool configured_on[2][kMaxDeviceSlots] = {};   // the attribute is per GPU (and per instantiation)
  PairMoeParams params = params_in;
  params.profile = g_pair_moe_profile;                   // gate/up: first half of the buffer
  const int slot = current_device_slot();
  if (params.profile != nullptr)
    return launch_pair_kernel(pair_moe_gate_up_kernel<true>, gu::kThreads, gu::kSmemBytes, params, sm_count,
                              &configured_on[1][slot], stream);
  return launch_pair_kernel(pair_moe_gate_up_kernel<false>, gu::kThreads, gu::kSmemBytes, params, sm_count,
                            &configured_on[0][slot], stream);
}

cudaError_t launch_pair_moe_down(const PairMoeParams& params_in, int sm_count, cudaStream_t stream) {
  static bool configured_on[2][kMaxDeviceSlots] = {};
  PairMoeParams params = params_in;
  params.profile = g_pair_moe_profile ? g_pair_moe_profile + 148 * 8 : nullptr;   // down: second half
  const int slot = current_device_slot();
  if (params.profile != nullptr)
    return launch_pair_kernel(pair_moe_down_kernel<true>, dn::kThreads, dn::kSmemBytes, params, sm_count,
                              &configured_on[1][slot], stream);
  return launch_pair_kernel(pair_moe_down_kernel<false>, dn::kThreads, dn::kSmemBytes, params, sm_count,
                            &configured_on[0][slot], stream);
}

}  // namespace gw
