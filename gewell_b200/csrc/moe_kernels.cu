// MoE routing, permutation, fused gather+quantise, GeGLU+quantise and the
// ordered combine for the 128-expert / top-8 layer (hidden 2816, expert MLP
// 704).  Everything stays on the device: no routing data is read back.
//
// Permutation.  The reference radix-sorts (expert, assignment) pairs; because
// the eight experts of a token are distinct, the stable order inside an expert
// is simply token order.  So the position of assignment (t, slot) is
//   offsets[e] + #tokens t' < t that chose e,
// computed here with per-64-token bitmaps and popcounts: kernel 1 routes and
// builds the bitmaps, kernel 2 scans the per-chunk counts, kernel 3 scatters.
#include "common.cuh"
#include "moe_kernels.h"
#include "ptx.cuh"

namespace gw {
namespace {

constexpr int kExperts = 128;
constexpr int kTopK = 8;
constexpr int kHidden = 2816;
constexpr int kInter = 704;
constexpr int kMapsPerExpert = kMoeMapsPerExpert;
constexpr int kChunkTokens = 64;   // tokens per routing block (two 32-bit bitmap words per expert)

__device__ __forceinline__ uint64_t ptx_global_timer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void unpack8(const uint4& raw, float* out) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
  }
}

// One token (one warp): FP32 softmax over its 128 logits, eight winners, renormalised weights, and the
// winners' bits in the chunk's bitmaps.  The FP32 operation order is that of the reference's select
// kernel (models/gemma4/26b_a4b/sm120/moe.cu:104-157), so ids and FP32 weights match it bit for bit.
__device__ __forceinline__ void route_token(const bf16* __restrict__ scores, const bf16* __restrict__ expert_scales,
                                            uint32_t row, uint32_t local, unsigned lane, int32_t* __restrict__ keys,
                                            float* __restrict__ weights, uint32_t (*bitmap)[2]) {
  // Softmax over the token's 128 logits; this lane owns experts lane, lane + 32, lane + 64, lane + 96.
  // The FP32 additions keep the order the reference's weights depend on: the lane's four terms in
  // ascending expert order first, then the xor butterfly 16, 8, 4, 2, 1 over the lanes.
  const bf16* token_scores = scores + size_t(row) * kExperts;
  float prob[4];
  float peak = -INFINITY;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    prob[q] = __bfloat162float(token_scores[lane + 32 * q]);
    peak = fmaxf(peak, prob[q]);
  }
#pragma unroll
  for (int step = 16; step > 0; step >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, step));
  float denominator = 0.0F;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    prob[q] = expf(prob[q] - peak);
    denominator += prob[q];
  }
#pragma unroll
  for (int step = 16; step > 0; step >>= 1) denominator += __shfl_xor_sync(0xffffffffu, denominator, step);
  // Eight winners, one 64-bit maximum per round: the probability's bit pattern (probabilities are
  // not negative, so their patterns order like unsigned integers) in the high word and 128 - id
  // in the low word, so that the larger probability wins and, among equal ones, the smaller id.
  // A candidate that has won is replaced by key 0, below every live key.
  unsigned long long candidate[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    prob[q] = __fdiv_rn(prob[q], denominator);
    candidate[q] = (static_cast<unsigned long long>(__float_as_uint(prob[q])) << 32) | uint32_t(kExperts - (lane + 32 * q));
  }
  int ids[kTopK];
  float chosen[kTopK];
#pragma unroll
  for (int round = 0; round < kTopK; ++round) {
    unsigned long long winner = candidate[0];
#pragma unroll
    for (int q = 1; q < 4; ++q) winner = candidate[q] > winner ? candidate[q] : winner;
#pragma unroll
    for (int step = 16; step > 0; step >>= 1) {
      const unsigned long long theirs = __shfl_xor_sync(0xffffffffu, winner, step);
      winner = theirs > winner ? theirs : winner;
    }
    const int id = kExperts - int(uint32_t(winner));
    ids[round] = id;
    chosen[round] = __uint_as_float(uint32_t(winner >> 32));
#pragma unroll
    for (int q = 0; q < 4; ++q)
      if (id == int(lane) + 32 * q) candidate[q] = 0;
  }
  // renormalisation: ((p0+p4)+(p2+p6)) + ((p1+p5)+(p3+p7)), the pairwise order of a stride-4/2/1 fold
  float fold[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) fold[q] = chosen[q] + chosen[q + 4];
  const float sum = (fold[0] + fold[2]) + (fold[1] + fold[3]);
  int my_id = 0;
  float my_p = 0;
#pragma unroll
  for (int i = 0; i < kTopK; ++i) if (lane == unsigned(i)) { my_id = ids[i]; my_p = chosen[i]; }
  if (lane < kTopK) {
    int rank = 0;
#pragma unroll
    for (int i = 0; i < kTopK; ++i) rank += ids[i] < my_id;
    const float weight = __fmul_rn(__fdiv_rn(my_p, sum), __bfloat162float(expert_scales[my_id]));
    keys[size_t(row) * kTopK + rank] = my_id;
    weights[size_t(row) * kTopK + rank] = weight;
    atomicOr(&bitmap[my_id][local / 32], 1u << (local % 32));
  }
}

// ---------------------------------------------------------------------------
// 1. route: FP32 softmax over 128 BF16 logits, eight winners (lower id wins
//    ties), renormalise, times the per-expert scale, sort the eight by id.
//    The FP32 operation order is that of the reference's select kernel
//    (models/gemma4/26b_a4b/sm120/moe.cu:104-157), so ids and FP32 weights match
//    it bit for bit.  One warp per token, eight tokens per warp.
// ---------------------------------------------------------------------------
//    (route_token below; used by the single-block kernel and by the grid-wide kernel)
//    With at most 64 tokens there is one block: it then also does the work of kernels 2
//    and 3 (`offsets` != nullptr), which saves two dependent launches on the decode path.
__global__ void __launch_bounds__(1024)
moe_route_kernel(const bf16* __restrict__ scores, const bf16* __restrict__ expert_scales, uint32_t rows,
                 int32_t* __restrict__ keys, float* __restrict__ weights, uint32_t* __restrict__ bitmaps,
                 int32_t* __restrict__ chunk_counts, int32_t* __restrict__ offsets,
                 int32_t* __restrict__ sorted_assignments, int32_t* __restrict__ sorted_keys,
                 int32_t* __restrict__ inverse) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  __shared__ uint32_t bitmap[kExperts][2];
  const unsigned lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  if (threadIdx.x < kExperts) { bitmap[threadIdx.x][0] = 0; bitmap[threadIdx.x][1] = 0; }
  __syncthreads();
  const uint32_t chunk = blockIdx.x;
  const int tokens_per_warp = kChunkTokens / int(blockDim.x / 32);     // 8 warps: 8 tokens each; 32 warps: 2
  for (int t = 0; t < tokens_per_warp; ++t) {
    const uint32_t local = warp * tokens_per_warp + t;
    const uint32_t row = chunk * kChunkTokens + local;
    if (row >= rows) break;
    route_token(scores, expert_scales, row, local, lane, keys, weights, bitmap);
  }
  __syncthreads();
  if (threadIdx.x < kExperts) {
    const uint32_t w0 = bitmap[threadIdx.x][0], w1 = bitmap[threadIdx.x][1];
    bitmaps[(size_t(chunk) * kExperts + threadIdx.x) * 2] = w0;
    bitmaps[(size_t(chunk) * kExperts + threadIdx.x) * 2 + 1] = w1;
    chunk_counts[size_t(chunk) * kExperts + threadIdx.x] = offsets != nullptr ? 0 : __popc(w0) + __popc(w1);
  }
  if (offsets == nullptr) return;
  // single block: offsets, positions, inverse (the scan and scatter steps of kernels 2 and 3)
  __shared__ int32_t base[kExperts];
  if (warp == 0) {
    // exclusive scan of the 128 expert counts in one warp: four consecutive experts per lane
    int32_t count[4], mine = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      count[q] = __popc(bitmap[4 * lane + q][0]) + __popc(bitmap[4 * lane + q][1]);
      mine += count[q];
    }
    int32_t running = mine;
#pragma unroll
    for (int step = 1; step < 32; step <<= 1) {
      const int32_t below = __shfl_up_sync(0xffffffffu, running, step);
      if (lane >= unsigned(step)) running += below;
    }
    int32_t acc = running - mine;        // rows of all experts before this lane's four
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      base[4 * lane + q] = acc;
      offsets[4 * lane + q] = acc;
      acc += count[q];
    }
    if (lane == 31) offsets[kExperts] = acc;
  }
  __syncthreads();                       // also orders this block's writes of `keys` before the reads below
  for (uint32_t i = threadIdx.x; i < kChunkTokens * kTopK; i += blockDim.x) {
    const uint32_t local = i / kTopK;
    if (local >= rows) continue;
    const uint32_t assignment = local * kTopK + i % kTopK;
    const int32_t e = keys[assignment];
    const uint32_t w0 = bitmap[e][0], w1 = bitmap[e][1];
    const int rank = local < 32 ? __popc(w0 & ((1u << local) - 1u))
                                : __popc(w0) + __popc(w1 & ((1u << (local - 32)) - 1u));
    const int32_t position = base[e] + rank;
    sorted_assignments[position] = int32_t(assignment);
    sorted_keys[position] = e;
    inverse[assignment] = position;
  }
}

// ---------------------------------------------------------------------------
// 1b. route + scan + scatter in ONE launch for more than 64 tokens.  At most
//     kRouteGridBlocksPerSm blocks per SM, each walking chunks b, b + grid, ...:
//       phase 1  route the block's chunks (bitmaps and per-chunk counts to global memory)
//       barrier  every block has published its counts
//       phase 2  every block walks all chunk counts once: the running sums at its own chunks are
//                their bases, the totals give the expert offsets (block 0 stores them)
//       phase 3  scatter the block's chunks
//     The barrier is a counter plus a generation word in the workspace (the last block to arrive
//     resets the counter and bumps the generation, so replays need no host-side reset).  All blocks
//     are resident together -- the grid is sized below what the GPU holds at once -- and the wait is
//     bounded: on a timeout the block reports through the error word and returns.
// ---------------------------------------------------------------------------
constexpr int kRouteGridBlocksPerSm = 1;
constexpr int kRouteGridThreads = 1024;
constexpr int kRouteOwnChunks = 16;     // chunks per block the launch sizes the grid for (65536 tokens / 64 / 148 < 8)
constexpr int kRouteParts = kRouteGridThreads / kExperts;   // phase 2: eight threads share an expert's chunk list

__device__ __forceinline__ bool route_grid_barrier(uint32_t* state, uint32_t blocks, uint32_t* error) {
  __shared__ int passed;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();                                        // this block's counts are visible before it arrives
    const uint32_t generation = atomicAdd(state + 1, 0u);
    int ok = 1;
    if (atomicAdd(state, 1u) == blocks - 1) {
      atomicExch(state, 0u);                                // ready for the next launch
      __threadfence();
      atomicAdd(state + 1, 1u);
    } else {
      const uint64_t start = ptx_global_timer();
      for (uint32_t spin = 1; atomicAdd(state + 1, 0u) == generation; ++spin) {
        if ((spin & 63u) == 0 && ptx_global_timer() - start > 2000000000ull) { ok = 0; break; }
        __nanosleep(32);
      }
    }
    __threadfence();
    if (!ok && error != nullptr) atomicCAS(error, 0u, 0x80000000u | blockIdx.x);
    passed = ok;
  }
  __syncthreads();
  return passed != 0;
}

__global__ void __launch_bounds__(kRouteGridThreads)
moe_route_grid_kernel(const bf16* __restrict__ scores, const bf16* __restrict__ expert_scales, uint32_t rows,
                      uint32_t chunks, int32_t* __restrict__ keys, float* __restrict__ weights,
                      uint32_t* __restrict__ bitmaps, int32_t* __restrict__ chunk_counts, int32_t* __restrict__ offsets,
                      int32_t* __restrict__ sorted_assignments, int32_t* __restrict__ sorted_keys,
                      int32_t* __restrict__ inverse, uint32_t* __restrict__ barrier_state, uint32_t* __restrict__ error) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  __shared__ uint32_t bitmap[kExperts][2];
  __shared__ int32_t own_base[kRouteOwnChunks][kExperts];
  __shared__ int32_t part_sum[kRouteParts][kExperts];
  __shared__ int32_t expert_offset[kExperts];
  __shared__ int32_t warp_totals[4];
  const unsigned lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  constexpr int kTokensPerWarp = kChunkTokens / (kRouteGridThreads / 32);     // 2
  // ---- phase 1: 32 warps, two tokens each, per chunk
  for (uint32_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x) {
    if (threadIdx.x < kExperts) { bitmap[threadIdx.x][0] = 0; bitmap[threadIdx.x][1] = 0; }
    __syncthreads();
#pragma unroll
    for (int t = 0; t < kTokensPerWarp; ++t) {
      const uint32_t local = warp * kTokensPerWarp + t;
      const uint32_t row = chunk * kChunkTokens + local;
      if (row < rows) route_token(scores, expert_scales, row, local, lane, keys, weights, bitmap);
    }
    __syncthreads();
    if (threadIdx.x < kExperts) {
      const uint32_t w0 = bitmap[threadIdx.x][0], w1 = bitmap[threadIdx.x][1];
      bitmaps[(size_t(chunk) * kExperts + threadIdx.x) * 2] = w0;
      bitmaps[(size_t(chunk) * kExperts + threadIdx.x) * 2 + 1] = w1;
      chunk_counts[size_t(chunk) * kExperts + threadIdx.x] = __popc(w0) + __popc(w1);
    }
    __syncthreads();
  }
  if (!route_grid_barrier(barrier_state, gridDim.x, error)) return;
  // ---- phase 2: expert e's counts summed over the chunks in order; eight threads share the list (contiguous
  // ranges of chunks), their partial sums are combined in order afterwards
  {
    const unsigned e = threadIdx.x % kExperts, part = threadIdx.x / kExperts;
    const uint32_t per_part = (chunks + kRouteParts - 1) / kRouteParts;
    const uint32_t c_begin = min(part * per_part, chunks), c_end = min(c_begin + per_part, chunks);
    int32_t running = 0;
#pragma unroll 8
    for (uint32_t c = c_begin; c < c_end; ++c) running += __ldcg(chunk_counts + size_t(c) * kExperts + e);
    part_sum[part][e] = running;
    __syncthreads();
    // bases of this block's own chunks: sum of the parts before the chunk's part plus the counts inside it
    if (part == 0) {
      int32_t before[kRouteParts];
      int32_t total = 0;
#pragma unroll
      for (int q = 0; q < kRouteParts; ++q) { before[q] = total; total += part_sum[q][e]; }
      uint32_t own = 0;
      for (uint32_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x, ++own) {
        const uint32_t q = chunk / per_part;
        int32_t base = before[q];
        for (uint32_t c = q * per_part; c < chunk; ++c) base += __ldcg(chunk_counts + size_t(c) * kExperts + e);
        own_base[own][e] = base;
      }
      // exclusive scan of the totals over the 128 experts (threads 0..127 are four whole warps)
      int32_t scan = total;
#pragma unroll
      for (int step = 1; step < 32; step *= 2) {
        const int32_t other = __shfl_up_sync(0xffffffffu, scan, step);
        if (lane >= unsigned(step)) scan += other;
      }
      if (lane == 31) warp_totals[warp] = scan;
      expert_offset[e] = scan - total;
    }
  }
  __syncthreads();
  if (threadIdx.x < kExperts) {
    int32_t base = 0;
    for (unsigned w = 0; w < warp; ++w) base += warp_totals[w];
    expert_offset[threadIdx.x] += base;
    if (blockIdx.x == 0) {
      offsets[threadIdx.x] = expert_offset[threadIdx.x];
      if (threadIdx.x == kExperts - 1) offsets[kExperts] = base + warp_totals[3];
    }
  }
  __syncthreads();
  // ---- phase 3
  uint32_t own = 0;
  for (uint32_t chunk = blockIdx.x; chunk < chunks; chunk += gridDim.x, ++own) {
    if (threadIdx.x < kExperts) {
      bitmap[threadIdx.x][0] = __ldcg(bitmaps + (size_t(chunk) * kExperts + threadIdx.x) * 2);
      bitmap[threadIdx.x][1] = __ldcg(bitmaps + (size_t(chunk) * kExperts + threadIdx.x) * 2 + 1);
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < kChunkTokens * kTopK; i += kRouteGridThreads) {
      const uint32_t local = i / kTopK;
      const uint32_t row = chunk * kChunkTokens + local;
      if (row >= rows) continue;
      const uint32_t assignment = row * kTopK + i % kTopK;
      const int32_t e = keys[assignment];
      const uint32_t w0 = bitmap[e][0], w1 = bitmap[e][1];
      const int rank = local < 32 ? __popc(w0 & ((1u << local) - 1u))
                                  : __popc(w0) + __popc(w1 & ((1u << (local - 32)) - 1u));
      const int32_t position = expert_offset[e] + own_base[own][e] + rank;
      sorted_assignments[position] = int32_t(assignment);
      sorted_keys[position] = e;
      inverse[assignment] = position;
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// 2. scan: per expert, exclusive prefix of the chunk counts (in place) and the
//    expert offsets (== searchsorted of the sorted keys, moe.cu:158-167).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kExperts)
moe_scan_kernel(int32_t* __restrict__ chunk_counts, uint32_t chunks, int32_t* __restrict__ offsets) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  __shared__ int32_t totals[kExperts];
  const unsigned e = threadIdx.x;
  int32_t running = 0;
#pragma unroll 8
  for (uint32_t c = 0; c < chunks; ++c) {
    const int32_t v = chunk_counts[size_t(c) * kExperts + e];
    chunk_counts[size_t(c) * kExperts + e] = running;
    running += v;
  }
  totals[e] = running;
  __syncthreads();
  if (e == 0) {
    int32_t acc = 0;
    for (int i = 0; i < kExperts; ++i) { offsets[i] = acc; acc += totals[i]; }
    offsets[kExperts] = acc;
  }
}

// ---------------------------------------------------------------------------
// 3. scatter: stable position of every assignment, sorted assignments/keys and
//    the inverse permutation (moe.cu:179-182).
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_scatter_kernel(const int32_t* __restrict__ keys, const uint32_t* __restrict__ bitmaps,
                   const int32_t* __restrict__ chunk_base, const int32_t* __restrict__ offsets, uint32_t rows,
                   int32_t* __restrict__ sorted_assignments, int32_t* __restrict__ sorted_keys,
                   int32_t* __restrict__ inverse) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  __shared__ uint32_t bitmap[kExperts][2];
  __shared__ int32_t base[kExperts];
  const uint32_t chunk = blockIdx.x;
  if (threadIdx.x < kExperts) {
    bitmap[threadIdx.x][0] = bitmaps[(size_t(chunk) * kExperts + threadIdx.x) * 2];
    bitmap[threadIdx.x][1] = bitmaps[(size_t(chunk) * kExperts + threadIdx.x) * 2 + 1];
    base[threadIdx.x] = offsets[threadIdx.x] + chunk_base[size_t(chunk) * kExperts + threadIdx.x];
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < kChunkTokens * kTopK; i += 256) {
    const uint32_t local = i / kTopK;
    const uint32_t row = chunk * kChunkTokens + local;
    if (row >= rows) continue;
    const uint32_t assignment = row * kTopK + i % kTopK;
    const int32_t e = keys[assignment];
    const uint32_t w0 = bitmap[e][0], w1 = bitmap[e][1];
    const int rank = local < 32 ? __popc(w0 & ((1u << local) - 1u))
                                : __popc(w0) + __popc(w1 & ((1u << (local - 32)) - 1u));
    const int32_t position = base[e] + rank;
    sorted_assignments[position] = int32_t(assignment);
    sorted_keys[position] = e;
    inverse[assignment] = position;
  }
}

// Expert id of every row of an already sorted buffer (expert-parallel entry).
__global__ void __launch_bounds__(256)
moe_keys_from_offsets_kernel(const int32_t* __restrict__ offsets, uint32_t first_expert, uint32_t expert_count,
                             uint32_t rows, int32_t* __restrict__ sorted_keys, int32_t* __restrict__ full_offsets) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  const uint32_t i = blockIdx.x * 256 + threadIdx.x;
  if (blockIdx.x == 0 && threadIdx.x <= kExperts) {
    // offsets over all 128 experts: empty outside [first, first+count)
    const uint32_t e = threadIdx.x;
    int32_t v;
    if (e < first_expert) v = 0;
    else if (e <= first_expert + expert_count) v = offsets[e - first_expert];
    else v = offsets[expert_count];
    full_offsets[e] = v;
  }
  if (i >= rows || i >= uint32_t(offsets[expert_count])) return;   // `rows` may be an upper bound
  uint32_t lo = 0, hi = expert_count;   // largest e with offsets[e] <= i
  while (lo + 1 < hi) {
    const uint32_t mid = (lo + hi) / 2;
    if (uint32_t(offsets[mid]) <= i) lo = mid; else hi = mid;
  }
  sorted_keys[i] = int32_t(first_expert + lo);
}

// ---------------------------------------------------------------------------
// 4. group descriptors of the grouped GEMMs, from the offsets (the role of
//    grouped_nvfp4::prepare, moe_nvfp4.cuh:51-78).  Three plans:
//      swap    weights on the lane operand, an expert's tokens on the column operand
//              (small batches): 256 gate/up groups + 128 down groups
//      direct  tokens on the lane operand, weights on the column operand, plain BF16
//              output: 256 gate/up groups + 128 down groups
//      fused   direct form with gate and up as the two halves of the column operand
//              and GeGLU + FP4 quantisation in the epilogue: 128 groups (+128 down)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_prepare_groups_kernel(MoeGroupPlan plan, GemmGroup* __restrict__ first_groups, GemmGroup* __restrict__ down_groups) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  __shared__ int32_t items_first[2 * kExperts], items_down[kExperts];
  const unsigned g = threadIdx.x;            // 0..255: expert = g/2, part = g%2
  const unsigned e = g / 2, part = g % 2;
  // Offsets that come from other ranks' histograms (expert parallelism) may describe more rows than
  // the buffers hold: clamp every group to the capacity and report, so that no tile is scheduled
  // over rows that do not exist.
  int32_t first = plan.offsets[e], last = plan.offsets[e + 1];
  const int32_t capacity = int32_t(plan.n);
  if (first < 0 || last < first || last > capacity) {
    if (plan.error != nullptr && part == 0) atomicCAS(plan.error, 0u, 0x70000100u | e);
    first = min(max(first, 0), capacity);
    last = min(max(last, first), capacity);
  }
  const MoeExpertInfo info = plan.experts[e];
  // A projection gets work in this launch only if it runs as the launch's kind.
  const bool nv = plan.kind == kMoeKindNvfp4;
  auto runs_here = [&](int proj) { return moe_effective_kind(info.storage[proj], plan.fp4) == plan.kind; };
  const int map_base = int32_t(e) * kMapsPerExpert + (nv ? 0 : 4);
  // BF16 operands carry no scales (the info's alpha belongs to the NVFP4 form of a W4A16 projection)
  auto alpha_of = [&](int proj) { return plan.kind == kMoeKindBf16 ? 1.0F : info.alpha[proj]; };
  const int32_t count = last - first;
  const int32_t token_tiles_swap = (count + plan.block_n_first - 1) / plan.block_n_first;
  const int32_t token_tiles_direct = (count + 127) / 128;
  const int32_t padded_first = (first / 128 + int32_t(e)) * 128;
  // which copy of the quantised input a gate/up projection reads: NVFP4 keeps one copy when gate and up
  // share their input scale, FP8 always keeps two, BF16 rows are not quantised at all
  const int src_part = nv ? (plan.shared_gate_up ? 0 : int(part)) : (plan.kind == kMoeKindFp8 ? int(part) : 0);
  const uint8_t* in_scales = nv ? plan.scales_in + (size_t(src_part) * plan.scale_rows + padded_first) * (kHidden / 16) : nullptr;
  const uint8_t* act_scales = nv ? plan.scales_act + size_t(padded_first) * (kInter / 16) : nullptr;
  {
    GemmGroup grp{};
    if (plan.form == kMoeFormFused) {
      // one group per expert (threads with part == 1 write nothing); NVFP4 only
      const bool active = runs_here(0) && runs_here(1);
      grp.sf_l = in_scales;
      grp.map_l = -1;
      grp.l_row0 = first;
      grp.l_rows = count;
      grp.l_tiles = active ? token_tiles_direct : 0;
      grp.sf_c[0] = info.scales[0];
      grp.sf_c[1] = info.scales[1];
      grp.map_c[0] = map_base;
      grp.map_c[1] = map_base + 1;
      grp.c_row0 = 0;
      grp.c_rows = kInter;
      grp.c_tiles = (kInter + 127) / 128;
      grp.c_half_stride = 0;
      grp.alpha[0] = info.alpha[0];
      grp.alpha[1] = info.alpha[1];
      grp.quant_inverse_scale = info.inverse_input_scale[2];
      grp.out_row0 = first;
      grp.out_col0 = 0;
      grp.sf_out_row0 = padded_first;
      items_first[g] = part == 0 ? grp.l_tiles * grp.c_tiles : 0;
      if (part == 0) first_groups[e] = grp;
    } else if (plan.form == kMoeFormDirect) {
      const int proj = part;
      grp.sf_l = in_scales;
      grp.map_l = -1;
      grp.l_row0 = src_part * int32_t(plan.n) + first;
      grp.l_rows = count;
      grp.l_tiles = runs_here(proj) ? token_tiles_direct : 0;
      grp.sf_c[0] = grp.sf_c[1] = info.scales[proj];
      grp.map_c[0] = grp.map_c[1] = map_base + proj;
      grp.c_row0 = 0;
      grp.c_rows = kInter;
      grp.c_tiles = (kInter + plan.block_n_first - 1) / plan.block_n_first;
      grp.c_half_stride = plan.block_n_first > 128 ? 128 : 0;
      grp.alpha[0] = grp.alpha[1] = alpha_of(proj);
      grp.channel_alpha = nv ? nullptr : info.channel_alpha[proj];
      grp.out_row0 = first;
      grp.out_col0 = proj * kInter;
      items_first[g] = grp.l_tiles * grp.c_tiles;
      first_groups[g] = grp;
    } else {
      const int proj = part;
      grp.sf_l = info.scales[proj];
      grp.map_l = map_base + proj;
      grp.l_row0 = 0;
      grp.l_rows = kInter;
      grp.l_tiles = runs_here(proj) ? (kInter + 127) / 128 : 0;
      grp.sf_c[0] = grp.sf_c[1] = in_scales;
      grp.map_c[0] = grp.map_c[1] = -1;
      grp.c_row0 = src_part * int32_t(plan.n) + first;
      grp.c_rows = count;
      grp.c_tiles = token_tiles_swap;
      grp.c_half_stride = 0;
      grp.alpha[0] = grp.alpha[1] = alpha_of(proj);
      grp.channel_alpha = nv ? nullptr : info.channel_alpha[proj];
      grp.out_row0 = first;
      grp.out_col0 = proj * kInter;
      items_first[g] = grp.l_tiles * grp.c_tiles;
      first_groups[g] = grp;
    }
  }
  if (part == 0) {
    GemmGroup grp{};
    const bool active = runs_here(2);
    if (plan.form == kMoeFormSwap) {
      grp.sf_l = info.scales[2];
      grp.map_l = map_base + 2;
      grp.l_row0 = 0;
      grp.l_rows = kHidden;
      grp.l_tiles = active ? kHidden / 128 : 0;
      grp.sf_c[0] = grp.sf_c[1] = act_scales;
      grp.map_c[0] = grp.map_c[1] = -1;
      grp.c_row0 = first;
      grp.c_rows = count;
      grp.c_tiles = (count + plan.block_n_down - 1) / plan.block_n_down;
      grp.c_half_stride = 0;
    } else {
      grp.sf_l = act_scales;
      grp.map_l = -1;
      grp.l_row0 = first;
      grp.l_rows = count;
      grp.l_tiles = active ? token_tiles_direct : 0;
      grp.sf_c[0] = grp.sf_c[1] = info.scales[2];
      grp.map_c[0] = grp.map_c[1] = map_base + 2;
      grp.c_row0 = 0;
      grp.c_rows = kHidden;
      grp.c_tiles = kHidden / plan.block_n_down;
      grp.c_half_stride = plan.block_n_down > 128 ? 128 : 0;
    }
    grp.alpha[0] = grp.alpha[1] = alpha_of(2);
    grp.channel_alpha = nv ? nullptr : info.channel_alpha[2];
    grp.out_row0 = first;
    grp.out_col0 = 0;
    items_down[e] = grp.l_tiles * grp.c_tiles;
    down_groups[e] = grp;
  }
  __syncthreads();
  if (g == 0) {
    const int count_first = plan.form == kMoeFormFused ? kExperts : 2 * kExperts;
    int32_t acc = 0;
    for (int i = 0; i < count_first; ++i) {
      first_groups[i].work_begin = acc;
      acc += plan.form == kMoeFormFused ? items_first[2 * i] : items_first[i];
    }
    GemmGroup sentinel{};
    sentinel.work_begin = acc;
    sentinel.l_tiles = sentinel.c_tiles = 1;
    first_groups[count_first] = sentinel;
  }
  if (g == 1) {
    int32_t acc = 0;
    for (int i = 0; i < kExperts; ++i) { down_groups[i].work_begin = acc; acc += items_down[i]; }
    GemmGroup sentinel{};
    sentinel.work_begin = acc;
    sentinel.l_tiles = sentinel.c_tiles = 1;
    down_groups[kExperts] = sentinel;
  }
}

// ---------------------------------------------------------------------------
// 5. NVFP4 quantisation of sorted rows with the destination expert's input
//    scale (recipe of moe.cu:254-304 == src/nvfp4_linear.cu:61-116), reading
//    either through the permutation (fused gather, moe.cu:183-186) or in place.
//    One thread per K16 block.  Scales go to the expert's 128-row aligned
//    region ((first/128 + e) * 128, moe.cu:296-300) in the tiled layout.
//    Source modes: plain rows of width K, or [rows, 2K] gate|up with GeGLU
//    (moe.cu:439-445) whose BF16 result is also stored for the capture accessor.
// ---------------------------------------------------------------------------
template <int K, bool Gelu>
__global__ void __launch_bounds__(256)
moe_quantize_kernel(const uint4* __restrict__ input, const int32_t* __restrict__ gather_index,
                    const int32_t* __restrict__ sorted_keys, const int32_t* __restrict__ offsets,
                    const MoeExpertInfo* __restrict__ experts, uint32_t n, uint32_t scale_rows, int projection,
                    uint32_t gather_divisor, uint2* __restrict__ packed, uint8_t* __restrict__ scales,
                    uint4* __restrict__ activated) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  constexpr uint32_t kBlocks = K / 16;
  const size_t index = size_t(blockIdx.x) * 256 + threadIdx.x;
  const uint32_t part = blockIdx.y;             // gate/up copy (0 unless the scales differ)
  if (index >= size_t(n) * kBlocks) return;
  const uint32_t row = index / kBlocks, kb = index % kBlocks;
  if (row >= uint32_t(offsets[kExperts])) return;       // n may be an upper bound (expert parallelism)
  const int32_t e = sorted_keys[row];
  const int32_t first = offsets[e];
  const float inverse_scale = experts[e].inverse_input_scale[projection + part];
  float values[16];
  if constexpr (Gelu) {
    const size_t gate = size_t(row) * (2 * kBlocks) + kb;
    float g[16], u[16];
    unpack8(input[2 * gate], g);
    unpack8(input[2 * gate + 1], g + 8);
    unpack8(input[2 * (gate + kBlocks)], u);
    unpack8(input[2 * (gate + kBlocks) + 1], u + 8);
    uint32_t words[8];
#pragma unroll
    for (int i = 0; i < 16; ++i) values[i] = gelu_tanh_multiply_bf16(g[i], u[i]);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      words[i] = (__float_as_uint(values[2 * i]) >> 16) | (__float_as_uint(values[2 * i + 1]) & 0xFFFF0000u);
    if (activated != nullptr) {
      activated[2 * index] = make_uint4(words[0], words[1], words[2], words[3]);
      activated[2 * index + 1] = make_uint4(words[4], words[5], words[6], words[7]);
    }
  } else {
    const size_t source_row = gather_index ? size_t(uint32_t(gather_index[row]) / gather_divisor) : row;
    const size_t block = source_row * kBlocks + kb;
    unpack8(input[2 * block], values);
    unpack8(input[2 * block + 1], values + 8);
  }
  float amax = 0.0F;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(values[i]));
  const uint8_t scale_code = float_to_e4m3(inverse_scale * (amax * rcp_approx_ftz(6.0F)));
  const float block_scale = e4m3_to_float(scale_code);
  const float factor =
      block_scale == 0.0F ? 0.0F : rcp_approx_ftz(block_scale * rcp_approx_ftz(inverse_scale));
  uint32_t out[2] = {0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i)
    out[i / 4] |= uint32_t(float2_to_e2m1x2(values[2 * i] * factor, values[2 * i + 1] * factor)) << (8 * (i % 4));
  packed[(size_t(part) * n + row) * kBlocks + kb] = make_uint2(out[0], out[1]);
  const size_t region = (size_t(part) * scale_rows + size_t(first / 128 + e) * 128) * kBlocks;
  scales[region + scale_offset(row - first, kb, K)] = scale_code;
}

// ---------------------------------------------------------------------------
// 5b. The same quantisation, token-major: two warps read a token's row once
//     (a lane keeps three K16 blocks as packed BF16 and their maxima) and write
//     the token's eight quantised copies, one per chosen expert, each with that
//     expert's input scale, at the copy's sorted position.  Arithmetic per
//     value is that of kernel 5, so the bytes are identical; the input is read
//     from memory once instead of eight times.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_quantize_tokens_kernel(const uint4* __restrict__ input, const int32_t* __restrict__ keys,
                           const int32_t* __restrict__ inverse, const int32_t* __restrict__ offsets,
                           const MoeExpertInfo* __restrict__ experts, uint32_t tokens, uint32_t scale_rows, int parts,
                           uint2* __restrict__ packed, uint8_t* __restrict__ scales) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  // Two warps per token, each with one half of the row (88 K16 blocks, three per lane): half the
  // registers of a whole row per warp, so twice as many warps are resident to cover the loads.
  constexpr uint32_t kBlocks = kHidden / 16;            // 176
  constexpr uint32_t kHalfBlocks = kBlocks / 2;         // 88
  constexpr int kPerLane = (kHalfBlocks + 31) / 32;     // 3
  const uint32_t warp_index = (blockIdx.x * 256 + threadIdx.x) / 32, lane = threadIdx.x % 32;
  const uint32_t token = warp_index / 2, half = warp_index % 2;
  if (token >= tokens) return;
  const uint32_t n = tokens * kTopK;
  // Lane j < 8 fetches what copy j needs (expert, destination row, the expert's first row and input
  // scales): one round of dependent loads for the token instead of one per copy.
  int32_t copy_expert = 0, copy_first = 0;
  uint32_t copy_row = 0;
  float copy_scale[2] = {0.0F, 0.0F};
  if (lane < kTopK) {
    copy_expert = keys[token * kTopK + lane];
    copy_row = uint32_t(inverse[token * kTopK + lane]);
    copy_first = offsets[copy_expert];
    copy_scale[0] = experts[copy_expert].inverse_input_scale[0];
    if (parts > 1) copy_scale[1] = experts[copy_expert].inverse_input_scale[1];
  }
  uint32_t raw[kPerLane][8];
  float amax[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const uint32_t local = lane + 32 * i;
    const uint32_t kb = half * kHalfBlocks + local;
    amax[i] = 0.0F;
    if (local < kHalfBlocks) {
      const uint4 a = input[2 * (size_t(token) * kBlocks + kb)], b = input[2 * (size_t(token) * kBlocks + kb) + 1];
      raw[i][0] = a.x; raw[i][1] = a.y; raw[i][2] = a.z; raw[i][3] = a.w;
      raw[i][4] = b.x; raw[i][5] = b.y; raw[i][6] = b.z; raw[i][7] = b.w;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        amax[i] = fmaxf(amax[i], fabsf(__uint_as_float(raw[i][k] << 16)));
        amax[i] = fmaxf(amax[i], fabsf(__uint_as_float(raw[i][k] & 0xFFFF0000u)));
      }
    }
  }
  // The quantised row depends on the input scale only: consecutive copies with the same scale (experts
  // calibrated together, or one scale for the whole layer) reuse the codes of the copy before them.
  uint32_t out[kPerLane][2];
  uint8_t scale_code[kPerLane];
  float quantised_with = -1.0F;        // input scales are positive
  for (int j = 0; j < kTopK; ++j) {
    const int32_t e = __shfl_sync(0xffffffffu, copy_expert, j);
    const uint32_t row = __shfl_sync(0xffffffffu, copy_row, j);
    const int32_t first = __shfl_sync(0xffffffffu, copy_first, j);
    const float scale_of_part[2] = {__shfl_sync(0xffffffffu, copy_scale[0], j), __shfl_sync(0xffffffffu, copy_scale[1], j)};
    for (int part = 0; part < parts; ++part) {
      const float inverse_scale = scale_of_part[part];
      const size_t region = (size_t(part) * scale_rows + size_t(first / 128 + e) * 128) * kBlocks;
      if (inverse_scale != quantised_with) {     // the same for every lane of the warp
        quantised_with = inverse_scale;
#pragma unroll
        for (int i = 0; i < kPerLane; ++i) {
          scale_code[i] = float_to_e4m3(inverse_scale * (amax[i] * rcp_approx_ftz(6.0F)));
          const float block_scale = e4m3_to_float(scale_code[i]);
          const float factor =
              block_scale == 0.0F ? 0.0F : rcp_approx_ftz(block_scale * rcp_approx_ftz(inverse_scale));
          out[i][0] = out[i][1] = 0;
#pragma unroll
          for (int k = 0; k < 8; ++k)
            out[i][k / 4] |= uint32_t(float2_to_e2m1x2(__uint_as_float(raw[i][k] << 16) * factor,
                                                       __uint_as_float(raw[i][k] & 0xFFFF0000u) * factor)) << (8 * (k % 4));
        }
      }
#pragma unroll
      for (int i = 0; i < kPerLane; ++i) {
        const uint32_t local = lane + 32 * i;
        const uint32_t kb = half * kHalfBlocks + local;
        if (local >= kHalfBlocks) continue;
        packed[(size_t(part) * n + row) * kBlocks + kb] = make_uint2(out[i][0], out[i][1]);
        scales[region + scale_offset(row - first, kb, kHidden)] = scale_code[i];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// 5c. FP8 expert inputs (the role of pack_fp8 inside the reference's grouped_fp8,
//     moe.cu:187-251, which quantises in registers): e4m3_satfinite(x * 1/input_scale)
//     with the input scale of the row's expert and projection; eight values per thread.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_quantize_fp8_kernel(const uint4* __restrict__ input, const int32_t* __restrict__ gather_index,
                        uint32_t gather_divisor, const int32_t* __restrict__ sorted_keys,
                        const int32_t* __restrict__ offsets, const MoeExpertInfo* __restrict__ experts, uint32_t n,
                        uint32_t vectors, int first_projection, uint2* __restrict__ packed) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  const size_t index = size_t(blockIdx.x) * 256 + threadIdx.x;
  const uint32_t part = blockIdx.y;
  if (index >= size_t(n) * vectors) return;
  const uint32_t row = index / vectors, v = index % vectors;
  if (row >= uint32_t(offsets[kExperts])) return;       // n may be an upper bound
  const int32_t e = sorted_keys[row];
  const float inverse_scale = experts[e].inverse_input_scale[first_projection + part];
  const size_t source_row = gather_index ? size_t(uint32_t(gather_index[row]) / gather_divisor) : row;
  float x[8];
  unpack8(input[source_row * vectors + v], x);
  uint32_t words[2] = {0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i)
    words[i / 4] |= uint32_t(float_to_e4m3(__fmul_rn(x[i], inverse_scale))) << (8 * (i % 4));
  packed[(size_t(part) * n + row) * vectors + v] = make_uint2(words[0], words[1]);
}

// GeGLU alone (moe.cu:439-445) for expert tables without FP4 activations.
__global__ void __launch_bounds__(256)
moe_activate_kernel(const uint4* __restrict__ gate_up, const int32_t* __restrict__ offsets, uint32_t n,
                    uint4* __restrict__ activated) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  constexpr uint32_t kVectors = kInter / 8;
  const size_t index = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (index >= size_t(n) * kVectors) return;
  const uint32_t row = index / kVectors, v = index % kVectors;
  if (row >= uint32_t(offsets[kExperts])) return;
  float g[8], u[8];
  unpack8(gate_up[size_t(row) * (2 * kVectors) + v], g);
  unpack8(gate_up[size_t(row) * (2 * kVectors) + kVectors + v], u);
  uint32_t words[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float a = gelu_tanh_multiply_bf16(g[2 * i], u[2 * i]), b = gelu_tanh_multiply_bf16(g[2 * i + 1], u[2 * i + 1]);
    words[i] = (__float_as_uint(a) >> 16) | (__float_as_uint(b) & 0xFFFF0000u);
  }
  activated[index] = make_uint4(words[0], words[1], words[2], words[3]);
}

// ---------------------------------------------------------------------------
// 6. combine: out[t,:] = ordered BF16 fold over the token's eight slots
//    (ascending expert id) of bf16(down[inverse[8t+j],:] * w[8t+j])
//    (moe.cu:446-456).  Eight columns per thread.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
moe_combine_kernel(const uint4* __restrict__ down, const int32_t* __restrict__ inverse,
                   const float* __restrict__ weights, uint32_t rows, uint32_t width, uint4* __restrict__ output) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  const uint32_t vectors = width / 8;
  const size_t index = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (index >= size_t(rows) * vectors) return;
  const uint32_t row = index / vectors, v = index % vectors;
  uint4 raw[kTopK];
  float w[kTopK];
#pragma unroll
  for (int j = 0; j < kTopK; ++j) {        // all eight gathered loads are in flight before the fold starts
    const uint32_t assignment = row * kTopK + j;
    raw[j] = down[size_t(inverse[assignment]) * vectors + v];
    w[j] = weights[assignment];
  }
  float sum[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sum[i] = 0.0F;
#pragma unroll
  for (int j = 0; j < kTopK; ++j) {
    float x[8];
    unpack8(raw[j], x);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float product = __bfloat162float(__float2bfloat16_rn(__fmul_rn(x[i], w[j])));
      sum[i] = __bfloat162float(__float2bfloat16_rn(__fadd_rn(sum[i], product)));
    }
  }
  uint32_t words[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    words[i] = (__float_as_uint(sum[2 * i]) >> 16) | (__float_as_uint(sum[2 * i + 1]) & 0xFFFF0000u);
  output[index] = make_uint4(words[0], words[1], words[2], words[3]);
}

// The same fold for the layer's own width (2816 = 352 vectors), one block per token: the eight row
// numbers and weights are fetched once per block, and the arithmetic is packed -- the product of two
// channels is rounded to BF16 by one cvt.rn.bf16x2.f32, and the BF16 add of the running sum is a
// single bfloat162 add.  That add rounds the exact sum once; the reference rounds FP32(a + b) to BF16,
// which is the same value: the exact sum of two BF16 numbers either fits FP32's 24 bits or its smaller
// term lies far below half a BF16 ulp of the larger one.
__global__ void __launch_bounds__(kHidden / 8)
moe_combine_token_kernel(const uint4* __restrict__ down, const int32_t* __restrict__ inverse,
                         const float* __restrict__ weights, uint32_t rows, uint4* __restrict__ output) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  constexpr uint32_t kVectors = kHidden / 8;
  __shared__ int32_t slot_row[kTopK];
  __shared__ float slot_weight[kTopK];
  const uint32_t token = blockIdx.x;
  if (threadIdx.x < kTopK) {
    slot_row[threadIdx.x] = inverse[size_t(token) * kTopK + threadIdx.x];
    slot_weight[threadIdx.x] = weights[size_t(token) * kTopK + threadIdx.x];
  }
  __syncthreads();
  const uint32_t v = threadIdx.x;
  uint4 raw[kTopK];
#pragma unroll
  for (int j = 0; j < kTopK; ++j)          // all eight gathered loads are in flight before the fold starts
    raw[j] = __ldcs(down + size_t(slot_row[j]) * kVectors + v);
  __nv_bfloat162 sum[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) sum[i] = __floats2bfloat162_rn(0.0F, 0.0F);
#pragma unroll
  for (int j = 0; j < kTopK; ++j) {
    const float w = slot_weight[j];
    const uint32_t words[4] = {raw[j].x, raw[j].y, raw[j].z, raw[j].w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 product = __floats2bfloat162_rn(__fmul_rn(__uint_as_float(words[i] << 16), w),
                                                           __fmul_rn(__uint_as_float(words[i] & 0xFFFF0000u), w));
      sum[i] = __hadd2(sum[i], product);
    }
  }
  uint4 result;
  result.x = *reinterpret_cast<const uint32_t*>(&sum[0]);
  result.y = *reinterpret_cast<const uint32_t*>(&sum[1]);
  result.z = *reinterpret_cast<const uint32_t*>(&sum[2]);
  result.w = *reinterpret_cast<const uint32_t*>(&sum[3]);
  __stcs(output + size_t(token) * kVectors + v, result);
  (void)rows;
}

__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ input, const int32_t* __restrict__ index, uint32_t divisor,
                   uint32_t rows, uint32_t vectors, uint4* __restrict__ output) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  const size_t i = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (i >= size_t(rows) * vectors) return;
  const uint32_t row = i / vectors, v = i % vectors;
  output[i] = input[size_t(uint32_t(index[row]) / divisor) * vectors + v];
}

// ---------------------------------------------------------------------------
// Expert parallelism: small all-to-all exchange + barrier over peer memory (replaces an NCCL
// all-gather / all-reduce whose latency, not its bytes, is what a step pays for).  Every rank
// owns a mailbox of 2 x 8 slots of 1024 bytes: slot (parity, source rank) = {flag, payload}.
// A call takes the next epoch from a device counter (so a replay of a captured step keeps
// counting), writes its payload into its slot of every rank's mailbox, orders those stores with
// a system-scope fence, raises the slot's flag to the epoch in every mailbox, then waits -- with
// a bound, after which it reports through the error word and returns -- until all `world` flags of
// its own mailbox show the epoch, and copies the payloads out.  Flags and payloads of consecutive
// epochs alternate between the two parities: a rank can be at most one exchange ahead of the
// slowest, which has then finished reading the parity that is written next.
// Ranks are different GPUs; one block per rank.
// ---------------------------------------------------------------------------
constexpr uint32_t kMailboxSlotBytes = 1024, kMailboxRanks = 8, kMailboxPayloadOffset = 16;

__global__ void __launch_bounds__(256)
ep_exchange_kernel(const int32_t* __restrict__ payload, uint32_t count, uint8_t* const* __restrict__ mailboxes,
                   uint32_t rank, uint32_t world, uint32_t* __restrict__ epoch_counter, int32_t* __restrict__ gathered,
                   uint32_t* __restrict__ error) {
  __shared__ uint32_t shared_epoch;
  if (threadIdx.x == 0) shared_epoch = ++(*epoch_counter);
  __syncthreads();
  const uint32_t epoch = shared_epoch, parity = epoch & 1u;
  const size_t my_slot = (size_t(parity) * kMailboxRanks + rank) * kMailboxSlotBytes;
  for (uint32_t i = threadIdx.x; i < world * count; i += blockDim.x) {
    const uint32_t peer = i / count, word = i % count;
    reinterpret_cast<int32_t*>(mailboxes[peer] + my_slot + kMailboxPayloadOffset)[word] = payload[word];
  }
  __threadfence_system();            // this thread's payload stores (and everything this GPU wrote before) first ...
  __syncthreads();
  if (threadIdx.x < world) {
    __threadfence_system();
    uint32_t* flag = reinterpret_cast<uint32_t*>(mailboxes[threadIdx.x] + my_slot);
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");   // ... then the flag
    const uint32_t* theirs = reinterpret_cast<const uint32_t*>(
        mailboxes[rank] + (size_t(parity) * kMailboxRanks + threadIdx.x) * kMailboxSlotBytes);
    const uint64_t start = ptx_global_timer();
    for (uint32_t spin = 1;; ++spin) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(theirs) : "memory");
      if (seen == epoch) break;
      if ((spin & 63u) == 0 && ptx_global_timer() - start > 2000000000ull) {
        if (error != nullptr) atomicCAS(error, 0u, 0x90000000u | (threadIdx.x << 8) | rank);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  for (uint32_t i = threadIdx.x; i < world * count; i += blockDim.x) {
    const uint32_t source = i / count, word = i % count;
    const int32_t* slot = reinterpret_cast<const int32_t*>(
        mailboxes[rank] + (size_t(parity) * kMailboxRanks + source) * kMailboxSlotBytes + kMailboxPayloadOffset);
    gathered[i] = __ldcv(slot + word);
  }
}

// ---------------------------------------------------------------------------
// 7. Expert parallelism over peer memory (no counterpart in the reference, which
//    is single GPU).  A travelling row is a 1584-byte record: 1408 bytes of
//    packed E2M1 (K = 2816) followed by its 176 E4M3 block scales in K order.
//    The dispatch kernel quantises a routed row with the destination expert's
//    input scale (same arithmetic as kernel 5), builds the record in shared memory
//    and sends it into the owning rank's buffer with one bulk copy (shared ->
//    global, no cluster fan-out); the owner re-tiles the scale bytes locally
//    and runs the grouped GEMMs on the records in place; the combine kernel
//    reads the eight result rows of a token from their owners' buffers and folds
//    them as kernel 6 does.  All other remote accesses are plain loads and stores.
// ---------------------------------------------------------------------------
constexpr uint32_t kRecordBytes = kHidden / 2 + kHidden / 16;   // 1584
static_assert(kRecordBytes % 16 == 0, "a record leaves as one bulk copy: 16-byte granules");

constexpr uint32_t kDispatchTokensPerBlock = 2;

__global__ void __launch_bounds__(64 * kDispatchTokensPerBlock)
ep_dispatch_kernel(const uint4* __restrict__ input, const int32_t* __restrict__ keys,
                   const int32_t* __restrict__ inverse, const int32_t* __restrict__ offsets,
                   const float* __restrict__ inverse_input_scale, const int32_t* __restrict__ dest_rank,
                   const int32_t* __restrict__ dest_row0, uint8_t* const* __restrict__ peer_records, uint32_t tokens,
                   uint32_t capacity_rows, uint32_t* __restrict__ error) {
  // The eight records of a token are built in shared memory and leave as eight bulk copies of 1584 bytes
  // each: the copy engine keeps the NVLink writes in flight, the warps do not wait on remote stores.
  __shared__ __align__(16) uint8_t staged[kDispatchTokensPerBlock][kTopK][kRecordBytes];
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  // token-major like kernel 5b: two warps per token, each with one half of the row (88 K16 blocks, three
  // per lane), read once for the token's eight records
  constexpr uint32_t kBlocks = kHidden / 16;            // 176
  constexpr uint32_t kHalfBlocks = kBlocks / 2;         // 88
  constexpr int kPerLane = (kHalfBlocks + 31) / 32;     // 3
  const uint32_t slot = threadIdx.x / 64, half = (threadIdx.x / 32) % 2, lane = threadIdx.x % 32;
  const uint32_t token = blockIdx.x * kDispatchTokensPerBlock + slot;
  if (token >= tokens) return;                          // both warps of a token leave together
  // lane j < 8 fetches the input scale of copy j's expert: one round of dependent loads for the token
  const float copy_scale = lane < kTopK ? inverse_input_scale[keys[token * kTopK + lane]] : 0.0F;
  uint32_t raw[kPerLane][8];
  float amax[kPerLane];
#pragma unroll
  for (int i = 0; i < kPerLane; ++i) {
    const uint32_t local = lane + 32 * i;
    const uint32_t kb = half * kHalfBlocks + local;
    amax[i] = 0.0F;
    if (local < kHalfBlocks) {
      const uint4 a = input[2 * (size_t(token) * kBlocks + kb)], b = input[2 * (size_t(token) * kBlocks + kb) + 1];
      raw[i][0] = a.x; raw[i][1] = a.y; raw[i][2] = a.z; raw[i][3] = a.w;
      raw[i][4] = b.x; raw[i][5] = b.y; raw[i][6] = b.z; raw[i][7] = b.w;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        amax[i] = fmaxf(amax[i], fabsf(__uint_as_float(raw[i][k] << 16)));
        amax[i] = fmaxf(amax[i], fabsf(__uint_as_float(raw[i][k] & 0xFFFF0000u)));
      }
    }
  }
  // A record depends on the input scale only: a copy whose expert has the scale of the copy before it
  // is sent from that copy's staged record (four bits per copy say which record it leaves from).
  uint32_t staged_in = 0;
  int last_built = 0;
  float built_with = -1.0F;            // input scales are positive
  for (int j = 0; j < kTopK; ++j) {
    const float inverse_scale = __shfl_sync(0xffffffffu, copy_scale, j);
    if (inverse_scale == built_with) {           // the same for every thread of the token
      staged_in |= uint32_t(last_built) << (4 * j);
      continue;
    }
    built_with = inverse_scale;
    last_built = j;
    staged_in |= uint32_t(j) << (4 * j);
    uint8_t* record = staged[slot][j];
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const uint32_t local = lane + 32 * i;
      const uint32_t kb = half * kHalfBlocks + local;
      if (local >= kHalfBlocks) continue;
      const uint8_t scale_code = float_to_e4m3(inverse_scale * (amax[i] * rcp_approx_ftz(6.0F)));
      const float block_scale = e4m3_to_float(scale_code);
      const float factor =
          block_scale == 0.0F ? 0.0F : rcp_approx_ftz(block_scale * rcp_approx_ftz(inverse_scale));
      uint32_t out[2] = {0, 0};
#pragma unroll
      for (int k = 0; k < 8; ++k)
        out[k / 4] |= uint32_t(float2_to_e2m1x2(__uint_as_float(raw[i][k] << 16) * factor,
                                                __uint_as_float(raw[i][k] & 0xFFFF0000u) * factor)) << (8 * (k % 4));
      *reinterpret_cast<uint2*>(record + kb * 8) = make_uint2(out[0], out[1]);
      record[kHidden / 2 + kb] = scale_code;
    }
  }
  ptx::fence_proxy_async_smem();                        // the copy engine reads what these threads wrote
  asm volatile("bar.sync %0, 64;" ::"r"(int(slot) + 1) : "memory");     // the token's two warps
  if (half == 0 && lane < kTopK) {
    const uint32_t assignment = token * kTopK + lane;
    const int32_t e = keys[assignment];
    const uint32_t dest_row = uint32_t(dest_row0[e] + inverse[assignment] - offsets[e]);
    if (dest_row >= capacity_rows) {          // the owner's buffer is too small: report, never write outside it
      if (error != nullptr) atomicCAS(error, 0u, 0x70000000u | uint32_t(e));
    } else {
      ptx::bulk_store(peer_records[dest_rank[e]] + size_t(dest_row) * kRecordBytes,
                      staged[slot][(staged_in >> (4 * lane)) & 15u], kRecordBytes);
      ptx::bulk_store_commit();
      ptx::bulk_store_wait_all();
    }
  }
}

// Where every rank's rows of every expert go, from the all-gathered histogram
// counts[source rank][expert id]: experts are laid out expert-major in physical order on
// their owner, source ranks in rank order inside an expert.  One block of 128 threads.
__global__ void __launch_bounds__(kExperts)
ep_tables_kernel(const int32_t* __restrict__ counts, const int32_t* __restrict__ physical, uint32_t rank,
                 uint32_t world, int32_t* __restrict__ dest_row0, int32_t* __restrict__ local_offsets,
                 int32_t* __restrict__ segment_start, int32_t* __restrict__ home_base) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  __shared__ int32_t total_at[kExperts];       // rows of the expert at a physical position, over all sources
  __shared__ int32_t sorted_base[8][kExperts]; // a source rank's own offsets: rows of experts with a lower id
  const uint32_t e = threadIdx.x, per_rank = kExperts / world;
  int32_t total = 0, before_me = 0;
  for (uint32_t s = 0; s < world; ++s) {
    const int32_t c = counts[s * kExperts + e];
    total += c;
    if (s < rank) before_me += c;
  }
  const uint32_t position = uint32_t(physical[e]);
  total_at[position] = total;
  if (e < world && world <= 8) {               // thread s scans source s's histogram
    int32_t running = 0;
    for (uint32_t x = 0; x < kExperts; ++x) { sorted_base[e][x] = running; running += counts[e * kExperts + x]; }
  }
  __syncthreads();
  int32_t first = 0;                            // rows of the owner's experts placed before this one
  for (uint32_t q = position / per_rank * per_rank; q < position; ++q) first += total_at[q];
  dest_row0[e] = first + before_me;
  if (position / per_rank == rank) {
    const uint32_t slot = position % per_rank;
    local_offsets[slot] = first;
    if (slot == per_rank - 1) local_offsets[per_rank] = first + total;
    if (segment_start != nullptr && world <= 8) {
      // the way home: rows [segment_start[s][slot], +counts[s][e]) of this rank's buffers came
      // from source s, where they are rows home_base[s][slot].. of its expert-sorted order
      int32_t running = first;
      for (uint32_t s = 0; s < world; ++s) {
        segment_start[s * per_rank + slot] = running;
        home_base[s * per_rank + slot] = sorted_base[s][e];
        running += counts[s * kExperts + e];
      }
    }
  }
}

// Byte address, in its source rank's memory, of the home of every row this rank's experts
// produce: the down GEMM's epilogue stores its rows there directly.
__global__ void __launch_bounds__(256)
ep_row_home_kernel(const int32_t* __restrict__ sorted_keys, const int32_t* __restrict__ offsets,
                   const int32_t* __restrict__ segment_start, const int32_t* __restrict__ home_base,
                   uint8_t* const* __restrict__ peer_returned, uint32_t first_expert, uint32_t per_rank,
                   uint32_t world, uint32_t n, uint32_t home_capacity_rows, uint32_t* __restrict__ error,
                   uint64_t* __restrict__ row_home) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  const uint32_t row = blockIdx.x * 256 + threadIdx.x;
  if (row >= n || row >= uint32_t(offsets[kExperts])) return;
  const uint32_t slot = uint32_t(sorted_keys[row]) - first_expert;
  uint32_t source = 0;
  for (uint32_t s = 1; s < world; ++s)
    if (uint32_t(segment_start[s * per_rank + slot]) <= row) source = s;     // starts are non-decreasing in s
  const uint32_t home_row = uint32_t(home_base[source * per_rank + slot]) + row - uint32_t(segment_start[source * per_rank + slot]);
  if (home_row >= home_capacity_rows) {      // inconsistent tables: park the row in this rank's own buffer, report
    if (error != nullptr) atomicCAS(error, 0u, 0x70000300u | slot);
    row_home[row] = 0;
    return;
  }
  row_home[row] = reinterpret_cast<uint64_t>(peer_returned[source]) + uint64_t(home_row) * (kHidden * 2);
}

// scale bytes of the local records -> the tiled per-expert regions the GEMM reads
__global__ void __launch_bounds__(256)
ep_retile_scales_kernel(const uint8_t* __restrict__ records, const int32_t* __restrict__ sorted_keys,
                        const int32_t* __restrict__ offsets, uint32_t n, uint8_t* __restrict__ scales) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  constexpr uint32_t kWords = kHidden / 64;        // 44 four-byte words of scales per row
  const size_t index = size_t(blockIdx.x) * 256 + threadIdx.x;
  if (index >= size_t(n) * kWords) return;
  const uint32_t row = index / kWords, word = index % kWords;
  if (row >= uint32_t(offsets[kExperts])) return;       // n may be an upper bound
  const int32_t e = sorted_keys[row];
  const int32_t first = offsets[e];
  const uint32_t value = *reinterpret_cast<const uint32_t*>(records + size_t(row) * kRecordBytes + kHidden / 2 + word * 4);
  const size_t region = size_t(first / 128 + e) * 128 * (kHidden / 16);
  *reinterpret_cast<uint32_t*>(scales + region + scale_offset(row - first, word * 4, kHidden)) = value;
}

// Expert parallelism with the down projection at the tokens' home: the owner of an expert runs gate/up
// + GeGLU + FP4 quantisation only and exports every row of its expert-major order as a 416-byte
// activation record (352 B of E2M1, 44 scale bytes in K order, padding to 16 bytes) that the row's home
// rank fetches -- 14 times fewer bytes over NVLink than the BF16 result row of the down projection.
//   export: one warp per row, from the workspace's packed rows and tiled scales
__global__ void __launch_bounds__(256)
ep_export_activations_kernel(const uint4* __restrict__ packed, const uint8_t* __restrict__ scales,
                             const int32_t* __restrict__ sorted_keys, const int32_t* __restrict__ offsets, uint32_t rows,
                             uint4* __restrict__ records) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  const uint32_t row = (blockIdx.x * 256 + threadIdx.x) / 32, lane = threadIdx.x % 32;
  if (row >= rows || row >= uint32_t(offsets[kExperts])) return;      // `rows` may be an upper bound
  constexpr uint32_t kPackedVectors = kInter / 2 / 16;                // 22
  constexpr uint32_t kScaleWords = kInter / 16 / 4;                   // 11
  constexpr uint32_t kRecordVectors = kEpActivationRecordBytes / 16;  // 26
  const int32_t e = sorted_keys[row];
  const int32_t first = offsets[e];
  uint4* record = records + size_t(row) * kRecordVectors;
  if (lane < kPackedVectors) record[lane] = packed[size_t(row) * kPackedVectors + lane];
  if (lane < kScaleWords) {
    const size_t region = size_t(first / 128 + e) * 128 * (kInter / 16);
    const uint32_t word = *reinterpret_cast<const uint32_t*>(scales + region + scale_offset(row - first, lane * 4, kInter));
    reinterpret_cast<uint32_t*>(record + kPackedVectors)[lane] = word;
  }
}

//   import: one warp per routed assignment of this rank; the record comes from the expert's owner
//   (row dest_row0[e] + position of the assignment among this rank's rows of e) and lands at the
//   assignment's position in this rank's own expert-sorted order, scales in the local tiled layout.
__global__ void __launch_bounds__(128, 8)
ep_import_activations_kernel(const int32_t* __restrict__ keys, const int32_t* __restrict__ inverse,
                             const int32_t* __restrict__ offsets, const int32_t* __restrict__ dest_rank,
                             const int32_t* __restrict__ dest_row0, const uint4* const* __restrict__ peer_records,
                             uint32_t assignments, uint32_t capacity_rows, uint32_t* __restrict__ error,
                             uint4* __restrict__ packed, uint8_t* __restrict__ scales) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  const uint32_t assignment = (blockIdx.x * 128 + threadIdx.x) / 32, lane = threadIdx.x % 32;
  if (assignment >= assignments) return;
  constexpr uint32_t kPackedVectors = kInter / 2 / 16, kScaleWords = kInter / 16 / 4;
  constexpr uint32_t kRecordVectors = kEpActivationRecordBytes / 16;
  const int32_t e = keys[assignment];
  const int32_t position = inverse[assignment], first = offsets[e];
  const size_t remote_row = size_t(dest_row0[e] + position - first);
  if (remote_row >= capacity_rows) {          // outside the owner's buffer: never read there, report
    if (error != nullptr && lane == 0) atomicCAS(error, 0u, 0x70000400u | uint32_t(e));
    return;
  }
  const uint4* record = peer_records[dest_rank[e]] + remote_row * kRecordVectors;
  if (lane < kPackedVectors) packed[size_t(position) * kPackedVectors + lane] = record[lane];
  if (lane < kScaleWords) {
    const uint32_t word = reinterpret_cast<const uint32_t*>(record + kPackedVectors)[lane];
    const size_t region = size_t(first / 128 + e) * 128 * (kInter / 16);
    *reinterpret_cast<uint32_t*>(scales + region + scale_offset(position - first, lane * 4, kInter)) = word;
  }
}

// Small blocks (128 threads, at most 64 registers): many independent blocks keep enough
// remote loads in flight to cover the NVLink latency.
__global__ void __launch_bounds__(128, 8)
ep_combine_kernel(const int32_t* __restrict__ keys, const int32_t* __restrict__ inverse,
                  const float* __restrict__ weights, const int32_t* __restrict__ offsets,
                  const int32_t* __restrict__ dest_rank, const int32_t* __restrict__ dest_row0,
                  const uint4* const* __restrict__ peer_down, uint32_t rows, uint32_t capacity_rows,
                  uint32_t* __restrict__ error, uint4* __restrict__ output) {
  griddep_launch();
  griddep_wait();     // results of earlier kernels in the stream are read from here on
  constexpr uint32_t kVectors = kHidden / 8;
  const size_t index = size_t(blockIdx.x) * 128 + threadIdx.x;
  if (index >= size_t(rows) * kVectors) return;
  const uint32_t row = index / kVectors, v = index % kVectors;
  uint4 raw[kTopK];
  float w[kTopK];
#pragma unroll
  for (int j = 0; j < kTopK; ++j) {      // all eight remote loads are in flight before the fold starts
    const uint32_t assignment = row * kTopK + j;
    const int32_t e = keys[assignment];
    const size_t remote_row = size_t(dest_row0[e] + inverse[assignment] - offsets[e]);
    if (remote_row >= capacity_rows) {       // outside the owner's buffer: never read there, report
      if (error != nullptr && v == 0) atomicCAS(error, 0u, 0x70000200u | uint32_t(e));
      raw[j] = make_uint4(0, 0, 0, 0);
    } else {
      raw[j] = peer_down[dest_rank[e]][remote_row * kVectors + v];
    }
    w[j] = weights[assignment];
  }
  float sum[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sum[i] = 0.0F;
#pragma unroll
  for (int j = 0; j < kTopK; ++j) {
    float x[8];
    unpack8(raw[j], x);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float product = __bfloat162float(__float2bfloat16_rn(__fmul_rn(x[i], w[j])));
      sum[i] = __bfloat162float(__float2bfloat16_rn(__fadd_rn(sum[i], product)));
    }
  }
  uint32_t words[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    words[i] = (__float_as_uint(sum[2 * i]) >> 16) | (__float_as_uint(sum[2 * i + 1]) & 0xFFFF0000u);
  output[index] = make_uint4(words[0], words[1], words[2], words[3]);
}

unsigned blocks_for(size_t items) { return unsigned((items + 255) / 256); }

}  // namespace

uint32_t moe_chunks(uint32_t rows) { return (rows + kChunkTokens - 1) / kChunkTokens; }

cudaError_t launch_moe_dispatch(const void* scores, const void* expert_scales, uint32_t rows, int32_t* keys,
                                float* weights, uint32_t* bitmaps, int32_t* chunk_counts, int32_t* offsets,
                                int32_t* sorted_assignments, int32_t* sorted_keys, int32_t* inverse,
                                uint32_t* barrier_state, uint32_t* error, int sm_count, bool one_launch,
                                cudaStream_t stream) {
  const uint32_t chunks = moe_chunks(rows);
  if (chunks == 1) {     // decode sizes: one block (32 warps, two tokens each) routes, scans and scatters
    launch_pdl(moe_route_kernel, chunks, 1024, stream, static_cast<const bf16*>(scores),
               static_cast<const bf16*>(expert_scales), rows, keys, weights, bitmaps, chunk_counts, offsets,
               sorted_assignments, sorted_keys, inverse);
    return cudaGetLastError();
  }
  const uint32_t resident = uint32_t(sm_count) * kRouteGridBlocksPerSm;
  if (one_launch && barrier_state != nullptr && chunks <= resident * kRouteOwnChunks) {
    launch_pdl(moe_route_grid_kernel, chunks < resident ? chunks : resident, kRouteGridThreads, stream,
               static_cast<const bf16*>(scores), static_cast<const bf16*>(expert_scales), rows, chunks, keys, weights,
               bitmaps, chunk_counts, offsets, sorted_assignments, sorted_keys, inverse, barrier_state, error);
    return cudaGetLastError();
  }
  launch_pdl(moe_route_kernel, chunks, 256, stream, static_cast<const bf16*>(scores),
             static_cast<const bf16*>(expert_scales), rows, keys, weights, bitmaps, chunk_counts,
             static_cast<int32_t*>(nullptr), static_cast<int32_t*>(nullptr), static_cast<int32_t*>(nullptr),
             static_cast<int32_t*>(nullptr));
  launch_pdl(moe_scan_kernel, 1, kExperts, stream, chunk_counts, chunks, offsets);
  launch_pdl(moe_scatter_kernel, chunks, 256, stream, keys, bitmaps, chunk_counts, offsets, rows, sorted_assignments,
             sorted_keys, inverse);
  return cudaGetLastError();
}

cudaError_t launch_moe_keys_from_offsets(const int32_t* offsets, uint32_t first_expert, uint32_t expert_count,
                                         uint32_t rows, int32_t* sorted_keys, int32_t* full_offsets,
                                         cudaStream_t stream) {
  launch_pdl(moe_keys_from_offsets_kernel, blocks_for(rows > 256 ? rows : 256), 256, stream, 
      offsets, first_expert, expert_count, rows, sorted_keys, full_offsets);
  return cudaGetLastError();
}

cudaError_t launch_moe_prepare_groups(const MoeGroupPlan& plan, GemmGroup* first_groups, GemmGroup* down_groups,
                                      cudaStream_t stream) {
  launch_pdl(moe_prepare_groups_kernel, 1, 256, stream, plan, first_groups, down_groups);
  return cudaGetLastError();
}

cudaError_t launch_moe_quantize_input(const void* input, const int32_t* gather_index, uint32_t gather_divisor,
                                      const int32_t* sorted_keys, const int32_t* offsets,
                                      const MoeExpertInfo* experts, uint32_t n, uint32_t scale_rows, int parts,
                                      uint8_t* packed, uint8_t* scales, cudaStream_t stream) {
  const dim3 grid(blocks_for(size_t(n) * (kHidden / 16)), parts);
  launch_pdl(moe_quantize_kernel<kHidden, false>, grid, 256, stream, 
      static_cast<const uint4*>(input), gather_index, sorted_keys, offsets, experts, n, scale_rows, 0,
      gather_divisor ? gather_divisor : 1, reinterpret_cast<uint2*>(packed), scales, nullptr);
  return cudaGetLastError();
}

cudaError_t launch_moe_quantize_tokens(const void* input, const int32_t* keys, const int32_t* inverse,
                                       const int32_t* offsets, const MoeExpertInfo* experts, uint32_t tokens,
                                       uint32_t scale_rows, int parts, uint8_t* packed, uint8_t* scales,
                                       cudaStream_t stream) {
  launch_pdl(moe_quantize_tokens_kernel, blocks_for(size_t(tokens) * 64), 256, stream, 
      static_cast<const uint4*>(input), keys, inverse, offsets, experts, tokens, scale_rows, parts,
      reinterpret_cast<uint2*>(packed), scales);
  return cudaGetLastError();
}

cudaError_t launch_moe_activate_quantize(const void* gate_up, const int32_t* sorted_keys, const int32_t* offsets,
                                         const MoeExpertInfo* experts, uint32_t n, uint32_t scale_rows, uint8_t* packed,
                                         uint8_t* scales, void* activated, cudaStream_t stream) {
  const dim3 grid(blocks_for(size_t(n) * (kInter / 16)), 1);
  launch_pdl(moe_quantize_kernel<kInter, true>, grid, 256, stream, 
      static_cast<const uint4*>(gate_up), nullptr, sorted_keys, offsets, experts, n, scale_rows, 2, 1,
      reinterpret_cast<uint2*>(packed), scales, static_cast<uint4*>(activated));
  return cudaGetLastError();
}

cudaError_t launch_moe_quantize_fp8(const void* input, const int32_t* gather_index, uint32_t gather_divisor,
                                    const int32_t* sorted_keys, const int32_t* offsets, const MoeExpertInfo* experts,
                                    uint32_t n, uint32_t width, int first_projection, int parts, uint8_t* packed,
                                    cudaStream_t stream) {
  const dim3 grid(blocks_for(size_t(n) * (width / 8)), parts);
  launch_pdl(moe_quantize_fp8_kernel, grid, 256, stream, static_cast<const uint4*>(input), gather_index,
             gather_divisor ? gather_divisor : 1, sorted_keys, offsets, experts, n, width / 8, first_projection,
             reinterpret_cast<uint2*>(packed));
  return cudaGetLastError();
}

cudaError_t launch_moe_activate(const void* gate_up, const int32_t* offsets, uint32_t n, void* activated,
                                cudaStream_t stream) {
  launch_pdl(moe_activate_kernel, blocks_for(size_t(n) * (kInter / 8)), 256, stream, static_cast<const uint4*>(gate_up),
             offsets, n, static_cast<uint4*>(activated));
  return cudaGetLastError();
}

cudaError_t launch_moe_combine(const void* down, const int32_t* inverse, const float* weights, uint32_t rows,
                               uint32_t width, void* output, cudaStream_t stream) {
  if (width == kHidden) {
    launch_pdl(moe_combine_token_kernel, rows, kHidden / 8, stream, static_cast<const uint4*>(down), inverse, weights, rows,
               static_cast<uint4*>(output));
    return cudaGetLastError();
  }
  launch_pdl(moe_combine_kernel, blocks_for(size_t(rows) * (width / 8)), 256, stream, 
      static_cast<const uint4*>(down), inverse, weights, rows, width, static_cast<uint4*>(output));
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const void* input, const int32_t* index, uint32_t divisor, uint32_t rows,
                               uint32_t width, void* output, cudaStream_t stream) {
  launch_pdl(gather_rows_kernel, blocks_for(size_t(rows) * (width / 8)), 256, stream, 
      static_cast<const uint4*>(input), index, divisor, rows, width / 8, static_cast<uint4*>(output));
  return cudaGetLastError();
}

cudaError_t launch_ep_dispatch(const void* input, const int32_t* keys, const int32_t* inverse, const int32_t* offsets,
                               const float* inverse_input_scale, const int32_t* dest_rank, const int32_t* dest_row0,
                               void* const* peer_records, uint32_t tokens, uint32_t capacity_rows, uint32_t* error,
                               cudaStream_t stream) {
  launch_pdl(ep_dispatch_kernel, (tokens + kDispatchTokensPerBlock - 1) / kDispatchTokensPerBlock,
             64 * kDispatchTokensPerBlock, stream,
      static_cast<const uint4*>(input), keys, inverse, offsets, inverse_input_scale, dest_rank, dest_row0,
      reinterpret_cast<uint8_t* const*>(peer_records), tokens, capacity_rows, error);
  return cudaGetLastError();
}

cudaError_t launch_ep_export_activations(const void* packed, const uint8_t* scales, const int32_t* sorted_keys,
                                         const int32_t* offsets, uint32_t rows, void* records, cudaStream_t stream) {
  launch_pdl(ep_export_activations_kernel, blocks_for(size_t(rows) * 32), 256, stream, static_cast<const uint4*>(packed), scales,
             sorted_keys, offsets, rows, static_cast<uint4*>(records));
  return cudaGetLastError();
}

cudaError_t launch_ep_import_activations(const int32_t* keys, const int32_t* inverse, const int32_t* offsets,
                                         const int32_t* dest_rank, const int32_t* dest_row0, void* const* peer_records,
                                         uint32_t assignments, uint32_t capacity_rows, uint32_t* error, void* packed,
                                         uint8_t* scales, cudaStream_t stream) {
  launch_pdl(ep_import_activations_kernel, unsigned((size_t(assignments) * 32 + 127) / 128), 128, stream, keys, inverse, offsets,
             dest_rank, dest_row0, reinterpret_cast<const uint4* const*>(peer_records), assignments, capacity_rows, error,
             static_cast<uint4*>(packed), scales);
  return cudaGetLastError();
}

cudaError_t launch_ep_exchange(const int32_t* payload, uint32_t count, void* const* mailboxes, uint32_t rank,
                               uint32_t world, uint32_t* epoch_counter, int32_t* gathered, uint32_t* error,
                               cudaStream_t stream) {
  // an ordinary launch: it must not start before the kernels queued before it have finished
  ep_exchange_kernel<<<1, 256, 0, stream>>>(payload, count, reinterpret_cast<uint8_t* const*>(mailboxes), rank, world,
                                            epoch_counter, gathered, error);
  note_launch();
  return cudaGetLastError();
}

cudaError_t launch_ep_tables(const int32_t* counts, const int32_t* physical, uint32_t rank, uint32_t world,
                             int32_t* dest_row0, int32_t* local_offsets, int32_t* segment_start, int32_t* home_base,
                             cudaStream_t stream) {
  launch_pdl(ep_tables_kernel, 1, kExperts, stream, counts, physical, rank, world, dest_row0, local_offsets, segment_start,
                                               home_base);
  return cudaGetLastError();
}

cudaError_t launch_ep_row_home(const int32_t* sorted_keys, const int32_t* offsets, const int32_t* segment_start,
                               const int32_t* home_base, void* const* peer_returned, uint32_t first_expert,
                               uint32_t per_rank, uint32_t world, uint32_t n, uint32_t home_capacity_rows,
                               uint32_t* error, uint64_t* row_home, cudaStream_t stream) {
  launch_pdl(ep_row_home_kernel, blocks_for(n), 256, stream, sorted_keys, offsets, segment_start, home_base,
                                                        reinterpret_cast<uint8_t* const*>(peer_returned), first_expert,
                                                        per_rank, world, n, home_capacity_rows, error, row_home);
  return cudaGetLastError();
}

cudaError_t launch_ep_retile_scales(const void* records, const int32_t* sorted_keys, const int32_t* offsets,
                                    uint32_t n, uint8_t* scales, cudaStream_t stream) {
  launch_pdl(ep_retile_scales_kernel, blocks_for(size_t(n) * (kHidden / 64)), 256, stream, 
      static_cast<const uint8_t*>(records), sorted_keys, offsets, n, scales);
  return cudaGetLastError();
}

cudaError_t launch_ep_combine(const int32_t* keys, const int32_t* inverse, const float* weights,
                              const int32_t* offsets, const int32_t* dest_rank, const int32_t* dest_row0,
                              void* const* peer_down, uint32_t rows, uint32_t capacity_rows, uint32_t* error,
                              void* output, cudaStream_t stream) {
  launch_pdl(ep_combine_kernel, unsigned((size_t(rows) * (kHidden / 8) + 127) / 128), 128, stream, 
      keys, inverse, weights, offsets, dest_rank, dest_row0, reinterpret_cast<const uint4* const*>(peer_down), rows,
      capacity_rows, error, static_cast<uint4*>(output));
  return cudaGetLastError();
}

}  // namespace gw
