// MoE workspace and expert table behind the C ABI: owns every buffer, strings
// the routing / permutation / quantise kernels and the two grouped tcgen05
// GEMMs together on one stream.  Mirrors sm120::MoeWorkspace
// (models/gemma4/26b_a4b/sm120/moe.cuh:20-48, moe.cu:462-545).
#include <nvtx3/nvToolsExt.h>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "common.cuh"
#include "gemm_pair_moe.h"
#include "gemm_tc.cuh"
#include "moe_kernels.h"

using namespace gw;

namespace {

constexpr uint32_t kExperts = 128;
constexpr uint32_t kHidden = 2816;
constexpr uint32_t kInter = 704;
constexpr uint32_t kMaxRows = 65536;

bool finite_positive(float v) { return v > 0.0F && std::isfinite(v); }

struct DeviceBuffer {
  void* data = nullptr;
  size_t bytes = 0;
  cudaError_t allocate(size_t n) {
    bytes = n;
    return cudaMalloc(&data, n ? n : 1);
  }
  ~DeviceBuffer() { if (data) cudaFree(data); }
  template <typename T> T* as() const { return static_cast<T*>(data); }
};

}  // namespace

struct gw_expert_table {
  DeviceBuffer maps;    // CUtensorMap[128 * kMoeMapsPerExpert] (see moe_kernels.h)
  DeviceBuffer info;    // MoeExpertInfo[128]
  DeviceBuffer bf16_copies;      // W4A16: BF16 copies of every NVFP4 matrix (gw_moe_expert_table_enable_w4a16)
  std::vector<CUtensorMap> host_maps;
  std::vector<MoeExpertInfo> host_info;
  std::vector<gw_expert_weights> bound;   // the bindings as given
  bool shared_gate_up = false;   // every expert quantises gate and up inputs with one scale
  bool all_nvfp4 = false;        // every present projection is NVFP4
  bool any_nvfp4 = false, any_bf16 = false, any_fp8 = false;
  bool w4a16 = false;            // BF16 copies exist
};

// Tuning overrides, read from the environment once, when a workspace is created:
//   GW_MOE_FORM          swap / direct / fused: plan of the grouped GEMMs (default: by batch size)
//   GW_MOE_NO_PAIR       1: never use the CTA-pair kernels (single-CTA kernels for every batch size)
//   GW_MOE_ROUTE_THREE_LAUNCHES  1: route, scan and scatter as three launches instead of one with a grid barrier
//   GW_MOE_BLOCK_N, GW_MOE_BLOCK_N_DOWN, GW_MOE_CHUNK_FIRST, GW_MOE_CHUNK_DOWN: tile / schedule of the
//                        single-CTA kernels
struct MoeTuning {
  char form = 0;
  bool no_pair = false, route_three_launches = false;
  int block_n = 0, block_n_down = 0, chunk_first = 0, chunk_down = 0;
  static int number(const char* name) {
    const char* value = std::getenv(name);
    return value ? std::atoi(value) : 0;
  }
  void read() {
    const char* forced = std::getenv("GW_MOE_FORM");
    form = forced ? forced[0] : 0;
    no_pair = number("GW_MOE_NO_PAIR") != 0;
    route_three_launches = number("GW_MOE_ROUTE_THREE_LAUNCHES") != 0;
    block_n = number("GW_MOE_BLOCK_N");
    block_n_down = number("GW_MOE_BLOCK_N_DOWN");
    chunk_first = number("GW_MOE_CHUNK_FIRST");
    chunk_down = number("GW_MOE_CHUNK_DOWN");
  }
};

// An activation tensor map, re-encoded only when what it describes changes.
struct CachedMap {
  CUtensorMap map{};
  const void* base = nullptr;
  uint64_t rows = 0, pitch = 0;
  uint32_t box = 0;
  bool get(const void* b, uint64_t row_bytes, uint64_t r, uint32_t box_rows, uint64_t pitch_bytes, std::string* error) {
    if (b == base && r == rows && box_rows == box && pitch_bytes == pitch) return true;
    if (!encode_tensor_map_2d(&map, b, row_bytes, r, box_rows, error, pitch_bytes)) return false;
    base = b; rows = r; box = box_rows; pitch = pitch_bytes;
    return true;
  }
};

struct gw_moe_workspace {
  uint32_t max_rows = 0, n = 0, scale_rows = 0, chunks = 0;
  MoeTuning tuning;
  CachedMap first_map, down_map;
  DeviceBuffer metadata, bitmaps, groups, packed_in, scales_in, gate_up, activated, packed_act, scales_act, down;
  DeviceBuffer route_barrier;   // counter and generation of the routing kernel's grid-wide barrier
  DeviceBuffer row_home;   // expert parallelism: address of every produced row's home in its source rank
  DeviceBuffer fp8_in, fp8_act;   // FP8 experts (GW_MOE_FP8_EXPERTS): E4M3 gate / up inputs [2][n, 2816], down input [n, 704]
  DeviceBuffer kind_groups;       // group descriptors of the BF16 and FP8 launches of a mixed table
  CachedMap bf16_first_map, bf16_down_map, fp8_first_map, fp8_down_map;
  int32_t *keys = nullptr, *sorted_keys = nullptr, *sorted_assignments = nullptr, *inverse = nullptr;
  int32_t *offsets = nullptr, *chunk_counts = nullptr, *local_offsets = nullptr;
  float* weights = nullptr;
  bool timing = false;
  bool capture = false;   // materialise the BF16 gate/up and activated intermediates on the fused path too
  cudaEvent_t events[7] = {};
  ~gw_moe_workspace() { for (auto& e : events) if (e) cudaEventDestroy(e); }
  // Stage boundary i of a pass (0 = start ... 6 = end): closes the NVTX range of the stage that ends here and
  // opens the next one (visible to a profiler that collects NVTX; near-free otherwise), and records the
  // timing event when stage timing is on.
  void mark(int i, cudaStream_t s) const {
    static const char* const kStageNames[6] = {"gw.moe.route_permute", "gw.moe.gather_quantise", "gw.moe.gate_up_gemm",
                                               "gw.moe.geglu_quantise", "gw.moe.down_gemm", "gw.moe.combine"};
    if (i > 0) nvtxRangePop();
    if (i < 6) nvtxRangePushA(kStageNames[i]);
    if (timing) cudaEventRecord(events[i], s);
  }
};

extern "C" {

gw_status gw_moe_expert_table_create(const gw_expert_weights* experts, uint32_t count, gw_expert_table** table) {
  clear_error();
  if (!experts || !table || count != kExperts)
    return fail(GW_INVALID_ARGUMENT, "expert table requires 128 host-resident entries");
  std::vector<CUtensorMap> maps(kExperts * kMoeMapsPerExpert);
  std::vector<MoeExpertInfo> info(kExperts);
  bool shared = true, all_nvfp4 = true, any_nvfp4 = false, any_bf16 = false, any_fp8 = false;
  std::string error;
  const auto address = [](const void* p) { return reinterpret_cast<uintptr_t>(p); };
  for (uint32_t e = 0; e < kExperts; ++e) {
    const gw_projection* proj[3] = {&experts[e].gate, &experts[e].up, &experts[e].down};
    info[e] = MoeExpertInfo{};
    for (int i = 0; i < 3; ++i) info[e].storage[i] = GW_STORAGE_ABSENT;
    if (proj[0]->storage == GW_STORAGE_ABSENT && proj[1]->storage == GW_STORAGE_ABSENT &&
        proj[2]->storage == GW_STORAGE_ABSENT)
      continue;     // lives on another rank: no rows may be routed to it here
    const std::string who = " (expert " + std::to_string(e) + ")";
    for (int i = 0; i < 3; ++i) {
      const gw_projection& p = *proj[i];
      // a projection kept elsewhere (expert parallelism with the down projection at the tokens' home:
      // the owner's table may lack nothing, the home table holds only the down matrices)
      if (p.storage == GW_STORAGE_ABSENT) continue;
      const uint32_t want_in = i < 2 ? kHidden : kInter, want_out = i < 2 ? kInter : kHidden;
      CUtensorMap* slot = &maps[e * kMoeMapsPerExpert];
      if (p.input != want_in || p.output != want_out)
        return fail(GW_INVALID_ARGUMENT, "invalid 26B expert projection shape" + who);
      info[e].storage[i] = int32_t(p.storage);
      info[e].alpha[i] = 1.0F;
      info[e].inverse_input_scale[i] = 1.0F;
      if (p.storage == GW_STORAGE_NVFP4_W4A4) {
        if (p.physical_output != (want_out + 127) / 128 * 128 || !p.nvfp4_data || !p.nvfp4_scales ||
            address(p.nvfp4_data) % 16 || address(p.nvfp4_scales) % 16 || !finite_positive(p.nvfp4_input_scale) ||
            !finite_positive(p.nvfp4_weight_scale) || !std::isfinite(1.0F / p.nvfp4_input_scale) ||
            !finite_positive(p.nvfp4_input_scale * p.nvfp4_weight_scale))
          return fail(GW_INVALID_ARGUMENT, "invalid 26B expert projection binding" + who);
        if (!encode_tensor_map_2d(slot + i, p.nvfp4_data, p.input / 2, p.physical_output, 128, &error) ||
            (i == 2 && !encode_tensor_map_2d(slot + 3, p.nvfp4_data, p.input / 2, p.physical_output, 64, &error)))
          return fail(GW_CUDA_ERROR, "expert weight descriptor: " + error);
        info[e].scales[i] = p.nvfp4_scales;
        info[e].alpha[i] = p.nvfp4_input_scale * p.nvfp4_weight_scale;   // == __fmul_rn on the device
        info[e].inverse_input_scale[i] = 1.0F / p.nvfp4_input_scale;
        any_nvfp4 = true;
      } else if (p.storage == GW_STORAGE_BF16) {
        if (!p.bf16 || address(p.bf16) % 16 || p.physical_output != p.output)
          return fail(GW_INVALID_ARGUMENT, "invalid 26B BF16 expert projection binding" + who);
        if (!encode_tensor_map_2d(slot + 4 + i, p.bf16, size_t(p.input) * 2, p.output, 128, &error))
          return fail(GW_CUDA_ERROR, "expert weight descriptor: " + error);
        any_bf16 = true;
        all_nvfp4 = false;
      } else if (p.storage == GW_STORAGE_FP8_W8A8) {
        if (!p.fp8_data || address(p.fp8_data) % 16 || p.physical_output != p.output ||
            !finite_positive(p.fp8_input_scale) || !finite_positive(p.fp8_weight_scale) ||
            !std::isfinite(1.0F / p.fp8_input_scale) || !finite_positive(p.fp8_input_scale * p.fp8_weight_scale) ||
            address(p.fp8_channel_scales) % 16)
          return fail(GW_INVALID_ARGUMENT, "invalid 26B FP8 expert projection binding" + who);
        if (!encode_tensor_map_2d(slot + 4 + i, p.fp8_data, p.input, p.output, 128, &error))
          return fail(GW_CUDA_ERROR, "expert weight descriptor: " + error);
        info[e].alpha[i] = p.fp8_input_scale * p.fp8_weight_scale;
        info[e].inverse_input_scale[i] = 1.0F / p.fp8_input_scale;
        info[e].channel_alpha[i] = p.fp8_channel_scales;
        any_fp8 = true;
        all_nvfp4 = false;
      } else {
        return fail(GW_INVALID_ARGUMENT, "invalid 26B expert projection storage" + who);
      }
    }
    const bool no_first = experts[e].gate.storage == GW_STORAGE_ABSENT && experts[e].up.storage == GW_STORAGE_ABSENT;
    if (!no_first && (experts[e].gate.storage != GW_STORAGE_NVFP4_W4A4 || experts[e].up.storage != GW_STORAGE_NVFP4_W4A4 ||
                      experts[e].gate.nvfp4_input_scale != experts[e].up.nvfp4_input_scale))
      shared = false;
  }
  auto* t = new (std::nothrow) gw_expert_table();
  if (!t) return fail(GW_CUDA_ERROR, "out of host memory");
  t->shared_gate_up = shared && all_nvfp4;
  t->all_nvfp4 = all_nvfp4;
  t->any_nvfp4 = any_nvfp4;
  t->any_bf16 = any_bf16;
  t->any_fp8 = any_fp8;
  t->host_maps = maps;
  t->host_info = info;
  t->bound.assign(experts, experts + kExperts);
  cudaError_t status = t->maps.allocate(maps.size() * sizeof(CUtensorMap));
  if (status == cudaSuccess) status = t->info.allocate(info.size() * sizeof(MoeExpertInfo));
  if (status == cudaSuccess)
    status = cudaMemcpy(t->maps.data, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
  if (status == cudaSuccess)
    status = cudaMemcpy(t->info.data, info.data(), info.size() * sizeof(MoeExpertInfo), cudaMemcpyHostToDevice);
  if (status != cudaSuccess) {
    delete t;
    return fail(GW_CUDA_ERROR, std::string("expert table upload: ") + cudaGetErrorString(status));
  }
  *table = t;
  return GW_OK;
}

gw_status gw_moe_expert_table_enable_w4a16(gw_expert_table* t, void* stream) {
  clear_error();
  if (!t) return fail(GW_INVALID_ARGUMENT, "W4A16 preparation requires an expert table");
  if (t->w4a16 || !t->any_nvfp4) return GW_OK;
  // one BF16 copy per NVFP4 matrix, padding rows included (they decode to zero)
  size_t bytes = 0;
  for (const auto& e : t->bound)
    for (const gw_projection* p : {&e.gate, &e.up, &e.down})
      if (p->storage == GW_STORAGE_NVFP4_W4A4) bytes += align_up(size_t(p->physical_output) * p->input * sizeof(bf16), 256);
  GW_CUDA_CHECK(t->bf16_copies.allocate(bytes), "BF16 copies of the NVFP4 expert weights");
  cudaStream_t s = as_stream(stream);
  std::string error;
  size_t cursor = 0;
  for (uint32_t e = 0; e < kExperts; ++e) {
    const gw_projection* proj[3] = {&t->bound[e].gate, &t->bound[e].up, &t->bound[e].down};
    for (int i = 0; i < 3; ++i) {
      const gw_projection& p = *proj[i];
      if (p.storage != GW_STORAGE_NVFP4_W4A4) continue;
      auto* copy = t->bf16_copies.as<uint8_t>() + cursor;
      cursor += align_up(size_t(p.physical_output) * p.input * sizeof(bf16), 256);
      const gw_status status = gw_nvfp4_dequantize(p.nvfp4_data, p.nvfp4_scales, p.nvfp4_weight_scale, p.input,
                                                   p.physical_output, copy, s);
      if (status != GW_OK) return status;
      if (!encode_tensor_map_2d(&t->host_maps[e * kMoeMapsPerExpert + 4 + i], copy, size_t(p.input) * 2, p.physical_output,
                                128, &error))
        return fail(GW_CUDA_ERROR, "expert weight descriptor: " + error);
    }
    t->host_info[e].bf16_copy = 1;
  }
  GW_CUDA_CHECK(cudaMemcpyAsync(t->maps.data, t->host_maps.data(), t->host_maps.size() * sizeof(CUtensorMap),
                                cudaMemcpyHostToDevice, s), "expert table upload");
  GW_CUDA_CHECK(cudaMemcpyAsync(t->info.data, t->host_info.data(), t->host_info.size() * sizeof(MoeExpertInfo),
                                cudaMemcpyHostToDevice, s), "expert table upload");
  GW_CUDA_CHECK(cudaStreamSynchronize(s), "W4A16 preparation");
  t->w4a16 = true;
  return GW_OK;
}

void gw_moe_expert_table_destroy(gw_expert_table* table) { delete table; }

gw_status gw_moe_create(uint32_t max_rows, gw_moe_workspace** workspace) {
  return gw_moe_create_ex(max_rows, 0, workspace);
}

gw_status gw_moe_create_ex(uint32_t max_rows, uint32_t flags, gw_moe_workspace** workspace) {
  clear_error();
  if (flags & ~uint32_t(GW_MOE_FP8_EXPERTS)) return fail(GW_INVALID_ARGUMENT, "unknown MoE workspace flag");
  if (!workspace || max_rows == 0 || max_rows > kMaxRows)
    return fail(GW_INVALID_ARGUMENT, "MoE capacity must be in 1..65536");
  auto* w = new (std::nothrow) gw_moe_workspace();
  if (!w) return fail(GW_CUDA_ERROR, "out of host memory");
  w->max_rows = max_rows;
  w->n = 8 * max_rows;
  const size_t n = w->n;
  // per-expert 128-row aligned regions (at most 128 blocks of padding) plus two blocks that the
  // pair kernels may read past an expert's last block (never used in a result)
  w->scale_rows = uint32_t(((n + 127) / 128 + 128 + 2) * 128);
  w->tuning.read();
  w->chunks = moe_chunks(max_rows);
  const size_t metadata_ints = 5 * n + 2 * 132 + size_t(w->chunks) * kExperts;
  cudaError_t status = w->metadata.allocate((metadata_ints + n) * sizeof(int32_t));
  if (status == cudaSuccess) status = w->bitmaps.allocate(size_t(w->chunks) * kExperts * 2 * sizeof(uint32_t));
  if (status == cudaSuccess) status = w->groups.allocate((2 * kExperts + 1 + kExperts + 1) * sizeof(GemmGroup));
  if (status == cudaSuccess) status = w->packed_in.allocate(2 * n * (kHidden / 2));
  if (status == cudaSuccess) status = w->scales_in.allocate(2 * size_t(w->scale_rows) * (kHidden / 16));
  if (status == cudaSuccess) status = w->gate_up.allocate(n * 2 * kInter * sizeof(bf16));
  if (status == cudaSuccess) status = w->activated.allocate(n * kInter * sizeof(bf16));
  if (status == cudaSuccess) status = w->packed_act.allocate(n * (kInter / 2));
  if (status == cudaSuccess) status = w->scales_act.allocate(size_t(w->scale_rows) * (kInter / 16));
  if (status == cudaSuccess) status = w->down.allocate(n * kHidden * sizeof(bf16));
  if (status == cudaSuccess) status = w->row_home.allocate(n * sizeof(uint64_t));
  if (status == cudaSuccess) status = w->route_barrier.allocate(2 * sizeof(uint32_t));
  if (status == cudaSuccess) status = cudaMemset(w->route_barrier.data, 0, 2 * sizeof(uint32_t));
  if (status == cudaSuccess) status = w->kind_groups.allocate(2 * (2 * kExperts + 1 + kExperts + 1) * sizeof(GemmGroup));
  if (status == cudaSuccess && (flags & GW_MOE_FP8_EXPERTS)) {
    status = w->fp8_in.allocate(2 * n * kHidden);
    if (status == cudaSuccess) status = w->fp8_act.allocate(n * kInter);
  }
  // Scale regions contain rows no kernel writes (tile padding); start from zero so
  // that they never hold NaN patterns.
  if (status == cudaSuccess) status = cudaMemset(w->scales_in.data, 0, w->scales_in.bytes);
  if (status == cudaSuccess) status = cudaMemset(w->scales_act.data, 0, w->scales_act.bytes);
  if (status != cudaSuccess) {
    delete w;
    return fail(GW_CUDA_ERROR, std::string("MoE workspace allocation: ") + cudaGetErrorString(status));
  }
  auto* p = w->metadata.as<int32_t>();
  w->keys = p;
  w->sorted_keys = p + n;
  w->sorted_assignments = p + 2 * n;
  w->inverse = p + 3 * n;
  w->weights = reinterpret_cast<float*>(p + 4 * n);
  w->offsets = p + 5 * n;
  w->local_offsets = p + 5 * n + 132;
  w->chunk_counts = p + 5 * n + 264;
  *workspace = w;
  return GW_OK;
}

void gw_moe_destroy(gw_moe_workspace* workspace) { delete workspace; }

gw_status gw_moe_dispatch(gw_moe_workspace* w, const void* scores_bf16, const void* expert_scales_bf16, uint32_t rows,
                          void* stream) {
  clear_error();
  if (!w) return fail(GW_INVALID_ARGUMENT, "MoE dispatch requires a workspace");
  if (rows > w->max_rows) return fail(GW_INVALID_ARGUMENT, "MoE rows exceed workspace");
  if (!rows) return GW_OK;
  if (!scores_bf16 || !expert_scales_bf16) return fail(GW_INVALID_ARGUMENT, "MoE dispatch requires scores and expert scales");
  GW_CUDA_CHECK(launch_moe_dispatch(scores_bf16, expert_scales_bf16, rows, w->keys, w->weights, w->bitmaps.as<uint32_t>(),
                                    w->chunk_counts, w->offsets, w->sorted_assignments, w->sorted_keys, w->inverse,
                                    w->route_barrier.as<uint32_t>(), device_error_word(), sm_count(),
                                    !w->tuning.route_three_launches, as_stream(stream)),
                "MoE dispatch");
  return GW_OK;
}

}  // extern "C"

namespace {

// Expert MLP over rows sorted by expert: quantise -> gate/up GEMM -> GeGLU +
// quantise -> down GEMM.  `gather_index` != nullptr reads input rows through
// the permutation (input row = index / gather_divisor); otherwise input row i
// is sorted row i.
//
// Three plans (see moe_prepare_groups_kernel): small batches put the weights on
// the 128-lane operand and an expert's few tokens on the column operand; large
// batches put tokens on the lanes, and when gate and up share their input scale
// the first GEMM's epilogue applies GeGLU and quantises the down input itself.
//
// `records` != nullptr (expert parallelism): the rows arrive already quantised as 1584-byte
// records (packed E2M1 + K-ordered scale bytes) written by the ranks that routed them; the
// GEMM reads the packed part in place and only the scale bytes are re-tiled here.
//
// `stages`: kStageFirst runs up to the quantised down input (in the workspace's packed_act / scales_act),
// kStageDown only the down GEMM over what those buffers hold; both by default.
constexpr int kStageFirst = 1, kStageDown = 2;
gw_status run_experts(gw_moe_workspace* w, const void* input, const int32_t* gather_index, uint32_t gather_divisor,
                      const int32_t* offsets, uint32_t n, const gw_expert_table* table, void* down_out, cudaStream_t s,
                      const void* records = nullptr, const uint64_t* row_home = nullptr,
                      int stages = kStageFirst | kStageDown, void* activation_records = nullptr,
                      bool* exported = nullptr) {
  if (!table->all_nvfp4)
    return fail(GW_UNSUPPORTED, "this entry point runs NVFP4 (W4A4) expert tables only; mixed tables run through gw_moe_run");
  const auto* info = table->info.as<MoeExpertInfo>();
  auto* first_groups = w->groups.as<GemmGroup>();
  auto* down_groups = first_groups + 2 * kExperts + 1;
  const MoeTuning& tune = w->tuning;
  int form = n <= 8 * 512 ? kMoeFormSwap : (table->shared_gate_up ? kMoeFormFused : kMoeFormDirect);
  if (tune.form == 's') form = kMoeFormSwap;
  if (tune.form == 'd') form = kMoeFormDirect;
  if (tune.form == 'f' && table->shared_gate_up) form = kMoeFormFused;
  // Large batches run on CTA pairs: the gate/up GEMM when one quantised copy of a row serves both
  // projections (the fused plan), the down GEMM whenever tokens sit on the lanes.
  const bool pair_first = form == kMoeFormFused && !tune.no_pair;
  const bool pair_down = form != kMoeFormSwap && !tune.no_pair;
  int block_n_first, block_n_down;
  if (form == kMoeFormSwap) {
    block_n_first = n <= 8 * 64 ? 32 : (n <= 8 * 256 ? 64 : 128);
    if (tune.block_n == 32 || tune.block_n == 64 || tune.block_n == 128) block_n_first = tune.block_n;
    block_n_down = block_n_first;
  } else {
    block_n_first = form == kMoeFormFused ? 256 : (tune.block_n == 256 ? 256 : 128);
    block_n_down = tune.block_n_down == 256 ? 256 : 128;
  }
  const int parts = table->shared_gate_up ? 1 : 2;
  w->mark(1, s);
  if (!(pair_first && pair_down)) {
    MoeGroupPlan plan{offsets, info, w->scales_in.as<uint8_t>(), w->scales_act.as<uint8_t>(), n, w->scale_rows, form,
                      block_n_first, block_n_down, table->shared_gate_up ? 1 : 0, device_error_word(), kMoeKindNvfp4, 1};
    GW_CUDA_CHECK(launch_moe_prepare_groups(plan, first_groups, down_groups, s), "MoE group descriptors");
  }
  if (!(stages & kStageFirst)) {
    // the down input is in place already
  } else if (records != nullptr) {
    GW_CUDA_CHECK(launch_ep_retile_scales(records, w->sorted_keys, offsets, n, w->scales_in.as<uint8_t>(), s),
                  "MoE scale re-tiling of received rows");
  } else if (gather_index == w->sorted_assignments && gather_divisor == 8 && n % 8 == 0 && n >= 8 * 512) {
    // whole-layer path with enough tokens to fill the GPU with one warp per token: rows are the
    // routed copies of n / 8 tokens
    GW_CUDA_CHECK(launch_moe_quantize_tokens(input, w->keys, w->inverse, offsets, info, n / 8, w->scale_rows, parts,
                                             w->packed_in.as<uint8_t>(), w->scales_in.as<uint8_t>(), s),
                  "MoE quantise (token-major)");
  } else {
    GW_CUDA_CHECK(launch_moe_quantize_input(input, gather_index, gather_divisor, w->sorted_keys, offsets, info, n,
                                            w->scale_rows, parts, w->packed_in.as<uint8_t>(), w->scales_in.as<uint8_t>(), s),
                  "MoE gather + quantise");
  }
  std::string error;
  const bool swap = form == kMoeFormSwap;
  if ((stages & kStageFirst) &&
      !w->first_map.get(records ? records : w->packed_in.data, kHidden / 2, size_t(parts) * n,
                        swap ? block_n_first : 128, records ? kEpRecordBytes : kHidden / 2, &error))
    return fail(GW_CUDA_ERROR, "MoE activation descriptor: " + error);
  if (!w->down_map.get(w->packed_act.data, kInter / 2, n, swap ? block_n_down : 128, kInter / 2, &error))
    return fail(GW_CUDA_ERROR, "MoE activation descriptor: " + error);
  w->mark(2, s);
  if (!(stages & kStageFirst)) {
    w->mark(3, s);
  } else if (pair_first) {
    PairMoeParams first{};
    first.map_tokens = w->first_map.map;
    first.map_table = table->maps.as<CUtensorMap>();
    first.experts = info;
    first.offsets = offsets;
    first.sf_tokens = w->scales_in.as<uint8_t>();
    first.capacity = n;
    first.packed_out = w->packed_act.as<uint8_t>();
    first.scales_out = w->scales_act.as<uint8_t>();
    // expert parallelism with the down projection elsewhere: the epilogue writes the travelling records itself
    if (activation_records != nullptr && !(stages & kStageDown) && !w->capture) {
      first.records_out = static_cast<uint8_t*>(activation_records);
      if (exported) *exported = true;
    }
    first.capture_gate_up = w->capture ? w->gate_up.data : nullptr;
    first.capture_activated = w->capture ? w->activated.data : nullptr;
    first.error = device_error_word();
    GW_CUDA_CHECK(launch_pair_moe_gate_up(first, sm_count(), s), "MoE grouped gate/up GEMM on CTA pairs");
    w->mark(3, s);
  } else {
    GemmParams first{};
    (swap ? first.map_c : first.map_l) = w->first_map.map;
    first.map_table = table->maps.as<CUtensorMap>();
    first.groups = first_groups;
    first.num_groups = form == kMoeFormFused ? kExperts : 2 * kExperts;
    first.k = kHidden;
    first.c_rows_per_tile = form == kMoeFormFused ? 128 : block_n_first;
    // two consecutive tiles per CTA (same token tile, same expert) before it strides on: measured best
    first.work_chunk = tune.chunk_first > 0 ? tune.chunk_first : (swap ? 1 : 2);
    first.error = device_error_word();
    if (form == kMoeFormFused) {
      first.out = w->packed_act.data;
      first.ld_out = kInter / 2;
      first.out_scales = w->scales_act.as<uint8_t>();
      first.out_width = kInter;
      first.capture_gate_up = w->capture ? w->gate_up.data : nullptr;
      first.capture_activated = w->capture ? w->activated.data : nullptr;
      GW_CUDA_CHECK(launch_gemm_tc(GemmKind::nvfp4, GemmEpilogue::geglu_quant, 256, first, sm_count(), s),
                    "MoE grouped gate/up GEMM with fused GeGLU + quantise");
      w->mark(3, s);
    } else {
      first.out = w->gate_up.data;
      first.ld_out = 2 * kInter;
      GW_CUDA_CHECK(launch_gemm_tc(GemmKind::nvfp4, swap ? GemmEpilogue::swap_store : GemmEpilogue::direct_store,
                                   block_n_first, first, sm_count(), s),
                    "MoE grouped gate/up GEMM");
      w->mark(3, s);
      GW_CUDA_CHECK(launch_moe_activate_quantize(w->gate_up.data, w->sorted_keys, offsets, info, n, w->scale_rows,
                                                 w->packed_act.as<uint8_t>(), w->scales_act.as<uint8_t>(),
                                                 w->activated.data, s),
                    "MoE GeGLU + quantise");
    }
  }
  w->mark(4, s);
  if (!(stages & kStageDown)) {
    // the caller takes the quantised activations from the workspace
  } else if (pair_down) {
    PairMoeParams down{};
    down.map_tokens = w->down_map.map;
    down.map_table = table->maps.as<CUtensorMap>();
    down.experts = info;
    down.offsets = offsets;
    down.sf_tokens = w->scales_act.as<uint8_t>();
    down.capacity = n;
    down.out = down_out;
    down.row_dest = row_home;   // rows go to their homes (possibly on other GPUs) instead of down_out
    down.error = device_error_word();
    GW_CUDA_CHECK(launch_pair_moe_down(down, sm_count(), s), "MoE grouped down GEMM on CTA pairs");
  } else {
    GemmParams down{};
    (swap ? down.map_c : down.map_l) = w->down_map.map;
    down.map_table = table->maps.as<CUtensorMap>();
    down.groups = down_groups;
    down.num_groups = kExperts;
    down.k = kInter;
    down.c_rows_per_tile = block_n_down;
    down.work_chunk = tune.chunk_down > 0 ? tune.chunk_down : (swap ? 1 : 2);
    down.out = down_out;
    down.ld_out = kHidden;
    down.row_dest = row_home;   // rows go to their homes (possibly on other GPUs) instead of down_out
    down.error = device_error_word();
    GW_CUDA_CHECK(launch_gemm_tc(GemmKind::nvfp4, swap ? GemmEpilogue::swap_store : GemmEpilogue::direct_store,
                                 block_n_down, down, sm_count(), s),
                  "MoE grouped down GEMM");
  }
  w->mark(5, s);
  return GW_OK;
}

// Expert MLP of one whole layer pass for tables with BF16 / FP8 projections, or NVFP4 weights used with
// BF16 activations (W4A16, through their BF16 copies) -- the storage mixes of MoeWorkspace::run
// (moe.cu:489-534), where each kernel of the reference skips the projections that are not of its kind.
// Every kind that is present runs its own grouped gate/up and down GEMM over the projections that run as
// that kind (the others get no work items); all of them write the shared BF16 gate_up and down buffers.
// GeGLU runs unfused, as in the reference.
gw_status run_experts_general(gw_moe_workspace* w, const void* input, uint32_t n, const gw_expert_table* table,
                              bool run_nvfp4, bool run_bf16, bool run_fp8, int fp4, cudaStream_t s) {
  const auto* info = table->info.as<MoeExpertInfo>();
  const int32_t* offsets = w->offsets;
  const MoeTuning& tune = w->tuning;
  int form = n <= 8 * 512 ? kMoeFormSwap : kMoeFormDirect;
  if (tune.form == 's') form = kMoeFormSwap;
  if (tune.form == 'd' || tune.form == 'f') form = kMoeFormDirect;
  const bool swap = form == kMoeFormSwap;
  int block_n = 128;
  if (swap) {
    block_n = n <= 8 * 64 ? 32 : (n <= 8 * 256 ? 64 : 128);
    if (tune.block_n == 32 || tune.block_n == 64 || tune.block_n == 128) block_n = tune.block_n;
  }
  const GemmEpilogue epilogue = swap ? GemmEpilogue::swap_store : GemmEpilogue::direct_store;
  const uint32_t token_box = swap ? uint32_t(block_n) : 128;
  void* expanded = w->down.data;     // the gathered BF16 rows are dead once gate/up has run: share the down buffer
  std::string error;
  w->mark(1, s);
  // ---- inputs of the gate/up GEMMs, per kind
  if (run_bf16)
    GW_CUDA_CHECK(launch_gather_rows(input, w->sorted_assignments, 8, n, kHidden, expanded, s), "MoE gather");
  if (run_nvfp4)
    GW_CUDA_CHECK(launch_moe_quantize_input(input, w->sorted_assignments, 8, w->sorted_keys, offsets, info, n, w->scale_rows,
                                            2, w->packed_in.as<uint8_t>(), w->scales_in.as<uint8_t>(), s),
                  "MoE gather + quantise");
  if (run_fp8)
    GW_CUDA_CHECK(launch_moe_quantize_fp8(input, w->sorted_assignments, 8, w->sorted_keys, offsets, info, n, kHidden, 0, 2,
                                          w->fp8_in.as<uint8_t>(), s),
                  "MoE gather + FP8 quantise");
  struct KindRun {
    bool enabled;
    int kind;
    GemmKind gemm;
    GemmGroup* groups;
    CachedMap* first_map;
    CachedMap* down_map;
    const void* first_rows;
    uint64_t first_row_bytes, first_row_count;
    const void* down_rows;
    uint64_t down_row_bytes;
  };
  auto* extra = w->kind_groups.as<GemmGroup>();
  constexpr size_t kGroupSet = 2 * kExperts + 1 + kExperts + 1;
  KindRun runs[3] = {
      {run_nvfp4, kMoeKindNvfp4, GemmKind::nvfp4, w->groups.as<GemmGroup>(), &w->first_map, &w->down_map,
       w->packed_in.data, kHidden / 2, uint64_t(2) * n, w->packed_act.data, kInter / 2},
      {run_bf16, kMoeKindBf16, GemmKind::bf16, extra, &w->bf16_first_map, &w->bf16_down_map, expanded, kHidden * 2,
       uint64_t(n), w->activated.data, kInter * 2},
      {run_fp8, kMoeKindFp8, GemmKind::fp8, extra + kGroupSet, &w->fp8_first_map, &w->fp8_down_map, w->fp8_in.data, kHidden,
       uint64_t(2) * n, w->fp8_act.data, kInter}};
  w->mark(2, s);
  for (KindRun& run : runs) {
    if (!run.enabled) continue;
    MoeGroupPlan plan{offsets, info, w->scales_in.as<uint8_t>(), w->scales_act.as<uint8_t>(), n, w->scale_rows, form,
                      block_n, block_n, 0, device_error_word(), run.kind, fp4};
    GW_CUDA_CHECK(launch_moe_prepare_groups(plan, run.groups, run.groups + 2 * kExperts + 1, s), "MoE group descriptors");
    if (!run.first_map->get(run.first_rows, run.first_row_bytes, run.first_row_count, token_box, run.first_row_bytes, &error) ||
        !run.down_map->get(run.down_rows, run.down_row_bytes, n, token_box, run.down_row_bytes, &error))
      return fail(GW_CUDA_ERROR, "MoE activation descriptor: " + error);
    GemmParams first{};
    (swap ? first.map_c : first.map_l) = run.first_map->map;
    first.map_table = table->maps.as<CUtensorMap>();
    first.groups = run.groups;
    first.num_groups = 2 * kExperts;
    first.k = kHidden;
    first.c_rows_per_tile = block_n;
    first.work_chunk = swap ? 1 : 2;
    first.out = w->gate_up.data;
    first.ld_out = 2 * kInter;
    first.error = device_error_word();
    GW_CUDA_CHECK(launch_gemm_tc(run.gemm, epilogue, block_n, first, sm_count(), s), "MoE grouped gate/up GEMM");
  }
  w->mark(3, s);
  // ---- GeGLU and the inputs of the down GEMMs
  if (run_nvfp4)
    GW_CUDA_CHECK(launch_moe_activate_quantize(w->gate_up.data, w->sorted_keys, offsets, info, n, w->scale_rows,
                                               w->packed_act.as<uint8_t>(), w->scales_act.as<uint8_t>(), w->activated.data, s),
                  "MoE GeGLU + quantise");
  else
    GW_CUDA_CHECK(launch_moe_activate(w->gate_up.data, offsets, n, w->activated.data, s), "MoE GeGLU");
  if (run_fp8)
    GW_CUDA_CHECK(launch_moe_quantize_fp8(w->activated.data, nullptr, 1, w->sorted_keys, offsets, info, n, kInter, 2, 1,
                                          w->fp8_act.as<uint8_t>(), s),
                  "MoE FP8 quantise of the down input");
  w->mark(4, s);
  for (KindRun& run : runs) {
    if (!run.enabled) continue;
    GemmParams down{};
    (swap ? down.map_c : down.map_l) = run.down_map->map;
    down.map_table = table->maps.as<CUtensorMap>();
    down.groups = run.groups + 2 * kExperts + 1;
    down.num_groups = kExperts;
    down.k = kInter;
    down.c_rows_per_tile = block_n;
    down.work_chunk = swap ? 1 : 2;
    down.out = w->down.data;
    down.ld_out = kHidden;
    down.error = device_error_word();
    GW_CUDA_CHECK(launch_gemm_tc(run.gemm, epilogue, block_n, down, sm_count(), s), "MoE grouped down GEMM");
  }
  w->mark(5, s);
  return GW_OK;
}

}  // namespace

extern "C" {

gw_status gw_moe_run(gw_moe_workspace* w, const void* input_bf16, const void* scores_bf16,
                     const void* expert_scales_bf16, const gw_expert_table* table, void* output_bf16, uint32_t rows,
                     int has_bf16, int has_fp8, int has_nvfp4, int fp4, void* stream) {
  clear_error();
  if (!w) return fail(GW_INVALID_ARGUMENT, "MoE run requires a workspace");
  if (rows > w->max_rows) return fail(GW_INVALID_ARGUMENT, "MoE rows exceed workspace");
  if (!rows) return GW_OK;
  if (!input_bf16 || !scores_bf16 || !expert_scales_bf16 || !table || !output_bf16 ||
      reinterpret_cast<uintptr_t>(input_bf16) % 16 || reinterpret_cast<uintptr_t>(output_bf16) % 16)
    return fail(GW_INVALID_ARGUMENT, "MoE run requires 16-byte aligned input/output, scores, expert scales and a bound expert table");
  // The storage flags say which kinds of expert weights the caller's table holds (the reference launches
  // one set of kernels per flag); fp4 == 0 runs NVFP4 weights with BF16 activations (W4A16).
  const bool fast = table->all_nvfp4 && has_nvfp4 && fp4;
  const bool run_nvfp4 = has_nvfp4 && fp4 && table->any_nvfp4;
  const bool w4a16 = has_nvfp4 && !fp4 && table->any_nvfp4;
  const bool run_bf16 = (has_bf16 && table->any_bf16) || w4a16;
  const bool run_fp8 = has_fp8 && table->any_fp8;
  if (!fast) {
    if (!run_nvfp4 && !run_bf16 && !run_fp8)
      return fail(GW_INVALID_ARGUMENT, "MoE run: the storage flags select none of the table's expert weights");
    if (w4a16 && !table->w4a16)
      return fail(GW_UNSUPPORTED,
                  "NVFP4 experts with BF16 activations (W4A16) need their BF16 copies: call "
                  "gw_moe_expert_table_enable_w4a16 once, at set-up");
    if (run_fp8 && !w->fp8_in.data)
      return fail(GW_UNSUPPORTED, "FP8 experts need a workspace created with GW_MOE_FP8_EXPERTS (gw_moe_create_ex)");
  }
  cudaStream_t s = as_stream(stream);
  w->mark(0, s);
  gw_status status = gw_moe_dispatch(w, scores_bf16, expert_scales_bf16, rows, stream);
  if (status != GW_OK) return status;
  if (fast)
    status = run_experts(w, input_bf16, w->sorted_assignments, 8, w->offsets, 8 * rows, table, w->down.data, s);
  else
    status = run_experts_general(w, input_bf16, 8 * rows, table, run_nvfp4, run_bf16, run_fp8, fp4, s);
  if (status != GW_OK) return status;
  GW_CUDA_CHECK(launch_moe_combine(w->down.data, w->inverse, w->weights, rows, kHidden, output_bf16, s), "MoE combine");
  w->mark(6, s);
  return GW_OK;
}

gw_status gw_moe_capture(gw_moe_workspace* w, int enable) {
  clear_error();
  if (!w) return fail(GW_INVALID_ARGUMENT, "capture switch requires a workspace");
  w->capture = enable != 0;
  return GW_OK;
}

gw_status gw_moe_stage_timing(gw_moe_workspace* w, int enable) {
  clear_error();
  if (!w) return fail(GW_INVALID_ARGUMENT, "stage timing requires a workspace");
  if (enable && !w->events[0])
    for (auto& e : w->events) GW_CUDA_CHECK(cudaEventCreate(&e), "create stage timing event");
  w->timing = enable != 0;
  return GW_OK;
}

gw_status gw_moe_stage_elapsed_ms(gw_moe_workspace* w, float* milliseconds) {
  clear_error();
  if (!w || !milliseconds || !w->events[0]) return fail(GW_INVALID_ARGUMENT, "stage timing was never enabled");
  GW_CUDA_CHECK(cudaEventSynchronize(w->events[6]), "wait for the last stage event");
  for (int i = 0; i < 6; ++i)
    GW_CUDA_CHECK(cudaEventElapsedTime(milliseconds + i, w->events[i], w->events[i + 1]), "stage elapsed time");
  return GW_OK;
}

gw_status gw_moe_run_sorted(gw_moe_workspace* w, const void* input_bf16, const int32_t* row_index,
                            const int32_t* offsets, uint32_t first_expert, uint32_t expert_count, uint32_t total_rows,
                            const gw_expert_table* table, void* output_bf16, void* stream) {
  clear_error();
  if (!w || !table) return fail(GW_INVALID_ARGUMENT, "sorted MoE run requires a workspace and an expert table");
  if (total_rows > w->n) return fail(GW_INVALID_ARGUMENT, "sorted MoE rows exceed workspace (8 x max_rows)");
  if (!total_rows) return GW_OK;
  if (!input_bf16 || !offsets || !output_bf16 || expert_count == 0 || first_expert + expert_count > kExperts ||
      reinterpret_cast<uintptr_t>(input_bf16) % 16 || reinterpret_cast<uintptr_t>(output_bf16) % 16)
    return fail(GW_INVALID_ARGUMENT, "sorted MoE run requires aligned buffers and an expert range inside 0..128");
  cudaStream_t s = as_stream(stream);
  w->mark(0, s);
  GW_CUDA_CHECK(launch_moe_keys_from_offsets(offsets, first_expert, expert_count, total_rows, w->sorted_keys,
                                             w->local_offsets, s),
                "MoE keys from offsets");
  const gw_status status = run_experts(w, input_bf16, row_index, 1, w->local_offsets, total_rows, table, output_bf16, s);
  w->mark(6, s);
  return status;
}

gw_status gw_gather_rows_bf16(const void* input_bf16, const int32_t* index, uint32_t divisor, uint32_t rows,
                              uint32_t width, void* output_bf16, void* stream) {
  clear_error();
  if (!rows) return GW_OK;
  if (!input_bf16 || !index || !output_bf16 || !divisor || !width || width % 8 ||
      reinterpret_cast<uintptr_t>(input_bf16) % 16 || reinterpret_cast<uintptr_t>(output_bf16) % 16)
    return fail(GW_INVALID_ARGUMENT, "row gather requires 16-byte aligned buffers and a width divisible by 8");
  GW_CUDA_CHECK(launch_gather_rows(input_bf16, index, divisor, rows, width, output_bf16, as_stream(stream)), "row gather");
  return GW_OK;
}

gw_status gw_moe_combine(const void* down_bf16, const int32_t* inverse, const float* weights, uint32_t rows,
                         uint32_t width, void* output_bf16, void* stream) {
  clear_error();
  if (!rows) return GW_OK;
  if (!down_bf16 || !inverse || !weights || !output_bf16 || !width || width % 8 ||
      reinterpret_cast<uintptr_t>(down_bf16) % 16 || reinterpret_cast<uintptr_t>(output_bf16) % 16)
    return fail(GW_INVALID_ARGUMENT, "MoE combine requires 16-byte aligned buffers and a width divisible by 8");
  GW_CUDA_CHECK(launch_moe_combine(down_bf16, inverse, weights, rows, width, output_bf16, as_stream(stream)), "MoE combine");
  return GW_OK;
}

// --------------------------------------------------------------------------- expert parallelism over peer memory

gw_status gw_ipc_alloc(size_t bytes, void** pointer, uint8_t* handle) {
  clear_error();
  if (!pointer || !handle || bytes == 0) return fail(GW_INVALID_ARGUMENT, "shared buffer needs a size, a pointer slot and a 64-byte handle slot");
  static_assert(sizeof(cudaIpcMemHandle_t) == GW_IPC_HANDLE_BYTES, "handle size");
  void* p = nullptr;
  GW_CUDA_CHECK(cudaMalloc(&p, bytes), "allocate shared buffer");
  cudaIpcMemHandle_t h;
  const cudaError_t status = cudaIpcGetMemHandle(&h, p);
  if (status != cudaSuccess) {
    cudaFree(p);
    return fail(GW_CUDA_ERROR, std::string("export shared buffer: ") + cudaGetErrorString(status));
  }
  std::memcpy(handle, &h, sizeof(h));
  *pointer = p;
  return GW_OK;
}

gw_status gw_ipc_open(const uint8_t* handle, void** pointer) {
  clear_error();
  if (!handle || !pointer) return fail(GW_INVALID_ARGUMENT, "opening a shared buffer needs its handle and a pointer slot");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  GW_CUDA_CHECK(cudaIpcOpenMemHandle(pointer, h, cudaIpcMemLazyEnablePeerAccess), "open a peer's shared buffer");
  return GW_OK;
}

gw_status gw_ipc_close(void* pointer) {
  clear_error();
  if (pointer) GW_CUDA_CHECK(cudaIpcCloseMemHandle(pointer), "close a peer's shared buffer");
  return GW_OK;
}

gw_status gw_ipc_free(void* pointer) {
  clear_error();
  if (pointer) GW_CUDA_CHECK(cudaFree(pointer), "free shared buffer");
  return GW_OK;
}

size_t gw_moe_ep_mailbox_bytes(void) { return kEpMailboxBytes; }

gw_status gw_moe_ep_exchange(const int32_t* payload, uint32_t count, void* const* peer_mailboxes, uint32_t rank,
                             uint32_t world, uint32_t* epoch_counter, int32_t* gathered, void* stream) {
  clear_error();
  if (!peer_mailboxes || !epoch_counter || world == 0 || world > 8 || rank >= world || count > kEpMailboxMaxInts ||
      (count != 0 && (!payload || !gathered)))
    return fail(GW_INVALID_ARGUMENT, "exchange requires the ranks' mailboxes, an epoch counter, at most 8 ranks and 252 values");
  GW_CUDA_CHECK(launch_ep_exchange(payload, count, peer_mailboxes, rank, world, epoch_counter, gathered, device_error_word(),
                                   as_stream(stream)),
                "exchange over peer memory");
  return GW_OK;
}

gw_status gw_moe_ep_tables(const int32_t* counts, const int32_t* physical, uint32_t rank, uint32_t world,
                           int32_t* dest_row0, int32_t* local_offsets, int32_t* segment_start, int32_t* home_base,
                           void* stream) {
  clear_error();
  if (!counts || !physical || !dest_row0 || !local_offsets || world == 0 || kExperts % world || rank >= world ||
      (segment_start == nullptr) != (home_base == nullptr))
    return fail(GW_INVALID_ARGUMENT, "destination tables need the gathered histogram, the placement and a rank count that divides 128");
  if (segment_start != nullptr && world > 8)
    return fail(GW_UNSUPPORTED, "the way-home tables are built for at most 8 ranks (one node)");
  GW_CUDA_CHECK(launch_ep_tables(counts, physical, rank, world, dest_row0, local_offsets, segment_start, home_base,
                                 as_stream(stream)),
                "expert-parallel destination tables");
  return GW_OK;
}

gw_status gw_moe_ep_dispatch(gw_moe_workspace* w, const void* input_bf16, uint32_t rows,
                             const float* inverse_input_scales, const int32_t* dest_rank, const int32_t* dest_row0,
                             void* const* peer_records, uint32_t capacity_rows, void* stream) {
  clear_error();
  if (!w) return fail(GW_INVALID_ARGUMENT, "expert-parallel dispatch requires the workspace that routed the rows");
  if (rows > w->max_rows) return fail(GW_INVALID_ARGUMENT, "MoE rows exceed workspace");
  if (!rows) return GW_OK;
  if (!input_bf16 || !inverse_input_scales || !dest_rank || !dest_row0 || !peer_records ||
      reinterpret_cast<uintptr_t>(input_bf16) % 16)
    return fail(GW_INVALID_ARGUMENT, "expert-parallel dispatch requires a 16-byte aligned input and the destination tables");
  GW_CUDA_CHECK(launch_ep_dispatch(input_bf16, w->keys, w->inverse, w->offsets, inverse_input_scales, dest_rank,
                                   dest_row0, peer_records, rows, capacity_rows, device_error_word(), as_stream(stream)),
                "expert-parallel dispatch");
  return GW_OK;
}

gw_status gw_moe_ep_run_experts(gw_moe_workspace* w, const void* records, const int32_t* offsets, uint32_t first_expert,
                                uint32_t expert_count, uint32_t total_rows, const gw_expert_table* table,
                                void* down_bf16, const int32_t* segment_start, const int32_t* home_base,
                                void* const* peer_returned, uint32_t home_capacity_rows, uint32_t world,
                                void* stream) {
  clear_error();
  if (!w || !table) return fail(GW_INVALID_ARGUMENT, "expert run requires a workspace and an expert table");
  if (!table->shared_gate_up)
    return fail(GW_UNSUPPORTED, "records carry one quantised copy of a row: gate and up must share their input scale");
  if (total_rows > w->n) return fail(GW_INVALID_ARGUMENT, "received rows exceed workspace (8 x max_rows)");
  if (!total_rows) return GW_OK;
  const bool push = peer_returned != nullptr;
  if (!records || !offsets || (!down_bf16 && !push) || expert_count == 0 || first_expert + expert_count > kExperts ||
      reinterpret_cast<uintptr_t>(records) % 16 || reinterpret_cast<uintptr_t>(down_bf16) % 16)
    return fail(GW_INVALID_ARGUMENT, "expert run requires aligned buffers and an expert range inside 0..128");
  if (push && (!segment_start || !home_base || world == 0 || world > 8 || expert_count * world != kExperts))
    return fail(GW_INVALID_ARGUMENT, "sending rows home requires the way-home tables of gw_moe_ep_tables and 128 / world experts");
  cudaStream_t s = as_stream(stream);
  w->mark(0, s);
  GW_CUDA_CHECK(launch_moe_keys_from_offsets(offsets, first_expert, expert_count, total_rows, w->sorted_keys,
                                             w->local_offsets, s),
                "MoE keys from offsets");
  if (push)
    GW_CUDA_CHECK(launch_ep_row_home(w->sorted_keys, w->local_offsets, segment_start, home_base, peer_returned,
                                     first_expert, expert_count, world, total_rows, home_capacity_rows,
                                     device_error_word(), w->row_home.as<uint64_t>(), s),
                  "addresses of the rows' homes");
  const gw_status status = run_experts(w, nullptr, nullptr, 1, w->local_offsets, total_rows, table,
                                       push ? w->down.data : down_bf16, s, records,
                                       push ? w->row_home.as<uint64_t>() : nullptr);
  w->mark(6, s);
  return status;
}

size_t gw_moe_ep_activation_record_bytes(void) { return kEpActivationRecordBytes; }

gw_status gw_moe_ep_run_gate_up(gw_moe_workspace* w, const void* records, const int32_t* offsets, uint32_t first_expert,
                                uint32_t expert_count, uint32_t total_rows, const gw_expert_table* table,
                                void* activation_records, void* stream) {
  clear_error();
  if (!w || !table) return fail(GW_INVALID_ARGUMENT, "expert run requires a workspace and an expert table");
  if (!table->shared_gate_up)
    return fail(GW_UNSUPPORTED, "records carry one quantised copy of a row: gate and up must share their input scale");
  if (total_rows > w->n) return fail(GW_INVALID_ARGUMENT, "received rows exceed workspace (8 x max_rows)");
  if (!total_rows) return GW_OK;
  if (!records || !offsets || !activation_records || expert_count == 0 || first_expert + expert_count > kExperts ||
      reinterpret_cast<uintptr_t>(records) % 16 || reinterpret_cast<uintptr_t>(activation_records) % 16)
    return fail(GW_INVALID_ARGUMENT, "expert run requires aligned buffers and an expert range inside 0..128");
  cudaStream_t s = as_stream(stream);
  w->mark(0, s);
  GW_CUDA_CHECK(launch_moe_keys_from_offsets(offsets, first_expert, expert_count, total_rows, w->sorted_keys,
                                             w->local_offsets, s),
                "MoE keys from offsets");
  bool exported = false;
  const gw_status status = run_experts(w, nullptr, nullptr, 1, w->local_offsets, total_rows, table, nullptr, s, records, nullptr,
                                       kStageFirst, activation_records, &exported);
  if (status != GW_OK) return status;
  if (!exported)      // plans whose gate/up epilogue does not write the records itself
    GW_CUDA_CHECK(launch_ep_export_activations(w->packed_act.data, w->scales_act.as<uint8_t>(), w->sorted_keys,
                                               w->local_offsets, total_rows, activation_records, s),
                  "export of the quantised activations");
  w->mark(6, s);
  return GW_OK;
}

gw_status gw_moe_ep_finish_at_home(gw_moe_workspace* w, uint32_t rows, const int32_t* dest_rank, const int32_t* dest_row0,
                                   void* const* peer_activation_records, uint32_t capacity_rows,
                                   const gw_expert_table* down_table, void* output_bf16, void* stream) {
  clear_error();
  if (!w || !down_table) return fail(GW_INVALID_ARGUMENT, "finishing at home requires the workspace that routed the rows and a table of down projections");
  if (rows > w->max_rows) return fail(GW_INVALID_ARGUMENT, "MoE rows exceed workspace");
  if (!rows) return GW_OK;
  if (!dest_rank || !dest_row0 || !peer_activation_records || !output_bf16 || reinterpret_cast<uintptr_t>(output_bf16) % 16)
    return fail(GW_INVALID_ARGUMENT, "finishing at home requires the destination tables and a 16-byte aligned output");
  for (const MoeExpertInfo& e : down_table->host_info)
    if (e.storage[2] != GW_STORAGE_NVFP4_W4A4)
      return fail(GW_INVALID_ARGUMENT, "the home table must hold the NVFP4 down projection of all 128 experts");
  cudaStream_t s = as_stream(stream);
  w->mark(0, s);
  GW_CUDA_CHECK(launch_ep_import_activations(w->keys, w->inverse, w->offsets, dest_rank, dest_row0, peer_activation_records,
                                             8 * rows, capacity_rows, device_error_word(), w->packed_act.data,
                                             w->scales_act.as<uint8_t>(), s),
                "import of the quantised activations");
  const gw_status status = run_experts(w, nullptr, nullptr, 1, w->offsets, 8 * rows, down_table, w->down.data, s, nullptr,
                                       nullptr, kStageDown);
  if (status != GW_OK) return status;
  GW_CUDA_CHECK(launch_moe_combine(w->down.data, w->inverse, w->weights, rows, kHidden, output_bf16, s), "MoE combine");
  w->mark(6, s);
  return GW_OK;
}

gw_status gw_moe_ep_combine(gw_moe_workspace* w, uint32_t rows, const int32_t* dest_rank, const int32_t* dest_row0,
                            void* const* peer_down, uint32_t capacity_rows, void* output_bf16, void* stream) {
  clear_error();
  if (!w) return fail(GW_INVALID_ARGUMENT, "expert-parallel combine requires the workspace that routed the rows");
  if (rows > w->max_rows) return fail(GW_INVALID_ARGUMENT, "MoE rows exceed workspace");
  if (!rows) return GW_OK;
  if (!dest_rank || !dest_row0 || !peer_down || !output_bf16 || reinterpret_cast<uintptr_t>(output_bf16) % 16)
    return fail(GW_INVALID_ARGUMENT, "expert-parallel combine requires the destination tables and a 16-byte aligned output");
  GW_CUDA_CHECK(launch_ep_combine(w->keys, w->inverse, w->weights, w->offsets, dest_rank, dest_row0, peer_down, rows,
                                  capacity_rows, device_error_word(), output_bf16, as_stream(stream)),
                "expert-parallel combine");
  return GW_OK;
}

gw_status gw_debug_moe_quantized_input(const gw_moe_workspace* w, const uint8_t** packed, const uint8_t** scales,
                                       uint32_t* scale_rows, uint32_t* part_rows) {
  clear_error();
  if (!w || !packed || !scales || !scale_rows || !part_rows)
    return fail(GW_INVALID_ARGUMENT, "quantised-input accessor requires a workspace and four result slots");
  *packed = w->packed_in.as<uint8_t>();
  *scales = w->scales_in.as<uint8_t>();
  *scale_rows = w->scale_rows;
  *part_rows = w->n;
  return GW_OK;
}

const int32_t* gw_moe_selected_experts(const gw_moe_workspace* w) { return w ? w->keys : nullptr; }
const float* gw_moe_routing_weights(const gw_moe_workspace* w) { return w ? w->weights : nullptr; }
const int32_t* gw_moe_offsets(const gw_moe_workspace* w) { return w ? w->offsets : nullptr; }
const int32_t* gw_moe_inverse(const gw_moe_workspace* w) { return w ? w->inverse : nullptr; }
const int32_t* gw_moe_sorted_assignments(const gw_moe_workspace* w) { return w ? w->sorted_assignments : nullptr; }
const void* gw_moe_gate_up_capture(const gw_moe_workspace* w) { return w ? w->gate_up.data : nullptr; }
const void* gw_moe_activated_capture(const gw_moe_workspace* w) { return w ? w->activated.data : nullptr; }
const void* gw_moe_down_capture(const gw_moe_workspace* w) { return w ? w->down.data : nullptr; }
size_t gw_moe_routing_bytes(const gw_moe_workspace* w) { return w ? w->metadata.bytes + w->bitmaps.bytes + w->groups.bytes : 0; }
size_t gw_moe_projection_bytes(const gw_moe_workspace* w) {
  return w ? w->packed_in.bytes + w->scales_in.bytes + w->gate_up.bytes + w->activated.bytes + w->packed_act.bytes +
                 w->scales_act.bytes : 0;
}
size_t gw_moe_reduction_bytes(const gw_moe_workspace* w) { return w ? w->down.bytes : 0; }
size_t gw_moe_bytes(const gw_moe_workspace* w) {
  return gw_moe_routing_bytes(w) + gw_moe_projection_bytes(w) + gw_moe_reduction_bytes(w);
}

}  // extern "C"
