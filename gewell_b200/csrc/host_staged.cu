// MoE layer passes whose tokens and results live in pinned HOST memory, behind
// the C ABI (gw_moe_host_runner_*).  The reference keeps activations on the
// device throughout (its callers are its own executors), so this runner has no
// counterpart there; it is the entry point for a caller that holds activations
// on the host and therefore pays a host->device copy of the token rows and
// router logits and a device->host copy of the layer output on every pass.
//
// Issued on one stream those three steps would run one after another.  The
// runner gives each its own stream and a ring of `depth` device buffers, so the
// upload of pass i+1 and the download of pass i-1 overlap the kernels of pass i
// (PCIe is full duplex; the copies use the copy engines, not the SMs).  Kernels
// of consecutive passes still run in order on the compute stream -- a
// workspace is one set of scratch buffers -- and results are bit-identical to
// gw_moe_run on device buffers.
#include <new>
#include <string>
#include <vector>

#include "common.cuh"

using namespace gw;

namespace {
constexpr uint32_t kHidden = 2816, kExperts = 128;
}

struct gw_moe_host_runner {
  gw_moe_workspace* workspace = nullptr;
  const gw_expert_table* table = nullptr;
  const void* expert_scales = nullptr;
  uint32_t max_rows = 0, depth = 0;
  cudaStream_t upload = nullptr, compute = nullptr, download = nullptr;
  struct Slot {
    void *x = nullptr, *scores = nullptr, *y = nullptr;
    cudaEvent_t uploaded = nullptr, computed = nullptr, downloaded = nullptr;
    bool used = false;
  };
  std::vector<Slot> slots;
  uint64_t submitted = 0, h2d_bytes = 0, d2h_bytes = 0;

  ~gw_moe_host_runner() {
    for (auto& s : slots) {
      if (s.x) cudaFree(s.x);
      if (s.scores) cudaFree(s.scores);
      if (s.y) cudaFree(s.y);
      for (cudaEvent_t e : {s.uploaded, s.computed, s.downloaded})
        if (e) cudaEventDestroy(e);
    }
    for (cudaStream_t s : {upload, compute, download})
      if (s) cudaStreamDestroy(s);
  }
};

extern "C" {

gw_status gw_moe_host_runner_create(gw_moe_workspace* workspace, const gw_expert_table* table,
                                    const void* expert_scales_bf16, uint32_t max_rows, uint32_t depth,
                                    gw_moe_host_runner** runner) {
  clear_error();
  if (!workspace || !table || !expert_scales_bf16 || !runner || max_rows == 0 || depth == 0 || depth > 16)
    return fail(GW_INVALID_ARGUMENT,
                "host runner requires a workspace, a bound expert table, device expert scales, rows > 0 and a ring "
                "depth in 1..16");
  auto* r = new (std::nothrow) gw_moe_host_runner();
  if (!r) return fail(GW_CUDA_ERROR, "out of host memory");
  r->workspace = workspace;
  r->table = table;
  r->expert_scales = expert_scales_bf16;
  r->max_rows = max_rows;
  r->depth = depth;
  r->slots.resize(depth);
  cudaError_t status = cudaStreamCreateWithFlags(&r->upload, cudaStreamNonBlocking);
  if (status == cudaSuccess) status = cudaStreamCreateWithFlags(&r->compute, cudaStreamNonBlocking);
  if (status == cudaSuccess) status = cudaStreamCreateWithFlags(&r->download, cudaStreamNonBlocking);
  for (auto& s : r->slots) {
    if (status == cudaSuccess) status = cudaMalloc(&s.x, size_t(max_rows) * kHidden * 2);
    if (status == cudaSuccess) status = cudaMalloc(&s.scores, size_t(max_rows) * kExperts * 2);
    if (status == cudaSuccess) status = cudaMalloc(&s.y, size_t(max_rows) * kHidden * 2);
    if (status == cudaSuccess) status = cudaEventCreateWithFlags(&s.uploaded, cudaEventDisableTiming);
    if (status == cudaSuccess) status = cudaEventCreateWithFlags(&s.computed, cudaEventDisableTiming);
    if (status == cudaSuccess) status = cudaEventCreateWithFlags(&s.downloaded, cudaEventDisableTiming);
  }
  if (status != cudaSuccess) {
    delete r;
    return fail(GW_CUDA_ERROR, std::string("host runner set-up: ") + cudaGetErrorString(status));
  }
  *runner = r;
  return GW_OK;
}

void gw_moe_host_runner_destroy(gw_moe_host_runner* runner) {
  if (runner) {
    for (cudaStream_t s : {runner->upload, runner->compute, runner->download})
      if (s) cudaStreamSynchronize(s);
    delete runner;
  }
}

gw_status gw_moe_host_runner_submit(gw_moe_host_runner* r, const void* host_x, const void* host_scores,
                                    void* host_y, uint32_t rows, uint64_t* ticket) {
  clear_error();
  if (!r) return fail(GW_INVALID_ARGUMENT, "submit requires a host runner");
  if (rows > r->max_rows) return fail(GW_INVALID_ARGUMENT, "rows exceed the host runner's capacity");
  if (rows != 0 && (!host_x || !host_scores || !host_y))
    return fail(GW_INVALID_ARGUMENT, "submit requires host buffers for tokens, router logits and output");
  const uint64_t number = r->submitted;
  if (rows != 0) {
    auto& s = r->slots[number % r->depth];
    // the slot's previous pass no longer reads its inputs / its output has left the device
    if (s.used) GW_CUDA_CHECK(cudaStreamWaitEvent(r->upload, s.computed, 0), "host runner: order upload after compute");
    GW_CUDA_CHECK(cudaMemcpyAsync(s.x, host_x, size_t(rows) * kHidden * 2, cudaMemcpyHostToDevice, r->upload),
                  "host runner: upload tokens");
    GW_CUDA_CHECK(cudaMemcpyAsync(s.scores, host_scores, size_t(rows) * kExperts * 2, cudaMemcpyHostToDevice, r->upload),
                  "host runner: upload router logits");
    GW_CUDA_CHECK(cudaEventRecord(s.uploaded, r->upload), "host runner: record upload");
    GW_CUDA_CHECK(cudaStreamWaitEvent(r->compute, s.uploaded, 0), "host runner: order compute after upload");
    if (s.used) GW_CUDA_CHECK(cudaStreamWaitEvent(r->compute, s.downloaded, 0), "host runner: order compute after download");
    const gw_status status = gw_moe_run(r->workspace, s.x, s.scores, r->expert_scales, r->table, s.y, rows, 0, 0, 1, 1,
                                        r->compute);
    if (status != GW_OK) return status;
    GW_CUDA_CHECK(cudaEventRecord(s.computed, r->compute), "host runner: record compute");
    GW_CUDA_CHECK(cudaStreamWaitEvent(r->download, s.computed, 0), "host runner: order download after compute");
    GW_CUDA_CHECK(cudaMemcpyAsync(host_y, s.y, size_t(rows) * kHidden * 2, cudaMemcpyDeviceToHost, r->download),
                  "host runner: download output");
    GW_CUDA_CHECK(cudaEventRecord(s.downloaded, r->download), "host runner: record download");
    s.used = true;
    r->h2d_bytes += uint64_t(rows) * (kHidden + kExperts) * 2;
    r->d2h_bytes += uint64_t(rows) * kHidden * 2;
  }
  if (ticket) *ticket = number;
  r->submitted = number + 1;
  return GW_OK;
}

gw_status gw_moe_host_runner_wait(gw_moe_host_runner* r, uint64_t ticket) {
  clear_error();
  if (!r || ticket >= r->submitted) return fail(GW_INVALID_ARGUMENT, "no such pass");
  // downloads run in order: the newest download queued on the pass's slot is not earlier than its own
  auto& s = r->slots[ticket % r->depth];
  if (s.used) GW_CUDA_CHECK(cudaEventSynchronize(s.downloaded), "host runner: wait for a pass");
  return GW_OK;
}

gw_status gw_moe_host_runner_synchronize(gw_moe_host_runner* r) {
  clear_error();
  if (!r) return fail(GW_INVALID_ARGUMENT, "synchronize requires a host runner");
  for (cudaStream_t s : {r->upload, r->compute, r->download})
    GW_CUDA_CHECK(cudaStreamSynchronize(s), "host runner: synchronize");
  return GW_OK;
}

gw_status gw_moe_host_runner_streams(gw_moe_host_runner* r, void** upload, void** compute, void** download) {
  clear_error();
  if (!r || !upload || !compute || !download) return fail(GW_INVALID_ARGUMENT, "stream query requires a host runner");
  *upload = r->upload;
  *compute = r->compute;
  *download = r->download;
  return GW_OK;
}

uint64_t gw_moe_host_runner_h2d_bytes(const gw_moe_host_runner* r) { return r ? r->h2d_bytes : 0; }
uint64_t gw_moe_host_runner_d2h_bytes(const gw_moe_host_runner* r) { return r ? r->d2h_bytes : 0; }

}  // extern "C"
